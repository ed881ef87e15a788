// The dense part of an encoder layer boundary in ONE kernel (inference):
//
//     tail of layer l      y  = x + attn Wo^T + bo
//                          x' = y + relu(y W1^T + b1) W2^T + b2            (hidden units in chunks of 128, never stored)
//     head of layer l+1    q|k|v = x' Wqkv^T + bqkv ;  a = width(q . w_pos) ;  q <- q / sqrt(16)
//
// (models/indexed_latticeformer_encoder.py:848-890 without LayerNorm, and the in-projection and Gaussian-width
// pipeline of models/indexed_lattice_multi_head_attention_cuda.py:582-722.)  The reference - and the cuBLAS path of
// cf_encoder_forward - runs this as four GEMMs and two element-wise passes per layer, each a separate launch over a
// few thousand rows.  Here a thread block owns a tile of 16 MT atom rows and carries it through all four
// products; only x', q, k, v and a are written.
//
// Arithmetic: fp32-level accuracy on the tensor cores by splitting both operands, a = a_hi + a_lo with a_hi = tf32(a)
// (so |a_lo| <= 2^-11 |a|), and summing
//     a b ~ a_hi b_hi  +  ( a_lo b_hi + a_hi b_lo ),
// the first product in TF32 (exact products of 11-bit mantissas, fp32 accumulation), the bracket - 2^-11 of the
// result - in bfloat16 with fp32 accumulation as ONE 16-deep product: its A operand interleaves (a_lo, a_hi) along k
// and its B operand (b_hi, b_lo), so that a k step of 8 costs two tensor instructions (m16n8k8 TF32 + m16n8k16 BF16)
// instead of the three of an all-TF32 split; every legacy MMA shape issues at the same rate on this GPU (0.46 per
// clock and SM, measured), so that is a third less tensor time.  Error per term: 2^-22 (a_lo b_lo dropped) + about
// 2^-20 (bfloat16 rounding of the bracket's operands), i.e. 1e-6 relative, the level of an fp32 dot product of this
// length.  Warp-level mma (a 16-row tile per instruction) fits the ragged, few-thousand-row batches; the 64/128-row
// tiles of the block-level tensor instructions would leave most SMs idle at these sizes.  Weights are pre-split and
// stored in fragment order by the host (pack order documented at DensePacked), so a B fragment is one 16-byte load
// per lane; activations are split when they are written to shared memory: the `hi` tile holds TF32 words, the `lo`
// tile the words { lower half: bf16(a_lo), upper half: bf16(a_hi) }, which ldmatrix delivers as the A fragment of the
// 16-deep bfloat16 product with the same addresses as the TF32 fragment of the hi tile.
#include <type_traits>
#include "common.cuh"
#include "dense_block.cuh"

namespace cf {
namespace {

// Warp w = 8 kh + cp: column pair cp owns output columns 16 cp .. 16 cp + 15 of every 128-wide product, k half kh the
// k steps 8 kh .. 8 kh + 7 of it.  The two halves of a product are added through shared memory by the kh = 0 warp,
// which also holds biases and residuals and does the epilogues.  Sixteen warps instead of eight halve the dependent
// chain of a product and double the warps a scheduler can choose from; the tile has too few rows to give them more
// columns.
constexpr int KSPLIT = 2;
constexpr int KSTEPS = 16 / KSPLIT;       // k steps of a 128-deep product per warp
constexpr int DB_THREADS = 256 * KSPLIT;
constexpr int DB_WARPS = DB_THREADS / 32;
constexpr int LDA = 132;                  // row stride of the operand tiles (words): 528 bytes, so the eight 16-byte rows
                                          // of an ldmatrix fall into distinct bank groups

__device__ __forceinline__ unsigned tf32_hi(float x)
{
    unsigned r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

// ldmatrix from the 32-bit shared address `addr` + a compile-time byte offset (no address arithmetic at run time)
template <int OFFSET>
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr), "n"(OFFSET));
}

// f(integral_constant<int, I>) for I = FIRST .. LAST - 1: loops whose index must be a compile-time constant (immediate
// operands of the inline assembly)
template <int FIRST, int LAST, typename F>
__device__ __forceinline__ void static_for(F &&f)
{
    if constexpr (FIRST < LAST) {
        f(std::integral_constant<int, FIRST>{});
        static_for<FIRST + 1, LAST>(f);
    }
}

// the word of the correction operand: lower half bf16(lo), upper half bf16(hi)
__device__ __forceinline__ unsigned corr_word(float hi, float lo)
{
    unsigned r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ void mma_bf16_k16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- weight stream ---------------------------------------------------------------------------------------------------
// A warp consumes its B fragments in an order that is fixed in advance: panel after panel (a panel = the 16 k steps of
// one 128-deep product for the warp's two column tiles), the same sequence for every row tile.  The packed layout
// makes a fragment lane-private (a lane reads back exactly the 16 bytes it fetched), so each warp runs its own
// cp.async ring with no block-level synchronisation: weights stream from L2 continuously, across product, barrier
// and tile boundaries alike, while the tensor cores work.  The ring holds exactly one product (DEPTH = KSTEPS slots
// of two 512-byte fragments), so slot s always carries k step s of a product: every shared-memory address of the
// inner loop is a compile-time offset from one register.  The k steps are consumed in groups of G; right after a
// group's fragments have been read into registers its slots are refilled with the same k steps of the NEXT product
// (one commit per group), so the stream runs one product ahead.
constexpr int DEPTH = KSTEPS;             // slots per warp, 1 KB each
constexpr int RING_WORDS = DEPTH * 2 * 32 * 4;

struct Panel {
    const float4 *base;   // fragments of column pair cp's first column tile at k step 0
    size_t tile_stride;   // float4 between the pair's two column tiles
};

struct StreamPlan {
    const float4 *Wo, *W1, *W2, *Wqkv, *Wembed;
    int ff, tail, panels;

    __device__ __forceinline__ Panel panel(int idx, int cp) const
    {
        const int chunks = ff / 128;
        Panel r;
        if (Wembed != nullptr && idx == 0) {  // the embedding comes first (never together with a tail)
            r.base = Wembed + (size_t)(2 * cp) * 16 * 32;
            r.tile_stride = 16 * 32;
        } else if (tail && idx == 0) {
            r.base = Wo + (size_t)(2 * cp) * 16 * 32;
            r.tile_stride = 16 * 32;
        } else if (tail && idx <= 2 * chunks) {
            const int ch = (idx - 1) >> 1;
            if ((idx - 1) & 1) {  // W2, k steps 16 ch .. 16 ch + 15 of column tiles 2 cp, 2 cp + 1
                r.base = W2 + ((size_t)(2 * cp) * (ff / 8) + 16 * ch) * 32;
                r.tile_stride = (size_t)(ff / 8) * 32;
            } else {              // W1, column tiles of the chunk's hidden units
                r.base = W1 + (size_t)(16 * ch + 2 * cp) * 16 * 32;
                r.tile_stride = 16 * 32;
            }
        } else {                  // Wqkv, group 0..2 of the pair's 48 output columns
            const int grp = idx - (tail ? 1 + 2 * chunks : 0) - (Wembed != nullptr ? 1 : 0);
            r.base = Wqkv + (size_t)((48 * cp + 16 * grp) / 8) * 16 * 32;
            r.tile_stride = 16 * 32;
        }
        return r;
    }
};

// 16 bytes global -> shared (this lane's part of a fragment), OFFSET bytes into the warp's ring
template <int OFFSET>
__device__ __forceinline__ void cp_async_16(unsigned ring, const float4 *src)
{
    asm volatile("cp.async.cg.shared.global [%0+%1], [%2], 16;" ::"r"(ring), "n"(OFFSET), "l"(src));
}

// Requests k steps FIRST .. FIRST + COUNT - 1 of a product whose fragments for this lane start at src0 / src1 (the
// warp's two column tiles) into their slots, as one group; with src0 == nullptr only the (empty) group is committed,
// so that the group count stays in step.
template <int FIRST, int COUNT>
__device__ __forceinline__ void request_steps(unsigned ring, const float4 *src0, const float4 *src1)
{
    if (src0 != nullptr) {
        static_for<FIRST, FIRST + COUNT>([&](auto step) {
            constexpr int S = decltype(step)::value;
            cp_async_16<S * 1024>(ring, src0 + S * 32);
            cp_async_16<S * 1024 + 512>(ring, src1 + S * 32);
        });
    }
    asm volatile("cp.async.commit_group;");
}

// acc[mt][nt] += A (rows of the tile x 128, split in shared memory) . B (the product whose fragments are in the ring).
// a_hi / a_lo: shared addresses of this lane's ldmatrix row at the warp's first k step; frag: this lane's fragment of
// the warp's first column tile in slot 0 of its ring (ring: the same as a shared address); next0 / next1: this lane's
// fragments of the next product (null after the block's last one), requested into the slots as they are read.
template <int MT>
__device__ __forceinline__ void product_128(float (&acc)[MT][2][4], unsigned a_hi, unsigned a_lo, const float4 *frag,
                                            unsigned ring, const float4 *next0, const float4 *next1)
{
    // the correction product goes to an accumulator of its own: two independent dependency chains per tile, and the
    // small terms are summed among themselves before they meet the large ones
    float corr[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int u = 0; u < 4; ++u) corr[mt][nt][u] = 0.f;
    constexpr int G = MT == 1 ? 4 : 2;     // k steps fetched and issued together: loads of all G before the first MMA
    constexpr int GROUPS = KSTEPS / G;     // cp.async groups per product
    static_for<0, GROUPS>([&](auto group) {
        constexpr int KS0 = decltype(group)::value * G;
        // this group's fragments were requested one product ago; GROUPS - 1 younger groups may still be in flight
        asm volatile("cp.async.wait_group %0;" ::"n"(GROUPS - 1) : "memory");
        float4 b[G][2];
#pragma unroll
        for (int i = 0; i < G; ++i) {
            b[i][0] = frag[(KS0 + i) * 64];
            b[i][1] = frag[(KS0 + i) * 64 + 32];
        }
        request_steps<KS0, G>(ring, next0, next1);
        // ldmatrix hands a lane the 32-bit words (row lane/4, word lane%4) of four 8-row x 16-byte matrices, which for
        // 32-bit elements are exactly the a0..a3 of the m16n8k8 A fragment: rows 0-7 / 8-15 of the m tile, words 0-3 /
        // 4-7 of the k step (and, read as 16-bit elements, the A fragment of the 16-deep product of the lo tile).
        // Lane l supplies the address of row l%8 of matrix l/8.
        unsigned ah[G][MT][4], al[G][MT][4];
        static_for<0, G>([&](auto step) {
            constexpr int I = decltype(step)::value;
            static_for<0, MT>([&](auto mtile) {
                constexpr int M = decltype(mtile)::value;
                ldmatrix_x4<4 * (16 * M * LDA + 8 * (KS0 + I))>(ah[I][M], a_hi);
                ldmatrix_x4<4 * (16 * M * LDA + 8 * (KS0 + I))>(al[I][M], a_lo);
            });
        });
#pragma unroll
        for (int i = 0; i < G; ++i)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const unsigned bh0 = __float_as_uint(b[i][nt].x), bh1 = __float_as_uint(b[i][nt].y);
                const unsigned bc0 = __float_as_uint(b[i][nt].z), bc1 = __float_as_uint(b[i][nt].w);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_bf16_k16(corr[mt][nt], al[i][mt], bc0, bc1);
                    mma_tf32(acc[mt][nt], ah[i][mt], bh0, bh1);
                }
            }
    });
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[mt][nt][u] += corr[mt][nt][u];
}

// Writes this lane's accumulator entries of a 128-wide product (columns 16 warp + 8 nt + 2 t + {0,1}) into an operand tile.
template <int MT>
__device__ __forceinline__ void store_split(unsigned *a_hi, unsigned *a_lo, const float (&v)[MT][2][4], int warp, int lane)
{
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int row = 16 * mt + g + (u >= 2 ? 8 : 0), col = 16 * warp + 8 * nt + 2 * t + (u & 1);
                const unsigned hi = tf32_hi(v[mt][nt][u]);
                a_hi[row * LDA + col] = hi;
                a_lo[row * LDA + col] = corr_word(__uint_as_float(hi), v[mt][nt][u] - __uint_as_float(hi));
            }
}

template <int MT>
__global__ void __launch_bounds__(DB_THREADS) dense_block_kernel(const DenseArgs p)
{
    extern __shared__ __align__(16) unsigned smem_u[];
    constexpr int ROWS = 16 * MT;
    unsigned *a1_hi = smem_u, *a1_lo = a1_hi + ROWS * LDA;       // operand tile 1: attn, then y, then x'
    unsigned *a2_hi = a1_lo + ROWS * LDA, *a2_lo = a2_hi + ROWS * LDA;  // operand tile 2: a chunk of hidden units
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = (tid >> 5) & 7;      // column pair of this warp
    const int kh = tid >> 8;              // k half of this warp
    const bool owner = kh == 0;           // holds biases and residuals, does the epilogues
    const int g = lane >> 2, t = lane & 3;

    const long long tiles = (p.N + ROWS - 1) / ROWS;
    const long long my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // shared memory after the operand tiles: the warps' rings (16 x 8 KB) and the exchange buffers for the halves of a
    // product ([2][8 column pairs][32 lanes][8 MT floats])
    const int wid = tid >> 5;  // = 8 kh + warp
    float4 *rings = reinterpret_cast<float4 *>(a2_lo + ROWS * LDA);
    float *xch = reinterpret_cast<float *>(rings + (size_t)DB_WARPS * DEPTH * 64);
    const float4 *frag = rings + (size_t)wid * DEPTH * 64 + lane;   // this lane's 16 bytes of slot 0, first column tile
    const unsigned ring = smem_u32(frag);
    StreamPlan plan;
    plan.Wo = p.Wo; plan.W1 = p.W1; plan.W2 = p.W2; plan.Wqkv = p.Wqkv; plan.ff = p.ff; plan.tail = p.tail;
    plan.Wembed = p.tail ? nullptr : p.Wembed;
    plan.panels = (p.tail ? 1 + 2 * (p.ff / 128) : 0) + (p.head ? 3 : 0) + (plan.Wembed != nullptr ? 1 : 0);
    const long long total_products = my_tiles * plan.panels;
    long long products = 0;  // products done by this block
    int next_panel = plan.panels > 1 ? 1 : 0;  // panel of product `products + 1` within the row tile's sequence
    // this lane's fragments of the k steps of this warp's half of a panel, for its two column tiles
    auto panel_src = [&](int idx, const float4 *&src0, const float4 *&src1) {
        const Panel pn = plan.panel(idx, warp);
        src0 = pn.base + (size_t)(kh * KSTEPS) * 32 + lane;
        src1 = src0 + pn.tile_stride;
    };
    // this lane's ldmatrix row of the operand tiles at the warp's first k step
    const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8, lcol = (lane >> 4) * 4;
    const unsigned lane_off = 4u * (unsigned)(lrow * LDA + 8 * kh * KSTEPS + lcol);
    const unsigned a1h = smem_u32(a1_hi) + lane_off, a1l = smem_u32(a1_lo) + lane_off;
    const unsigned a2h = smem_u32(a2_hi) + lane_off, a2l = smem_u32(a2_lo) + lane_off;
    auto product = [&](float (&acc)[MT][2][4], unsigned a_hi, unsigned a_lo) {
        const float4 *next0 = nullptr, *next1 = nullptr;
        if (products + 1 < total_products) panel_src(next_panel, next0, next1);
        product_128<MT>(acc, a_hi, a_lo, frag, ring, next0, next1);
        ++products;
        if (++next_panel == plan.panels) next_panel = 0;
    };
    int xsel = 0;
    // acc <- acc(kh = 0) + acc(kh = 1), valid in the owner warps afterwards; contains one block barrier
    auto combine = [&](float (&acc)[MT][2][4]) {
        if (KSPLIT == 1) return;
        float4 *mine = reinterpret_cast<float4 *>(xch + ((size_t)(xsel * 8 + warp) * 32 + lane) * 8 * MT);
        if (!owner) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
                    mine[2 * mt + nt] = make_float4(acc[mt][nt][0], acc[mt][nt][1], acc[mt][nt][2], acc[mt][nt][3]);
        }
        __syncthreads();
        if (owner) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const float4 o = mine[2 * mt + nt];
                    acc[mt][nt][0] += o.x; acc[mt][nt][1] += o.y; acc[mt][nt][2] += o.z; acc[mt][nt][3] += o.w;
                }
        }
        xsel ^= 1;  // the next exchange uses the other buffer, so no barrier is needed before it
    };
    auto zero = [&](float (&acc)[MT][2][4]) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[mt][nt][u] = 0.f;
    };
    grid_launch_dependents();
    {   // weights are constants: the stream of the first product starts while the previous kernel drains
        constexpr int G = MT == 1 ? 4 : 2;
        const float4 *src0 = nullptr, *src1 = nullptr;
        if (total_products > 0) panel_src(0, src0, src1);
        static_for<0, KSTEPS / G>([&](auto group) { request_steps<decltype(group)::value * G, G>(ring, src0, src1); });
    }
    grid_dependency_wait();   // activations of the previous kernel (attention output, x) from here on

    for (long long tile = blockIdx.x; tile * ROWS < p.N; tile += gridDim.x) {
        const long long row0 = tile * ROWS;
        float xo[MT][2][4];  // the rows' current features at this lane's accumulator positions (x, then y, then x')
        __syncthreads();     // the previous tile's readers are done with the operand tiles
        if (p.tail) {
            // ---- operand 1 <- attention output of the tile, split
            for (int idx = tid; idx < ROWS * 32; idx += DB_THREADS) {
                const int r = idx >> 5, c4 = idx & 31;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (row0 + r < p.N) v = reinterpret_cast<const float4 *>(p.attn + (row0 + r) * 128)[c4];
                const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const unsigned hi = tf32_hi(vv[u]);
                    a1_hi[r * LDA + 4 * c4 + u] = hi;
                    a1_lo[r * LDA + 4 * c4 + u] = corr_word(__uint_as_float(hi), vv[u] - __uint_as_float(hi));
                }
            }
            // ---- y = x + bo + attn Wo^T
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int col = 16 * warp + 8 * nt + 2 * t;
                    const float2 bo = *reinterpret_cast<const float2 *>(p.bo + col);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const long long row = row0 + 16 * mt + g + 8 * half;
                        float2 xv = make_float2(0.f, 0.f);
                        if (row < p.N) xv = *reinterpret_cast<const float2 *>(p.x + row * 128 + col);
                        xo[mt][nt][2 * half] = xv.x + bo.x;
                        xo[mt][nt][2 * half + 1] = xv.y + bo.y;
                    }
                }
            if (!owner) zero(xo);
            __syncthreads();
            product(xo, a1h, a1l);
            combine(xo);      // (its barrier: every warp has read attn)
            if (KSPLIT == 1) __syncthreads();
            if (owner) store_split<MT>(a1_hi, a1_lo, xo, warp, lane);
            // ---- x' = y + b2 + sum over chunks of relu(y W1_c^T + b1_c) W2_c^T
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float2 b2 = *reinterpret_cast<const float2 *>(p.b2 + 16 * warp + 8 * nt + 2 * t);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    xo[mt][nt][0] += b2.x; xo[mt][nt][1] += b2.y; xo[mt][nt][2] += b2.x; xo[mt][nt][3] += b2.y;
                }
            }
            if (!owner) zero(xo);  // from here on the second half collects its own part of the feed-forward output
            __syncthreads();  // y is in operand 1
            const int chunks = p.ff / 128;
            for (int ch = 0; ch < chunks; ++ch) {
                float h[MT][2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const float2 b1 = *reinterpret_cast<const float2 *>(p.b1 + 128 * ch + 16 * warp + 8 * nt + 2 * t);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) { h[mt][nt][0] = b1.x; h[mt][nt][1] = b1.y; h[mt][nt][2] = b1.x; h[mt][nt][3] = b1.y; }
                }
                if (!owner) zero(h);
                product(h, a1h, a1l);  // W1, the chunk's hidden units
                combine(h);       // (its barrier: the previous chunk's readers are done with operand 2)
                if (KSPLIT == 1) __syncthreads();
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int u = 0; u < 4; ++u) h[mt][nt][u] = fmaxf(h[mt][nt][u], 0.f);
                if (owner) store_split<MT>(a2_hi, a2_lo, h, warp, lane);
                __syncthreads();
                product(xo, a2h, a2l);  // W2, the chunk's k steps
            }
            combine(xo);
            // ---- write x'
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const long long row = row0 + 16 * mt + g + 8 * half;
                        if (owner && row < p.N)
                            *reinterpret_cast<float2 *>(p.x + row * 128 + 16 * warp + 8 * nt + 2 * t) =
                                make_float2(xo[mt][nt][2 * half], xo[mt][nt][2 * half + 1]);
                    }
        } else if (plan.Wembed != nullptr) {
            // ---- x = features W_embed^T: operand 1 <- the tile's feature rows, zero beyond feature_dim
            for (int idx = tid; idx < ROWS * 128; idx += DB_THREADS) {
                const int r = idx >> 7, col = idx & 127;
                float v = 0.f;
                if (row0 + r < p.N && col < p.feature_dim)
                    v = p.features != nullptr ? p.features[(row0 + r) * p.feature_dim + col]
                                              : (p.species[row0 + r] == (long long)col ? 1.0f : 0.0f);
                const unsigned hi = tf32_hi(v);
                a1_hi[r * LDA + col] = hi;
                a1_lo[r * LDA + col] = corr_word(__uint_as_float(hi), v - __uint_as_float(hi));
            }
            zero(xo);
            __syncthreads();
            product(xo, a1h, a1l);
            combine(xo);
            if (KSPLIT == 1) __syncthreads();
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const long long row = row0 + 16 * mt + g + 8 * half;
                        if (owner && row < p.N)
                            *reinterpret_cast<float2 *>(p.x + row * 128 + 16 * warp + 8 * nt + 2 * t) =
                                make_float2(xo[mt][nt][2 * half], xo[mt][nt][2 * half + 1]);
                    }
        } else {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const long long row = row0 + 16 * mt + g + 8 * half;
                        float2 xv = make_float2(0.f, 0.f);
                        if (row < p.N) xv = *reinterpret_cast<const float2 *>(p.x + row * 128 + 16 * warp + 8 * nt + 2 * t);
                        xo[mt][nt][2 * half] = xv.x;
                        xo[mt][nt][2 * half + 1] = xv.y;
                    }
        }
        if (!p.head) continue;  // (block-uniform)

        // ---- in-projection of the next layer: operand 1 <- x'
        __syncthreads();  // every warp is done with y in operand 1
        if (owner) store_split<MT>(a1_hi, a1_lo, xo, warp, lane);
        __syncthreads();
        // warp w owns the 48 output columns 48 w .. 48 w + 47 of q|k|v = three 16-column groups (one head each)
#pragma unroll
        for (int grp = 0; grp < 3; ++grp) {
            const int col0 = 48 * warp + 16 * grp;  // 0..127 q, 128..255 k, 256..383 v
            float acc[MT][2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float2 bq = *reinterpret_cast<const float2 *>(p.bqkv + col0 + 8 * nt + 2 * t);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) { acc[mt][nt][0] = bq.x; acc[mt][nt][1] = bq.y; acc[mt][nt][2] = bq.x; acc[mt][nt][3] = bq.y; }
            }
            if (!owner) zero(acc);
            product(acc, a1h, a1l);
            combine(acc);
            if (!owner) continue;  // (warp-uniform; the epilogue below has no block barrier)
            const int which = col0 >> 7;           // 0 q, 1 k, 2 v (warp-uniform)
            const int hc0 = col0 & 127;            // first column within q, k or v; the head is hc0 / 16
            float *dst = which == 0 ? p.q : (which == 1 ? p.k : p.v);
            if (which == 0) {
                // the head's Gaussian width from alpha = q . w_pos (…attention_cuda.py:647-722), then q / sqrt(16)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        float alpha = 0.f;
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt) {
                            const float2 wq = *reinterpret_cast<const float2 *>(p.w_pos + hc0 + 8 * nt + 2 * t);
                            alpha = fmaf(acc[mt][nt][2 * half], wq.x, alpha);
                            alpha = fmaf(acc[mt][nt][2 * half + 1], wq.y, alpha);
                        }
                        alpha += __shfl_xor_sync(FULL, alpha, 1);
                        alpha += __shfl_xor_sync(FULL, alpha, 2);
                        const long long row = row0 + 16 * mt + g + 8 * half;
                        if (t == 0 && row < p.N) {
                            const float xn = (alpha + p.gauss_shift) * p.gauss_scale;
                            const float tt = xn * (p.elu_beta / (1.0f - p.lower_bound));
                            const float elu = tt > 0.f ? tt : expm1f(tt);
                            p.a[row * HEADS + (hc0 >> 4)] = ((1.0f - p.lower_bound) * elu + 1.0f) * p.a_factor;
                        }
                    }
            }
            const float scale = which == 0 ? 0.25f : 1.0f;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const long long row = row0 + 16 * mt + g + 8 * half;
                        if (row < p.N)
                            *reinterpret_cast<float2 *>(dst + row * 128 + hc0 + 8 * nt + 2 * t) =
                                make_float2(acc[mt][nt][2 * half] * scale, acc[mt][nt][2 * half + 1] * scale);
                    }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

}  // namespace

int launch_dense_block(const DenseArgs &p, cudaStream_t s)
{
    if (p.N == 0) return CF_OK;
    if (p.tail && (p.ff <= 0 || p.ff % 128 != 0))
        return fail(CF_ERR_UNSUPPORTED, "dense block: ff_dim=%d must be a positive multiple of 128", p.ff);
    if (!p.tail && p.Wembed != nullptr && ((p.features == nullptr && p.species == nullptr) || p.feature_dim < 1 || p.feature_dim > 128))
        return fail(CF_ERR_UNSUPPORTED, "dense block: embedding of %d features (1..128)", p.feature_dim);
    // 16-row tiles while they fit one wave of the SMs (more SMs busy), 32-row tiles beyond (half the weight traffic;
    // a block is tensor-pipe bound either way, so what counts is the number of waves) - unless the caller chose:
    // with several forwards side by side on the GPU the 32-row tiles' smaller total of SM time is worth more than
    // the single forward's latency
    const long long tiles16 = (p.N + 15) / 16;
    const int sms = sm_count();
    const int choice = dense_tile_rows_choice();
    const bool small = choice == 16 || (choice != 32 && tiles16 <= sms);
    const size_t smem = sizeof(unsigned) * (4 * (small ? 16 : 32) * LDA + DB_WARPS * RING_WORDS +
                                            (KSPLIT > 1 ? 2 * 8 * 32 * 8 * (small ? 1 : 2) : 0));
    auto kernel = small ? dense_block_kernel<1> : dense_block_kernel<2>;
    if (smem > 48 * 1024) {
        static thread_local bool raised_small = false, raised_large = false;
        bool &raised = small ? raised_small : raised_large;
        if (!raised) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
                cudaGetLastError();
                return fail(CF_ERR_CUDA, "dense block: %zu bytes of shared memory not available", smem);
            }
            raised = true;
        }
    }
    const long long tiles = small ? tiles16 : (p.N + 31) / 32;
    const long long cap = sms;  // one block per SM: the weight rings fill most of the shared memory
    if (launch_chained(kernel, dim3((unsigned)(tiles < cap ? tiles : cap)), dim3(DB_THREADS), smem, s, p.chained != 0, p) != cudaSuccess)
        return launch_status("dense_block_kernel");
    return launch_status("dense_block_kernel");
}

}  // namespace cf
