// cuBLAS resolved at run time from the copy already loaded in the process (the caller passes its handle), so that the
// handle and the functions come from the same library.  Shared by the one-call encoder and model forwards.
#pragma once
#include <cublas_v2.h>
#include <dlfcn.h>

#include <mutex>

namespace cf {

using SgemmFn = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const float *,
                                   const float *, int, const float *, int, const float *, float *, int);
using SetStreamFn = cublasStatus_t (*)(cublasHandle_t, cudaStream_t);
using GetStreamFn = cublasStatus_t (*)(cublasHandle_t, cudaStream_t *);
using SetMathFn = cublasStatus_t (*)(cublasHandle_t, cublasMath_t);
using GetMathFn = cublasStatus_t (*)(cublasHandle_t, cublasMath_t *);

struct Blas {
    SgemmFn sgemm = nullptr;
    SetStreamFn set_stream = nullptr;
    GetStreamFn get_stream = nullptr;
    SetMathFn set_math = nullptr;
    GetMathFn get_math = nullptr;
    bool ok = false;
};

inline const Blas &blas()
{
    static Blas b;
    static std::once_flag once;
    std::call_once(once, [] {
        void *lib = dlopen("libcublas.so.12", RTLD_NOW | RTLD_NOLOAD);
        if (!lib) lib = dlopen("libcublas.so.12", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libcublas.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) return;
        b.sgemm = (SgemmFn)dlsym(lib, "cublasSgemm_v2");
        b.set_stream = (SetStreamFn)dlsym(lib, "cublasSetStream_v2");
        b.get_stream = (GetStreamFn)dlsym(lib, "cublasGetStream_v2");
        b.set_math = (SetMathFn)dlsym(lib, "cublasSetMathMode");
        b.get_math = (GetMathFn)dlsym(lib, "cublasGetMathMode");
        b.ok = b.sgemm && b.set_stream && b.get_stream && b.set_math && b.get_math;
    });
    return b;
}

// Y (rows x out) = [beta] Y + X (rows x in) W^T, W (out x in), all row-major.
inline cublasStatus_t linear(const Blas &b, cublasHandle_t h, const float *X, const float *W, float *Y, int rows, int in,
                             int out, float beta)
{
    const float one = 1.0f;
    return b.sgemm(h, CUBLAS_OP_T, CUBLAS_OP_N, out, rows, in, &one, W, in, X, in, &beta, Y, out);
}


// Points the handle at a stream with plain fp32 math for the lifetime of the object, then restores both.
struct BlasScope {
    const Blas &bl;
    cublasHandle_t handle;
    cudaStream_t old_stream = nullptr;
    cublasMath_t old_math = CUBLAS_DEFAULT_MATH;
    BlasScope(const Blas &b, cublasHandle_t h, cudaStream_t s) : bl(b), handle(h)
    {
        bl.get_stream(handle, &old_stream);
        bl.get_math(handle, &old_math);
        bl.set_stream(handle, s);
        bl.set_math(handle, CUBLAS_DEFAULT_MATH);  // no TF32, as the reference's train.py:61-62 asks
    }
    ~BlasScope()
    {
        bl.set_math(handle, old_math);
        bl.set_stream(handle, old_stream);
    }
};

}  // namespace cf
