// One host call per batch of a streaming inference loop: host -> device copies of the inputs on a copy stream, the
// one-call model forward on a compute stream (its preparation beside the batches before it), device -> host copy of
// the outputs, and the events that order the three - issued from C++, because at the sizes of a crystal batch the
// step is a few hundred microseconds and a framework-level loop (a dozen tensor and stream operations per batch)
// spends as long issuing it as the GPU spends running it.
//
// The function keeps no state and owns nothing: streams, events and every buffer are the caller's (cf_serve_slot), so
// one caller can keep several batches in flight (one slot each) and alternate between compute streams.
#include "common.cuh"
#include "dense_block.cuh"

extern "C" int cf_serve_submit(const cf_model_desc *model, const cf_serve_slot *slot, const float *x_host,
                               const float *pos_host, const float *trans_host, const int64_t *sizes_host, int64_t N,
                               int64_t B, int64_t E, int64_t max_atoms, int inputs_in_use,
                               const cf_serve_gather *gather, const int64_t *species_host)
{
    using namespace cf;
    CF_REQUIRE(model != nullptr && slot != nullptr, CF_ERR_INVALID, "cf_serve_submit: null description");
    CF_REQUIRE(N >= 0 && B >= 0 && E >= 0, CF_ERR_INVALID, "cf_serve_submit: negative size");
    CF_REQUIRE(N <= slot->max_atoms_total && B <= slot->max_crystals && E <= slot->max_edges, CF_ERR_RANGE,
               "cf_serve_submit: batch of %lld atoms, %lld crystals, %lld edges exceeds the slot's buffers (%lld, %lld, %lld)",
               (long long)N, (long long)B, (long long)E, (long long)slot->max_atoms_total, (long long)slot->max_crystals,
               (long long)slot->max_edges);
    CF_REQUIRE(gather != nullptr || B > 0, CF_ERR_INVALID, "cf_serve_submit: empty batch");  // (an empty shard still gathers)
    CF_REQUIRE(model->dense_tile_rows == 0 || model->dense_tile_rows == 16 || model->dense_tile_rows == 32, CF_ERR_INVALID,
               "cf_serve_submit: dense_tile_rows = %d (0, 16 or 32)", (int)model->dense_tile_rows);
    if (gather != nullptr)
        CF_REQUIRE(gather->store && gather->stored && gather->collected && gather->own_cells && gather->index &&
                       gather->y_all && gather->y_all_host && gather->status && gather->status_host && gather->total_rows >= 0,
                   CF_ERR_INVALID, "cf_serve_submit: incomplete gather");
    CF_REQUIRE((x_host || species_host) && pos_host && trans_host && sizes_host, CF_ERR_INVALID, "cf_serve_submit: null input");
    CF_REQUIRE(x_host || slot->species, CF_ERR_INVALID, "cf_serve_submit: species indices given, but the slot has no buffer for them");
    // (a null stream handle is the default stream: valid for either role, though copies then do not overlap compute)
    CF_REQUIRE(slot->copied && slot->inputs_free && slot->done && slot->x && slot->pos && slot->trans && slot->sizes &&
                   slot->workspace && slot->y && slot->y_host,
               CF_ERR_INVALID, "cf_serve_submit: incomplete slot");
    cudaStream_t copy = as_stream(slot->copy_stream), compute = as_stream(slot->compute_stream);
    cudaEvent_t copied = reinterpret_cast<cudaEvent_t>(slot->copied), inputs_free = reinterpret_cast<cudaEvent_t>(slot->inputs_free);
    cudaEvent_t done = reinterpret_cast<cudaEvent_t>(slot->done);
    bool ok = true;
    // the forward that last read the slot's input buffers has run
    if (inputs_in_use) ok = ok && cudaStreamWaitEvent(copy, inputs_free, 0) == cudaSuccess;
    if (N > 0 && x_host) ok = ok && cudaMemcpyAsync(slot->x, x_host, sizeof(float) * (size_t)N * (size_t)model->feature_dim, cudaMemcpyHostToDevice, copy) == cudaSuccess;
    if (N > 0 && !x_host) ok = ok && cudaMemcpyAsync(slot->species, species_host, sizeof(int64_t) * (size_t)N, cudaMemcpyHostToDevice, copy) == cudaSuccess;
    if (N > 0) ok = ok && cudaMemcpyAsync(slot->pos, pos_host, sizeof(float) * 3 * (size_t)N, cudaMemcpyHostToDevice, copy) == cudaSuccess;
    if (B > 0) ok = ok && cudaMemcpyAsync(slot->trans, trans_host, sizeof(float) * 9 * (size_t)B, cudaMemcpyHostToDevice, copy) == cudaSuccess;
    if (B > 0) ok = ok && cudaMemcpyAsync(slot->sizes, sizes_host, sizeof(int64_t) * (size_t)B, cudaMemcpyHostToDevice, copy) == cudaSuccess;
    ok = ok && cudaEventRecord(copied, copy) == cudaSuccess;
    ok = ok && cudaStreamWaitEvent(compute, copied, 0) == cudaSuccess;
    if (!ok) return launch_status("cf_serve_submit: input copies");
    // (the slot's workspace was last used by the slot's previous batch, whose result the caller has collected: no
    // slot-free event is needed; the inputs-ready event lets the preparation start beside the batches in flight)
    if (gather != nullptr && gather->store_after != nullptr)
        ok = ok && cudaStreamWaitEvent(compute, reinterpret_cast<cudaEvent_t>(gather->store_after), 0) == cudaSuccess;
    if (!ok) return launch_status("cf_serve_submit: wait for the gather slot");
    DenseTileRows tile_rows(model->dense_tile_rows);  // for the launches of this call, on this thread
    const int rc = model_forward_impl(nullptr, x_host ? slot->x : nullptr, x_host ? nullptr : slot->species, model->feature_dim, slot->pos, slot->trans, slot->sizes, N, B, E,
                                    max_atoms, model->W_embed, model->W_embed_packed, model->num_layers, model->weights,
                                    model->scalars, model->K, model->ff_dim, model->wscale, model->cutoff_radius,
                                    model->lattice_range, model->minimum_range, model->W1, model->b1, model->hidden,
                                    model->W2, model->b2, model->targets, model->order_reach, slot->workspace, slot->y,
                                    nullptr, gather != nullptr ? gather->store : nullptr, slot->copied, nullptr,
                                    slot->compute_stream);
    if (rc != CF_OK) return rc;
    ok = ok && cudaEventRecord(inputs_free, compute) == cudaSuccess;
    if (gather != nullptr) {
        cudaStream_t collect = as_stream(gather->collect_stream);
        ok = ok && cudaEventRecord(reinterpret_cast<cudaEvent_t>(gather->stored), compute) == cudaSuccess;
        if (collect != compute) ok = ok && cudaStreamWaitEvent(collect, reinterpret_cast<cudaEvent_t>(gather->stored), 0) == cudaSuccess;
        if (!ok) return launch_status("cf_serve_submit: gather events");
        const int rc2 = cf_peer_gather_collect(gather->own_cells, gather->store->step, gather->index, gather->total_rows,
                                               model->targets, gather->store->rows_per_rank, gather->y_all, gather->status,
                                               gather->timeout_s, gather->collect_stream);
        if (rc2 != CF_OK) return rc2;
        ok = ok && cudaEventRecord(reinterpret_cast<cudaEvent_t>(gather->collected), collect) == cudaSuccess;
        if (gather->total_rows > 0)
            ok = ok && cudaMemcpyAsync(gather->y_all_host, gather->y_all, sizeof(float) * (size_t)gather->total_rows * (size_t)model->targets,
                                       cudaMemcpyDeviceToHost, collect) == cudaSuccess;
        ok = ok && cudaMemcpyAsync(gather->status_host, gather->status, sizeof(int32_t), cudaMemcpyDeviceToHost, collect) == cudaSuccess;
        ok = ok && cudaEventRecord(done, collect) == cudaSuccess;
        if (!ok) return launch_status("cf_serve_submit: gathered output copy");
        return CF_OK;
    }
    ok = ok && cudaMemcpyAsync(slot->y_host, slot->y, sizeof(float) * (size_t)B * (size_t)model->targets, cudaMemcpyDeviceToHost, compute) == cudaSuccess;
    ok = ok && cudaEventRecord(done, compute) == cudaSuccess;
    if (!ok) return launch_status("cf_serve_submit: output copy");
    return CF_OK;
}
