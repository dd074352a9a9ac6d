// KV-head sharding over the GPUs of one box: buffers that other processes can map, and the
// decode call whose combine kernel stores its output rows straight into every rank's gathered
// buffer (see tq_gather_desc in the public header).  The reference has no multi-GPU path.
#include "tq_common.cuh"
#include "tq_decode_shared.cuh"

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the public header promises a 64-byte handle");

extern "C" int32_t tq_peer_buffer_create(size_t bytes, void **dev_ptr, void *handle64_out) {
    if (!dev_ptr || !handle64_out || bytes == 0) return TQ_ERR_ARG;
    void *p = nullptr;
    TQ_CUDA_CHECK(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        tq_set_cuda_error(e, "tq_peer_buffer_create");
        return TQ_ERR_CUDA;
    }
    memcpy(handle64_out, &h, sizeof(h));
    *dev_ptr = p;
    return TQ_OK;
}

extern "C" int32_t tq_peer_buffer_open(const void *handle64, void **dev_ptr) {
    if (!handle64 || !dev_ptr) return TQ_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    TQ_CUDA_CHECK(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return TQ_OK;
}

extern "C" int32_t tq_peer_buffer_close(void *dev_ptr) {
    if (!dev_ptr) return TQ_OK;
    TQ_CUDA_CHECK(cudaIpcCloseMemHandle(dev_ptr));
    return TQ_OK;
}

extern "C" int32_t tq_peer_buffer_destroy(void *dev_ptr) {
    if (!dev_ptr) return TQ_OK;
    TQ_CUDA_CHECK(cudaFree(dev_ptr));
    return TQ_OK;
}

int tq_check_gather(const tq_gather_desc *g) {
    if (!g || g->world < 1 || g->world > TQ_MAX_PEERS || g->rank < 0 || g->rank >= g->world) return TQ_ERR_ARG;
    if ((g->seq == 0 && !g->seq_dev) || !g->counter || g->q_heads_total <= 0) return TQ_ERR_ARG;
    if (g->out_stride < 0 || (g->out_stride & 15) || ((uintptr_t)g->seq_dev & 3)) return TQ_ERR_ARG;
    for (int p = 0; p < g->world; ++p)
        if (!g->out[p] || !g->flags[p] || ((uintptr_t)g->out[p] & 15) || ((uintptr_t)g->flags[p] & 3)) return TQ_ERR_ARG;
    return TQ_OK;
}

extern "C" int32_t tq_decode_attn_gather(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                                         const tq_cache_desc *cache, int32_t seq_len, int32_t n_splits,
                                         void *workspace, size_t workspace_bytes, const tq_gather_desc *gather,
                                         tq_stream stream) {
    TqRange range_("tq_decode_attn_gather");
    if (!ctx || !q || !workspace) return TQ_ERR_ARG;
    int rc = tq_check_gather(gather);
    if (rc) return rc;
    rc = tq_check_cache(ctx, cache);
    if (rc) return rc;
    if (q_dtype != TQ_DTYPE_F16 && q_dtype != TQ_DTYPE_BF16) return TQ_ERR_UNSUPPORTED;
    if (seq_len <= 0 || seq_len > cache->capacity || n_splits < 1) return TQ_ERR_ARG;
    if (q_heads <= 0 || q_heads % cache->kv_heads || q_heads / cache->kv_heads > TQ_MAX_GROUPS) return TQ_ERR_ARG;
    if (gather->q_heads_total != q_heads * gather->world) return TQ_ERR_ARG;
    if (((uintptr_t)q | (uintptr_t)workspace) & 15) return TQ_ERR_ARG;
    if (workspace_bytes < tq_decode_workspace_bytes(cache->batch, q_heads, n_splits)) return TQ_ERR_WORKSPACE;
    const TqStepExtras extras = {nullptr, nullptr, gather, nullptr, 0};
    return tq_launch_decode_mma4(ctx, q, q_dtype, q_heads, cache, seq_len, nullptr, nullptr, 0, n_splits, workspace,
                                 /*out=*/nullptr, &extras, (cudaStream_t)stream);
}

extern "C" int32_t tq_gather_wait(tq_ctx *ctx, const tq_gather_desc *gather, int32_t batch, int32_t dtype,
                                  void *out_final, tq_stream stream) {
    TqRange range_("tq_gather_wait");
    if (!ctx) return TQ_ERR_ARG;
    int rc = tq_check_gather(gather);
    if (rc) return rc;
    if (batch <= 0 || gather->q_heads_total % gather->world) return TQ_ERR_ARG;
    if (out_final && ((dtype != TQ_DTYPE_F16 && dtype != TQ_DTYPE_BF16) || ((uintptr_t)out_final & 15))) return TQ_ERR_ARG;
    return tq_launch_gather_wait(gather, ctx->error_flag, ctx->wait_limit_ms, batch, 2, out_final, (cudaStream_t)stream);
}

// ---- sequence split: fewer KV heads than ranks -------------------------------------------------

extern "C" size_t tq_parts_exchange_bytes(int32_t batch, int32_t q_heads_total, int32_t parts) {
    if (batch <= 0 || q_heads_total <= 0 || parts <= 0) return 0;
    const size_t floats = (size_t)batch * q_heads_total * parts * (TQ_D + 2);
    return (floats * 4 + 255) / 256 * 256;
}

static int check_parts(const tq_gather_desc *g, int32_t parts, int32_t q_heads) {
    int rc = tq_check_gather(g);
    if (rc) return rc;
    if (parts < 1 || g->world % parts || g->seq_dev || g->seq == 0) return TQ_ERR_ARG;
    if (g->q_heads_total != q_heads * (g->world / parts)) return TQ_ERR_ARG;
    return TQ_OK;
}

extern "C" int32_t tq_decode_attn_parts(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                                        const tq_cache_desc *cache, int32_t seq_len, int32_t n_splits, void *workspace,
                                        size_t workspace_bytes, const tq_gather_desc *gather, int32_t parts,
                                        tq_stream stream) {
    TqRange range_("tq_decode_attn_parts");
    if (!ctx || !q || !workspace) return TQ_ERR_ARG;
    int rc = check_parts(gather, parts, q_heads);
    if (rc) return rc;
    rc = tq_check_cache(ctx, cache);
    if (rc) return rc;
    if (q_dtype != TQ_DTYPE_F16 && q_dtype != TQ_DTYPE_BF16) return TQ_ERR_UNSUPPORTED;
    if (seq_len < 0 || seq_len > cache->capacity || n_splits < 1) return TQ_ERR_ARG;
    if (q_heads <= 0 || q_heads % cache->kv_heads || q_heads / cache->kv_heads > TQ_MAX_GROUPS) return TQ_ERR_ARG;
    if (cache->seq_start) return TQ_ERR_UNSUPPORTED;  // token indices are per part: no per-row start offsets here
    if (((uintptr_t)q | (uintptr_t)workspace) & 15) return TQ_ERR_ARG;
    if (workspace_bytes < tq_decode_workspace_bytes(cache->batch, q_heads, n_splits)) return TQ_ERR_WORKSPACE;
    const TqStepExtras extras = {nullptr, nullptr, gather, nullptr, parts};
    if (seq_len > 0)
        return tq_launch_decode_mma4(ctx, q, q_dtype, q_heads, cache, seq_len, nullptr, nullptr, 0, n_splits, workspace,
                                     /*out=*/nullptr, &extras, (cudaStream_t)stream);
    // this part holds no token yet: report an empty partial (max = -inf, sum = 0) for every row
    CombineArgs c = {};
    c.n_splits = 0, c.Hq = q_heads, c.G = q_heads / cache->kv_heads;
    c.gather_world = gather->world, c.gather_rank = gather->rank, c.gather_heads_total = gather->q_heads_total;
    c.gather_seq = gather->seq, c.gather_out_stride = gather->out_stride;
    for (int p = 0; p < gather->world; ++p) c.gather_out[p] = gather->out[p], c.gather_flags[p] = gather->flags[p];
    c.parts = parts, c.part = gather->rank % parts, c.head_group = gather->rank / parts;
    c.exch_rows = (int64_t)cache->batch * gather->q_heads_total;
    c.rot_v = ctx->rot_v;
    return tq_launch_combine(c, q_dtype, (int64_t)cache->batch * q_heads, (cudaStream_t)stream, false);
}

extern "C" int32_t tq_decode_parts_finish(tq_ctx *ctx, const tq_gather_desc *gather, int32_t batch, int32_t dtype,
                                          int32_t parts, int32_t heads_per_block, void *out, tq_stream stream) {
    TqRange range_("tq_decode_parts_finish");
    if (!ctx || !out || batch <= 0 || ((uintptr_t)out & 15)) return TQ_ERR_ARG;
    if (dtype != TQ_DTYPE_F16 && dtype != TQ_DTYPE_BF16) return TQ_ERR_UNSUPPORTED;
    int rc = tq_check_gather(gather);
    if (rc) return rc;
    if (parts < 1 || gather->world % parts || gather->seq_dev || gather->seq == 0) return TQ_ERR_ARG;
    const int heads_total = gather->q_heads_total;
    if (heads_per_block < 1 || heads_per_block > TQ_MAX_GROUPS || heads_total % heads_per_block) return TQ_ERR_ARG;
    if (heads_total % (gather->world / parts)) return TQ_ERR_ARG;
    // every rank reports batch x (its group's query heads) partial rows per step
    const int64_t rows_per_step = (int64_t)batch * (heads_total / (gather->world / parts));
    rc = tq_launch_gather_wait(gather, ctx->error_flag, ctx->wait_limit_ms, batch, 2, nullptr, (cudaStream_t)stream,
                               rows_per_step);
    if (rc) return rc;
    const int64_t rows = (int64_t)batch * heads_total;
    const float *base = reinterpret_cast<const float *>(static_cast<const char *>(gather->out[gather->rank]) +
                                                        ((gather->seq & 1u) ? gather->out_stride : 0));
    CombineArgs c = {};
    c.part_m = base, c.part_l = base + rows * parts, c.part_acc = base + 2 * rows * parts;
    c.n_splits = parts, c.Hq = heads_total, c.G = heads_per_block;
    c.rot_v = ctx->rot_v;
    c.out = out;
    return tq_launch_combine(c, dtype, rows, (cudaStream_t)stream, false);
}

extern "C" int32_t tq_set_wait_limit_ms(tq_ctx *ctx, int32_t limit_ms) {
    if (!ctx || limit_ms < 1 || limit_ms > 60000) return TQ_ERR_ARG;
    ctx->wait_limit_ms = limit_ms;
    return TQ_OK;
}
