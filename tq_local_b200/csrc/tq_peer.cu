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
    const TqStepExtras extras = {nullptr, nullptr, gather, nullptr};
    return tq_launch_decode_mma4(ctx, q, q_dtype, q_heads, cache, seq_len, nullptr, nullptr, 0, n_splits, workspace,
                                 /*out=*/nullptr, &extras, (cudaStream_t)stream);
}

extern "C" int32_t tq_gather_wait(tq_ctx *ctx, const tq_gather_desc *gather, int32_t batch, int32_t dtype,
                                  void *out_final, tq_stream stream) {
    if (!ctx) return TQ_ERR_ARG;
    int rc = tq_check_gather(gather);
    if (rc) return rc;
    if (batch <= 0 || gather->q_heads_total % gather->world) return TQ_ERR_ARG;
    if (out_final && ((dtype != TQ_DTYPE_F16 && dtype != TQ_DTYPE_BF16) || ((uintptr_t)out_final & 15))) return TQ_ERR_ARG;
    return tq_launch_gather_wait(gather, ctx->error_flag, ctx->wait_limit_ms, batch, 2, out_final, (cudaStream_t)stream);
}

extern "C" int32_t tq_set_wait_limit_ms(tq_ctx *ctx, int32_t limit_ms) {
    if (!ctx || limit_ms < 1 || limit_ms > 60000) return TQ_ERR_ARG;
    ctx->wait_limit_ms = limit_ms;
    return TQ_OK;
}
