// tq_decode_attn_static: decode attention for callers that cannot allocate.
//
// Some hosts of this library may not call cudaMalloc (or any allocator) once they are
// running: an inference server that gives all device memory to its own pool at start-up, or
// a plug-in hook that the host framework forbids from allocating.  Such a caller has nowhere
// to get the scratch workspace that tq_decode_attn asks for.  This entry point runs the same
// kernels with the scratch placed in a fixed array that is part of the library image, so the
// call itself allocates nothing.
//
// Limits and rules:
//   * the array is kStaticScratchBytes (8 MiB) and every GPU that loads the library holds it
//     until the process exits; a shape whose scratch need (tq_decode_workspace_bytes) is larger
//     is rejected with TQ_ERR_WORKSPACE;
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress) and
//     remembers it; make that first call before any stream capture begins;
//   * all calls share the one array, which keeps whatever the previous call left in it.  The
//     kernels overwrite every word they later read, so nothing has to be cleared, but two calls
//     that overlap on the GPU (different streams, or the same context from two threads) race on
//     it: serialise them;
//   * the context's device must be the current device.
#include <mutex>

#include "tq_common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_scratch_mutex;
void *g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the array on `device`, which must be the current device.
int32_t static_scratch_for(int device, void **out) {
    if (device < 0 || device >= kMaxDevices) return TQ_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[device]) {
        void *p = nullptr;
        TQ_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
        g_scratch_ptr[device] = p;
    }
    *out = g_scratch_ptr[device];
    return TQ_OK;
}

}  // namespace

extern "C" size_t tq_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int32_t tq_decode_attn_static(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                                         const tq_cache_desc *cache, int32_t seq_len, int32_t n_splits, void *out,
                                         tq_stream stream) {
    TqRange range_("tq_decode_attn_static");
    if (!ctx || !q || !out) return TQ_ERR_ARG;
    int32_t rc = tq_check_cache(ctx, cache);  // the same descriptor checks as tq_decode_attn
    if (rc) return rc;
    if (q_dtype < 0 || q_dtype > 2 || n_splits < 1) return TQ_ERR_ARG;
    if (seq_len <= 0 || seq_len > cache->capacity) return TQ_ERR_ARG;
    if (q_heads <= 0 || q_heads % cache->kv_heads) return TQ_ERR_ARG;
    const int groups = q_heads / cache->kv_heads;
    if (groups > TQ_MAX_GROUPS) return TQ_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)out) & 15) return TQ_ERR_ARG;
    if (tq_decode_workspace_bytes(cache->batch, q_heads, n_splits) > kStaticScratchBytes) {
        tq_set_cuda_error(cudaErrorMemoryAllocation,
                          "tq_decode_attn_static: shape needs more scratch than the 8 MiB built-in array; "
                          "use fewer splits or tq_decode_attn with a caller workspace");
        return TQ_ERR_WORKSPACE;
    }
    int current = -1;
    TQ_CUDA_CHECK(cudaGetDevice(&current));
    if (current != ctx->device) return TQ_ERR_ARG;
    void *scratch = nullptr;
    rc = static_scratch_for(current, &scratch);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (q_dtype == TQ_DTYPE_F32)
        return tq_launch_decode_exact(ctx, q, q_dtype, q_heads, cache, seq_len, nullptr, nullptr, 0, n_splits, scratch,
                                      out, s);
    return tq_launch_decode_mma4(ctx, q, q_dtype, q_heads, cache, seq_len, nullptr, nullptr, 0, n_splits, scratch, out,
                                 nullptr, s);
}
