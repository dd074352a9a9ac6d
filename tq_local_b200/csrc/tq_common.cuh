// Shared declarations for the sm_100a TurboQuant kernels: context layout, dtype
// helpers, error plumbing.  Internal to the library; the public surface is
// include/tq_b200.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tq_b200.h"

#define TQ_D 128
#define TQ_MAX_DEVICES 64  // devices one process may hold contexts on

// Device-resident codec tables.  Matrices are [128][128] fp32, row-major.
struct tq_ctx {
    int device;
    int bits;      // total bits
    int key_bits;  // bits-1 with QJL, else bits
    int use_qjl;
    int sm_count;
    float *rot_k;    // R_k[j][d]
    float *rot_k_t;  // R_k^T[d][j]
    float *rot_v;    // R_v[j][d]
    float *rot_v_t;
    float *qjl;      // S[i][d]
    float *qjl_t;    // S^T[d][i]
    float *centers_k;  // [16] (padded)
    float *bounds_k;   // [16] (padded with +inf)
    float *centers_v;
    float *bounds_v;
    // Shared-memory images for the tensor-core encoder: each [128][128] K-major operand split
    // into three bf16 terms, two 64-wide slabs per term, 128-byte swizzle (96 KB per matrix).
    uint16_t *img_rot_k;   // rows j, k = d:  R_k[j][d]      (B operand of u @ R_k^T)
    uint16_t *img_rot_v;
    uint16_t *img_rot_kt;  // rows d, k = j:  R_k[j][d]      (B operand of c @ R_k)
    uint16_t *img_qjl;     // rows i, k = d:  S[i][d]        (B operand of r @ S^T)
    void *base;       // one allocation holding everything above
    size_t base_bytes;
    struct tq_prof *prof;  // measurement hooks, see tq_profile_enable
    int *error_flag;       // device word, set by a kernel whose bounded wait ran out
    int wait_limit_ms;     // how long tq_gather_wait polls for a peer before it gives up (tq_set_wait_limit_ms)
    int64_t splits_cache_key;  // last (rows, length bucket) asked of tq_decode_suggest_splits
    int splits_cache_val;
};

// Measurement hooks: bracket the main decode kernel with events, count launches.
void tq_prof_begin(tq_ctx *ctx, cudaStream_t stream);
void tq_prof_end(tq_ctx *ctx, cudaStream_t stream);
void tq_prof_count(tq_ctx *ctx, int n_launches);

void tq_set_cuda_error(cudaError_t e, const char *where);

// Named NVTX range around the host side of an entry point (header-only NVTX: a no-op unless a
// profiler is attached), so that a timeline shows pack / append / decode / gather calls by name.
#include <nvtx3/nvToolsExt.h>
struct TqRange {
    explicit TqRange(const char *name) { nvtxRangePushA(name); }
    ~TqRange() { nvtxRangePop(); }
    TqRange(const TqRange &) = delete;
    TqRange &operator=(const TqRange &) = delete;
};

#define TQ_CUDA_CHECK(expr)                         \
    do {                                            \
        cudaError_t _e = (expr);                    \
        if (_e != cudaSuccess) {                    \
            tq_set_cuda_error(_e, #expr);           \
            return TQ_ERR_CUDA;                     \
        }                                           \
    } while (0)

// Kernel launch with the optional "programmatic stream serialization" attribute: the kernel may
// start while the preceding kernel of the stream is still running and must call
// griddepcontrol.wait before it touches anything that kernel writes.
template <typename... KArgs, typename... Args>
cudaError_t tq_launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             bool programmatic, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename T> __device__ __forceinline__ float tq_to_float(T x);
template <> __device__ __forceinline__ float tq_to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float tq_to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float tq_to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T tq_from_float(float x);
template <> __device__ __forceinline__ float tq_from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __half tq_from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 tq_from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Round a float through storage type T and back (the reference's `.to(dtype).float()`).
template <typename T> __device__ __forceinline__ float tq_round_through(float x) {
    return tq_to_float<T>(tq_from_float<T>(x));
}

__device__ __forceinline__ float tq_half_bits_to_float(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ uint16_t tq_float_to_half_bits(float x) {
    return __half_as_ushort(__float2half_rn(x));
}

__device__ __forceinline__ float tq_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float tq_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Argument validators shared by every entry point that takes the descriptor (nothing is
// launched before they pass): all stream pointers present and 16-byte aligned, strides
// multiples of 8 tokens that do not overlap rows; every peer pointer and the counter present.
int tq_check_cache(const tq_ctx *ctx, const tq_cache_desc *c);
int tq_check_gather(const tq_gather_desc *g);

// Entry points implemented in the other translation units.
int32_t tq_launch_pack(tq_ctx *ctx, const tq_dense_desc *k, const tq_dense_desc *v, int32_t n_tokens,
                       const tq_cache_desc *cache, int32_t pos0, cudaStream_t stream);
int32_t tq_launch_decode_exact(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                               const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                               const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits,
                               void *workspace, void *out, cudaStream_t stream);
// What a whole-step entry point adds to a plain decode launch (all optional).
struct TqStepExtras {
    const struct TqPackArgs *append;  // encode and append the step's new token in the query-preparation launch
    const int *len_ptr;               // the sequence length lives in device memory
    const tq_gather_desc *gather;     // KV-head shard: write the outputs into every rank's gathered buffer
    float *out_f32;                   // write the result unrounded (fp32) here instead of `out`
    int parts;                        // sequence split: ranks per KV-head group (0: off), see tq_decode_attn_parts
};
int tq_mma4_tokens_per_cta_step();
int32_t tq_launch_decode_mma4(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                              const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                              const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits,
                              void *workspace, void *out, const TqStepExtras *extras, cudaStream_t stream);
void tq_build_operand_image(const float *m, uint16_t *image);
int32_t tq_launch_pack_tc(tq_ctx *ctx, const tq_dense_desc *x, int which, int32_t n_tokens,
                          const tq_cache_desc *cache, int32_t pos0, cudaStream_t stream);
int32_t tq_launch_dequant(tq_ctx *ctx, const tq_cache_desc *cache, int32_t which, int32_t pos0,
                          int32_t n_tokens, const tq_dense_desc *out, cudaStream_t stream);
