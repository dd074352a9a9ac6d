// C-ABI entry points: context life-cycle, argument checking, dispatch.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <queue>
#include <vector>

#include "tq_common.cuh"
#include "tq_step_blocks.cuh"

static thread_local char g_err[256] = "";

void tq_set_cuda_error(cudaError_t e, const char *where) {
    snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
}

extern "C" const char *tq_last_cuda_error(void) { return g_err; }

struct tq_prof {
    bool on = false;
    std::vector<cudaEvent_t> events;  // start/stop pairs, created on first use
    size_t used = 0;                  // events recorded since the last read
    int64_t launches = 0;
};

void tq_prof_count(tq_ctx *ctx, int n) {
    if (ctx->prof && ctx->prof->on) ctx->prof->launches += n;
}

static void prof_record(tq_ctx *ctx, cudaStream_t stream) {
    tq_prof *p = ctx->prof;
    if (!p || !p->on || p->used >= 8192) return;
    if (p->used == p->events.size()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return;
        p->events.push_back(e);
    }
    cudaEventRecord(p->events[p->used++], stream);
}
void tq_prof_begin(tq_ctx *ctx, cudaStream_t stream) { prof_record(ctx, stream); }
void tq_prof_end(tq_ctx *ctx, cudaStream_t stream) { prof_record(ctx, stream); }

extern "C" int32_t tq_profile_enable(tq_ctx *ctx, int32_t on) {
    if (!ctx) return TQ_ERR_ARG;
    if (!ctx->prof) ctx->prof = new tq_prof();
    ctx->prof->on = on != 0;
    ctx->prof->used = 0;
    ctx->prof->launches = 0;
    return TQ_OK;
}

extern "C" int32_t tq_profile_read(tq_ctx *ctx, double *main_ms, int64_t *main_launches, int64_t *all_launches) {
    if (!ctx || !ctx->prof) return TQ_ERR_ARG;
    tq_prof *p = ctx->prof;
    double total = 0.0;
    int64_t n = 0;
    for (size_t i = 0; i + 1 < p->used; i += 2) {
        TQ_CUDA_CHECK(cudaEventSynchronize(p->events[i + 1]));
        float ms = 0.f;
        TQ_CUDA_CHECK(cudaEventElapsedTime(&ms, p->events[i], p->events[i + 1]));
        total += ms;
        ++n;
    }
    if (main_ms) *main_ms = total;
    if (main_launches) *main_launches = n;
    if (all_launches) *all_launches = p->launches;
    p->used = 0;
    p->launches = 0;
    return TQ_OK;
}
extern "C" int32_t tq_abi_version(void) { return 1; }

namespace {
// Makes `device` current for the lifetime of the guard and puts the caller's device back
// afterwards: creating or destroying a context must not change the device the host program
// (PyTorch, say) believes to be current - least of all from a destructor run by a garbage collector.
struct DeviceGuard {
    int previous = -1;
    cudaError_t status;
    explicit DeviceGuard(int device) {
        status = cudaGetDevice(&previous);
        if (status == cudaSuccess && previous != device) status = cudaSetDevice(device);
        else if (status != cudaSuccess) previous = -1;
    }
    ~DeviceGuard() {
        if (previous >= 0) cudaSetDevice(previous);
    }
};
}  // namespace

extern "C" int32_t tq_ctx_create(tq_ctx **out, int32_t device, const tq_codec_desc *c) {
    if (!out || !c || !c->rot_k || !c->rot_v || !c->centers_k || !c->bounds_k || !c->centers_v || !c->bounds_v)
        return TQ_ERR_ARG;
    if (c->head_dim != TQ_D || c->bits < 2 || c->bits > 4) return TQ_ERR_UNSUPPORTED;
    if (c->use_qjl && !c->qjl) return TQ_ERR_ARG;
    DeviceGuard guard(device);
    TQ_CUDA_CHECK(guard.status);

    const int kb = c->use_qjl ? c->bits - 1 : c->bits;
    const size_t M = (size_t)TQ_D * TQ_D;
    // 6 plain matrices + 8 matrix-sized slots holding four 96 KB operand images + 4 tables of 16 floats.
    const size_t n_float = 14 * M + 4 * 16 + 4;  // + the device status word
    std::vector<float> h(n_float, 0.0f);
    auto mat = [&](int i) { return h.data() + (size_t)i * M; };
    auto transpose = [&](const float *src, float *dst) {
        for (int r = 0; r < TQ_D; ++r)
            for (int cc = 0; cc < TQ_D; ++cc) dst[(size_t)cc * TQ_D + r] = src[(size_t)r * TQ_D + cc];
    };
    memcpy(mat(0), c->rot_k, M * 4);
    transpose(c->rot_k, mat(1));
    memcpy(mat(2), c->rot_v, M * 4);
    transpose(c->rot_v, mat(3));
    if (c->use_qjl) {
        memcpy(mat(4), c->qjl, M * 4);
        transpose(c->qjl, mat(5));
    }
    // operand images (49152 bf16 = 24576 floats each) in the 8 matrix-sized slots after the plain matrices
    uint16_t *img = reinterpret_cast<uint16_t *>(mat(6));
    const size_t kImg = 3 * M;  // bf16 elements per image
    tq_build_operand_image(mat(0), img);             // R_k
    tq_build_operand_image(mat(2), img + kImg);      // R_v
    tq_build_operand_image(mat(1), img + 2 * kImg);  // R_k^T
    tq_build_operand_image(mat(4), img + 3 * kImg);  // S
    float *tab = h.data() + 14 * M;
    for (int i = 0; i < 16; ++i) {
        tab[i] = i < (1 << kb) ? c->centers_k[i] : 0.0f;
        tab[16 + i] = i < (1 << kb) - 1 ? c->bounds_k[i] : INFINITY;
        tab[32 + i] = i < (1 << c->bits) ? c->centers_v[i] : 0.0f;
        tab[48 + i] = i < (1 << c->bits) - 1 ? c->bounds_v[i] : INFINITY;
    }

    tq_ctx *ctx = new tq_ctx();
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    ctx->bits = c->bits;
    ctx->key_bits = kb;
    ctx->use_qjl = c->use_qjl ? 1 : 0;
    ctx->wait_limit_ms = 2000;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
        tq_set_cuda_error(e, "cudaGetDeviceProperties");
        delete ctx;
        return TQ_ERR_CUDA;
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->base_bytes = n_float * sizeof(float);
    e = cudaMalloc(&ctx->base, ctx->base_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(ctx->base, h.data(), ctx->base_bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        tq_set_cuda_error(e, "tq_ctx_create upload");
        if (ctx->base) cudaFree(ctx->base);
        delete ctx;
        return TQ_ERR_CUDA;
    }
    float *d = (float *)ctx->base;
    auto dm = [&](int i) { return d + (size_t)i * M; };
    ctx->rot_k = dm(0);
    ctx->rot_k_t = dm(1);
    ctx->rot_v = dm(2);
    ctx->rot_v_t = dm(3);
    ctx->qjl = dm(4);
    ctx->qjl_t = dm(5);
    uint16_t *dimg = reinterpret_cast<uint16_t *>(dm(6));
    ctx->img_rot_k = dimg;
    ctx->img_rot_v = dimg + 3 * M;
    ctx->img_rot_kt = dimg + 6 * M;
    ctx->img_qjl = dimg + 9 * M;
    ctx->centers_k = d + 14 * M;
    ctx->bounds_k = ctx->centers_k + 16;
    ctx->centers_v = ctx->centers_k + 32;
    ctx->bounds_v = ctx->centers_k + 48;
    ctx->error_flag = reinterpret_cast<int *>(ctx->centers_k + 64);  // uploaded as zero
    *out = ctx;
    return TQ_OK;
}

extern "C" int32_t tq_ctx_destroy(tq_ctx *ctx) {
    if (!ctx) return TQ_OK;
    DeviceGuard guard(ctx->device);
    if (ctx->base) cudaFree(ctx->base);
    if (ctx->prof) {
        for (cudaEvent_t e : ctx->prof->events) cudaEventDestroy(e);
        delete ctx->prof;
    }
    delete ctx;
    return TQ_OK;
}

int tq_check_cache(const tq_ctx *ctx, const tq_cache_desc *c) {
    if (!c || !c->k_codes || !c->k_norms || !c->v_codes || !c->v_norms) return TQ_ERR_ARG;
    if (ctx->use_qjl && (!c->k_signs || !c->k_rnorms)) return TQ_ERR_ARG;
    if (c->batch <= 0 || c->kv_heads <= 0 || c->capacity <= 0) return TQ_ERR_ARG;
    if (c->stride_h < c->capacity || c->stride_b < (int64_t)c->kv_heads * c->stride_h) return TQ_ERR_ARG;
    if ((c->stride_b & 7) || (c->stride_h & 7)) return TQ_ERR_ARG;
    const uintptr_t all = (uintptr_t)c->k_codes | (uintptr_t)c->k_norms | (uintptr_t)c->v_codes |
                          (uintptr_t)c->v_norms | (uintptr_t)c->k_signs | (uintptr_t)c->k_rnorms;
    if (all & 15) return TQ_ERR_ARG;
    if ((uintptr_t)c->seq_start & 3) return TQ_ERR_ARG;
    return TQ_OK;
}

extern "C" int32_t tq_pack(tq_ctx *ctx, const tq_dense_desc *k, const tq_dense_desc *v, int32_t n_tokens,
                           const tq_cache_desc *cache, int32_t pos0, tq_stream stream) {
    TqRange range_("tq_pack");
    if (!ctx || !k || !v || !k->data || !v->data) return TQ_ERR_ARG;
    int rc = tq_check_cache(ctx, cache);
    if (rc) return rc;
    if (n_tokens < 0 || pos0 < 0 || (int64_t)pos0 + n_tokens > cache->capacity) return TQ_ERR_ARG;
    if (k->dtype != v->dtype || k->dtype < 0 || k->dtype > 2) return TQ_ERR_ARG;
    if (n_tokens == 0) return TQ_OK;
    return tq_launch_pack(ctx, k, v, n_tokens, cache, pos0, (cudaStream_t)stream);
}

extern "C" size_t tq_decode_workspace_bytes(int32_t batch, int32_t q_heads, int32_t n_splits) {
    if (batch <= 0 || q_heads <= 0 || n_splits <= 0) return 0;
    // rotated query + projected query (+ padding row), then (max, sum, acc[128]) per split.
    size_t rows = (size_t)batch * q_heads;
    size_t floats = rows * (2 * TQ_D + 8) + rows * (size_t)n_splits * (TQ_D + 2);
    return ((floats * 4 + 255) / 256) * 256;
}

extern "C" int32_t tq_decode_suggest_splits(tq_ctx *ctx, int32_t batch, int32_t kv_heads, int32_t seq_len) {
    if (!ctx || batch <= 0 || kv_heads <= 0 || seq_len <= 0) return 1;
    // The decode kernel cuts the rows, laid end to end, into one equal chunk per SM; a row then
    // spans at most ceil(row / chunk) + 1 chunks, which is the number of partial slots to provide.
    const int step = tq_mma4_tokens_per_cta_step();
    const int64_t n_pad = (seq_len + step - 1) / step * step;
    const int64_t total = (int64_t)batch * kv_heads * n_pad;
    const int64_t chunk = ((total + ctx->sm_count - 1) / ctx->sm_count + step - 1) / step * step;
    int64_t splits = (n_pad + chunk - 1) / chunk + 1;
    if (chunk >= n_pad && total % chunk == 0 && chunk % n_pad == 0) splits = 1;  // whole rows per CTA
    return (int32_t)(splits > 1024 ? 1024 : splits);
}

extern "C" int32_t tq_device_status(tq_ctx *ctx, int32_t *status_out) {
    if (!ctx || !status_out) return TQ_ERR_ARG;
    int v = 0;
    TQ_CUDA_CHECK(cudaMemcpy(&v, ctx->error_flag, sizeof(int), cudaMemcpyDeviceToHost));
    *status_out = v;
    return TQ_OK;
}

// tq_decode_attn, plus what the whole-step entry points add (`extras`, tensor-core path only).
static int32_t decode_attn_impl(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                                const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                                const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits, void *workspace,
                                size_t workspace_bytes, void *out, const TqStepExtras *extras, tq_stream stream) {
    if (!ctx || !q || !out || !workspace) return TQ_ERR_ARG;
    int rc = tq_check_cache(ctx, cache);
    if (rc) return rc;
    if (q_dtype < 0 || q_dtype > 2) return TQ_ERR_ARG;
    if (seq_len < 0 || seq_len > cache->capacity || n_tail < 0 || n_splits < 1) return TQ_ERR_ARG;
    if (seq_len + n_tail == 0) return TQ_ERR_ARG;
    if (n_tail > 0 && (!tail_k || !tail_v || !tail_k->data || !tail_v->data)) return TQ_ERR_ARG;
    if (q_heads <= 0 || q_heads % cache->kv_heads) return TQ_ERR_ARG;
    if (q_heads / cache->kv_heads > TQ_MAX_GROUPS) return TQ_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)workspace) & 15) return TQ_ERR_ARG;
    if (workspace_bytes < tq_decode_workspace_bytes(cache->batch, q_heads, n_splits)) return TQ_ERR_WORKSPACE;
    if (q_dtype == TQ_DTYPE_F32 || seq_len == 0)
        return tq_launch_decode_exact(ctx, q, q_dtype, q_heads, cache, seq_len, tail_k, tail_v, n_tail, n_splits,
                                      workspace, out, (cudaStream_t)stream);
    return tq_launch_decode_mma4(ctx, q, q_dtype, q_heads, cache, seq_len, tail_k, tail_v, n_tail, n_splits,
                                 workspace, out, extras, (cudaStream_t)stream);
}

extern "C" int32_t tq_decode_attn(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                                  const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                                  const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits,
                                  void *workspace, size_t workspace_bytes, void *out, tq_stream stream) {
    TqRange range_("tq_decode_attn");
    return decode_attn_impl(ctx, q, q_dtype, q_heads, cache, seq_len, tail_k, tail_v, n_tail, n_splits, workspace,
                            workspace_bytes, out, nullptr, stream);
}

extern "C" int32_t tq_decode_attn_f32out(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                                         const tq_cache_desc *cache, int32_t seq_len, int32_t n_splits,
                                         void *workspace, size_t workspace_bytes, float *out, tq_stream stream) {
    TqRange range_("tq_decode_attn_f32out");
    if (q_dtype != TQ_DTYPE_F16 && q_dtype != TQ_DTYPE_BF16) return TQ_ERR_UNSUPPORTED;
    if (seq_len <= 0) return TQ_ERR_ARG;
    const TqStepExtras extras = {nullptr, nullptr, nullptr, out, 0};
    return decode_attn_impl(ctx, q, q_dtype, q_heads, cache, seq_len, nullptr, nullptr, 0, n_splits, workspace,
                            workspace_bytes, out, &extras, stream);
}

extern "C" size_t tq_decode_step_workspace_bytes(int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t n_splits) {
    const size_t ws = tq_decode_workspace_bytes(batch, q_heads, n_splits);
    if (!ws || kv_heads <= 0) return 0;
    // device staging: q and out (batch x q_heads x 128), k and v (batch x kv_heads x 128), fp32-sized
    const size_t staging = ((size_t)batch * (2 * (size_t)q_heads + 2 * (size_t)kv_heads) * TQ_D * 4 + 255) / 256 * 256;
    return ws + staging;
}

// Device-side address of a caller buffer the GPU can reach directly (page-locked host memory
// mapped into the device's address space, managed or device memory), else nullptr.
static void *device_view(const void *p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (at.type == cudaMemoryTypeUnregistered || !at.devicePointer) return nullptr;
    return ((uintptr_t)at.devicePointer & 15) ? nullptr : at.devicePointer;
}

extern "C" int32_t tq_decode_step_host(tq_ctx *ctx, const void *q_host, const void *k_host, const void *v_host,
                                       int32_t dtype, int32_t q_heads, const tq_cache_desc *cache, int32_t pos,
                                       int32_t n_splits, void *workspace, size_t workspace_bytes, void *out_host,
                                       tq_stream stream) {
    TqRange range_("tq_decode_step_host");
    // every check comes before the first copy or launch: a call that fails leaves the cache and
    // the workspace untouched
    if (!ctx || !q_host || !k_host || !v_host || !out_host || !workspace || !cache) return TQ_ERR_ARG;
    int32_t rc = tq_check_cache(ctx, cache);
    if (rc) return rc;
    if (dtype < 0 || dtype > 2 || pos < 0 || pos >= cache->capacity || n_splits < 1) return TQ_ERR_ARG;
    if (q_heads <= 0 || q_heads % cache->kv_heads) return TQ_ERR_ARG;
    if (q_heads / cache->kv_heads > TQ_MAX_GROUPS) return TQ_ERR_UNSUPPORTED;
    if ((uintptr_t)workspace & 15) return TQ_ERR_ARG;
    const size_t need = tq_decode_step_workspace_bytes(cache->batch, q_heads, cache->kv_heads, n_splits);
    if (need == 0) return TQ_ERR_ARG;
    if (workspace_bytes < need) return TQ_ERR_WORKSPACE;
    const size_t es = dtype == TQ_DTYPE_F32 ? 4 : 2;
    const size_t q_bytes = (size_t)cache->batch * q_heads * TQ_D * es;
    const size_t kv_bytes = (size_t)cache->batch * cache->kv_heads * TQ_D * es;
    const size_t ws = tq_decode_workspace_bytes(cache->batch, q_heads, n_splits);
    cudaStream_t s = (cudaStream_t)stream;
    // Page-locked, device-mapped host buffers are read and written by the kernels themselves
    // (no copy engine round trips); anything else is staged through the workspace.
    void *d_q = device_view(q_host), *d_k = device_view(k_host), *d_v = device_view(v_host);
    void *d_out = device_view(out_host);
    const bool direct = d_q && d_k && d_v && d_out;
    if (!direct) {
        uint8_t *stage = (uint8_t *)workspace + ws;
        const size_t q_slot = (size_t)cache->batch * q_heads * TQ_D * 4;
        const size_t kv_slot = (size_t)cache->batch * cache->kv_heads * TQ_D * 4;
        d_q = stage, d_out = stage + q_slot, d_k = stage + 2 * q_slot, d_v = stage + 2 * q_slot + kv_slot;
        TQ_CUDA_CHECK(cudaMemcpyAsync(d_q, q_host, q_bytes, cudaMemcpyHostToDevice, s));
        TQ_CUDA_CHECK(cudaMemcpyAsync(d_k, k_host, kv_bytes, cudaMemcpyHostToDevice, s));
        TQ_CUDA_CHECK(cudaMemcpyAsync(d_v, v_host, kv_bytes, cudaMemcpyHostToDevice, s));
    }
    tq_dense_desc kd = {d_k, dtype, (int64_t)cache->kv_heads * TQ_D, TQ_D, TQ_D};
    tq_dense_desc vd = {d_v, dtype, (int64_t)cache->kv_heads * TQ_D, TQ_D, TQ_D};
    TqPackArgs append;
    TqStepExtras extras = {nullptr, nullptr, nullptr, nullptr, 0};
    if (dtype != TQ_DTYPE_F32) {
        // the tensor-core decode path encodes the new token in its own query-preparation launch
        tq_fill_pack_args(ctx, &kd, &vd, 1, cache, pos, &append);
        extras.append = &append;
    } else {
        rc = tq_pack(ctx, &kd, &vd, 1, cache, pos, stream);
        if (rc) return rc;
    }
    rc = decode_attn_impl(ctx, d_q, dtype, q_heads, cache, pos + 1, nullptr, nullptr, 0, n_splits, workspace, ws, d_out,
                          extras.append ? &extras : nullptr, stream);
    if (rc) return rc;
    if (!direct) TQ_CUDA_CHECK(cudaMemcpyAsync(out_host, d_out, q_bytes, cudaMemcpyDeviceToHost, s));
    return TQ_OK;
}

extern "C" int32_t tq_decode_step_host_gather(tq_ctx *ctx, const void *q_host, const void *k_host, const void *v_host,
                                              int32_t dtype, int32_t q_heads, const tq_cache_desc *cache, int32_t pos,
                                              int32_t n_splits, void *workspace, size_t workspace_bytes,
                                              const tq_gather_desc *gather, void *out_host, tq_stream stream) {
    TqRange range_("tq_decode_step_host_gather");
    if (!ctx || !q_host || !k_host || !v_host || !out_host || !workspace || !cache || !gather) return TQ_ERR_ARG;
    if (pos < 0 || pos >= cache->capacity || n_splits < 1) return TQ_ERR_ARG;
    if (dtype != TQ_DTYPE_F16 && dtype != TQ_DTYPE_BF16) return TQ_ERR_UNSUPPORTED;
    int32_t rc = tq_check_cache(ctx, cache);
    if (rc) return rc;
    if (q_heads <= 0 || q_heads % cache->kv_heads) return TQ_ERR_ARG;
    if (q_heads / cache->kv_heads > TQ_MAX_GROUPS) return TQ_ERR_UNSUPPORTED;
    rc = tq_check_gather(gather);  // before any launch: the combine kernel stores through these pointers
    if (rc) return rc;
    if (gather->q_heads_total != q_heads * gather->world || (uintptr_t)workspace & 15) return TQ_ERR_ARG;
    if (workspace_bytes < tq_decode_workspace_bytes(cache->batch, q_heads, n_splits)) return TQ_ERR_WORKSPACE;
    // the kernels read and write the host buffers themselves: they must be page-locked and mapped
    void *d_q = device_view(q_host), *d_k = device_view(k_host), *d_v = device_view(v_host);
    void *d_out = device_view(out_host);
    if (!d_q || !d_k || !d_v || !d_out) return TQ_ERR_ARG;
    tq_dense_desc kd = {d_k, dtype, (int64_t)cache->kv_heads * TQ_D, TQ_D, TQ_D};
    tq_dense_desc vd = {d_v, dtype, (int64_t)cache->kv_heads * TQ_D, TQ_D, TQ_D};
    TqPackArgs append;
    tq_fill_pack_args(ctx, &kd, &vd, 1, cache, pos, &append);
    const TqStepExtras extras = {&append, nullptr, gather, nullptr, 0};
    rc = tq_launch_decode_mma4(ctx, d_q, dtype, q_heads, cache, pos + 1, nullptr, nullptr, 0, n_splits, workspace,
                               nullptr, &extras, (cudaStream_t)stream);
    if (rc) return rc;
    return tq_gather_wait(ctx, gather, cache->batch, dtype, d_out, stream);
}

extern "C" int32_t tq_decode_step_dev(tq_ctx *ctx, const void *q, const void *k_new, const void *v_new, int32_t dtype,
                                      int32_t q_heads, const tq_cache_desc *cache, const int32_t *pos_dev,
                                      int32_t n_splits, void *workspace, size_t workspace_bytes, void *out,
                                      const tq_gather_desc *gather, tq_stream stream) {
    TqRange range_("tq_decode_step_dev");
    if (!ctx || !q || !k_new || !v_new || !out || !workspace || !pos_dev) return TQ_ERR_ARG;
    int32_t rc = tq_check_cache(ctx, cache);
    if (rc) return rc;
    if (gather) {  // validated before any launch: the combine kernel stores through these pointers
        rc = tq_check_gather(gather);
        if (rc) return rc;
        if (!gather->seq_dev || gather->q_heads_total != q_heads * gather->world) return TQ_ERR_ARG;
    }
    if (dtype < 0 || dtype > 2 || n_splits < 1) return TQ_ERR_ARG;
    if (q_heads <= 0 || q_heads % cache->kv_heads) return TQ_ERR_ARG;
    if (dtype == TQ_DTYPE_F32 || q_heads / cache->kv_heads > TQ_MAX_GROUPS) return TQ_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)workspace | (uintptr_t)k_new | (uintptr_t)v_new) & 15) return TQ_ERR_ARG;
    if ((uintptr_t)pos_dev & 3) return TQ_ERR_ARG;
    if (workspace_bytes < tq_decode_workspace_bytes(cache->batch, q_heads, n_splits)) return TQ_ERR_WORKSPACE;
    tq_dense_desc kd = {k_new, dtype, (int64_t)cache->kv_heads * TQ_D, TQ_D, TQ_D};
    tq_dense_desc vd = {v_new, dtype, (int64_t)cache->kv_heads * TQ_D, TQ_D, TQ_D};
    TqPackArgs append;
    tq_fill_pack_args(ctx, &kd, &vd, 1, cache, 0, &append);
    append.pos_ptr = pos_dev;
    const TqStepExtras extras = {&append, pos_dev, gather, nullptr, 0};
    rc = tq_launch_decode_mma4(ctx, q, dtype, q_heads, cache, cache->capacity, nullptr, nullptr, 0, n_splits, workspace,
                               gather ? nullptr : out, &extras, (cudaStream_t)stream);
    if (rc || !gather) return rc;
    return tq_gather_wait(ctx, gather, cache->batch, dtype, out, stream);
}

extern "C" int32_t tq_dequant(tq_ctx *ctx, const tq_cache_desc *cache, int32_t which, int32_t pos0,
                              int32_t n_tokens, const tq_dense_desc *out, tq_stream stream) {
    TqRange range_("tq_dequant");
    if (!ctx || !out || !out->data) return TQ_ERR_ARG;
    int rc = tq_check_cache(ctx, cache);
    if (rc) return rc;
    if (which < 0 || which > 1 || out->dtype < 0 || out->dtype > 2) return TQ_ERR_ARG;
    if (n_tokens < 0 || pos0 < 0 || (int64_t)pos0 + n_tokens > cache->capacity) return TQ_ERR_ARG;
    if (n_tokens == 0) return TQ_OK;
    return tq_launch_dequant(ctx, cache, which, pos0, n_tokens, out, (cudaStream_t)stream);
}
