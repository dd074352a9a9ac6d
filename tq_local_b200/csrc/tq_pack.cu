// CUDA-core (fp32 FMA) encode / dequantise kernels: one warp per vector.
//
// tq_pack_rows_kernel is the arithmetic-exact encoder: fp32 accumulation in a
// fixed order, true division, the reference's tie rule (a value equal to a
// boundary goes to the lower bin) and the reference's dtype round trip of the
// reconstruction before the QJL residual.  It serves the O(1) append of decoded
// tokens and small prefills; large prefills go to the tensor-core kernel.
#include "tq_common.cuh"
#include "tq_step_blocks.cuh"

namespace {

constexpr int kWarpsPerBlock = 8;

using PackArgs = TqPackArgs;

template <typename T, bool QJL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) tq_pack_rows_kernel(PackArgs a) {
    __shared__ float s_vec[kWarpsPerBlock][TQ_D];
    __shared__ float s_cq[kWarpsPerBlock][TQ_D];
    __shared__ uint8_t s_code[kWarpsPerBlock][TQ_D];
    __shared__ float s_bnd[2][16];
    __shared__ float s_cen[16];
    if (threadIdx.x < 32) {
        const int i = threadIdx.x & 15, kind = threadIdx.x >> 4;
        s_bnd[kind][i] = a.bounds[kind][i];
        if (kind == 0) s_cen[i] = a.centers_k[i];
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t n_vec = (int64_t)a.B * a.H * a.S;
    const int64_t n_items = a.n_kinds * n_vec;
    float *vec = s_vec[warp];
    float *cq = s_cq[warp];
    uint8_t *code = s_code[warp];

    for (int64_t item = (int64_t)blockIdx.x * kWarpsPerBlock + warp; item < n_items;
         item += (int64_t)gridDim.x * kWarpsPerBlock) {
        const int kind = a.first_kind + (item >= n_vec ? 1 : 0);
        const int64_t vid = item >= n_vec ? item - n_vec : item;
        const int t = (int)(vid % a.S);
        const int h = (int)((vid / a.S) % a.H);
        const int b = (int)(vid / ((int64_t)a.S * a.H));
        const T *src = (const T *)a.x[kind] + b * a.sb[kind] + h * a.sh[kind] + (int64_t)t * a.st[kind];
        const int64_t row = b * a.cache_sb + h * a.cache_sh + a.pos0 + t;
        const int bits = a.bits[kind];

        float x[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = tq_to_float<T>(src[4 * lane + i]);
        float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
        const float nrm = sqrtf(tq_warp_sum(ss));
        const float safe = nrm > 0.0f ? nrm : 1.0f;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) vec[4 * lane + i] = x[i] / safe;
        __syncwarp();

        // z_j = sum_d u_d * R[j][d] for j = 4*lane .. 4*lane+3
        float z[4] = {0.f, 0.f, 0.f, 0.f};
        const float4 *rt = (const float4 *)a.rot_t[kind] + lane;
#pragma unroll 8
        for (int d = 0; d < TQ_D; ++d) {
            const float u = vec[d];
            const float4 r = __ldg(rt + d * (TQ_D / 4));
            z[0] = fmaf(u, r.x, z[0]);
            z[1] = fmaf(u, r.y, z[1]);
            z[2] = fmaf(u, r.z, z[2]);
            z[3] = fmaf(u, r.w, z[3]);
        }
        int idx[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int c = 0;
#pragma unroll
            for (int e = 0; e < 15; ++e) c += (s_bnd[kind][e] < z[i]) ? 1 : 0;
            idx[i] = c;
            code[4 * lane + i] = (uint8_t)c;
        }
        const uint16_t nh = tq_float_to_half_bits(safe);
        if (lane == 0) a.norms[kind][row] = nh;
        __syncwarp();
        if (lane < 4 * bits) {
            uint32_t *dst = (uint32_t *)(a.codes[kind] + row * (int64_t)(16 * bits));
            dst[lane] = tq_assemble_word(code, lane, bits);
        }

        if (QJL && kind == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) cq[4 * lane + i] = s_cen[idx[i]];
            __syncwarp();
            float rec[4] = {0.f, 0.f, 0.f, 0.f};
            const float4 *rk = (const float4 *)a.rot_k + lane;
#pragma unroll 8
            for (int j = 0; j < TQ_D; ++j) {
                const float c = cq[j];
                const float4 r = __ldg(rk + j * (TQ_D / 4));
                rec[0] = fmaf(c, r.x, rec[0]);
                rec[1] = fmaf(c, r.y, rec[1]);
                rec[2] = fmaf(c, r.z, rec[2]);
                rec[3] = fmaf(c, r.w, rec[3]);
            }
            const float nf = tq_half_bits_to_float(nh);
            float res[4];
            float rs = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                res[i] = x[i] - tq_round_through<T>(rec[i] * nf);
                rs = fmaf(res[i], res[i], rs);
            }
            const float rn = sqrtf(tq_warp_sum(rs));
            const float rsafe = rn > 0.0f ? rn : 1.0f;
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) vec[4 * lane + i] = res[i] / rsafe;
            __syncwarp();
            float pr[4] = {0.f, 0.f, 0.f, 0.f};
            const float4 *st = (const float4 *)a.qjl_t + lane;
#pragma unroll 8
            for (int d = 0; d < TQ_D; ++d) {
                const float u = vec[d];
                const float4 r = __ldg(st + d * (TQ_D / 4));
                pr[0] = fmaf(u, r.x, pr[0]);
                pr[1] = fmaf(u, r.y, pr[1]);
                pr[2] = fmaf(u, r.z, pr[2]);
                pr[3] = fmaf(u, r.w, pr[3]);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) code[4 * lane + i] = pr[i] >= 0.0f ? 1 : 0;
            __syncwarp();
            uint32_t mine = 0;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t m = __ballot_sync(0xffffffffu, code[32 * w + lane] != 0);
                if (lane == w) mine = m;
            }
            if (lane < 4) ((uint32_t *)(a.signs + row * 16))[lane] = mine;
            if (lane == 0) a.rnorms[row] = tq_float_to_half_bits(rsafe);
        }
        __syncwarp();
    }
}

// Latency-optimised encoder for a handful of vectors (the per-step append of decoded tokens):
// one 512-thread block per vector, see tq_pack_small_block.
template <typename T, bool QJL>
__global__ void __launch_bounds__(4 * TQ_D, 2) tq_pack_small_kernel(PackArgs a) {
    tq_pack_small_block<T, QJL>(a, blockIdx.x);
}

struct DequantArgs {
    const uint8_t *codes;
    const uint16_t *norms;
    const uint8_t *signs;
    const uint16_t *rnorms;
    int64_t cache_sb, cache_sh;
    int B, H, S, pos0, bits;
    void *out;
    int64_t ob, oh, ot;
    const float *rot;    // R[j][d]
    const float *qjl;    // S[i][d]
    const float *centers;
};

template <typename T, bool QJL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) tq_dequant_rows_kernel(DequantArgs a) {
    __shared__ float s_cq[kWarpsPerBlock][TQ_D];
    __shared__ float s_cen[16];
    if (threadIdx.x < 16) s_cen[threadIdx.x] = a.centers[threadIdx.x];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *cq = s_cq[warp];
    const int64_t n_vec = (int64_t)a.B * a.H * a.S;
    const int bits = a.bits;
    const uint32_t mask = (1u << bits) - 1u;
    const int row_bytes = 16 * bits;
    for (int64_t vid = (int64_t)blockIdx.x * kWarpsPerBlock + warp; vid < n_vec;
         vid += (int64_t)gridDim.x * kWarpsPerBlock) {
        const int t = (int)(vid % a.S);
        const int h = (int)((vid / a.S) % a.H);
        const int b = (int)(vid / ((int64_t)a.S * a.H));
        const int64_t row = b * a.cache_sb + h * a.cache_sh + a.pos0 + t;
        const uint8_t *rb = a.codes + row * row_bytes;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = 4 * lane + i;
            const int o = j * bits, by = o >> 3, sh = o & 7;
            uint32_t v = rb[by];
            if (by + 1 < row_bytes) v |= (uint32_t)rb[by + 1] << 8;
            cq[j] = s_cen[(v >> sh) & mask];
        }
        __syncwarp();
        float rec[4] = {0.f, 0.f, 0.f, 0.f};
        const float4 *rk = (const float4 *)a.rot + lane;
#pragma unroll 8
        for (int j = 0; j < TQ_D; ++j) {
            const float c = cq[j];
            const float4 r = __ldg(rk + j * (TQ_D / 4));
            rec[0] = fmaf(c, r.x, rec[0]);
            rec[1] = fmaf(c, r.y, rec[1]);
            rec[2] = fmaf(c, r.z, rec[2]);
            rec[3] = fmaf(c, r.w, rec[3]);
        }
        const float nf = tq_half_bits_to_float(a.norms[row]);
        float outv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) outv[i] = tq_round_through<T>(rec[i] * nf);
        if (QJL) {
            __syncwarp();
            const uint32_t *sw = (const uint32_t *)(a.signs + row * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = 4 * lane + i;
                cq[j] = ((sw[j >> 5] >> (j & 31)) & 1u) ? 1.0f : -1.0f;
            }
            __syncwarp();
            float cor[4] = {0.f, 0.f, 0.f, 0.f};
            const float4 *sq = (const float4 *)a.qjl + lane;
#pragma unroll 8
            for (int i = 0; i < TQ_D; ++i) {
                const float s = cq[i];
                const float4 r = __ldg(sq + i * (TQ_D / 4));
                cor[0] = fmaf(s, r.x, cor[0]);
                cor[1] = fmaf(s, r.y, cor[1]);
                cor[2] = fmaf(s, r.z, cor[2]);
                cor[3] = fmaf(s, r.w, cor[3]);
            }
            const float rn = tq_half_bits_to_float(a.rnorms[row]);
            const float scale = 1.2533141373155003f / (float)TQ_D;  // sqrt(pi/2)/D
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float c = tq_round_through<T>(cor[i] * rn * scale);
                outv[i] = tq_round_through<T>(outv[i] + c);
            }
        }
        T *dst = (T *)a.out + b * a.ob + h * a.oh + (int64_t)t * a.ot + 4 * lane;
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = tq_from_float<T>(outv[i]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) tq_norm_sum_kernel(const T *x, int64_t sb, int64_t sh, int64_t st, int B,
                                                          int H, int S, double *out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t n_vec = (int64_t)B * H * S;
    double acc = 0.0;
    for (int64_t vid = (int64_t)blockIdx.x * 8 + warp; vid < n_vec; vid += (int64_t)gridDim.x * 8) {
        const int t = (int)(vid % S);
        const int h = (int)((vid / S) % H);
        const int b = (int)(vid / ((int64_t)S * H));
        const T *src = x + b * sb + h * sh + (int64_t)t * st + 4 * lane;
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float v = tq_to_float<T>(src[i]);
            ss = fmaf(v, v, ss);
        }
        acc += (double)sqrtf(tq_warp_sum(ss));
    }
    __shared__ double s_acc[8];
    if (lane == 0) s_acc[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int i = 0; i < 8; ++i) tot += s_acc[i];
        atomicAdd(out, tot);
    }
}

int grid_for(int64_t items, int sm_count) {
    int64_t blocks = (items + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int64_t cap = (int64_t)sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace

void tq_fill_pack_args(tq_ctx *ctx, const tq_dense_desc *k, const tq_dense_desc *v, int32_t n_tokens,
                       const tq_cache_desc *cache, int32_t pos0, TqPackArgs *out) {
    TqPackArgs &a = *out;
    a.x[0] = k->data;
    a.x[1] = v->data;
    a.sb[0] = k->stride_b, a.sh[0] = k->stride_h, a.st[0] = k->stride_t;
    a.sb[1] = v->stride_b, a.sh[1] = v->stride_h, a.st[1] = v->stride_t;
    a.B = cache->batch, a.H = cache->kv_heads, a.S = n_tokens, a.pos0 = pos0;
    a.bits[0] = ctx->key_bits, a.bits[1] = ctx->bits;
    a.codes[0] = cache->k_codes, a.codes[1] = cache->v_codes;
    a.norms[0] = cache->k_norms, a.norms[1] = cache->v_norms;
    a.signs = cache->k_signs, a.rnorms = cache->k_rnorms;
    a.cache_sb = cache->stride_b, a.cache_sh = cache->stride_h;
    a.rot_t[0] = ctx->rot_k_t, a.rot_t[1] = ctx->rot_v_t;
    a.rot_k = ctx->rot_k, a.qjl_t = ctx->qjl_t;
    a.centers_k = ctx->centers_k;
    a.bounds[0] = ctx->bounds_k, a.bounds[1] = ctx->bounds_v;
    a.first_kind = 0, a.n_kinds = 2;
    a.pos_ptr = nullptr, a.capacity = cache->capacity, a.error_flag = ctx->error_flag;
}

int32_t tq_launch_pack(tq_ctx *ctx, const tq_dense_desc *k, const tq_dense_desc *v, int32_t n_tokens,
                       const tq_cache_desc *cache, int32_t pos0, cudaStream_t stream) {
    PackArgs a;
    tq_fill_pack_args(ctx, k, v, n_tokens, cache, pos0, &a);
    static bool configured = false;
    if (!configured) {  // same shared-memory carve-out as the decode kernels: no SM reconfiguration between them
        configured = true;
        cudaFuncSetAttribute(tq_pack_rows_kernel<float, true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaFuncSetAttribute(tq_pack_rows_kernel<float, false>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaFuncSetAttribute(tq_pack_rows_kernel<__half, true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaFuncSetAttribute(tq_pack_rows_kernel<__half, false>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaFuncSetAttribute(tq_pack_rows_kernel<__nv_bfloat16, true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaFuncSetAttribute(tq_pack_rows_kernel<__nv_bfloat16, false>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    }
    // Large encodes go to the tensor-core kernel; small appends (and tensors whose alignment
    // the tensor-core loader cannot take) stay on this one.
    a.first_kind = 0, a.n_kinds = 2;
    const int64_t n_vec = (int64_t)a.B * a.H * a.S;
    if (n_vec >= 1024) {
        if (tq_launch_pack_tc(ctx, v, 1, n_tokens, cache, pos0, stream) == TQ_OK) a.n_kinds = 1;
        if (a.n_kinds == 1 && tq_launch_pack_tc(ctx, k, 0, n_tokens, cache, pos0, stream) == TQ_OK) return TQ_OK;
    }
    const int64_t items = a.n_kinds * n_vec;
    if (n_vec < 1024) {  // appends: one block per vector
#define TQ_LAUNCH_SMALL(T)                                                                   \
    do {                                                                                     \
        if (ctx->use_qjl)                                                                    \
            tq_pack_small_kernel<T, true><<<(unsigned)items, 4 * TQ_D, 0, stream>>>(a);      \
        else                                                                                 \
            tq_pack_small_kernel<T, false><<<(unsigned)items, 4 * TQ_D, 0, stream>>>(a);     \
    } while (0)
        if (k->dtype == TQ_DTYPE_F32) TQ_LAUNCH_SMALL(float);
        else if (k->dtype == TQ_DTYPE_F16) TQ_LAUNCH_SMALL(__half);
        else TQ_LAUNCH_SMALL(__nv_bfloat16);
#undef TQ_LAUNCH_SMALL
        tq_prof_count(ctx, 1);
        TQ_CUDA_CHECK(cudaGetLastError());
        return TQ_OK;
    }
    const int grid = grid_for(items, ctx->sm_count);
    const int threads = kWarpsPerBlock * 32;
#define TQ_LAUNCH_PACK(T)                                                          \
    do {                                                                           \
        if (ctx->use_qjl)                                                          \
            tq_pack_rows_kernel<T, true><<<grid, threads, 0, stream>>>(a);         \
        else                                                                       \
            tq_pack_rows_kernel<T, false><<<grid, threads, 0, stream>>>(a);        \
    } while (0)
    if (k->dtype == TQ_DTYPE_F32) TQ_LAUNCH_PACK(float);
    else if (k->dtype == TQ_DTYPE_F16) TQ_LAUNCH_PACK(__half);
    else TQ_LAUNCH_PACK(__nv_bfloat16);
#undef TQ_LAUNCH_PACK
    tq_prof_count(ctx, 1);
    TQ_CUDA_CHECK(cudaGetLastError());
    return TQ_OK;
}

int32_t tq_launch_dequant(tq_ctx *ctx, const tq_cache_desc *cache, int32_t which, int32_t pos0,
                          int32_t n_tokens, const tq_dense_desc *out, cudaStream_t stream) {
    DequantArgs a;
    const bool key = which == 0;
    a.codes = key ? cache->k_codes : cache->v_codes;
    a.norms = key ? cache->k_norms : cache->v_norms;
    a.signs = cache->k_signs, a.rnorms = cache->k_rnorms;
    a.cache_sb = cache->stride_b, a.cache_sh = cache->stride_h;
    a.B = cache->batch, a.H = cache->kv_heads, a.S = n_tokens, a.pos0 = pos0;
    a.bits = key ? ctx->key_bits : ctx->bits;
    a.out = const_cast<void *>(out->data);
    a.ob = out->stride_b, a.oh = out->stride_h, a.ot = out->stride_t;
    a.rot = key ? ctx->rot_k : ctx->rot_v;
    a.qjl = ctx->qjl;
    a.centers = key ? ctx->centers_k : ctx->centers_v;
    const bool qjl = key && ctx->use_qjl;
    const int grid = grid_for((int64_t)a.B * a.H * a.S, ctx->sm_count);
    const int threads = kWarpsPerBlock * 32;
#define TQ_LAUNCH_DQ(T)                                                               \
    do {                                                                              \
        if (qjl)                                                                      \
            tq_dequant_rows_kernel<T, true><<<grid, threads, 0, stream>>>(a);         \
        else                                                                          \
            tq_dequant_rows_kernel<T, false><<<grid, threads, 0, stream>>>(a);        \
    } while (0)
    if (out->dtype == TQ_DTYPE_F32) TQ_LAUNCH_DQ(float);
    else if (out->dtype == TQ_DTYPE_F16) TQ_LAUNCH_DQ(__half);
    else TQ_LAUNCH_DQ(__nv_bfloat16);
#undef TQ_LAUNCH_DQ
    TQ_CUDA_CHECK(cudaGetLastError());
    return TQ_OK;
}

extern "C" int32_t tq_key_norm_sum(const tq_dense_desc *k, int32_t batch, int32_t heads, int32_t n_tokens,
                                   double *sum_out, tq_stream stream) {
    if (!k || !k->data || !sum_out || batch <= 0 || heads <= 0 || n_tokens <= 0) return TQ_ERR_ARG;
    const int64_t n_vec = (int64_t)batch * heads * n_tokens;
    int grid = (int)((n_vec + 7) / 8 < 1184 ? (n_vec + 7) / 8 : 1184);
    cudaStream_t s = (cudaStream_t)stream;
    if (k->dtype == TQ_DTYPE_F32)
        tq_norm_sum_kernel<float><<<grid, 256, 0, s>>>((const float *)k->data, k->stride_b, k->stride_h, k->stride_t,
                                                       batch, heads, n_tokens, sum_out);
    else if (k->dtype == TQ_DTYPE_F16)
        tq_norm_sum_kernel<__half><<<grid, 256, 0, s>>>((const __half *)k->data, k->stride_b, k->stride_h,
                                                        k->stride_t, batch, heads, n_tokens, sum_out);
    else if (k->dtype == TQ_DTYPE_BF16)
        tq_norm_sum_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16 *)k->data, k->stride_b,
                                                               k->stride_h, k->stride_t, batch, heads, n_tokens,
                                                               sum_out);
    else
        return TQ_ERR_ARG;
    TQ_CUDA_CHECK(cudaGetLastError());
    return TQ_OK;
}
