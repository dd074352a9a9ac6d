// Block-level bodies of the latency-bound kernels of a decode step: query preparation and
// the append of the step's new key / value vectors.  They live in a header so that one
// launch can run both kinds of block side by side (tq_step_prologue_kernel) and the
// stand-alone kernels share the same code.  Every body is written for 512 threads and at
// most 64 registers, so two blocks fit an SM and a whole step's prologue is one wave.
//
// All mat-vecs use the same shape: thread (j, dq) owns output column j and the 32 matrix
// rows [32 dq, 32 dq + 32); its 32 matrix elements are loaded into registers in one batch
// (one trip to L2 instead of a chain of them) before the data they multiply is ready.
#pragma once

#include "tq_common.cuh"

struct TqPackArgs {
    const void *x[2];  // K, V
    int64_t sb[2], sh[2], st[2];
    int B, H, S;
    int pos0;
    int bits[2];  // key_bits, value bits
    uint8_t *codes[2];
    uint16_t *norms[2];
    uint8_t *signs;
    uint16_t *rnorms;
    int64_t cache_sb, cache_sh;
    const float *rot_t[2];   // R^T[d][j] for the rotation
    const float *rot_k;      // R_k[j][d] for the reconstruction
    const float *qjl_t;      // S^T[d][i]
    const float *centers_k;
    const float *bounds[2];
    int first_kind, n_kinds;  // which of {keys, values} this launch encodes
    const int *pos_ptr;       // when set, the append position is read from device memory instead of pos0
    int capacity;             // tokens per cache row; an append past it is dropped and flagged
    int *error_flag;
};

struct TqQprepArgs {
    const void *q;          // [kv_rows * G][128] in the query dtype
    const float *rot_k_t;   // R_k^T[d][j]
    const float *qjl_t;     // S^T[d][i]
    uint32_t *frag;         // [kv_rows * G][TQ_FRAG_WORDS]
    int G, use_qjl;
    int64_t kv_rows;
};

// Words per query head in the fragment area: 8 lane variants of 26 words, padded to the size
// of the rotated + projected query rows the area overlays in the decode workspace.
#define TQ_FRAG_ROW_WORDS (2 * TQ_D + 8)

// How the decode kernel cuts the (batch, KV head) rows, laid end to end and each padded to
// `step` tokens, into one chunk per CTA.  A row then has at most n_splits partials.  Computed by
// the host for a length it knows and by the kernels themselves for a length kept on the device.
struct TqPlan {
    int n_pad, chunk;
};
__host__ __device__ inline TqPlan tq_make_plan(int seq_len, int rows, int n_ctas, int n_splits, int step) {
    TqPlan p;
    p.n_pad = (seq_len + step - 1) / step * step;
    const long long total = (long long)rows * p.n_pad;
    long long chunk = ((total + n_ctas - 1) / n_ctas + step - 1) / step * step;
    if (n_splits == 1) {
        chunk = p.n_pad;
    } else {
        const long long floor_chunk = ((p.n_pad + n_splits - 2) / (n_splits - 1) + step - 1) / step * step;
        if (chunk < floor_chunk) chunk = floor_chunk;
    }
    p.chunk = (int)chunk;
    return p;
}

void tq_fill_pack_args(tq_ctx *ctx, const tq_dense_desc *k, const tq_dense_desc *v, int32_t n_tokens,
                       const tq_cache_desc *cache, int32_t pos0, TqPackArgs *a);

// Programmatic dependent launch: `tq_grid_dependency_wait` returns once the preceding kernel
// of the stream has completed and its writes are visible (at once when the launch carried no
// programmatic attribute); `tq_launch_dependents` lets the next kernel's blocks start early.
__device__ __forceinline__ void tq_grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void tq_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

__device__ __forceinline__ void tq_load_column(float (&m)[32], const float *mat, int dq, int j) {
#pragma unroll
    for (int i = 0; i < 32; ++i) m[i] = __ldg(mat + (32 * dq + i) * TQ_D + j);
}

// Assemble 32-bit word `w` of the LSB-first bitstream from one-code-per-byte storage.
__device__ __forceinline__ uint32_t tq_assemble_word(const uint8_t *codes, int w, int bits) {
    uint32_t word = 0;
    const int lo = 32 * w;
    int j = lo / bits;
    for (; j < TQ_D && j * bits < lo + 32; ++j) {
        const int sh = j * bits - lo;
        const uint32_t c = codes[j];
        word |= sh >= 0 ? (c << sh) : (c >> (-sh));
    }
    return word;
}

// ---------------------------------------------------------------------------------------------
// Encode one vector (item < n_vec: kind first_kind, else the next kind) and write it at its
// cache row.  fp32 arithmetic in a fixed order: partial sums over four 32-row quarters, then
// (p0 + p1) + (p2 + p3).
template <typename T, bool QJL> __device__ __forceinline__ void tq_pack_small_block(const TqPackArgs &a, int64_t item) {
    __shared__ float s_x[TQ_D], s_u[TQ_D], s_part[4][TQ_D], s_red[4];
    __shared__ uint8_t s_code[TQ_D];
    __shared__ float s_bnd[16], s_cen[16];
    const int tid = threadIdx.x, j = tid & (TQ_D - 1), dq = tid >> 7, lane = tid & 31;
    const int64_t n_vec = (int64_t)a.B * a.H * a.S;
    const int kind = a.first_kind + (item >= n_vec ? 1 : 0);
    const int64_t vid = item >= n_vec ? item - n_vec : item;
    const int t = (int)(vid % a.S);
    const int h = (int)((vid / a.S) % a.H);
    const int b = (int)(vid / ((int64_t)a.S * a.H));
    const T *src = (const T *)a.x[kind] + b * a.sb[kind] + h * a.sh[kind] + (int64_t)t * a.st[kind];
    const int bits = a.bits[kind];
    float m[32];
    tq_load_column(m, a.rot_t[kind], dq, j);  // (codec constants: fetched before the wait)
    if (tid < 16) s_bnd[tid] = a.bounds[kind][tid], s_cen[tid] = a.centers_k[tid];
    // the new vectors and the append position come from, and the cache may still be read by, the
    // preceding kernel of the stream
    tq_grid_dependency_wait();
    tq_launch_dependents();
    const int pos0 = a.pos_ptr ? *a.pos_ptr : a.pos0;
    if (pos0 < 0 || pos0 + a.S > a.capacity) {  // (the whole block leaves together)
        if (tid == 0) atomicExch(a.error_flag, 4);
        return;
    }
    const int64_t row = b * a.cache_sb + h * a.cache_sh + pos0 + t;

    auto block_norm = [&](float v) {  // sqrt of the sum of v*v over the 128 threads with dq == 0
        float ss = dq == 0 ? v * v : 0.f;
        ss = tq_warp_sum(ss);
        if (dq == 0 && lane == 0) s_red[j >> 5] = ss;
        __syncthreads();
        const float tot = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
        __syncthreads();
        return sqrtf(tot);
    };
    // partial of out[j] = sum_d vec[d] * m[d][j] over this thread's quarter of d
    auto quarter = [&](const float *vec) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) acc = fmaf(vec[32 * dq + i], m[i], acc);
        s_part[dq][j] = acc;
    };
    auto finish = [&]() {
        __syncthreads();
        const float r = (s_part[0][j] + s_part[1][j]) + (s_part[2][j] + s_part[3][j]);
        __syncthreads();
        return r;
    };

    const float x = tq_to_float<T>(src[j]);
    const float nrm = block_norm(x);
    const float safe = nrm > 0.0f ? nrm : 1.0f;
    if (dq == 0) s_x[j] = x, s_u[j] = x / safe;
    __syncthreads();
    quarter(s_u);
    const bool residual = QJL && kind == 0;
    if (residual) tq_load_column(m, a.rot_k, dq, j);  // in flight while the codes are formed
    const float z = finish();
    int idx = 0;
#pragma unroll
    for (int e = 0; e < 15; ++e) idx += (s_bnd[e] < z) ? 1 : 0;
    if (dq == 0) s_code[j] = (uint8_t)idx;
    const uint16_t nh = tq_float_to_half_bits(safe);
    if (tid == 0) a.norms[kind][row] = nh;
    __syncthreads();
    if (tid < 4 * bits) ((uint32_t *)(a.codes[kind] + row * (int64_t)(16 * bits)))[tid] = tq_assemble_word(s_code, tid, bits);

    if (residual) {
        __syncthreads();
        if (dq == 0) s_u[j] = s_cen[idx];
        __syncthreads();
        quarter(s_u);  // sum_j c[j] * R_k[j][d], d = this thread's column
        tq_load_column(m, a.qjl_t, dq, j);
        const float rec = finish();
        const float res = s_x[j] - tq_round_through<T>(rec * tq_half_bits_to_float(nh));
        const float rn = block_norm(res);
        const float rsafe = rn > 0.0f ? rn : 1.0f;
        if (dq == 0) s_u[j] = res / rsafe;
        __syncthreads();
        quarter(s_u);
        const float pr = finish();
        const uint32_t mask = __ballot_sync(0xffffffffu, pr >= 0.0f);
        if (dq == 0 && lane == 0) ((uint32_t *)(a.signs + row * 16))[j >> 5] = mask;
        if (tid == 0) a.rnorms[row] = tq_float_to_half_bits(rsafe);
    }
}

// ---------------------------------------------------------------------------------------------
// Query preparation for the tensor-core decode kernel.  A block serves up to four query heads
// of one KV row (a row with G > 4 heads takes two blocks).  The first kv_rows * ceil(G / 4)
// blocks rotate their heads (q @ R_k^T) and write the f16 hi / lo MMA fragments; the next
// kv_rows * ceil(G / 4) blocks project them (q @ S^T), quantise the result to 16-bit fixed
// point and write the s8 hi / lo fragments with the scale and bias that undo it.
// Fragment layout per head: 8 lane variants (part * 4 + t) of 26 words: 16 rotated-query
// words, 8 projected-query words, scale, bias.
template <typename T> __device__ __forceinline__ void tq_qprep_block(const TqQprepArgs &a, int64_t blk) {
    __shared__ float s_q[4][TQ_D], s_o[4][TQ_D];
    __shared__ float s_part[4][4][TQ_D];  // [quarter of d][head][column]
    __shared__ int s_x[4][TQ_D];
    __shared__ float s_scale[4], s_bias[4];
    const int groups = (a.G + 3) >> 2;  // blocks per KV row
    const bool proj = blk >= a.kv_rows * groups;
    const int64_t item = proj ? blk - a.kv_rows * groups : blk;
    const int64_t R = item / groups;
    const int h0 = 4 * (int)(item % groups);                  // first head of this block
    const int G = a.G - h0 < 4 ? a.G - h0 : 4;                // heads of this block
    const int64_t head0 = R * a.G + h0;                       // their first row in q / frag
    const int tid = threadIdx.x, j = tid & (TQ_D - 1), dq = tid >> 7;
    const int warp = tid >> 5, lane = tid & 31;
    float m[32];
    tq_load_column(m, proj ? a.qjl_t : a.rot_k_t, dq, j);  // (codec constants: fetched before the wait)
    tq_grid_dependency_wait();   // the query comes from the preceding kernel of the stream
    tq_launch_dependents();      // the decode kernel may begin its set-up now
    if (dq < G) s_q[dq][j] = tq_to_float<T>(((const T *)a.q)[(head0 + dq) * TQ_D + j]);
    __syncthreads();
    {
        float r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int d = 32 * dq + i;
#pragma unroll
            for (int g = 0; g < 4; ++g) r[g] = fmaf(g < G ? s_q[g][d] : 0.f, m[i], r[g]);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) s_part[dq][g][j] = r[g];
    }
    __syncthreads();
    s_o[dq][j] = (s_part[0][dq][j] + s_part[1][dq][j]) + (s_part[2][dq][j] + s_part[3][dq][j]);  // head dq
    __syncthreads();
    if (!proj) {
        // one thread per word: G heads x 8 variants x 16 words; dims 32t + 4*(k/2) + 2*(k%2) + {0, 1}
        for (int w = tid; w < G * 8 * 16; w += blockDim.x) {
            const int variant = w >> 4, k = w & 15;
            const int hcol = variant >> 3, part = (variant >> 2) & 1, t = variant & 3;
            const int d0 = 32 * t + 4 * (k >> 1) + 2 * (k & 1);
            float x[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float v = s_o[hcol][d0 + i];
                const float hi = __half2float(__float2half_rn(v));
                x[i] = part ? (v - hi) : hi;
            }
            const __half2 hh = __floats2half2_rn(x[0], x[1]);
            a.frag[(head0 + hcol) * TQ_FRAG_ROW_WORDS + (variant & 7) * 26 + k] = *reinterpret_cast<const uint32_t *>(&hh);
        }
        return;
    }
    if (warp < G) {  // warp w quantises the projected query of head w to 16-bit fixed point
        float amax = 0.f;
        for (int i = lane; i < TQ_D; i += 32) amax = fmaxf(amax, fabsf(s_o[warp][i]));
        amax = tq_warp_max(amax);
        const float inv = amax > 0.f ? 32000.0f / amax : 0.f;
        int isum = 0;
        for (int i = lane; i < TQ_D; i += 32) {
            const int x = __float2int_rn(s_o[warp][i] * inv);
            s_x[warp][i] = x;
            isum += x;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
        if (lane == 0) {
            // <qp, sign> = scale * (2 * sum_{bit set} x - sum x); the MMA yields the sum over set bits
            const float scale = amax > 0.f ? amax / 32000.0f : 0.f;
            s_scale[warp] = 2.0f * scale;
            s_bias[warp] = -scale * (float)isum;
        }
    }
    __syncthreads();
    // G heads x 8 variants x 10 words: s8 hi / lo terms behind sign bits (n + 4 rr) + 8j, scale, bias.
    // The decode kernel's operand byte for such a bit is 2^n (the bit is masked in place, not moved),
    // so the term stored here is x / 2^n, rounded: at most three of the sixteen bits are given up.
    for (int w = tid; w < G * 8 * 10; w += blockDim.x) {
        const int variant = w / 10, k = w % 10;
        const int hcol = variant >> 3, part = (variant >> 2) & 1, t = variant & 3;
        uint32_t word = 0;
        if (k < 8) {
            const int n = k >> 1, rr = k & 1;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int x16 = (s_x[hcol][32 * t + (n + 4 * rr) + 8 * jj] + ((1 << n) >> 1)) >> n;
                const int hi8 = (x16 + 128) >> 8;
                const int lo8 = x16 - (hi8 << 8);
                word |= (uint32_t)((part ? lo8 : hi8) & 0xff) << (8 * jj);
            }
        } else {
            word = __float_as_uint(k == 8 ? s_scale[hcol] : s_bias[hcol]);
        }
        a.frag[(head0 + hcol) * TQ_FRAG_ROW_WORDS + (variant & 7) * 26 + 16 + k] = word;
    }
}
