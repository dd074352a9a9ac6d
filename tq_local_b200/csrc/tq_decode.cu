// Decode attention over the packed cache, fp32-exact CUDA-core variant, plus the
// pieces every variant shares: query preparation (rotate / project) and the
// split combine (+ dense tail merge + un-rotation).
//
//   logit[n] = (1/sqrt(D)) * ( |k_n| * <q R_k^T, c_k[idx_n]> + sqrt(pi/2)/D * |r_n| * <q S^T, sign_n> )
//   out      = ( sum_n softmax(logit)_n * |v_n| * c_v[idx_n] ) @ R_v
#include <math.h>

#include "tq_common.cuh"
#include "tq_decode_shared.cuh"

namespace {

constexpr int kExactWarps = 4;

struct ExactArgs {
    const uint8_t *k_codes;
    const uint16_t *k_norms;
    const uint8_t *k_signs;
    const uint16_t *k_rnorms;
    const uint8_t *v_codes;
    const uint16_t *v_norms;
    int64_t cache_sb, cache_sh;
    int Hkv, G, N, n_splits;
    const int *seq_start;  // per batch entry: first token attended (null: 0)
    const float *qrot;   // [B*Hq][128]
    const float *qproj;  // [B*Hq][128]
    float *part_m, *part_l, *part_acc;
    const float *centers_k, *centers_v;
};

template <int BITS> __device__ __forceinline__ uint32_t code_at(const uint32_t *w, int j) {
    const int o = j * BITS, wi = o >> 5, s = o & 31;
    uint32_t v = w[wi] >> s;
    if (s + BITS > 32) v |= w[wi + 1] << (32 - s);
    return v & ((1u << BITS) - 1u);
}

template <int KB, int VB, bool QJL>
__global__ void __launch_bounds__(kExactWarps * 32) tq_decode_exact_kernel(ExactArgs a) {
    __shared__ float s_q[TQ_MAX_GROUPS][TQ_D];
    __shared__ float s_qp[QJL ? TQ_MAX_GROUPS : 1][TQ_D];
    __shared__ float s_ck[16], s_cv[16];
    __shared__ float s_p[kExactWarps][TQ_MAX_GROUPS][32];
    __shared__ float s_m[kExactWarps][TQ_MAX_GROUPS], s_l[kExactWarps][TQ_MAX_GROUPS];
    __shared__ float s_acc[kExactWarps][TQ_MAX_GROUPS][TQ_D];

    const int split = blockIdx.x;
    const int bh = blockIdx.y;  // b * Hkv + h
    const int b = bh / a.Hkv, h = bh % a.Hkv;
    const int G = a.G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t q_row0 = ((int64_t)b * a.Hkv + h) * G;  // first query head of this KV head

    for (int i = threadIdx.x; i < G * TQ_D; i += blockDim.x) {
        s_q[i / TQ_D][i % TQ_D] = a.qrot[q_row0 * TQ_D + i];
        if (QJL) s_qp[i / TQ_D][i % TQ_D] = a.qproj[q_row0 * TQ_D + i];
    }
    if (threadIdx.x < 16) {
        s_ck[threadIdx.x] = a.centers_k[threadIdx.x];
        s_cv[threadIdx.x] = a.centers_v[threadIdx.x];
    }
    __syncthreads();

    const int chunks = (a.N + 31) / 32;
    const int chunks_per_split = (chunks + a.n_splits - 1) / a.n_splits;
    const int c_begin = split * chunks_per_split;
    const int c_end = min(chunks, c_begin + chunks_per_split);
    const int64_t row0 = (int64_t)b * a.cache_sb + (int64_t)h * a.cache_sh;
    const int t_lo = a.seq_start ? a.seq_start[b] : 0;        // tokens before it are masked (left padding)
    const float hs = 0.08838834764831845f;                    // 1/sqrt(128)
    const float qjl_scale = 1.2533141373155003f / (float)TQ_D;  // sqrt(pi/2)/D

    float m[TQ_MAX_GROUPS], l[TQ_MAX_GROUPS], acc[TQ_MAX_GROUPS][4];
#pragma unroll
    for (int g = 0; g < TQ_MAX_GROUPS; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
        acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
    }

    for (int c = c_begin + warp; c < c_end; c += kExactWarps) {
        const int base = c * 32;
        const int tok = base + lane;
        const bool valid = tok < a.N && tok >= t_lo;
        const int64_t row = row0 + (tok < a.N ? tok : base);
        // ---- phase A: one token per lane, all G logits
        uint32_t kw[4 * KB + 1];
        {
            const uint4 *src = (const uint4 *)(a.k_codes + row * (16 * KB));
#pragma unroll
            for (int i = 0; i < KB; ++i) {
                const uint4 t = __ldg(src + i);
                kw[4 * i] = t.x, kw[4 * i + 1] = t.y, kw[4 * i + 2] = t.z, kw[4 * i + 3] = t.w;
            }
            kw[4 * KB] = 0;
        }
        float dot[TQ_MAX_GROUPS];
#pragma unroll
        for (int g = 0; g < TQ_MAX_GROUPS; ++g) dot[g] = 0.f;
#pragma unroll
        for (int j = 0; j < TQ_D; ++j) {
            const float cv = s_ck[code_at<KB>(kw, j)];
#pragma unroll
            for (int g = 0; g < TQ_MAX_GROUPS; ++g)
                if (g < G) dot[g] = fmaf(cv, s_q[g][j], dot[g]);
        }
        const float kn = tq_half_bits_to_float(a.k_norms[row]);
        float logit[TQ_MAX_GROUPS];
#pragma unroll
        for (int g = 0; g < TQ_MAX_GROUPS; ++g) logit[g] = dot[g] * kn * hs;
        if (QJL) {
            const uint4 sw4 = __ldg((const uint4 *)(a.k_signs + row * 16));
            const uint32_t sw[4] = {sw4.x, sw4.y, sw4.z, sw4.w};
            float dq[TQ_MAX_GROUPS];
#pragma unroll
            for (int g = 0; g < TQ_MAX_GROUPS; ++g) dq[g] = 0.f;
#pragma unroll
            for (int j = 0; j < TQ_D; ++j) {
                const float sg = ((sw[j >> 5] >> (j & 31)) & 1u) ? 1.0f : -1.0f;
#pragma unroll
                for (int g = 0; g < TQ_MAX_GROUPS; ++g)
                    if (g < G) dq[g] = fmaf(sg, s_qp[g][j], dq[g]);
            }
            const float rn = tq_half_bits_to_float(a.k_rnorms[row]);
#pragma unroll
            for (int g = 0; g < TQ_MAX_GROUPS; ++g) logit[g] += qjl_scale * rn * dq[g] * hs;
        }
        // ---- phase B: online softmax over the 32 tokens of the chunk
        const float vn = tq_half_bits_to_float(a.v_norms[row]);
        __syncwarp();
#pragma unroll
        for (int g = 0; g < TQ_MAX_GROUPS; ++g) {
            if (g < G) {
                const float lg = valid ? logit[g] : -INFINITY;
                const float nm = fmaxf(m[g], tq_warp_max(lg));
                const float corr = (m[g] == -INFINITY) ? 0.f : expf(m[g] - nm);
                const float p = valid ? expf(lg - nm) : 0.f;
                l[g] = l[g] * corr + tq_warp_sum(p);
                acc[g][0] *= corr, acc[g][1] *= corr, acc[g][2] *= corr, acc[g][3] *= corr;
                m[g] = nm;
                s_p[warp][g][lane] = p * vn;
            }
        }
        __syncwarp();
        // ---- phase C: lane owns value dims 4*lane..4*lane+3
        const int n_here = min(32, a.N - base);
        for (int t = 0; t < n_here; ++t) {
            const uint8_t *vr = a.v_codes + (row0 + base + t) * (16 * VB);
            uint32_t v;
            if (VB == 2) {
                v = vr[lane];
            } else if (VB == 4) {
                v = ((const uint16_t *)vr)[lane];
            } else {  // 3 bits: 12 bits starting at bit 12*lane
                const int by = (3 * lane) >> 1;
                v = ((uint32_t)vr[by] | ((uint32_t)vr[by + 1] << 8)) >> ((lane & 1) * 4);
            }
            float cv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) cv[i] = s_cv[(v >> (VB * i)) & ((1u << VB) - 1u)];
#pragma unroll
            for (int g = 0; g < TQ_MAX_GROUPS; ++g) {
                if (g < G) {
                    const float w = s_p[warp][g][t];
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[g][i] = fmaf(w, cv[i], acc[g][i]);
                }
            }
        }
        __syncwarp();
    }

    // ---- merge the warps of this CTA and write the split partial
#pragma unroll
    for (int g = 0; g < TQ_MAX_GROUPS; ++g) {
        if (g < G) {
            if (lane == 0) s_m[warp][g] = m[g], s_l[warp][g] = l[g];
#pragma unroll
            for (int i = 0; i < 4; ++i) s_acc[warp][g][4 * lane + i] = acc[g][i];
        }
    }
    __syncthreads();
    const int d = threadIdx.x;  // 128 threads == 128 dims
    for (int g = 0; g < G; ++g) {
        float M = -INFINITY;
        for (int w = 0; w < kExactWarps; ++w) M = fmaxf(M, s_m[w][g]);
        float L = 0.f, A = 0.f;
        for (int w = 0; w < kExactWarps; ++w) {
            const float sc = (s_m[w][g] == -INFINITY) ? 0.f : expf(s_m[w][g] - M);
            L += s_l[w][g] * sc;
            A += s_acc[w][g][d] * sc;
        }
        const int64_t prow = (q_row0 + g) * a.n_splits + split;
        a.part_acc[prow * TQ_D + d] = A;
        if (d == 0) a.part_m[prow] = M, a.part_l[prow] = L;
    }
}

}  // namespace

// ---------------------------------------------------------------------------
// Shared pieces: query preparation and split combine
// ---------------------------------------------------------------------------

template <typename T>
__global__ void __launch_bounds__(TQ_D) tq_qprep_kernel(const T *q, const float *rot_k_t, const float *qjl_t,
                                                       float *qrot, float *qproj, int use_qjl) {
    __shared__ float s_q[TQ_D];
    const int64_t row = blockIdx.x;
    const int j = threadIdx.x;
    s_q[j] = tq_to_float<T>(q[row * TQ_D + j]);
    __syncthreads();
    float r = 0.f, p = 0.f;
#pragma unroll 8
    for (int d = 0; d < TQ_D; ++d) r = fmaf(s_q[d], __ldg(rot_k_t + d * TQ_D + j), r);
    qrot[row * TQ_D + j] = r;
    if (use_qjl) {
#pragma unroll 8
        for (int d = 0; d < TQ_D; ++d) p = fmaf(s_q[d], __ldg(qjl_t + d * TQ_D + j), p);
        qproj[row * TQ_D + j] = p;
    }
}

template <typename T>
__global__ void __launch_bounds__(TQ_D) tq_combine_kernel(CombineArgs a) {
    extern __shared__ float s_dyn[];  // tail logits
    __shared__ float s_o[TQ_D];
    __shared__ float s_q[TQ_D];
    __shared__ float s_red[4];
    const int64_t row = blockIdx.x;  // b * Hq + hq
    const int e = threadIdx.x;
    const int warp = e >> 5, lane = e & 31;
    const int b = (int)(row / a.Hq), hq = (int)(row % a.Hq);
    const float hs = 0.08838834764831845f;

    int n_valid = a.n_splits;
    if (a.seg_chunk > 0) {
        const int64_t lo = (row / a.G) * (int64_t)a.seg_npad;
        n_valid = (int)((lo + a.seg_npad - 1) / a.seg_chunk - lo / a.seg_chunk) + 1;
    }
    float M = -INFINITY;
    for (int s = 0; s < n_valid; ++s) M = fmaxf(M, a.part_m[row * a.n_splits + s]);

    // dense tail logits (quantize_decode = False buffer)
    const T *tk = nullptr, *tv = nullptr;
    if (a.n_tail > 0) {
        const int hkv = hq / a.G;
        tk = (const T *)a.tail_k + b * a.tk_sb + hkv * a.tk_sh;
        tv = (const T *)a.tail_v + b * a.tv_sb + hkv * a.tv_sh;
        s_q[e] = tq_to_float<T>(((const T *)a.q)[row * TQ_D + e]);
        __syncthreads();
        float wmax = -INFINITY;
        for (int t = warp; t < a.n_tail; t += 4) {
            const T *kr = tk + (int64_t)t * a.tk_st + 4 * lane;
            float dsum = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) dsum = fmaf(s_q[4 * lane + i], tq_to_float<T>(kr[i]), dsum);
            dsum = tq_warp_sum(dsum) * hs;
            if (lane == 0) s_dyn[t] = dsum;
            wmax = fmaxf(wmax, dsum);
        }
        if (lane == 0) s_red[warp] = wmax;
        __syncthreads();
        M = fmaxf(M, fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3])));
    }

    float L = 0.f, o = 0.f;
    for (int s = 0; s < n_valid; ++s) {
        const float ms = a.part_m[row * a.n_splits + s];
        const float w = (ms == -INFINITY) ? 0.f : expf(ms - M);
        L += a.part_l[row * a.n_splits + s] * w;
        o += a.part_acc[(row * a.n_splits + s) * TQ_D + e] * w;
    }
    s_o[e] = o;
    __syncthreads();
    float out = 0.f;
#pragma unroll 8
    for (int d = 0; d < TQ_D; ++d) out = fmaf(s_o[d], __ldg(a.rot_v + d * TQ_D + e), out);
    for (int t = 0; t < a.n_tail; ++t) {
        const float p = expf(s_dyn[t] - M);
        L += p;
        out = fmaf(p, tq_to_float<T>(tv[(int64_t)t * a.tv_st + e]), out);
    }
    ((T *)a.out)[row * TQ_D + e] = tq_from_float<T>(out / fmaxf(L, 1e-8f));
}

// Query preparation for the tensor-core kernel (see tq_qprep_block): kv_rows * ceil(G / 4) blocks
// rotate, another kv_rows blocks project when the keys carry a QJL sketch.  Launched as a
// programmatic dependent of whatever precedes it in the stream: a block fetches its matrix
// column, waits for that kernel, then lets the decode kernel begin its own set-up.
template <typename T>
__global__ void __launch_bounds__(4 * TQ_D, 2) tq_qprep_frag_kernel(TqQprepArgs a) {
    tq_qprep_block<T>(a, blockIdx.x);
}

// The whole latency-bound front of a decode step in one launch: query preparation blocks
// first, then one block per new key and value vector to append (tq_pack_small_block).
template <typename T, bool QJL>
__global__ void __launch_bounds__(4 * TQ_D, 2) tq_step_prologue_kernel(TqQprepArgs qa, TqPackArgs pa, int n_qprep) {
    if ((int)blockIdx.x < n_qprep)
        tq_qprep_block<T>(qa, blockIdx.x);
    else
        tq_pack_small_block<T, QJL>(pa, (int64_t)blockIdx.x - n_qprep);
}

// Split combine for up to four heads of one (batch, KV head) row per block (no dense tail):
// the un-rotation matrix is read once for the G heads.
// Publishing rows to the peers and waiting for theirs (system scope, PTX memory model):
// a block's threads store their rows with plain stores, the block barrier orders those stores
// before thread 0, which adds the block's row count to the flag word with a RELEASE reduction at
// system scope (cumulative over what the barrier ordered before it); the waiting side polls the
// word with ACQUIRE loads at system scope, and its own block barrier orders the data reads of
// the other threads behind the observation.  No separate fence on either side: on a B200 pair
// the two full system fences this replaces cost 3.3 us of a 92 us step.
__device__ __forceinline__ void tq_release_add_sys(unsigned *word, unsigned value) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;\n" ::"l"(word), "r"(value) : "memory");
}
__device__ __forceinline__ unsigned tq_acquire_load_sys(const unsigned *word) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(word) : "memory");
    return v;
}

template <typename T>
__global__ void __launch_bounds__(4 * TQ_D) tq_combine_group_kernel(CombineArgs a) {
    __shared__ __align__(16) float s_o[4][TQ_D];
    __shared__ float s_part[4][4][TQ_D];  // [quarter of d][head][column]
    __shared__ float s_L[4], s_M[4];
    const int groups = (a.G + 3) >> 2;           // a block serves up to four heads of a KV row
    const int64_t R = blockIdx.x / groups;
    const int h0 = 4 * (blockIdx.x % groups);
    const int n_heads = a.G - h0 < 4 ? a.G - h0 : 4;
    const int tid = threadIdx.x, e = tid & (TQ_D - 1), dq = tid >> 7;
    float rv[32];  // this thread's un-rotation elements, fetched while the decode kernel drains
    tq_load_column(rv, a.rot_v, dq, e);
    tq_grid_dependency_wait();
    int n_valid = a.n_splits;
    int seg_chunk = a.seg_chunk, seg_npad = a.seg_npad;
    if (a.len_ptr) {
        const TqPlan plan = tq_make_plan(min(*a.len_ptr + a.len_add, a.capacity), a.plan_rows, a.plan_ctas, a.n_splits,
                                         a.plan_step);
        seg_chunk = plan.chunk, seg_npad = plan.n_pad;
    }
    if (seg_chunk > 0) {
        const int64_t lo = R * (int64_t)seg_npad;
        n_valid = (int)((lo + seg_npad - 1) / seg_chunk - lo / seg_chunk) + 1;
    }
    {   // thread (e, dq) merges the splits of head dq
        const int g = dq;
        float o = 0.f, L = 0.f, Mx = -INFINITY;
        if (g < n_heads) {
            const int64_t row = R * a.G + h0 + g;
            if (n_valid <= 4) {  // the usual case: everything is requested in one batch of loads
                float pm[4], pl[4], pa[4];
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const bool on = s < n_valid;
                    pm[s] = on ? a.part_m[row * a.n_splits + s] : -INFINITY;
                    pl[s] = on ? a.part_l[row * a.n_splits + s] : 0.f;
                    pa[s] = on ? a.part_acc[(row * a.n_splits + s) * TQ_D + e] : 0.f;
                }
                const float M = fmaxf(fmaxf(pm[0], pm[1]), fmaxf(pm[2], pm[3]));
                Mx = M;
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const float w = (pm[s] == -INFINITY) ? 0.f : expf(pm[s] - M);
                    L += pl[s] * w;
                    o += pa[s] * w;
                }
            } else {
                float M = -INFINITY;
                for (int s = 0; s < n_valid; ++s) M = fmaxf(M, a.part_m[row * a.n_splits + s]);
                Mx = M;
                for (int s = 0; s < n_valid; ++s) {
                    const float ms = a.part_m[row * a.n_splits + s];
                    const float w = (ms == -INFINITY) ? 0.f : expf(ms - M);
                    L += a.part_l[row * a.n_splits + s] * w;
                    o += a.part_acc[(row * a.n_splits + s) * TQ_D + e] * w;
                }
            }
        }
        s_o[g][e] = o;
        if (e == 0) s_L[g] = L, s_M[g] = Mx;
        if (a.parts > 0 && g < n_heads) {
            // Sequence split: this rank holds only a part of the row's tokens.  Its merged partial goes,
            // unfinished, into slot `part` of every rank's exchange buffer [row][parts] (laid out like a
            // decode workspace: all maxima, then all sums, then the accumulators); whoever has waited for
            // all parts finishes the rows with this same kernel (n_splits = parts).
            const int64_t row0 = R * a.G + h0;
            const int64_t bi = row0 / a.Hq, hl = row0 % a.Hq;
            const int64_t grow = bi * a.gather_heads_total + (int64_t)a.head_group * a.Hq + hl + g;  // row of the whole model
            const unsigned seq = a.gather_seq;
            for (int p = 0; p < a.gather_world; ++p) {
                float *base = reinterpret_cast<float *>(static_cast<char *>(a.gather_out[p]) + ((seq & 1u) ? a.gather_out_stride : 0));
                const int64_t n_rows = a.exch_rows;
                float *xm = base, *xl = base + n_rows * a.parts, *xacc = base + 2 * n_rows * a.parts;
                const int64_t slot = grow * a.parts + a.part;
                xacc[slot * TQ_D + e] = o;
                if (e == 0) xm[slot] = Mx, xl[slot] = L;
            }
        }
    }
    if (a.parts > 0) {  // report the rows (see the gather below) and leave: nothing is finished here
        __syncthreads();
        // (lane p of the first warp reports to rank p: one instruction, so one wait for the stores)
        if (tid < a.gather_world) tq_release_add_sys(a.gather_flags[tid] + a.gather_rank, (unsigned)n_heads);
        return;
    }
    __syncthreads();
    {   // thread (e, dq) un-rotates rows d in [32 dq, 32 dq + 32) for all heads
        float out[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int d = 32 * dq + i;
#pragma unroll
            for (int g = 0; g < 4; ++g) out[g] = fmaf(s_o[g][d], rv[i], out[g]);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) s_part[dq][g][e] = out[g];
    }
    __syncthreads();
    if (dq < n_heads) {
        const int g = dq;
        const float v = (s_part[0][g][e] + s_part[1][g][e]) + (s_part[2][g][e] + s_part[3][g][e]);
        const T res = tq_from_float<T>(v / fmaxf(s_L[g], 1e-8f));
        const int64_t row = R * a.G + h0 + g;  // = batch index * local query heads + local head
        if (a.gather_world > 0) {
            reinterpret_cast<T *>(&s_o[0][0])[g * TQ_D + e] = res;  // staged: the peers get 16-byte stores below
        } else if (a.out_f32) {
            a.out_f32[row * TQ_D + e] = v / fmaxf(s_L[g], 1e-8f);
        } else {
            ((T *)a.out)[row * TQ_D + e] = res;
        }
    }
    if (a.gather_world > 0) {
        static_assert(sizeof(T) == 2 || sizeof(T) == 4, "");
        __syncthreads();
        // The block's heads are consecutive rows of one batch entry: one contiguous piece of every
        // rank's gathered buffer.  Thread (p, i) stores 16-byte piece i of it into rank p's buffer.
        const unsigned seq = a.gather_seq_ptr ? *a.gather_seq_ptr + 1u : a.gather_seq;
        const long long buf = (seq & 1u) ? a.gather_out_stride : 0;
        const int64_t row0 = R * a.G + h0;  // = batch index * local query heads + local head
        const int64_t bi = row0 / a.Hq, hl = row0 % a.Hq;
        const int64_t dst0 = (bi * a.gather_heads_total + (int64_t)a.gather_rank * a.Hq + hl) * TQ_D;  // elements
        const int pieces = n_heads * TQ_D * (int)sizeof(T) / 16;
        for (int w = tid; w < a.gather_world * pieces; w += blockDim.x) {
            const int p = w / pieces, i = w % pieces;
            uint4 *dst = reinterpret_cast<uint4 *>(static_cast<char *>(a.gather_out[p]) + buf + dst0 * sizeof(T));
            dst[i] = reinterpret_cast<const uint4 *>(&s_o[0][0])[i];
        }
        // Every block reports its own rows: after a system-scope fence (cumulative over the block's
        // stores, which the barrier ordered before it) it adds its row count to this rank's word in
        // every peer's flag block.  A peer has all of this rank's rows of step s once that word has
        // reached s * (rows per step); no block waits for another, no counter round trip.
        __syncthreads();
        // (lane p of the first warp reports to rank p: the release reductions of all peers are one
        // instruction and wait for the block's stores once; one after the other they cost one such
        // wait per peer)
        if (tid < a.gather_world) tq_release_add_sys(a.gather_flags[tid] + a.gather_rank, (unsigned)n_heads);
    }
}

__device__ __forceinline__ unsigned long long tq_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}

// Waits until every rank's word of this rank's flag block has reached step * rows_per_step (the
// peers' combine kernels add the rows they have stored), for at most `limit_ns` nanoseconds of the
// GPU's wall clock; a wait that runs out sets the status word to 5 and the kernel returns without
// copying.  Otherwise, optionally, every block copies its slice of this rank's gathered buffer of
// the step to `dst`.  A step numbered on the device (seq_ptr: the number of the last completed
// step) is number *seq_ptr + 1; the last block to finish stores it back, after every block has
// read it.
__global__ void tq_gather_wait_kernel(const unsigned *flags, int world, unsigned seq_arg, unsigned *seq_ptr,
                                      unsigned rows_per_step, unsigned *counter, int *error_flag,
                                      unsigned long long limit_ns, const uint4 *src0, long long stride, uint4 *dst,
                                      size_t n16, size_t row_len16, size_t row_stride16, size_t src_off16) {
    // (the combine kernel of a device-numbered step reads the same word: it must be complete
    // before this kernel may advance it; a host-numbered step may start polling early)
    if (seq_ptr) tq_grid_dependency_wait();
    tq_launch_dependents();  // the next kernel of the stream may be placed while this one polls
    const unsigned seq = seq_ptr ? *seq_ptr + 1u : seq_arg;
    const unsigned target = seq * rows_per_step;
    __shared__ int s_failed;
    if (threadIdx.x == 0) s_failed = 0;
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const unsigned long long t0 = tq_global_ns();
        unsigned polls = 0;
        while ((int)(tq_acquire_load_sys(flags + threadIdx.x) - target) < 0) {  // (the words only grow; a peer may already be a step ahead)
            if ((++polls & 63u) == 0 && tq_global_ns() - t0 > limit_ns) {
                atomicExch(error_flag, 5);
                s_failed = 1;
                break;
            }
        }
    }
    __syncthreads();
    if (dst && !s_failed) {
        // dst is dense; piece i of it is piece (i % row_len16) of source row (i / row_len16), rows being
        // row_stride16 apart and starting src_off16 into the buffer (a whole-buffer copy is one row)
        const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(src0) + ((seq & 1u) ? stride : 0));
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
            dst[i] = src[(i / row_len16) * row_stride16 + src_off16 + i % row_len16];
    }
    if (seq_ptr && !s_failed) {
        __syncthreads();
        if (threadIdx.x == 0 && atomicAdd(counter, 1u) == gridDim.x - 1) {
            *counter = 0;
            *seq_ptr = seq;
        }
    }
    // (a host-numbered wait began before the combine kernel was done: it ends only after it)
    if (!seq_ptr) tq_grid_dependency_wait();
}

// The decode kernels run with the largest shared-memory carve-out.  The small kernels around
// them ask for the same carve-out, so the SMs are not reconfigured (and drained) between the
// launches of one decode step.
template <typename K> static void prefer_max_shared(K kernel) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}
static void configure_small_kernels() {
    static bool done = false;
    if (done) return;
    done = true;
    prefer_max_shared(tq_qprep_kernel<float>);
    prefer_max_shared(tq_qprep_kernel<__half>);
    prefer_max_shared(tq_qprep_kernel<__nv_bfloat16>);
    prefer_max_shared(tq_combine_kernel<float>);
    prefer_max_shared(tq_combine_kernel<__half>);
    prefer_max_shared(tq_combine_kernel<__nv_bfloat16>);
    prefer_max_shared(tq_qprep_frag_kernel<float>);
    prefer_max_shared(tq_qprep_frag_kernel<__half>);
    prefer_max_shared(tq_qprep_frag_kernel<__nv_bfloat16>);
    prefer_max_shared(tq_combine_group_kernel<float>);
    prefer_max_shared(tq_combine_group_kernel<__half>);
    prefer_max_shared(tq_combine_group_kernel<__nv_bfloat16>);
    prefer_max_shared(tq_step_prologue_kernel<float, true>);
    prefer_max_shared(tq_step_prologue_kernel<float, false>);
    prefer_max_shared(tq_step_prologue_kernel<__half, true>);
    prefer_max_shared(tq_step_prologue_kernel<__half, false>);
    prefer_max_shared(tq_step_prologue_kernel<__nv_bfloat16, true>);
    prefer_max_shared(tq_step_prologue_kernel<__nv_bfloat16, false>);
}

int32_t tq_launch_qprep(tq_ctx *ctx, const void *q, int32_t q_dtype, int64_t rows, float *qrot, float *qproj,
                        cudaStream_t stream) {
    configure_small_kernels();
    if (q_dtype == TQ_DTYPE_F32)
        tq_qprep_kernel<float><<<(unsigned)rows, TQ_D, 0, stream>>>((const float *)q, ctx->rot_k_t, ctx->qjl_t, qrot,
                                                                    qproj, ctx->use_qjl);
    else if (q_dtype == TQ_DTYPE_F16)
        tq_qprep_kernel<__half><<<(unsigned)rows, TQ_D, 0, stream>>>((const __half *)q, ctx->rot_k_t, ctx->qjl_t,
                                                                     qrot, qproj, ctx->use_qjl);
    else
        tq_qprep_kernel<__nv_bfloat16><<<(unsigned)rows, TQ_D, 0, stream>>>((const __nv_bfloat16 *)q, ctx->rot_k_t,
                                                                            ctx->qjl_t, qrot, qproj, ctx->use_qjl);
    TQ_CUDA_CHECK(cudaGetLastError());
    return TQ_OK;
}

template <typename T>
static cudaError_t launch_prologue(tq_ctx *ctx, const TqQprepArgs &qa, const TqPackArgs *append, cudaStream_t stream) {
    const int n_qprep = (int)qa.kv_rows * ((qa.G + 3) / 4) * (qa.use_qjl ? 2 : 1);
    if (!append) return tq_launch_kernel(tq_qprep_frag_kernel<T>, dim3(n_qprep), dim3(4 * TQ_D), 0, stream, true, qa);
    const int n_pack = append->n_kinds * append->B * append->H * append->S;
    if (ctx->use_qjl)
        return tq_launch_kernel(tq_step_prologue_kernel<T, true>, dim3(n_qprep + n_pack), dim3(4 * TQ_D), 0, stream,
                                true, qa, *append, n_qprep);
    return tq_launch_kernel(tq_step_prologue_kernel<T, false>, dim3(n_qprep + n_pack), dim3(4 * TQ_D), 0, stream, true,
                            qa, *append, n_qprep);
}

int32_t tq_launch_qprep_frag(tq_ctx *ctx, const void *q, int32_t q_dtype, int64_t kv_rows, int G, uint32_t *frag,
                             const TqPackArgs *append, cudaStream_t stream) {
    configure_small_kernels();
    if (G > 8) return TQ_ERR_UNSUPPORTED;
    TqQprepArgs qa;
    qa.q = q, qa.rot_k_t = ctx->rot_k_t, qa.qjl_t = ctx->qjl_t, qa.frag = frag;
    qa.G = G, qa.use_qjl = ctx->use_qjl, qa.kv_rows = kv_rows;
    cudaError_t e;
    if (q_dtype == TQ_DTYPE_F32) e = launch_prologue<float>(ctx, qa, append, stream);
    else if (q_dtype == TQ_DTYPE_F16) e = launch_prologue<__half>(ctx, qa, append, stream);
    else e = launch_prologue<__nv_bfloat16>(ctx, qa, append, stream);
    TQ_CUDA_CHECK(e);
    return TQ_OK;
}

int32_t tq_launch_combine(const CombineArgs &a, int32_t q_dtype, int64_t rows, cudaStream_t stream, bool programmatic) {
    if (a.n_tail == 0 && a.G <= 8) {  // grouped variant: one block per four heads of a KV row
        const dim3 grid((unsigned)(rows / a.G) * ((a.G + 3) / 4)), block(4 * TQ_D);
        cudaError_t e;
        if (q_dtype == TQ_DTYPE_F32) e = tq_launch_kernel(tq_combine_group_kernel<float>, grid, block, 0, stream, programmatic, a);
        else if (q_dtype == TQ_DTYPE_F16) e = tq_launch_kernel(tq_combine_group_kernel<__half>, grid, block, 0, stream, programmatic, a);
        else e = tq_launch_kernel(tq_combine_group_kernel<__nv_bfloat16>, grid, block, 0, stream, programmatic, a);
        TQ_CUDA_CHECK(e);
        return TQ_OK;
    }
    const size_t dyn = (size_t)a.n_tail * sizeof(float);
    if (dyn > 40 * 1024) return TQ_ERR_UNSUPPORTED;
    if (q_dtype == TQ_DTYPE_F32)
        tq_combine_kernel<float><<<(unsigned)rows, TQ_D, dyn, stream>>>(a);
    else if (q_dtype == TQ_DTYPE_F16)
        tq_combine_kernel<__half><<<(unsigned)rows, TQ_D, dyn, stream>>>(a);
    else
        tq_combine_kernel<__nv_bfloat16><<<(unsigned)rows, TQ_D, dyn, stream>>>(a);
    TQ_CUDA_CHECK(cudaGetLastError());
    return TQ_OK;
}

int32_t tq_launch_gather_wait(const tq_gather_desc *g, int *error_flag, int limit_ms, int32_t batch, size_t elem_bytes,
                              void *out_final, cudaStream_t stream, int64_t rows_per_step) {
    if (rows_per_step <= 0) rows_per_step = (int64_t)batch * (g->q_heads_total / g->world);
    // out_final: the whole gathered output [batch, q_heads_total, 128], or (out_local_only) this
    // rank's heads of it [batch, q_heads_total / world, 128]
    size_t n16 = 0, row_len16 = 1, row_stride16 = 0, src_off16 = 0;
    if (out_final) {
        const size_t head16 = TQ_D * elem_bytes / 16;
        const size_t heads_local = (size_t)g->q_heads_total / g->world;
        if (g->out_local_only) {
            row_len16 = heads_local * head16, row_stride16 = (size_t)g->q_heads_total * head16;
            src_off16 = (size_t)g->rank * heads_local * head16, n16 = (size_t)batch * row_len16;
        } else {
            n16 = (size_t)batch * g->q_heads_total * head16, row_len16 = n16;
        }
    }
    const int blocks = out_final ? (int)((n16 + 255) / 256 < 64 ? (n16 + 255) / 256 : 64) : 1;
    // Launched as a programmatic dependent: with a host-side step number it begins polling while the
    // combine kernel that raises this rank's own flag is still finishing (harmless: the flags carry
    // the step number); what follows it in the stream still starts only after it has seen every
    // rank's flag, this rank's included.
    cudaError_t e = tq_launch_kernel(tq_gather_wait_kernel, dim3(blocks < 1 ? 1 : blocks), dim3(256), 0, stream, true,
                                     (const unsigned *)g->flags[g->rank], (int)g->world, (unsigned)g->seq,
                                     (unsigned *)g->seq_dev, (unsigned)rows_per_step,
                                     (unsigned *)g->counter, error_flag,
                                     (unsigned long long)(limit_ms < 1 ? 1 : limit_ms) * 1000000ull,
                                     reinterpret_cast<const uint4 *>(g->out[g->rank]), (long long)g->out_stride,
                                     reinterpret_cast<uint4 *>(out_final), n16, row_len16, row_stride16, src_off16);
    TQ_CUDA_CHECK(e);
    return TQ_OK;
}

DecodeWorkspace tq_carve_workspace(void *workspace, int64_t rows, int n_splits) {
    DecodeWorkspace w;
    float *p = (float *)workspace;
    w.qrot = p;
    p += rows * TQ_D;
    w.qproj = p;
    p += rows * TQ_D;
    p += rows * 8;
    w.part_m = p;
    p += rows * n_splits;
    w.part_l = p;
    p += rows * n_splits;
    w.part_acc = p;
    return w;
}

int32_t tq_launch_decode_exact(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                               const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                               const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits, void *workspace,
                               void *out, cudaStream_t stream) {
    const int64_t rows = (int64_t)cache->batch * q_heads;
    DecodeWorkspace w = tq_carve_workspace(workspace, rows, n_splits);
    int rc = tq_launch_qprep(ctx, q, q_dtype, rows, w.qrot, w.qproj, stream);
    if (rc) return rc;

    ExactArgs a;
    a.k_codes = cache->k_codes, a.k_norms = cache->k_norms;
    a.k_signs = cache->k_signs, a.k_rnorms = cache->k_rnorms;
    a.v_codes = cache->v_codes, a.v_norms = cache->v_norms;
    a.cache_sb = cache->stride_b, a.cache_sh = cache->stride_h;
    a.Hkv = cache->kv_heads, a.G = q_heads / cache->kv_heads, a.N = seq_len, a.n_splits = n_splits;
    a.seq_start = cache->seq_start;
    a.qrot = w.qrot, a.qproj = w.qproj;
    a.part_m = w.part_m, a.part_l = w.part_l, a.part_acc = w.part_acc;
    a.centers_k = ctx->centers_k, a.centers_v = ctx->centers_v;
    dim3 grid(n_splits, cache->batch * cache->kv_heads);
    const int threads = kExactWarps * 32;
    const int mode = ctx->use_qjl * 10 + ctx->bits;
    tq_prof_count(ctx, 3);
    tq_prof_begin(ctx, stream);
    switch (mode) {
        case 2: tq_decode_exact_kernel<2, 2, false><<<grid, threads, 0, stream>>>(a); break;
        case 3: tq_decode_exact_kernel<3, 3, false><<<grid, threads, 0, stream>>>(a); break;
        case 4: tq_decode_exact_kernel<4, 4, false><<<grid, threads, 0, stream>>>(a); break;
        case 12: tq_decode_exact_kernel<1, 2, true><<<grid, threads, 0, stream>>>(a); break;
        case 13: tq_decode_exact_kernel<2, 3, true><<<grid, threads, 0, stream>>>(a); break;
        case 14: tq_decode_exact_kernel<3, 4, true><<<grid, threads, 0, stream>>>(a); break;
        default: return TQ_ERR_UNSUPPORTED;
    }
    tq_prof_end(ctx, stream);
    TQ_CUDA_CHECK(cudaGetLastError());

    CombineArgs c;
    c.part_m = w.part_m, c.part_l = w.part_l, c.part_acc = w.part_acc;
    c.n_splits = n_splits, c.Hq = q_heads, c.G = a.G;
    c.seg_chunk = 0, c.seg_npad = 0;
    c.len_ptr = nullptr, c.len_add = 0, c.capacity = 0, c.plan_rows = 0, c.plan_ctas = 0, c.plan_step = 0;
    c.gather_world = 0, c.parts = 0, c.part = 0, c.head_group = 0, c.exch_rows = 0;
    c.rot_v = ctx->rot_v;
    c.q = q, c.out = out, c.out_f32 = nullptr;
    c.n_tail = n_tail;
    c.tail_k = n_tail ? tail_k->data : nullptr;
    c.tail_v = n_tail ? tail_v->data : nullptr;
    if (n_tail) {
        if (tail_k->dtype != q_dtype || tail_v->dtype != q_dtype) return TQ_ERR_ARG;
        c.tk_sb = tail_k->stride_b, c.tk_sh = tail_k->stride_h, c.tk_st = tail_k->stride_t;
        c.tv_sb = tail_v->stride_b, c.tv_sh = tail_v->stride_h, c.tv_st = tail_v->stride_t;
    } else {
        c.tk_sb = c.tk_sh = c.tk_st = c.tv_sb = c.tv_sh = c.tv_st = 0;
    }
    return tq_launch_combine(c, q_dtype, rows, stream);
}
