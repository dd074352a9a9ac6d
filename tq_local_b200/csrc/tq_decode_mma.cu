// Decode attention over the packed cache, tensor-core variant for fp16 / bf16 queries.
//
// One CTA owns one (batch, KV head) row and one contiguous token range (a "split")
// and serves all G <= 8 query heads of that KV head, so packed bytes are read once.
// Each warp walks its share of the range 64 tokens at a time:
//
//   S[16 tok x 8 heads]  = Kdeq[16 tok x 128] * Qrot^T         mma.m16n8k16 (f16 in, f32 acc)
//   S2[16 tok x 8 heads] = Sign2[16 tok x 128] * Qproj^T       (sign bit -> {0, 2.0})
//   logit = hs * ( |k| * S + sqrt(pi/2)/D * |r| * (S2 - sum(Qproj)) )
//   online softmax in registers (base-2), P * |v| packed to f16 and transposed with movmatrix
//   O^T[128 x 8 heads]  += Vdeq^T[128 x 16 tok] * P[16 tok x 8 heads]
//
// The A operands are built in registers straight from the packed words.  The
// contraction order of an MMA is free, so each lane is given the dims (logits) or
// the tokens (values) whose codes sit together in the words it loaded:
//   * keys: lane (g, t) holds dims [32t, 32t+32) of tokens g and g+8 of a 16-token tile;
//     two neighbouring codes index a per-lane-replicated shared-memory table of
//     f16x2 centre pairs (conflict-free: entry e of lane l lives in bank l);
//   * QJL signs: bit i and bit i+16 of the lane's sign word become one f16x2 with a
//     shift and a mask (bit -> 0x4000 = 2.0);
//   * values: lane (g, t) holds dims [16g, 16g+16) of tokens 2t, 2t+1, 2t+8, 2t+9; the
//     codes of two tokens are interleaved with two bit-selects so that one table
//     look-up yields the (token a, token b) f16x2 the MMA wants along its K axis.
#include <math.h>

#include "tq_common.cuh"
#include "tq_decode_shared.cuh"
#include "tq_mma_utils.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kTilesPerIter = 4;               // 16-token MMA tiles per warp iteration
constexpr int kTokPerIter = 16 * kTilesPerIter;  // 64

struct MmaArgs {
    const uint8_t *k_codes;
    const uint16_t *k_norms;
    const uint8_t *k_signs;
    const uint16_t *k_rnorms;
    const uint8_t *v_codes;
    const uint16_t *v_norms;
    int64_t cache_sb, cache_sh;
    int Hkv, G, N, n_splits, tok_per_split;
    const float *qrot;
    const float *qproj;
    float *part_m, *part_l, *part_acc;
    const float *centers_k, *centers_v;
};

// Byte offset, in a per-lane-replicated table (entry stride 128 bytes), of the entry
// selected by the WIDTH-bit field at bit `off` of the little-endian word array `w`.
// `off` is a compile-time constant after unrolling, so this folds to a shift and a mask
// (plus a funnel shift when the field straddles two words; w[off/32 + 1] must exist).
template <int WIDTH> __device__ __forceinline__ uint32_t entry_offset_dyn(const uint32_t *w, int off) {
    constexpr uint32_t kMask = ((1u << WIDTH) - 1u) << 7;
    const int wi = off >> 5, s = off & 31;
    uint32_t x;
    if (s + WIDTH <= 32) {
        x = s >= 7 ? (w[wi] >> (s - 7)) : (w[wi] << (7 - s));
    } else {
        x = __funnelshift_r(w[wi], w[wi + 1], s) << 7;
    }
    return x & kMask;
}

// Load the 16*VB-bit value chunk of lane group g from one token row (VB*16 bytes).
template <int VB> __device__ __forceinline__ uint64_t load_v_chunk(const uint8_t *row, int g) {
    if (VB == 4) {
        return __ldg((const unsigned long long *)(row + 8 * g));
    } else if (VB == 2) {
        return __ldg((const unsigned int *)(row + 4 * g));
    } else {  // 3 bits: 6 bytes at byte 6g; read the aligned 8-byte windows that cover it
        const int off = 6 * g, base = off & ~7, sh = (off & 7) * 8;
        const unsigned long long w0 = __ldg((const unsigned long long *)(row + base));
        unsigned long long v = w0 >> sh;
        if (sh > 16) v |= __ldg((const unsigned long long *)(row + base + 8)) << (64 - sh);
        return v & 0xffffffffffffull;
    }
}

template <int KB, int VB, bool QJL>
__global__ void __launch_bounds__(kWarps * 32, 2) tq_decode_mma_kernel(MmaArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kKEntries = 1 << (2 * KB), kVEntries = 1 << (2 * VB);
    uint32_t *lut_k = reinterpret_cast<uint32_t *>(smem);
    uint32_t *lut_v = lut_k + kKEntries * 32;

    const int split = blockIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / a.Hkv, h = bh % a.Hkv;
    const int G = a.G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t q_row0 = ((int64_t)b * a.Hkv + h) * G;

    // ---- per-lane replicated f16x2 centre-pair tables
    for (int i = threadIdx.x; i < kKEntries * 32; i += blockDim.x) {
        const int e = i >> 5;
        lut_k[i] = pack_half2(a.centers_k[e & ((1 << KB) - 1)], a.centers_k[e >> KB]);
    }
    for (int i = threadIdx.x; i < kVEntries * 32; i += blockDim.x) {
        const int e = i >> 5;
        lut_v[i] = pack_half2(a.centers_v[e & ((1 << VB) - 1)], a.centers_v[e >> VB]);
    }

    // ---- B fragments of the rotated / projected query (column g = head g)
    uint32_t bq[8][2], bp[QJL ? 8 : 1][2];
    float qsum = 0.f;
    {
        const bool live = g < G;
        const float *qr = a.qrot + (q_row0 + (live ? g : 0)) * TQ_D + 32 * t;
        const float *qp = a.qproj + (q_row0 + (live ? g : 0)) * TQ_D + 32 * t;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const float4 v = *reinterpret_cast<const float4 *>(qr + 4 * s);
            bq[s][0] = live ? pack_half2(v.x, v.y) : 0u;
            bq[s][1] = live ? pack_half2(v.z, v.w) : 0u;
            if (QJL) {
                const float x0 = qp[2 * s], x1 = qp[2 * s + 16], y0 = qp[2 * s + 1], y1 = qp[2 * s + 17];
                const __half2 h0 = __floats2half2_rn(x0, x1), h1 = __floats2half2_rn(y0, y1);
                bp[s][0] = live ? *reinterpret_cast<const uint32_t *>(&h0) : 0u;
                bp[s][1] = live ? *reinterpret_cast<const uint32_t *>(&h1) : 0u;
                if (live) qsum += __low2float(h0) + __high2float(h0) + __low2float(h1) + __high2float(h1);
            }
        }
    }
    float qs0 = 0.f, qs1 = 0.f;  // sum of the (f16-rounded) projected query for heads 2t, 2t+1
    if (QJL) {
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
        qs0 = __shfl_sync(0xffffffffu, qsum, (2 * t) * 4);
        qs1 = __shfl_sync(0xffffffffu, qsum, (2 * t + 1) * 4);
    }
    __syncthreads();

    const int64_t row0 = (int64_t)b * a.cache_sb + (int64_t)h * a.cache_sh;
    const int t_begin = split * a.tok_per_split;
    const int t_end = min(a.N, t_begin + a.tok_per_split);
    const int last = a.N - 1;
    const float kA = 0.08838834764831845f * 1.4426950408889634f;  // hs * log2(e)
    const float kB = kA * (1.2533141373155003f / (float)TQ_D);     // ... * sqrt(pi/2)/D
    const uint32_t lane_off = lane * 4;
    const uint8_t *lk = reinterpret_cast<const uint8_t *>(lut_k) + lane_off;
    const uint8_t *lv = reinterpret_cast<const uint8_t *>(lut_v) + lane_off;

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int base = t_begin + warp * kTokPerIter; base < t_end; base += kWarps * kTokPerIter) {
        // ------------------------------------------------------------ logits
        float lg[kTilesPerIter][4];
#pragma unroll
        for (int i = 0; i < kTilesPerIter; ++i) {
            const int tokA = base + 16 * i + g, tokB = tokA + 8;
            const int64_t rA = row0 + min(tokA, last), rB = row0 + min(tokB, last);
            uint32_t wa[KB + 1], wb[KB + 1];
            {
                const uint32_t *pa = reinterpret_cast<const uint32_t *>(a.k_codes + rA * (16 * KB)) + KB * t;
                const uint32_t *pb = reinterpret_cast<const uint32_t *>(a.k_codes + rB * (16 * KB)) + KB * t;
#pragma unroll
                for (int w = 0; w < KB; ++w) wa[w] = __ldg(pa + w), wb[w] = __ldg(pb + w);
                wa[KB] = wb[KB] = 0;
            }
            float d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                // pair 2s -> dims 4s, 4s+1; pair 2s+1 -> dims 4s+2, 4s+3 (of the lane's 32)
                constexpr int W = 2 * KB;
                const int o0 = (2 * s) * W, o1 = (2 * s + 1) * W;
                uint32_t a0, a1, a2, a3;
                a0 = *reinterpret_cast<const uint32_t *>(lk + entry_offset_dyn<W>(wa, o0));
                a1 = *reinterpret_cast<const uint32_t *>(lk + entry_offset_dyn<W>(wb, o0));
                a2 = *reinterpret_cast<const uint32_t *>(lk + entry_offset_dyn<W>(wa, o1));
                a3 = *reinterpret_cast<const uint32_t *>(lk + entry_offset_dyn<W>(wb, o1));
                mma_f16(d1, a0, a1, a2, a3, bq[s][0], bq[s][1]);
            }
            const float knA = tq_half_bits_to_float(__ldg(a.k_norms + rA)) * kA;
            const float knB = tq_half_bits_to_float(__ldg(a.k_norms + rB)) * kA;
            if (QJL) {
                const uint32_t sa = __ldg(reinterpret_cast<const uint32_t *>(a.k_signs + rA * 16) + t);
                const uint32_t sb = __ldg(reinterpret_cast<const uint32_t *>(a.k_signs + rB * 16) + t);
                float d2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    constexpr uint32_t kBit = 0x40004000u;  // f16 2.0 in both halves
                    const uint32_t a0 = (sa << (14 - 2 * s)) & kBit;
                    const uint32_t a1 = (sb << (14 - 2 * s)) & kBit;
                    const uint32_t a2 = (s < 7 ? (sa << (13 - 2 * s)) : (sa >> 1)) & kBit;
                    const uint32_t a3 = (s < 7 ? (sb << (13 - 2 * s)) : (sb >> 1)) & kBit;
                    mma_f16(d2, a0, a1, a2, a3, bp[s][0], bp[s][1]);
                }
                const float rnA = tq_half_bits_to_float(__ldg(a.k_rnorms + rA)) * kB;
                const float rnB = tq_half_bits_to_float(__ldg(a.k_rnorms + rB)) * kB;
                lg[i][0] = fmaf(knA, d1[0], rnA * (d2[0] - qs0));
                lg[i][1] = fmaf(knA, d1[1], rnA * (d2[1] - qs1));
                lg[i][2] = fmaf(knB, d1[2], rnB * (d2[2] - qs0));
                lg[i][3] = fmaf(knB, d1[3], rnB * (d2[3] - qs1));
            } else {
                lg[i][0] = knA * d1[0], lg[i][1] = knA * d1[1];
                lg[i][2] = knB * d1[2], lg[i][3] = knB * d1[3];
            }
            if (tokA >= t_end) lg[i][0] = lg[i][1] = -INFINITY;
            if (tokB >= t_end) lg[i][2] = lg[i][3] = -INFINITY;
        }
        // ------------------------------------------------------------ online softmax (base 2)
        float mx0 = lg[0][0], mx1 = lg[0][1];
#pragma unroll
        for (int i = 0; i < kTilesPerIter; ++i) {
            mx0 = fmaxf(mx0, fmaxf(lg[i][0], lg[i][2]));
            mx1 = fmaxf(mx1, fmaxf(lg[i][1], lg[i][3]));
        }
#pragma unroll
        for (int sft = 4; sft <= 16; sft <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sft));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sft));
        }
        const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
        if (__any_sync(0xffffffffu, (nm0 > m0) || (nm1 > m1))) {
            // rescale the running state; exp2(-inf) = 0 covers the first iteration
            const float s0 = (nm0 == -INFINITY) ? 1.f : fast_exp2(m0 - nm0);
            const float s1 = (nm1 == -INFINITY) ? 1.f : fast_exp2(m1 - nm1);
            l0 *= s0, l1 *= s1;
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i][0] *= s0, o[i][1] *= s1, o[i][2] *= s0, o[i][3] *= s1;
            m0 = nm0, m1 = nm1;
        }
        const float sub0 = (m0 == -INFINITY) ? 0.f : m0, sub1 = (m1 == -INFINITY) ? 0.f : m1;
        uint32_t pb[kTilesPerIter][2];
#pragma unroll
        for (int i = 0; i < kTilesPerIter; ++i) {
            const int tokA = base + 16 * i + g, tokB = tokA + 8;
            const float vnA = tq_half_bits_to_float(__ldg(a.v_norms + row0 + min(tokA, last)));
            const float vnB = tq_half_bits_to_float(__ldg(a.v_norms + row0 + min(tokB, last)));
            const float p0 = fast_exp2(lg[i][0] - sub0), p1 = fast_exp2(lg[i][1] - sub1);
            const float p2 = fast_exp2(lg[i][2] - sub0), p3 = fast_exp2(lg[i][3] - sub1);
            l0 += p0 + p2, l1 += p1 + p3;
            // rows = tokens (g / g+8), cols = heads (2t, 2t+1)  ->  transpose to rows = heads
            pb[i][0] = movmatrix_trans(pack_half2(p0 * vnA, p1 * vnA));
            pb[i][1] = movmatrix_trans(pack_half2(p2 * vnB, p3 * vnB));
        }
        // ------------------------------------------------------------ values
#pragma unroll
        for (int i = 0; i < kTilesPerIter; ++i) {
            const int tk = base + 16 * i + 2 * t;
            const uint8_t *vbase = a.v_codes + row0 * (16 * VB);
            const uint64_t wA = load_v_chunk<VB>(vbase + (int64_t)min(tk, last) * (16 * VB), g);
            const uint64_t wB = load_v_chunk<VB>(vbase + (int64_t)min(tk + 1, last) * (16 * VB), g);
            const uint64_t wC = load_v_chunk<VB>(vbase + (int64_t)min(tk + 8, last) * (16 * VB), g);
            const uint64_t wD = load_v_chunk<VB>(vbase + (int64_t)min(tk + 9, last) * (16 * VB), g);
            constexpr uint64_t me = even_field_mask<VB>();
            const uint64_t x01 = (wA & me) | ((wB << VB) & (me << VB));
            const uint64_t y01 = ((wA >> VB) & me) | (wB & (me << VB));
            const uint64_t x23 = (wC & me) | ((wD << VB) & (me << VB));
            const uint64_t y23 = ((wC >> VB) & me) | (wD & (me << VB));
            const uint32_t xw01[3] = {(uint32_t)x01, (uint32_t)(x01 >> 32), 0u};
            const uint32_t yw01[3] = {(uint32_t)y01, (uint32_t)(y01 >> 32), 0u};
            const uint32_t xw23[3] = {(uint32_t)x23, (uint32_t)(x23 >> 32), 0u};
            const uint32_t yw23[3] = {(uint32_t)y23, (uint32_t)(y23 >> 32), 0u};
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                constexpr int W = 2 * VB;
                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(lv + entry_offset_dyn<W>(xw01, mt * W));
                const uint32_t a1 = *reinterpret_cast<const uint32_t *>(lv + entry_offset_dyn<W>(yw01, mt * W));
                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(lv + entry_offset_dyn<W>(xw23, mt * W));
                const uint32_t a3 = *reinterpret_cast<const uint32_t *>(lv + entry_offset_dyn<W>(yw23, mt * W));
                mma_f16(o[mt], a0, a1, a2, a3, pb[i][0], pb[i][1]);
            }
        }
    }

    // ---- merge the warps of the CTA, write the split partial (same format as the exact kernel)
    __syncthreads();  // the tables are dead; reuse shared memory
    float *s_acc = reinterpret_cast<float *>(smem);                    // [kWarps][8][128]
    float *s_m = s_acc + kWarps * TQ_MAX_GROUPS * TQ_D;                // [kWarps][8]
    float *s_l = s_m + kWarps * TQ_MAX_GROUPS;
#pragma unroll
    for (int sft = 4; sft <= 16; sft <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, sft);
        l1 += __shfl_xor_sync(0xffffffffu, l1, sft);
    }
    if (g == 0) {
        s_m[warp * 8 + 2 * t] = m0, s_m[warp * 8 + 2 * t + 1] = m1;
        s_l[warp * 8 + 2 * t] = l0, s_l[warp * 8 + 2 * t + 1] = l1;
    }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        const int d0 = 16 * g + 2 * mt;
        float *r0 = s_acc + (warp * 8 + 2 * t) * TQ_D, *r1 = r0 + TQ_D;
        r0[d0] = o[mt][0], r1[d0] = o[mt][1];
        r0[d0 + 1] = o[mt][2], r1[d0 + 1] = o[mt][3];
    }
    __syncthreads();
    const int d = threadIdx.x;
    for (int hh = 0; hh < G; ++hh) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w * 8 + hh]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float mw = s_m[w * 8 + hh];
            const float sc = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            L += s_l[w * 8 + hh] * sc;
            A += s_acc[(w * 8 + hh) * TQ_D + d] * sc;
        }
        const int64_t prow = (q_row0 + hh) * a.n_splits + split;
        a.part_acc[prow * TQ_D + d] = A;
        // partial maxima are exchanged in natural-log units
        if (d == 0) a.part_m[prow] = M * 0.6931471805599453f, a.part_l[prow] = L;
    }
}

template <int KB, int VB, bool QJL> size_t mma_smem_bytes() {
    const size_t lut = ((size_t)(1 << (2 * KB)) + (size_t)(1 << (2 * VB))) * 128;
    const size_t merge = ((size_t)kWarps * TQ_MAX_GROUPS * TQ_D + 2 * kWarps * TQ_MAX_GROUPS) * sizeof(float);
    return lut > merge ? lut : merge;
}

template <int KB, int VB, bool QJL> cudaError_t launch_mma(const MmaArgs &a, dim3 grid, cudaStream_t stream) {
    const size_t smem = mma_smem_bytes<KB, VB, QJL>();
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(tq_decode_mma_kernel<KB, VB, QJL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    tq_decode_mma_kernel<KB, VB, QJL><<<grid, kWarps * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

int32_t tq_launch_decode_mma(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                             const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                             const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits, void *workspace,
                             void *out, cudaStream_t stream) {
    const int64_t rows = (int64_t)cache->batch * q_heads;
    DecodeWorkspace w = tq_carve_workspace(workspace, rows, n_splits);
    int rc = tq_launch_qprep(ctx, q, q_dtype, rows, w.qrot, w.qproj, stream);
    if (rc) return rc;

    MmaArgs a;
    a.k_codes = cache->k_codes, a.k_norms = cache->k_norms;
    a.k_signs = cache->k_signs, a.k_rnorms = cache->k_rnorms;
    a.v_codes = cache->v_codes, a.v_norms = cache->v_norms;
    a.cache_sb = cache->stride_b, a.cache_sh = cache->stride_h;
    a.Hkv = cache->kv_heads, a.G = q_heads / cache->kv_heads, a.N = seq_len, a.n_splits = n_splits;
    const int per_iter = kWarps * kTokPerIter;
    a.tok_per_split = ((seq_len + n_splits - 1) / n_splits + per_iter - 1) / per_iter * per_iter;
    if (a.tok_per_split < per_iter) a.tok_per_split = per_iter;
    a.qrot = w.qrot, a.qproj = w.qproj;
    a.part_m = w.part_m, a.part_l = w.part_l, a.part_acc = w.part_acc;
    a.centers_k = ctx->centers_k, a.centers_v = ctx->centers_v;
    dim3 grid(n_splits, cache->batch * cache->kv_heads);
    const int mode = ctx->use_qjl * 10 + ctx->bits;
    tq_prof_count(ctx, 3);
    tq_prof_begin(ctx, stream);
    cudaError_t e;
    switch (mode) {
        case 2: e = launch_mma<2, 2, false>(a, grid, stream); break;
        case 3: e = launch_mma<3, 3, false>(a, grid, stream); break;
        case 4: e = launch_mma<4, 4, false>(a, grid, stream); break;
        case 12: e = launch_mma<1, 2, true>(a, grid, stream); break;
        case 13: e = launch_mma<2, 3, true>(a, grid, stream); break;
        case 14: e = launch_mma<3, 4, true>(a, grid, stream); break;
        default: return TQ_ERR_UNSUPPORTED;
    }
    tq_prof_end(ctx, stream);
    TQ_CUDA_CHECK(e);

    CombineArgs c;
    c.part_m = w.part_m, c.part_l = w.part_l, c.part_acc = w.part_acc;
    c.n_splits = n_splits, c.Hq = q_heads, c.G = a.G;
    c.seg_chunk = 0, c.seg_npad = 0;
    c.len_ptr = nullptr, c.len_add = 0, c.capacity = 0, c.plan_rows = 0, c.plan_ctas = 0, c.plan_step = 0;
    c.rot_v = ctx->rot_v;
    c.q = q, c.out = out;
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
