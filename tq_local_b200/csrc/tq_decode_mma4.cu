// Decode attention over the packed cache: tensor-core kernel for fp16 / bf16 queries
// with at most 4 query heads per KV head (Llama-3.1-8B: 32 / 8).
//
// One CTA owns one (batch, KV head) row and one contiguous token range and serves all
// G <= 4 query heads, so packed bytes are read once.  The 8 columns of every MMA are
// used as (head, part) pairs, which gives each lane of a quad its own head:
//
//   logits   S  [16 tok x (4 heads x {hi, lo})] = Kdeq[16 x 128] * {Qrot_hi, Qrot_lo}   f16 m16n8k16
//            the rotated query is split in two f16 terms, so its rounding does not show;
//   QJL      S2 [16 tok x (4 heads x {hi, lo})] = -Bit[16 x 128] * {Qp_hi, Qp_lo}       s8 m16n8k32
//            sign bits become 0 / -1 bytes four at a time (byte permute with sign
//            replication); the projected query is 16-bit fixed point in two s8 terms;
//   values   O^T[128 x (4 heads x {P, 0})] += Vdeq^T[128 x 16 tok] * P                   f16 m16n8k16
//
// A operands are built in registers from the packed words.  The contraction order and
// the row order of an MMA are free, so every lane gets codes that sit together in memory:
//   keys    lane (g, t): dims [32t, 32t+32) of tokens 2g, 2g+1 of a 16-token tile; two
//           neighbouring codes index a per-lane-replicated shared-memory table of f16x2
//           centre pairs (entry e of lane l lives in bank l: no bank conflicts);
//   values  lane (g, t): dims [16g, 16g+16) of tokens 4t .. 4t+3; the codes of two tokens
//           are interleaved with bit-selects so one look-up yields the (token a, token b)
//           f16x2 that the MMA wants along its K axis.
// Softmax is online, base 2, in registers; P*|v| goes to f16 and is transposed with
// movmatrix.  Per-CTA partials (max, sum, acc) go to the workspace; tq_combine_kernel
// merges splits, un-rotates and casts.
#include <math.h>

#include "tq_common.cuh"
#include "tq_decode_shared.cuh"
#include "tq_mma_utils.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kTiles = 4;               // 16-token MMA tiles per warp iteration
constexpr int kTokIter = 16 * kTiles;   // 64
constexpr int kSlotWords = 64;          // table slot: 32 key words then 32 value words (256 B)

struct Mma4Args {
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

// Byte offset of this lane's copy of the table slot selected by the WIDTH-bit field at bit
// `off` of the little-endian word array `w`: slot * 256 + lane_bits, where lane_bits < 256
// is the lane's offset inside a slot.  `off` is a compile-time constant after unrolling.
// A byte-aligned 8-bit field takes one byte permute (field -> byte 1, lane_bits -> byte 0);
// any other field takes a shift and one three-input logic op (or a funnel shift first when
// it straddles two words; w[off/32+1] must exist).
template <int WIDTH> __device__ __forceinline__ uint32_t slot_offset(const uint32_t *w, int off, uint32_t lane_bits) {
    const int wi = off >> 5, s = off & 31;
    if (WIDTH == 8 && (s & 7) == 0) return prmt(w[wi], lane_bits, 0x5504u | ((uint32_t)(s >> 3) << 4));
    constexpr uint32_t kMask = ((1u << WIDTH) - 1u) << 8;
    uint32_t x;
    if (s + WIDTH <= 32) {
        x = s >= 8 ? (w[wi] >> (s - 8)) : (w[wi] << (8 - s));
    } else {
        x = __funnelshift_r(w[wi], w[wi + 1], s) << 8;
    }
    return (x & kMask) | lane_bits;
}

// The 16*VB-bit value chunk of lane group g of one token row (row = VB*16 bytes).
template <int VB> __device__ __forceinline__ uint64_t load_v_chunk(const uint8_t *row, int g) {
    if (VB == 4) {
        return __ldg((const unsigned long long *)(row + 8 * g));
    } else if (VB == 2) {
        return __ldg((const unsigned int *)(row + 4 * g));
    } else {  // 3 bits: 6 bytes at byte 6g; read the aligned 8-byte windows that cover it
        const int off = 6 * g, base = off & ~7, sh = (off & 7) * 8;
        unsigned long long v = __ldg((const unsigned long long *)(row + base)) >> sh;
        if (sh > 16) v |= __ldg((const unsigned long long *)(row + base + 8)) << (64 - sh);
        return v & 0xffffffffffffull;
    }
}

__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&u));
}

template <int KB, int VB, bool QJL>
__global__ void __launch_bounds__(kWarps * 32, 3) tq_decode_mma4_kernel(Mma4Args a) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kKEntries = 1 << (2 * KB), kVEntries = 1 << (2 * VB);
    constexpr int kEntries = kKEntries > kVEntries ? kKEntries : kVEntries;
    uint32_t *table = reinterpret_cast<uint32_t *>(smem);

    const int split = blockIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / a.Hkv, h = bh % a.Hkv;
    const int G = a.G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t q_row0 = ((int64_t)b * a.Hkv + h) * G;

    // ---- per-lane replicated f16x2 centre-pair tables (keys in the low half of each slot);
    // a warp fills one slot at a time, lane l writing words l and 32+l (no bank conflicts)
    for (int e = warp; e < kEntries; e += kWarps) {
        uint32_t *slot = table + e * kSlotWords;
        if (e < kKEntries) slot[lane] = pack_half2(a.centers_k[e & ((1 << KB) - 1)], a.centers_k[e >> KB]);
        if (e < kVEntries) slot[32 + lane] = pack_half2(a.centers_v[e & ((1 << VB) - 1)], a.centers_v[e >> VB]);
    }

    // ---- B fragments: column g = (head g/2, part g%2)
    const int hcol = g >> 1, part = g & 1;
    const bool live = hcol < G;
    uint32_t bq[8][2];
    uint32_t bp[QJL ? 4 : 1][2];
    float sign_scale = 0.f, sign_bias = 0.f;  // for the head this lane owns in the softmax (head t)
    {
        const float *qr = a.qrot + (q_row0 + (live ? hcol : 0)) * TQ_D + 32 * t;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const float4 v = *reinterpret_cast<const float4 *>(qr + 4 * s);
            float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float hi = __half2float(__float2half_rn(x[i]));
                x[i] = part ? (x[i] - hi) : hi;
            }
            bq[s][0] = live ? pack_half2(x[0], x[1]) : 0u;
            bq[s][1] = live ? pack_half2(x[2], x[3]) : 0u;
        }
        if (QJL) {
            const float *qp = a.qproj + (q_row0 + (live ? hcol : 0)) * TQ_D + 32 * t;
            float amax = 0.f;
#pragma unroll
            for (int d = 0; d < 32; ++d) amax = fmaxf(amax, fabsf(qp[d]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            const float inv = amax > 0.f ? 32000.0f / amax : 0.f;
            int isum = 0;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    uint32_t word = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int d = (7 - 2 * n - r) + 8 * j;  // bit of the sign word behind k-slot j
                        const int x16 = __float2int_rn(qp[d] * inv);
                        const int hi8 = (x16 + 128) >> 8;
                        const int lo8 = x16 - (hi8 << 8);
                        isum += x16;
                        word |= (uint32_t)((part ? lo8 : hi8) & 0xff) << (8 * j);
                    }
                    bp[n][r] = live ? word : 0u;
                }
            }
            isum += __shfl_xor_sync(0xffffffffu, isum, 1);
            isum += __shfl_xor_sync(0xffffffffu, isum, 2);
            // <qp, sign> = scale * (2 * sum_{bit set} x16 - sum x16), and the MMA returns
            // D = -(256 * hi + lo) summed over set bits
            const float scale = amax > 0.f ? amax / 32000.0f : 0.f;
            const float my_scale = -2.0f * scale, my_bias = -scale * (float)isum;
            sign_scale = __shfl_sync(0xffffffffu, my_scale, (2 * t) * 4);
            sign_bias = __shfl_sync(0xffffffffu, my_bias, (2 * t) * 4);
        }
    }
    __syncthreads();

    const int64_t row0 = (int64_t)b * a.cache_sb + (int64_t)h * a.cache_sh;
    const int t_begin = split * a.tok_per_split;
    const int t_end = min(a.N, t_begin + a.tok_per_split);
    const int last = a.N - 1;
    const float kA = 0.08838834764831845f * 1.4426950408889634f;  // (1/sqrt(128)) * log2(e)
    const float kB = kA * (1.2533141373155003f / (float)TQ_D);     // ... * sqrt(pi/2)/D
    const uint8_t *lk = smem;        // key copies: bytes [0, 128) of every slot
    const uint8_t *lv = smem + 128;  // value copies: bytes [128, 256)
    const uint32_t lane_bits = lane * 4;
    const bool head_live = t < G;

    float m_run = -INFINITY, l_run = 0.f;
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int base = t_begin + warp * kTokIter; base < t_end; base += kWarps * kTokIter) {
        const bool tail = base + kTokIter > t_end;
        // ------------------------------------------------------------ logits
        float lg[kTiles][2];
#pragma unroll
        for (int i = 0; i < kTiles; ++i) {
            int tokA = base + 16 * i + 2 * g;
            if (tail) tokA = min(tokA, last & ~1);  // stay on an even token inside the row
            const int64_t rA = row0 + tokA;
            uint32_t wa[KB + 1], wb[KB + 1];
            {
                const uint32_t *pa = reinterpret_cast<const uint32_t *>(a.k_codes + rA * (16 * KB)) + KB * t;
#pragma unroll
                for (int w = 0; w < KB; ++w) wa[w] = __ldg(pa + w), wb[w] = __ldg(pa + 4 * KB + w);
                wa[KB] = wb[KB] = 0;
            }
            float d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                constexpr int W = 2 * KB;
                const int o0 = (2 * s) * W, o1 = (2 * s + 1) * W;
                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(lk + slot_offset<W>(wa, o0, lane_bits));
                const uint32_t a1 = *reinterpret_cast<const uint32_t *>(lk + slot_offset<W>(wb, o0, lane_bits));
                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(lk + slot_offset<W>(wa, o1, lane_bits));
                const uint32_t a3 = *reinterpret_cast<const uint32_t *>(lk + slot_offset<W>(wb, o1, lane_bits));
                mma_f16(d1, a0, a1, a2, a3, bq[s][0], bq[s][1]);
            }
            const float2 kn = half2_bits_to_float2(__ldg(reinterpret_cast<const uint32_t *>(a.k_norms + rA)));
            float lgA = kn.x * kA * (d1[0] + d1[1]);
            float lgB = kn.y * kA * (d1[2] + d1[3]);
            if (QJL) {
                const uint32_t *ps = reinterpret_cast<const uint32_t *>(a.k_signs + rA * 16) + t;
                const uint32_t sa = __ldg(ps), sb = __ldg(ps + 4);
                int d2[4] = {0, 0, 0, 0};
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const uint32_t a0 = prmt(sa << (2 * n), 0u, 0xBA98u);
                    const uint32_t a1 = prmt(sb << (2 * n), 0u, 0xBA98u);
                    const uint32_t a2 = prmt(sa << (2 * n + 1), 0u, 0xBA98u);
                    const uint32_t a3 = prmt(sb << (2 * n + 1), 0u, 0xBA98u);
                    mma_s8(d2, a0, a1, a2, a3, bp[n][0], bp[n][1]);
                }
                const float2 rn = half2_bits_to_float2(__ldg(reinterpret_cast<const uint32_t *>(a.k_rnorms + rA)));
                const float sA = fmaf((float)(d2[0] * 256 + d2[1]), sign_scale, sign_bias);
                const float sB = fmaf((float)(d2[2] * 256 + d2[3]), sign_scale, sign_bias);
                lgA = fmaf(rn.x * kB, sA, lgA);
                lgB = fmaf(rn.y * kB, sB, lgB);
            }
            if (tail) {
                const int real = base + 16 * i + 2 * g;
                if (real >= t_end) lgA = -INFINITY;
                if (real + 1 >= t_end) lgB = -INFINITY;
            }
            lg[i][0] = head_live ? lgA : -INFINITY;
            lg[i][1] = head_live ? lgB : -INFINITY;
        }
        // ------------------------------------------------------------ online softmax (base 2), head t
        float mx = lg[0][0];
#pragma unroll
        for (int i = 0; i < kTiles; ++i) mx = fmaxf(mx, fmaxf(lg[i][0], lg[i][1]));
#pragma unroll
        for (int sft = 4; sft <= 16; sft <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
        const float nm = fmaxf(m_run, mx);
        if (__any_sync(0xffffffffu, nm > m_run)) {
            const float sc = (nm == -INFINITY) ? 1.f : fast_exp2(m_run - nm);
            l_run *= sc;
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i][0] *= sc, o[i][2] *= sc;
            m_run = nm;
        }
        const float sub = (m_run == -INFINITY) ? 0.f : m_run;
        uint32_t pb[kTiles][2];
#pragma unroll
        for (int i = 0; i < kTiles; ++i) {
            int tokA = base + 16 * i + 2 * g;
            if (tail) tokA = min(tokA, last & ~1);
            const float2 vn = half2_bits_to_float2(__ldg(reinterpret_cast<const uint32_t *>(a.v_norms + row0 + tokA)));
            const float pA = fast_exp2(lg[i][0] - sub), pB = fast_exp2(lg[i][1] - sub);
            l_run += pA + pB;
            // rows = token slots, cols = (head t, unused)  ->  transpose to rows = columns
            // (a masked token may sit on an unwritten row whose norm is not finite)
            pb[i][0] = movmatrix_trans(pack_half2(pA > 0.f ? pA * vn.x : 0.f, 0.f));
            pb[i][1] = movmatrix_trans(pack_half2(pB > 0.f ? pB * vn.y : 0.f, 0.f));
        }
        // ------------------------------------------------------------ values
#pragma unroll
        for (int i = 0; i < kTiles; ++i) {
            const int tk = base + 16 * i + 4 * t;
            const uint8_t *vrow = a.v_codes + (row0 + (tail ? min(tk, last) : tk)) * (16 * VB);
            const int step1 = tail ? (min(tk + 1, last) - min(tk, last)) * (16 * VB) : 16 * VB;
            const int step2 = tail ? (min(tk + 2, last) - min(tk, last)) * (16 * VB) : 32 * VB;
            const int step3 = tail ? (min(tk + 3, last) - min(tk, last)) * (16 * VB) : 48 * VB;
            const uint64_t w0 = load_v_chunk<VB>(vrow, g);
            const uint64_t w1 = load_v_chunk<VB>(vrow + step1, g);
            const uint64_t w2 = load_v_chunk<VB>(vrow + step2, g);
            const uint64_t w3 = load_v_chunk<VB>(vrow + step3, g);
            constexpr uint64_t me = even_field_mask<VB>();
            // k-slots (2t, 2t+1) hold tokens (4t, 4t+2); k-slots (2t+8, 2t+9) hold (4t+1, 4t+3)
            const uint64_t x02 = (w0 & me) | ((w2 << VB) & (me << VB));
            const uint64_t y02 = ((w0 >> VB) & me) | (w2 & (me << VB));
            const uint64_t x13 = (w1 & me) | ((w3 << VB) & (me << VB));
            const uint64_t y13 = ((w1 >> VB) & me) | (w3 & (me << VB));
            const uint32_t xa[3] = {(uint32_t)x02, (uint32_t)(x02 >> 32), 0u};
            const uint32_t ya[3] = {(uint32_t)y02, (uint32_t)(y02 >> 32), 0u};
            const uint32_t xb[3] = {(uint32_t)x13, (uint32_t)(x13 >> 32), 0u};
            const uint32_t yb[3] = {(uint32_t)y13, (uint32_t)(y13 >> 32), 0u};
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                constexpr int W = 2 * VB;
                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(lv + slot_offset<W>(xa, mt * W, lane_bits));
                const uint32_t a1 = *reinterpret_cast<const uint32_t *>(lv + slot_offset<W>(ya, mt * W, lane_bits));
                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(lv + slot_offset<W>(xb, mt * W, lane_bits));
                const uint32_t a3 = *reinterpret_cast<const uint32_t *>(lv + slot_offset<W>(yb, mt * W, lane_bits));
                mma_f16(o[mt], a0, a1, a2, a3, pb[i][0], pb[i][1]);
            }
        }
    }

    // ---- merge the warps of the CTA, write the split partial
    __syncthreads();  // the tables are dead; reuse shared memory
    float *s_acc = reinterpret_cast<float *>(smem);   // [kWarps][4][128]
    float *s_m = s_acc + kWarps * 4 * TQ_D;           // [kWarps][4]
    float *s_l = s_m + kWarps * 4;
#pragma unroll
    for (int sft = 4; sft <= 16; sft <<= 1) l_run += __shfl_xor_sync(0xffffffffu, l_run, sft);
    if (g == 0) s_m[warp * 4 + t] = m_run, s_l[warp * 4 + t] = l_run;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        float *r = s_acc + (warp * 4 + t) * TQ_D + 16 * g + 2 * mt;
        r[0] = o[mt][0], r[1] = o[mt][2];
    }
    __syncthreads();
    const int d = threadIdx.x;
    for (int hh = 0; hh < G; ++hh) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w * 4 + hh]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float mw = s_m[w * 4 + hh];
            const float sc = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            L += s_l[w * 4 + hh] * sc;
            A += s_acc[(w * 4 + hh) * TQ_D + d] * sc;
        }
        const int64_t prow = (q_row0 + hh) * a.n_splits + split;
        a.part_acc[prow * TQ_D + d] = A;
        if (d == 0) a.part_m[prow] = M * 0.6931471805599453f, a.part_l[prow] = L;  // natural-log units
    }
}

template <int KB, int VB> size_t mma4_smem_bytes() {
    const int kk = 1 << (2 * KB), kv = 1 << (2 * VB);
    const size_t lut = (size_t)(kk > kv ? kk : kv) * kSlotWords * 4;
    const size_t merge = ((size_t)kWarps * 4 * TQ_D + 2 * kWarps * 4) * sizeof(float);
    return lut > merge ? lut : merge;
}

template <int KB, int VB, bool QJL> cudaError_t launch_mma4(const Mma4Args &a, dim3 grid, cudaStream_t stream) {
    const size_t smem = mma4_smem_bytes<KB, VB>();
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(tq_decode_mma4_kernel<KB, VB, QJL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    tq_decode_mma4_kernel<KB, VB, QJL><<<grid, kWarps * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

int32_t tq_launch_decode_mma4(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                              const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                              const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits, void *workspace,
                              void *out, cudaStream_t stream) {
    const int64_t rows = (int64_t)cache->batch * q_heads;
    DecodeWorkspace w = tq_carve_workspace(workspace, rows, n_splits);
    int rc = tq_launch_qprep(ctx, q, q_dtype, rows, w.qrot, w.qproj, stream);
    if (rc) return rc;

    Mma4Args a;
    a.k_codes = cache->k_codes, a.k_norms = cache->k_norms;
    a.k_signs = cache->k_signs, a.k_rnorms = cache->k_rnorms;
    a.v_codes = cache->v_codes, a.v_norms = cache->v_norms;
    a.cache_sb = cache->stride_b, a.cache_sh = cache->stride_h;
    a.Hkv = cache->kv_heads, a.G = q_heads / cache->kv_heads, a.N = seq_len, a.n_splits = n_splits;
    const int per_iter = kWarps * kTokIter;
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
        case 2: e = launch_mma4<2, 2, false>(a, grid, stream); break;
        case 3: e = launch_mma4<3, 3, false>(a, grid, stream); break;
        case 4: e = launch_mma4<4, 4, false>(a, grid, stream); break;
        case 12: e = launch_mma4<1, 2, true>(a, grid, stream); break;
        case 13: e = launch_mma4<2, 3, true>(a, grid, stream); break;
        case 14: e = launch_mma4<3, 4, true>(a, grid, stream); break;
        default: return TQ_ERR_UNSUPPORTED;
    }
    tq_prof_end(ctx, stream);
    TQ_CUDA_CHECK(e);

    CombineArgs c;
    c.part_m = w.part_m, c.part_l = w.part_l, c.part_acc = w.part_acc;
    c.n_splits = n_splits, c.Hq = q_heads, c.G = a.G;
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
