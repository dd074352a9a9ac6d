// Decode attention over the packed cache: tensor-core kernel for fp16 / bf16 queries
// with at most 8 query heads per KV head (Llama-3.1-8B: 32 / 8; Qwen2.5-7B: 28 / 4).
//
// Persistent CTAs, one per SM: the (batch, KV head) rows are laid end to end and cut into
// equal token chunks, one per CTA, so every SM streams the same number of bytes; a CTA emits
// one partial (max, sum, acc) per row it touches.  Each CTA serves all G query heads of a
// row, so packed bytes are read from HBM once.  The description below is the G <= 4 variant;
// the wide variant (see the kernel's template note) differs in how the MMA columns are used.
//
// Data movement: every group of four warps runs its own ring of 128-token slots in shared
// memory (32 tokens per warp).  One lane of the group fills a slot with six TMA bulk copies
// (cp.async.bulk: key codes, QJL signs, value codes and the three fp16 norm streams are each
// contiguous in HBM) that complete on a "full" mbarrier; every warp hands the slot back on an
// "empty" mbarrier and the warps take turns to wait for it and request the refill.  All waits
// are bounded spins.  No registers and no load/store-unit issue slots are spent on global
// loads, and HBM latency is hidden by the ring rather than by occupancy.
//
// Math: the 8 columns of every MMA are (head, part) pairs, which gives each lane of a
// quad its own head:
//   logits   S  [16 tok x (4 heads x {hi, lo})] = Kdeq[16 x 128] * {Qrot_hi, Qrot_lo}   f16 m16n8k16
//            (the rotated query is split in two f16 terms, so its rounding does not show)
//   QJL      S2 [16 tok x (4 heads x {hi, lo})] = Bit[16 x 128] * {Qp_hi, Qp_lo}        s8 m16n8k32
//            (a mask keeps sign bit n of each of four bytes in place, so an operand byte is
//            2^n or 0 and costs one logic instruction per four signs; the projected query is
//            16-bit fixed point in two s8 terms, divided by 2^n behind bit n, n = 0..3)
//   values   O^T[128 x (4 heads x {P, 0})] += Vdeq^T[128 x 16 tok] * P                   f16 m16n8k16
// A operands are built in registers from the packed words.  The contraction order of an
// MMA is free, so every lane gets codes that sit together in memory:
//   keys    lane (g, t): dims [32t, 32t+32) of two tokens of a 16-token tile; two
//           neighbouring codes index a per-lane-replicated shared-memory table of f16x2
//           centre pairs (slot e, lane l -> bank l: no bank conflicts);
//   values  lane (g, t): dims [16g, 16g+16) of tokens t, t+4, t+8, t+12; the codes of two
//           tokens are interleaved with bit-selects so one look-up yields the (token a,
//           token b) f16x2 that the MMA wants along its K axis.
// Softmax is online, base 2, in registers; P*|v| goes to f16 and is transposed with
// movmatrix.  Per-CTA partials (max, sum, acc) go to the workspace; tq_combine_kernel
// merges splits, un-rotates and casts.
#include <math.h>

#include "tq_common.cuh"
#include "tq_decode_shared.cuh"
#include "tq_mma_utils.cuh"
#include "tq_step_blocks.cuh"

// Build with -DTQ_TIMELINE to make every CTA record wall-clock stamps of its phases
// (read back with tq_debug_stamps); compiled out otherwise.
#ifdef TQ_TIMELINE
__device__ unsigned long long g_stamps[160 * 16];
#define TQ_STAMP(i)                                                                          \
    do {                                                                                     \
        if (threadIdx.x == 0 && blockIdx.x < 160 && (i) < 16) {                              \
            unsigned long long t_;                                                           \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                           \
            g_stamps[blockIdx.x * 16 + (i)] = t_;                                            \
        }                                                                                    \
    } while (0)
extern "C" int tq_debug_stamps(unsigned long long *out) { return (int)cudaMemcpyFromSymbol(out, g_stamps, sizeof(g_stamps)); }
#else
#define TQ_STAMP(i) do {} while (0)
#endif

namespace {

constexpr int kWarps = 16;
constexpr int kStageTok = 32;  // tokens per warp per ring slot (two 16-token MMA tiles)
constexpr int kStages = 2;
constexpr int kGroupWarps = 4;  // warps that share a ring: one bulk copy per stream serves all of them
constexpr int kGroups = kWarps / kGroupWarps;
constexpr int kGroupTok = kGroupWarps * kStageTok;  // tokens per ring slot
constexpr int kSlotWords = 64;  // table slot: 32 key words then 32 value words (256 B)
constexpr uint32_t kSpinLimit = 1u << 22;  // mbarrier polls before a wait gives up

struct Mma4Args {
    const uint8_t *k_codes;
    const uint16_t *k_norms;
    const uint8_t *k_signs;
    const uint16_t *k_rnorms;
    const uint8_t *v_codes;
    const uint16_t *v_norms;
    int64_t cache_sb, cache_sh;
    int Hkv, G, N, n_splits;
    int rows;    // batch * kv_heads
    int n_pad;   // N rounded up to the CTA step: rows are laid end to end in units of n_pad tokens
    int chunk;   // tokens of that flattened (row, token) space per CTA
    const int *seq_start;  // per batch entry: first token attended (null: 0)
    int stable_len;  // tokens [0, stable_len) of every row were written before the preceding kernel began
    // Length kept on the device (launch sequences replayed from a CUDA graph): when len_ptr is
    // set, N = min(*len_ptr + len_add, capacity), stable_len = *len_ptr, and n_pad / chunk are
    // planned by the kernel for its own grid.
    const int *len_ptr;
    int len_add, capacity;
    const uint32_t *frag;  // per query head: TQ_FRAG_ROW_WORDS words, see tq_qprep_frag_kernel
    float *part_m, *part_l, *part_acc;
    const float *centers_k, *centers_v;
    int *error_flag;  // set to 1 when a bounded wait ran out
    int device;       // host side only: the context's device
};

template <int KB, int VB, bool QJL> struct StageLayout {
    static constexpr int kK = 0;
    static constexpr int kV = kK + kGroupTok * 16 * KB;
    static constexpr int kS = kV + kGroupTok * 16 * VB;
    static constexpr int kKN = kS + (QJL ? kGroupTok * 16 : 0);
    static constexpr int kVN = kKN + kGroupTok * 2;
    static constexpr int kRN = kVN + kGroupTok * 2;
    static constexpr int kBytes = (kRN + (QJL ? kGroupTok * 2 : 0) + 127) / 128 * 128;
};

// ---- mbarrier / TMA bulk-copy wrappers (shared::cta addresses) ----
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// Bounded wait: returns false (and the caller flags an error) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned),
// completion counted on `bar`.
__device__ __forceinline__ void tma_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// The centre-pair table sits at shared-memory address kTableAddr, a multiple of 65536, so
// that a complete address can be assembled without an add: bits 16+ are the table base,
// byte 1 is the slot index (slot stride 256 B) and byte 0 the lane's offset inside the slot.
constexpr uint32_t kTableAddr = 65536;

__device__ __forceinline__ uint32_t lds_abs(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

// Shared-memory address of this lane's copy of the table slot selected by the BYTE that
// starts at bit `off` of the little-endian word array `w` (w[off/32+1] must exist).  Every
// table has 256 slots and ignores the bits of the byte beyond the field it encodes, so a
// field never needs masking.  `lane_bits` = kTableAddr + the lane's offset inside a slot.
// `off` is a compile-time constant after unrolling: a byte-aligned field costs one byte
// permute; otherwise the word is first funnel-shifted by off % 8 (the shifted copies are
// shared by all fields with the same word and remainder).
__device__ __forceinline__ uint32_t slot_addr(const uint32_t *w, int off, uint32_t lane_bits) {
    const int wi = off >> 5, sh = off & 7, byte = (off & 31) >> 3;
    const uint32_t x = sh == 0 ? w[wi] : __funnelshift_r(w[wi], w[wi + 1], sh);
    return prmt(x, lane_bits, 0x7604u | ((uint32_t)byte << 4));
}

// The 16*VB-bit value chunk of lane group g of one staged token row (row = VB*16 bytes).
template <int VB> __device__ __forceinline__ uint64_t lds_v_chunk(const uint8_t *row, int g) {
    if (VB == 4) {
        return *reinterpret_cast<const unsigned long long *>(row + 8 * g);
    } else if (VB == 2) {
        return *reinterpret_cast<const unsigned int *>(row + 4 * g);
    } else {  // 3 bits: 6 bytes at byte 6g, inside the two aligned words that start at 6g rounded down to 4
        const uint32_t *p = reinterpret_cast<const uint32_t *>(row + ((6 * g) & ~3));
        const uint64_t w = (uint64_t)p[0] | ((uint64_t)p[1] << 32);
        return (g & 1) ? w >> 16 : w;  // (what lies beyond the 48 bits is never looked at)
    }
}

// WIDE = false: G <= 4 query heads per KV head, MMA columns = (head, hi / lo term of the query).
// WIDE = true : G <= 8, MMA columns = heads; the rotated query is a single f16 term and the two
//               s8 terms of the projected query go through two integer MMAs.  A lane then owns
//               two heads (columns 2t and 2t + 1) in the softmax and all four accumulator columns.
template <int KB, int VB, bool QJL, bool WIDE>
__global__ void __launch_bounds__(kWarps * 32, 1) tq_decode_mma4_kernel(Mma4Args a) {
    constexpr int NH = WIDE ? 2 : 1;  // heads per lane
    using L = StageLayout<KB, VB, QJL>;
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kEntries = 256;  // indexed by a whole byte; bits beyond the field are ignored
    constexpr int kTableBytes = kEntries * kSlotWords * 4;
    static_assert(kTableBytes <= 65536, "table must fit between two 64 KB boundaries");
    // Shared-memory map (absolute shared addresses): [dynamic base, 65536) the first rings,
    // [65536, 65536 + table) the centre-pair table, then the remaining rings and the mbarriers.
    const uint32_t dyn_base = smem_u32(smem);
    constexpr int kSlots = kGroups * kStages;  // ring slots of the CTA, placed one by one around the table
    constexpr int kMergeBytes = kWarps * 4 * (TQ_D + 2) * 4;
    const int slots_low = dyn_base <= kTableAddr ? min(kSlots, (int)((kTableAddr - dyn_base) / L::kBytes)) : 0;
    const uint32_t high_base = kTableAddr + ((kTableBytes + 127) / 128) * 128;
    const uint32_t bars_addr = high_base + (kSlots - slots_low) * L::kBytes;  // full[kSlots] then empty[kSlots]
    {
        uint32_t dyn_size;
        asm("mov.u32 %0, %%dynamic_smem_size;\n" : "=r"(dyn_size));
        if (dyn_base > kTableAddr || bars_addr + 2 * kSlots * 8 > dyn_base + dyn_size ||
            slots_low * L::kBytes < kMergeBytes) {
            if (threadIdx.x == 0) atomicExch(a.error_flag, 2);  // layout does not fit: refuse to run
            return;
        }
    }
    uint32_t *table = reinterpret_cast<uint32_t *>(smem + (kTableAddr - dyn_base));
    TQ_STAMP(0);
    int seg_no = 0;

    const int G = a.G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    // the centres the tables are built from: requested first, ahead of the bulk copies below,
    // so that these few bytes do not queue behind the ring's first fill
    const float ck = a.centers_k[lane & 15], cv = a.centers_v[lane & 15];

    int N = a.N, n_pad = a.n_pad, chunk = a.chunk, stable_len = a.stable_len;
    if (a.len_ptr) {
        stable_len = *a.len_ptr;
        N = max(1, min(stable_len + a.len_add, a.capacity));
        const TqPlan plan = tq_make_plan(N, a.rows, gridDim.x, a.n_splits, kWarps * kStageTok);
        n_pad = plan.n_pad, chunk = plan.chunk;
    }

    // ---- this CTA's contiguous piece of the flattened (row, token) space
    const int64_t flat_begin = (int64_t)blockIdx.x * chunk;
    const int64_t flat_end = min(flat_begin + chunk, (int64_t)a.rows * n_pad);

    // ---- ring set-up: group gq owns slots gq * kStages + s.  A group is the warps gq, gq + kGroups,
    // gq + 2 * kGroups, ...: with four groups these are the four warps of one of the SM's four warp
    // schedulers, so the schedulers carry identical loads and the groups finish together (with
    // consecutive warps per group every scheduler held one warp of each group, the groups ran at
    // different rates and the slowest one finished 4.5 us after the fastest, alone on the SM).
    const int gq = warp % kGroups, wq = warp / kGroups;
    auto slot_u32 = [&](int st) -> uint32_t {
        const int q = gq * kStages + st;
        return q < slots_low ? dyn_base + q * L::kBytes : high_base + (q - slots_low) * L::kBytes;
    };
    const uint32_t full_u32 = bars_addr + gq * kStages * 8;
    const uint32_t empty_u32 = bars_addr + (kSlots + gq * kStages) * 8;
    if (wq < kStages && lane == 0) {  // warp st of the group sets slot st up (and requests its first fill below)
        mbar_init(full_u32 + wq * 8, 1), mbar_init(empty_u32 + wq * 8, kGroupWarps);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    uint32_t ring_pos = 0;  // slots this group has consumed since the kernel began

    // ---- a segment = the part of one (batch, KV head) row inside this CTA's piece
    constexpr int kCtaStep = kWarps * kStageTok;
    struct Seg {
        int bh, seg_len, t_lo, t_end, grp_first, n_iter;
        int64_t row0;
    };
    auto seg_at = [&](int64_t flat) {
        Seg sg;
        // (the flattened space nearly always fits 32 bits, whose division is several times cheaper)
        sg.bh = flat_end <= 0xffffffffll ? (int)((uint32_t)flat / (uint32_t)n_pad) : (int)(flat / n_pad);
        const int seg_lo = (int)(flat - (int64_t)sg.bh * n_pad);
        sg.seg_len = (int)min((int64_t)(n_pad - seg_lo), flat_end - flat);
        sg.row0 = (int64_t)(sg.bh / a.Hkv) * a.cache_sb + (int64_t)(sg.bh % a.Hkv) * a.cache_sh;
        sg.t_end = min(N, seg_lo + sg.seg_len);
        // a left-padded row attends tokens [t_lo, N): CTA steps that lie wholly before t_lo are left out
        sg.t_lo = a.seq_start ? a.seq_start[sg.bh / a.Hkv] : 0;
        const int first_tok = min(max(seg_lo, sg.t_lo / kCtaStep * kCtaStep), seg_lo + sg.seg_len);
        sg.grp_first = first_tok + gq * kGroupTok;
        sg.n_iter = sg.grp_first < sg.t_end ? (sg.t_end - sg.grp_first + kCtaStep - 1) / kCtaStep : 0;
        return sg;
    };
    // one lane of the group: fill the ring slot of the segment's local iteration `it`
    auto issue = [&](const Seg &sg, int it) {
        const int base = sg.grp_first + it * kCtaStep;
        int n = min(kGroupTok, sg.t_end - base);
        n = (n + 7) & ~7;  // whole 16-byte pieces of the norm streams; rows stay inside the row's stride
        const int st = (ring_pos + it) % kStages;
        const uint32_t dst = slot_u32(st), bar = full_u32 + st * 8;
        const int64_t r = sg.row0 + base;
        const uint32_t total = n * (16 * KB + 16 * VB + 4 + (QJL ? 18 : 0));
#ifdef TQ_DEBUG_BOUNDS
        // Checked build: every bulk copy must read tokens [base, base + n) of a real row, inside the
        // row's allocation, and land inside this CTA's ring slot.  A request that does not is recorded
        // (status 6), dropped, and its barrier completed by hand so that nobody waits for it.
        {
            uint32_t dyn_size;
            asm("mov.u32 %0, %%dynamic_smem_size;\n" : "=r"(dyn_size));
            const bool ok = sg.bh >= 0 && sg.bh < a.rows && base >= 0 && n > 0 && n <= kGroupTok &&
                            base + n <= a.capacity && dst >= dyn_base && dst + L::kBytes <= dyn_base + dyn_size &&
                            (dst + L::kBytes <= kTableAddr || dst >= kTableAddr + kTableBytes);
            if (!ok) {
                atomicExch(a.error_flag, 6);
                mbar_arrive(bar);
                return;
            }
        }
#endif
        mbar_expect_tx(bar, total);
        tma_load_1d(dst + L::kK, a.k_codes + r * (16 * KB), n * 16 * KB, bar);
        tma_load_1d(dst + L::kV, a.v_codes + r * (16 * VB), n * 16 * VB, bar);
        tma_load_1d(dst + L::kKN, a.k_norms + r, n * 2, bar);
        tma_load_1d(dst + L::kVN, a.v_norms + r, n * 2, bar);
        if (QJL) {
            tma_load_1d(dst + L::kS, a.k_signs + r * 16, n * 16, bar);
            tma_load_1d(dst + L::kRN, a.k_rnorms + r, n * 2, bar);
        }
    };
    // The kernel is launched as a programmatic dependent of the query-preparation kernel, which
    // may also be appending this step's token: the first segment's ring slots that hold only
    // older tokens are requested right here, before the tables are built and before the
    // dependency wait; the others (`deferred`) after the wait.
    // (Slot `it` is requested by warp `it` of the group, so the requests of a group run side by
    // side; bit `it` of `deferred` is only ever set in that warp's lane 0.)
    uint32_t deferred = 0;
    static_assert(kStages <= kGroupWarps, "one warp per first slot");
    if (wq < kStages && lane == 0 && flat_begin < flat_end) {
        const Seg sg = seg_at(flat_begin);
        if (wq < sg.n_iter) {
            if (sg.grp_first + wq * kCtaStep + kGroupTok > stable_len) deferred = 1u << wq;
            else issue(sg, wq);
        }
    }

    // ---- per-lane replicated f16x2 centre-pair tables (keys in the low half of each slot);
    // a warp fills one slot at a time, lane l writing words l and 32+l (no bank conflicts)
    {
        constexpr int mk = (1 << KB) - 1, mv = (1 << VB) - 1;
        for (int e = warp; e < kEntries; e += kWarps) {
            uint32_t *slot = table + e * kSlotWords;
            const float klo = __shfl_sync(0xffffffffu, ck, e & mk), khi = __shfl_sync(0xffffffffu, ck, (e >> KB) & mk);
            const float vlo = __shfl_sync(0xffffffffu, cv, e & mv), vhi = __shfl_sync(0xffffffffu, cv, (e >> VB) & mv);
            slot[lane] = pack_half2(klo, khi);
            slot[32 + lane] = pack_half2(vlo, vhi);
        }
    }

    __syncthreads();  // tables complete
    TQ_STAMP(1);

    const float kA = 0.08838834764831845f * 1.4426950408889634f;  // (1/sqrt(128)) * log2(e)
    const float kB = kA * (1.2533141373155003f / (float)TQ_D);     // ... * sqrt(pi/2)/D
    const uint32_t lane_k = kTableAddr + lane * 4;        // key copies: bytes [0, 128) of every slot
    const uint32_t lane_v = kTableAddr + 128 + lane * 4;  // value copies: bytes [128, 256)
    bool timed_out = false;
    bool first_segment = true;

    // ---- one segment per row this CTA touches
    for (int64_t flat = flat_begin; flat < flat_end;) {
    const Seg sg = seg_at(flat);
    flat += sg.seg_len;
    const int bh = sg.bh;
    const int split = blockIdx.x - (int)(((int64_t)bh * n_pad) / chunk);  // partial slot inside the row
    const int64_t q_row0 = (int64_t)bh * G;
    const int t_end = sg.t_end, t_lo = sg.t_lo;
    const int my_first = sg.grp_first + wq * kStageTok;
    const int n_iter = sg.n_iter;
    const int n_first = min(n_iter, kStages);
    if (first_segment) {
        tq_grid_dependency_wait();
        TQ_STAMP(2);
        for (int it = 0; it < n_first; ++it)
            if (deferred >> it & 1) issue(sg, it);  // (only the issuing lane has bits set)
        first_segment = false;
    } else if (wq == 0 && lane == 0) {
        // The first slots of a later segment are requested by warp 0 of the group (the
        // __syncthreads that ended the previous segment guarantees that the whole group is done
        // with them); the ring area was last touched through ordinary loads/stores (the merge).
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (int it = 0; it < n_first; ++it) issue(sg, it);
    }

    // ---- B fragments: column g = (head g/2, part g%2), or head g in the wide variant
    const int hcol = WIDE ? g : g >> 1, part = WIDE ? 0 : g & 1;
    const bool live = hcol < G;
    uint32_t bq[8][2];
    uint32_t bp[QJL ? 4 * NH : 1][2];  // wide: [0, 4) hi terms, [4, 8) lo terms
    float sign_scale[NH], sign_bias[NH];  // for the heads this lane owns in the softmax
    {
        const uint32_t *head_frag = a.frag + (q_row0 + (live ? hcol : 0)) * TQ_FRAG_ROW_WORDS;
        const uint2 *fr = reinterpret_cast<const uint2 *>(head_frag + (part * 4 + t) * 26);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const uint2 v = __ldg(fr + s);
            bq[s][0] = live ? v.x : 0u, bq[s][1] = live ? v.y : 0u;
        }
        if (QJL) {
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const uint2 v = __ldg(fr + 8 + n);
                bp[n][0] = live ? v.x : 0u, bp[n][1] = live ? v.y : 0u;
            }
            if (WIDE) {
                const uint2 *fl = reinterpret_cast<const uint2 *>(head_frag + (4 + t) * 26);
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const uint2 v = __ldg(fl + 8 + n);
                    bp[(QJL && WIDE ? 4 : 0) + n][0] = live ? v.x : 0u, bp[(QJL && WIDE ? 4 : 0) + n][1] = live ? v.y : 0u;
                }
            }
        }
#pragma unroll
        for (int hl = 0; hl < NH; ++hl) {
            const int head = WIDE ? 2 * t + hl : t;
            const uint32_t *mine = a.frag + (q_row0 + (head < G ? head : 0)) * TQ_FRAG_ROW_WORDS;
            sign_scale[hl] = QJL ? __uint_as_float(__ldg(mine + 24)) : 0.f;
            sign_bias[hl] = QJL ? __uint_as_float(__ldg(mine + 25)) : 0.f;
        }
    }
    if (seg_no == 0) TQ_STAMP(3);
    float m_run[NH], l_run[NH];
#pragma unroll
    for (int hl = 0; hl < NH; ++hl) m_run[hl] = -INFINITY, l_run[hl] = 0.f;
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int it = 0; it < n_iter; ++it) {
        const int base = my_first + it * kCtaStep;
        const int st = (ring_pos + it) % kStages;
        const uint32_t use_parity = ((ring_pos + it) / kStages) & 1;
        const uint8_t *slot = smem + (slot_u32(st) - dyn_base);
        if (base < t_end) {  // (a warp whose tokens all lie past the end only takes part in the hand-shake)
        if (!mbar_wait(full_u32 + st * 8, use_parity)) timed_out = true;
        // `tail`: some of the warp's 32 tokens lie outside [t_lo, t_end) and get masked one by one;
        // a warp with all 32 before t_lo (only in a row's first step) has waited and now skips the math
        const bool tail = base + kStageTok > t_end || base < t_lo;
        if (base + kStageTok > t_lo) {
        // this warp's 32 tokens inside the slot
        const uint8_t *spK = slot + L::kK + wq * kStageTok * 16 * KB;
        const uint8_t *spV = slot + L::kV + wq * kStageTok * 16 * VB;
        const uint8_t *spS = slot + L::kS + wq * kStageTok * 16;
        const uint16_t *kn = reinterpret_cast<const uint16_t *>(slot + L::kKN) + wq * kStageTok;
        const uint16_t *vn = reinterpret_cast<const uint16_t *>(slot + L::kVN) + wq * kStageTok;
        const uint16_t *rn = reinterpret_cast<const uint16_t *>(slot + L::kRN) + wq * kStageTok;

        // ------------------------------------------------------------ logits
        float lg[2][2][NH];  // [tile][token A / B][head of this lane]
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            // token slot s of the tile holds token pi(s): pi(2j) = j, pi(2j+1) = j+4, pi(s+8) = pi(s)+8,
            // which lets the value reads below touch four consecutive rows per instruction
            const int slotA = 16 * i + (g >> 1) + 4 * (g & 1), slotB = slotA + 8;
            uint32_t wa[KB + 1], wb[KB + 1];
            {
                const uint32_t *pa = reinterpret_cast<const uint32_t *>(spK + slotA * (16 * KB)) + KB * t;
                const uint32_t *pb = reinterpret_cast<const uint32_t *>(spK + slotB * (16 * KB)) + KB * t;
#pragma unroll
                for (int w = 0; w < KB; ++w) wa[w] = pa[w], wb[w] = pb[w];
                wa[KB] = wb[KB] = 0;
            }
            float d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                constexpr int W = 2 * KB;
                const int o0 = (2 * s) * W, o1 = (2 * s + 1) * W;
                const uint32_t a0 = lds_abs(slot_addr(wa, o0, lane_k));
                const uint32_t a1 = lds_abs(slot_addr(wb, o0, lane_k));
                const uint32_t a2 = lds_abs(slot_addr(wa, o1, lane_k));
                const uint32_t a3 = lds_abs(slot_addr(wb, o1, lane_k));
                mma_f16(d1, a0, a1, a2, a3, bq[s][0], bq[s][1]);
            }
            float lgA[NH], lgB[NH];
            {
                const float knA = tq_half_bits_to_float(kn[slotA]) * kA, knB = tq_half_bits_to_float(kn[slotB]) * kA;
                if (WIDE) {
#pragma unroll
                    for (int hl = 0; hl < NH; ++hl) lgA[hl] = knA * d1[hl], lgB[hl] = knB * d1[2 + hl];
                } else {
                    lgA[0] = knA * (d1[0] + d1[1]), lgB[0] = knB * (d1[2] + d1[3]);
                }
            }
            if (QJL) {
                const uint32_t sa = reinterpret_cast<const uint32_t *>(spS + slotA * 16)[t];
                const uint32_t sb = reinterpret_cast<const uint32_t *>(spS + slotB * 16)[t];
                const uint32_t sa4 = sa >> 4, sb4 = sb >> 4;
                int d2[4] = {0, 0, 0, 0};
                int d2l[4] = {0, 0, 0, 0};  // wide: the lo-term products
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    // sign bit n of every byte stays where it is (value 2^n or 0); the projected
                    // query behind it was divided by 2^n when its fragment was built
                    const uint32_t a0 = sa & (0x01010101u << n);
                    const uint32_t a1 = sb & (0x01010101u << n);
                    const uint32_t a2 = sa4 & (0x01010101u << n);
                    const uint32_t a3 = sb4 & (0x01010101u << n);
                    mma_s8(d2, a0, a1, a2, a3, bp[n][0], bp[n][1]);
                    if (WIDE) mma_s8(d2l, a0, a1, a2, a3, bp[(WIDE ? 4 : 0) + n][0], bp[(WIDE ? 4 : 0) + n][1]);
                }
                const float rnA = tq_half_bits_to_float(rn[slotA]) * kB, rnB = tq_half_bits_to_float(rn[slotB]) * kB;
#pragma unroll
                for (int hl = 0; hl < NH; ++hl) {
                    const int xa = WIDE ? d2[hl] * 256 + d2l[hl] : d2[0] * 256 + d2[1];
                    const int xb = WIDE ? d2[2 + hl] * 256 + d2l[2 + hl] : d2[2] * 256 + d2[3];
                    lgA[hl] = fmaf(rnA, fmaf((float)xa, sign_scale[hl], sign_bias[hl]), lgA[hl]);
                    lgB[hl] = fmaf(rnB, fmaf((float)xb, sign_scale[hl], sign_bias[hl]), lgB[hl]);
                }
            }
#pragma unroll
            for (int hl = 0; hl < NH; ++hl) {
                if (tail) {  // rows past the range hold stale bytes, rows before it are masked
                    if (base + slotA >= t_end || base + slotA < t_lo) lgA[hl] = -INFINITY;
                    if (base + slotB >= t_end || base + slotB < t_lo) lgB[hl] = -INFINITY;
                }
                // (lanes whose head >= G see a zero query: their state is never read)
                lg[i][0][hl] = lgA[hl], lg[i][1][hl] = lgB[hl];
            }
        }
        // ------------------------------------------------------------ online softmax (base 2), this lane's heads
        float nm[NH];
        bool grew = false;
#pragma unroll
        for (int hl = 0; hl < NH; ++hl) {
            float mx = fmaxf(fmaxf(lg[0][0][hl], lg[0][1][hl]), fmaxf(lg[1][0][hl], lg[1][1][hl]));
#pragma unroll
            for (int sft = 4; sft <= 16; sft <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
            nm[hl] = fmaxf(m_run[hl], mx);
            grew |= nm[hl] > m_run[hl];
        }
        if (__any_sync(0xffffffffu, grew)) {
            // every iteration holds at least one real token, so nm is finite; exp2(-inf) = 0
#pragma unroll
            for (int hl = 0; hl < NH; ++hl) {
                const float sc = fast_exp2(m_run[hl] - nm[hl]);
                l_run[hl] *= sc;
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i][hl] *= sc, o[i][2 + hl] *= sc;
                m_run[hl] = nm[hl];
            }
        }
        uint32_t pb[2][2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int slotA = 16 * i + (g >> 1) + 4 * (g & 1);
            const float vnA = tq_half_bits_to_float(vn[slotA]), vnB = tq_half_bits_to_float(vn[slotA + 8]);
            float wA[2] = {0.f, 0.f}, wB[2] = {0.f, 0.f};
#pragma unroll
            for (int hl = 0; hl < NH; ++hl) {
                const float pA = fast_exp2(lg[i][0][hl] - m_run[hl]), pB = fast_exp2(lg[i][1][hl] - m_run[hl]);
                l_run[hl] += pA + pB;
                // (a masked token's staged norm may be stale and not finite)
                wA[hl] = pA * vnA, wB[hl] = pB * vnB;
                if (tail) wA[hl] = pA > 0.f ? wA[hl] : 0.f, wB[hl] = pB > 0.f ? wB[hl] : 0.f;
            }
            // rows = token slots, cols = this lane's heads (narrow: head t and an unused column)
            // -> transpose to rows = columns
            pb[i][0] = movmatrix_trans(pack_half2(wA[0], wA[1]));
            pb[i][1] = movmatrix_trans(pack_half2(wB[0], wB[1]));
        }
        // ------------------------------------------------------------ values
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint8_t *vrow = spV + (16 * i + t) * (16 * VB);
            const uint64_t w0 = lds_v_chunk<VB>(vrow, g);                    // token t      (k-slot 2t)
            const uint64_t w1 = lds_v_chunk<VB>(vrow + 4 * 16 * VB, g);      // token t+4    (k-slot 2t+1)
            const uint64_t w2 = lds_v_chunk<VB>(vrow + 8 * 16 * VB, g);      // token t+8    (k-slot 2t+8)
            const uint64_t w3 = lds_v_chunk<VB>(vrow + 12 * 16 * VB, g);     // token t+12   (k-slot 2t+9)
            constexpr uint64_t me = even_field_mask<VB>();
            const uint64_t x01 = (w0 & me) | ((w1 << VB) & (me << VB));
            const uint64_t y01 = ((w0 >> VB) & me) | (w1 & (me << VB));
            const uint64_t x23 = (w2 & me) | ((w3 << VB) & (me << VB));
            const uint64_t y23 = ((w2 >> VB) & me) | (w3 & (me << VB));
            const uint32_t xa[3] = {(uint32_t)x01, (uint32_t)(x01 >> 32), 0u};
            const uint32_t ya[3] = {(uint32_t)y01, (uint32_t)(y01 >> 32), 0u};
            const uint32_t xb[3] = {(uint32_t)x23, (uint32_t)(x23 >> 32), 0u};
            const uint32_t yb[3] = {(uint32_t)y23, (uint32_t)(y23 >> 32), 0u};
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                constexpr int W = 2 * VB;
                const uint32_t a0 = lds_abs(slot_addr(xa, mt * W, lane_v));
                const uint32_t a1 = lds_abs(slot_addr(ya, mt * W, lane_v));
                const uint32_t a2 = lds_abs(slot_addr(xb, mt * W, lane_v));
                const uint32_t a3 = lds_abs(slot_addr(yb, mt * W, lane_v));
                mma_f16(o[mt], a0, a1, a2, a3, pb[i][0], pb[i][1]);
            }
        }
        }  // at least one token at or after t_lo
        }  // base < t_end
        // ------------------------------------------------------------ hand the slot back; the warps of the
        // group take turns to wait until all of them have done so and to request the refill
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(empty_u32 + st * 8);
            if (it + kStages < n_iter && wq == (it % kGroupWarps)) {
                if (mbar_wait(empty_u32 + st * 8, use_parity)) issue(sg, it + kStages);
                else timed_out = true;
            }
        }
    }
    ring_pos += n_iter;
    TQ_STAMP(5 + 3 * seg_no);

    // ---- merge the warps of the CTA and write this segment's partial.  The merge buffer
    // reuses the first rings' memory, which is idle here: every issued stage was consumed.
    __syncthreads();
    TQ_STAMP(6 + 3 * seg_no);
    float *s_acc = reinterpret_cast<float *>(smem);   // [kWarps][4][128]
    float *s_m = s_acc + kWarps * 4 * TQ_D;           // [kWarps][4]
    float *s_l = s_m + kWarps * 4;
#pragma unroll
    for (int hl = 0; hl < NH; ++hl) {  // the wide variant merges its even heads, then its odd heads
        if (hl) __syncthreads();
        float l_all = l_run[hl];
#pragma unroll
        for (int sft = 4; sft <= 16; sft <<= 1) l_all += __shfl_xor_sync(0xffffffffu, l_all, sft);
        if (g == 0) s_m[warp * 4 + t] = m_run[hl], s_l[warp * 4 + t] = l_all;
        // A warp's 512 accumulators are laid out [mt][lane][2], so the 8-byte stores of a warp
        // and the reads of 32 consecutive elements below both touch every bank once.
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
            *reinterpret_cast<float2 *>(s_acc + warp * 4 * TQ_D + mt * 64 + lane * 2) = make_float2(o[mt][hl], o[mt][2 + hl]);
        __syncthreads();
        for (int idx = threadIdx.x; idx < 4 * TQ_D; idx += blockDim.x) {
            // element idx of that layout: accumulator tile mt of lane (gg, tt), column pair member j
            const int mt = idx >> 6, gg = (idx & 63) >> 3, tt = (idx >> 1) & 3, j = idx & 1;
            const int d = 16 * gg + 2 * mt + j;
            const int hh = WIDE ? 2 * tt + hl : tt;
            if (hh >= G) continue;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w * 4 + tt]);
            float Lsum = 0.f, A = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float mw = s_m[w * 4 + tt];
                const float sc = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
                Lsum += s_l[w * 4 + tt] * sc;
                A += s_acc[w * 4 * TQ_D + idx] * sc;
            }
            const int64_t prow = (q_row0 + hh) * a.n_splits + split;
#ifdef TQ_DEBUG_BOUNDS
            if (split < 0 || split >= a.n_splits || q_row0 + hh >= (int64_t)a.rows * G) {  // a partial slot the workspace does not have
                atomicExch(a.error_flag, 6);
                continue;
            }
#endif
            a.part_acc[prow * TQ_D + d] = A;
            if (d == 0) a.part_m[prow] = M * 0.6931471805599453f, a.part_l[prow] = Lsum;  // natural-log units
        }
    }
    __syncthreads();  // the merge buffer is free again before the next segment refills the rings
    TQ_STAMP(7 + 3 * seg_no);
    ++seg_no;
    }  // segment loop
    if (timed_out && lane == 0) atomicExch(a.error_flag, 1);
    // (a CTA without work still waits for the kernel before this one: a grid that completes must
    // imply that everything ordered before it has completed)
    if (first_segment) tq_grid_dependency_wait();
    TQ_STAMP(14);
}

template <int KB, int VB, bool QJL> size_t mma4_smem_bytes() { return 227 * 1024; }

template <int KB, int VB, bool QJL, bool WIDE>
cudaError_t launch_mma4_variant(const Mma4Args &a, dim3 grid, cudaStream_t stream) {
    const size_t smem = mma4_smem_bytes<KB, VB, QJL>();
    // the attribute belongs to the (kernel, device) pair: one flag per device of this instantiation
    static bool configured[TQ_MAX_DEVICES] = {};
    if (a.device < 0 || a.device >= TQ_MAX_DEVICES) return cudaErrorInvalidDevice;
    if (!configured[a.device]) {
        cudaError_t e = cudaFuncSetAttribute(tq_decode_mma4_kernel<KB, VB, QJL, WIDE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[a.device] = true;
    }
    return tq_launch_kernel(tq_decode_mma4_kernel<KB, VB, QJL, WIDE>, grid, dim3(kWarps * 32), smem, stream,
                            /*programmatic=*/true, a);
}

template <int KB, int VB, bool QJL> cudaError_t launch_mma4(const Mma4Args &a, dim3 grid, cudaStream_t stream) {
    return a.G > 4 ? launch_mma4_variant<KB, VB, QJL, true>(a, grid, stream)
                   : launch_mma4_variant<KB, VB, QJL, false>(a, grid, stream);
}

}  // namespace

int tq_mma4_tokens_per_cta_step() { return kWarps * kStageTok; }

int32_t tq_launch_decode_mma4(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                              const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                              const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits, void *workspace,
                              void *out, const TqStepExtras *extras, cudaStream_t stream) {
    const int64_t rows = (int64_t)cache->batch * q_heads;
    DecodeWorkspace w = tq_carve_workspace(workspace, rows, n_splits);
    // the fragment area overlays the rotated / projected query rows of the workspace
    uint32_t *frag = reinterpret_cast<uint32_t *>(w.qrot);
    const int groups = q_heads / cache->kv_heads;
    const TqPackArgs *append = extras ? extras->append : nullptr;  // this step's new token, encoded by the same launch
    const int *len_ptr = extras ? extras->len_ptr : nullptr;       // sequence length kept on the device
    const tq_gather_desc *gather = extras ? extras->gather : nullptr;
    if (gather && n_tail) return TQ_ERR_UNSUPPORTED;
    int rc = tq_launch_qprep_frag(ctx, q, q_dtype, rows / groups, groups, frag, append, stream);
    if (rc) return rc;

    Mma4Args a;
    a.k_codes = cache->k_codes, a.k_norms = cache->k_norms;
    a.k_signs = cache->k_signs, a.k_rnorms = cache->k_rnorms;
    a.v_codes = cache->v_codes, a.v_norms = cache->v_norms;
    a.cache_sb = cache->stride_b, a.cache_sh = cache->stride_h;
    a.Hkv = cache->kv_heads, a.G = q_heads / cache->kv_heads, a.N = seq_len, a.n_splits = n_splits;
    // Rows are laid end to end (each padded to the CTA step) and cut into equal chunks, one per
    // CTA, at most one CTA per SM; a row then has at most ceil(n_pad / chunk) + 1 partials,
    // which must fit the n_splits slots the caller's workspace provides.
    const int step = kWarps * kStageTok;
    a.rows = cache->batch * cache->kv_heads;
    const TqPlan plan = tq_make_plan(seq_len, a.rows, ctx->sm_count, n_splits, step);
    a.n_pad = plan.n_pad, a.chunk = plan.chunk;
    const int64_t total = (int64_t)a.rows * a.n_pad;
    a.seq_start = cache->seq_start;
    a.stable_len = append ? append->pos0 : seq_len;
    a.len_ptr = len_ptr, a.len_add = append ? 1 : 0, a.capacity = cache->capacity;
    a.frag = frag;
    a.part_m = w.part_m, a.part_l = w.part_l, a.part_acc = w.part_acc;
    a.centers_k = ctx->centers_k, a.centers_v = ctx->centers_v;
    a.error_flag = ctx->error_flag;
    a.device = ctx->device;
    // Length on the device: the kernel plans for its own grid.  One CTA per SM, except that a
    // single partial per row (n_splits == 1) means one CTA per row, however many rows there are.
    const unsigned dev_grid = n_splits == 1 && a.rows > ctx->sm_count ? (unsigned)a.rows : (unsigned)ctx->sm_count;
    dim3 grid(len_ptr ? dev_grid : (unsigned)((total + a.chunk - 1) / a.chunk));
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
    c.seg_chunk = a.chunk, c.seg_npad = a.n_pad;
    c.len_ptr = len_ptr, c.len_add = a.len_add, c.capacity = a.capacity;
    c.plan_rows = a.rows, c.plan_ctas = (int)grid.x, c.plan_step = step;
    c.gather_world = 0, c.parts = 0, c.part = 0, c.head_group = 0, c.exch_rows = 0;
    if (gather && extras->parts > 0) {
        c.parts = extras->parts, c.part = gather->rank % extras->parts, c.head_group = gather->rank / extras->parts;
        c.exch_rows = (int64_t)cache->batch * gather->q_heads_total;
    }
    if (gather) {
        c.gather_world = gather->world, c.gather_rank = gather->rank, c.gather_heads_total = gather->q_heads_total;
        c.gather_seq = gather->seq;
        c.gather_seq_ptr = gather->seq_dev, c.gather_out_stride = gather->out_stride;
        for (int p = 0; p < TQ_MAX_PEERS; ++p) {
            c.gather_out[p] = p < gather->world ? gather->out[p] : nullptr;
            c.gather_flags[p] = p < gather->world ? gather->flags[p] : nullptr;
        }
    }
    c.rot_v = ctx->rot_v;
    c.q = q, c.out = out, c.out_f32 = extras ? extras->out_f32 : nullptr;
    if (c.out_f32 && (gather || n_tail)) return TQ_ERR_UNSUPPORTED;
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
    return tq_launch_combine(c, q_dtype, rows, stream, /*programmatic=*/true);
}
