// Prefill encoder on the 5th-generation tensor cores: rotate 128 vectors at a time with
// tcgen05.mma, quantise and bit-pack in the epilogue.
//
//   z[128 tok x 128] = u[128 tok x 128] * R^T          (u = x / |x|, fp32 accuracy)
//
// fp32 accuracy on bf16 tensor cores: both operands are split into three bf16 terms
// (x = x1 + x2 + x3 exactly to 24 bits) and the six products down to 2^-16 relative weight
// are accumulated in the fp32 TMEM accumulator:  x1*r1 + x1*r2 + x2*r1 + x2*r2 + x1*r3 + x3*r1.
// bf16 x bf16 products are exact in fp32, so the only rounding is the accumulation.
//
// One CTA of 16 warps per SM, persistent over 128-vector tiles:
//   * the rotation's three bf16 terms (96 KB, already in the 128-byte-swizzled K-major image
//     the MMA wants) are fetched once with TMA bulk copies onto an mbarrier;
//   * four threads share a vector (warps w, w + 4, w + 8, w + 12 reach the same TMEM lanes), one
//     per quarter of its 128 coordinates: they add up the squared norm through shared memory,
//     each normalises, splits into three bf16 terms and stores its 32 coordinates swizzled into
//     the A tiles (96 KB);
//   * one thread issues 48 tcgen05.mma (M = N = 128, K = 16, kind::f16, bf16 in / fp32 out)
//     into 128 TMEM columns and commits to an mbarrier;
//   * each thread reads its 32 accumulator columns back with one tcgen05.ld, finds the
//     Lloyd-Max bin by binary search ("value equal to a boundary -> lower bin"), builds its
//     quarter of the LSB-first bitstream in registers and writes it.
// Every mbarrier wait is bounded and reports through the device status word.
#include <math.h>
#include <string.h>

#include "tq_common.cuh"

namespace {

constexpr int kTile = 128;                   // vectors per tile; four threads per vector
constexpr int kSplit = 4;
constexpr int kThreads = kSplit * kTile;
constexpr int kTermBytes = kTile * TQ_D * 2;  // one bf16 term of a 128 x 128 operand: 32 KB
constexpr int kSlabBytes = kTile * 128;       // 128 rows x 64 bf16 (one 128-byte swizzle row each): 16 KB
constexpr uint32_t kSpinLimit = 1u << 22;

struct PackTcArgs {
    const void *x;
    int64_t sb, sh, st;
    int B, H, S, pos0;
    uint8_t *codes;
    uint16_t *norms;
    int64_t cache_sb, cache_sh;
    const uint16_t *b_image;   // stage 1 operand: 3 terms x 2 slabs x 16 KB, swizzled (see tq_build_operand_image)
    const uint16_t *b_image2;  // Q_prod: R_k^T image (reconstruction)
    const uint16_t *b_image3;  // Q_prod: S image (QJL projection)
    const float *centers;      // 16 floats (key centres), Q_prod only
    uint8_t *signs;
    uint16_t *rnorms;
    const float *bounds;      // 16 floats, padded with +inf
    int *error_flag;
    int n_tiles;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
// Instruction descriptor: D = f32, A = B = bf16, both K-major, N = 128, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}

// Byte offset of element (row, k) inside one bf16 term image (two 64-wide slabs, 128-B swizzle).
__host__ __device__ inline int operand_offset(int row, int k) {
    const int slab = k >> 6, kk = k & 63;
    return slab * kSlabBytes + (row >> 3) * 1024 + (row & 7) * 128 + (((kk >> 3) ^ (row & 7)) << 4) + (kk & 7) * 2;
}

// (low half of a, low half of b) and (high half of a, high half of b) as one word
__device__ __forceinline__ uint32_t prmt_lo_lo(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x5410); }
__device__ __forceinline__ uint32_t prmt_hi_hi(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x7632); }

__device__ __forceinline__ void split3(float v, __nv_bfloat16 &t1, __nv_bfloat16 &t2, __nv_bfloat16 &t3) {
    t1 = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(t1);
    t2 = __float2bfloat16_rn(r1);
    t3 = __float2bfloat16_rn(r1 - __bfloat162float(t2));
}
// The same split for two values at a time: the conversions are packed (two floats -> one bf16x2),
// the way back to float is a shift / a mask.  Bit-identical to split3 on each value.
__device__ __forceinline__ void split3x2(float v0, float v1, uint32_t &t1, uint32_t &t2, uint32_t &t3) {
    auto pack = [](float lo, float hi) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    };
    t1 = pack(v0, v1);
    const float r0 = v0 - __uint_as_float(t1 << 16), r1 = v1 - __uint_as_float(t1 & 0xffff0000u);
    t2 = pack(r0, r1);
    t3 = pack(r0 - __uint_as_float(t2 << 16), r1 - __uint_as_float(t2 & 0xffff0000u));
}

// Two values rounded through the cache dtype and back (the reference's `.to(dtype).float()`), with
// one packed conversion for both.
template <typename T> __device__ __forceinline__ void round_through2(float &a, float &b);
template <> __device__ __forceinline__ void round_through2<float>(float &, float &) {}
template <> __device__ __forceinline__ void round_through2<__nv_bfloat16>(float &a, float &b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const uint32_t u = *reinterpret_cast<const uint32_t *>(&h);
    a = __uint_as_float(u << 16), b = __uint_as_float(u & 0xffff0000u);
}
template <> __device__ __forceinline__ void round_through2<__half>(float &a, float &b) {
    const float2 f = __half22float2(__floats2half2_rn(a, b));
    a = f.x, b = f.y;
}

template <typename T> struct RowLoader;
template <> struct RowLoader<float> {  // 8 floats = two 16-byte loads
    static __device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    }
};
template <> struct RowLoader<__half> {
    static __device__ __forceinline__ void load8(const __half *p, float (&v)[8]) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(p));
        const __half2 *h = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[2 * i] = __low2float(h[i]), v[2 * i + 1] = __high2float(h[i]);
    }
};
template <> struct RowLoader<__nv_bfloat16> {
    static __device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8]) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(p));
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&a);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[2 * i] = __low2float(h[i]), v[2 * i + 1] = __high2float(h[i]);
    }
};

// 32 consecutive fp32 accumulator columns of this thread's TMEM lane (= its vector).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// QJL = false: Q_mse encode (values, or keys without the sketch): one GEMM per tile.
// QJL = true : Q_prod key encode: three chained GEMMs per tile through the same TMEM columns
//   1. z     = u @ R_k^T                        -> codes (BITS = key bits), norm
//   2. recon = centers[codes] @ R_k             -> residual r = x - round_T(recon * fp16(norm)), |r|
//   3. proj  = (r / |r|) @ S^T                  -> sign bits, fp16 |r|
// The B operand (96 KB) is swapped between the stages with TMA bulk copies that are issued as
// soon as the previous stage's MMAs have completed, so they overlap with the epilogues.
template <typename T, int BITS, bool QJL>
__global__ void __launch_bounds__(kThreads, 1) tq_pack_tc_kernel(PackTcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ float s_bnd[16];
    __shared__ __align__(8) uint2 s_cen3[16];  // the three bf16 terms of a key centre: x = t1 | t2 << 16, y = t3
    __shared__ __align__(8) uint64_t s_bar[2];  // [0] B operand landed, [1] MMAs of a stage done
    __shared__ uint32_t s_tmem;
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
    uint8_t *a_tiles = smem_raw + (base - raw);    // three A terms, then three B terms
    const uint32_t a_addr = base, b_addr = base + 3 * kTermBytes;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int vrow = tid & (kTile - 1);  // this thread's vector within the tile (= its TMEM lane)
    const int hsel = tid >> 7;           // which quarter of the coordinates it works on
    __shared__ float s_sq[kSplit][kTile];  // partial squared norms of the four threads of a vector
    const uint32_t bar_b = smem_u32(&s_bar[0]), bar_mma = smem_u32(&s_bar[1]);
    bool timed_out = false;
    uint32_t b_phase = 0, mma_phase = 0;
    bool b_pending = false;  // thread 0: a B-operand copy has been issued and not yet waited for

    auto load_b = [&](const uint16_t *image) {  // thread 0 only; the B region must be idle
        mbar_expect_tx(bar_b, 3 * kTermBytes);
        for (int i = 0; i < 6; ++i)
            tma_load_1d(b_addr + i * kSlabBytes, reinterpret_cast<const uint8_t *>(image) + i * kSlabBytes, kSlabBytes,
                        bar_b);
        b_pending = true;
    };
    // Everybody has stored its A row: make the stores visible to the tensor core and let thread 0
    // wait for B and issue the 48 MMAs of one GEMM (gemm_issue); later everybody waits for their
    // completion (gemm_wait).  Work that does not touch the operands goes in between.
    auto gemm_issue = [&]() {
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (b_pending) {
                if (!mbar_wait(bar_b, b_phase)) timed_out = true;
                b_phase ^= 1;
                b_pending = false;
            }
            uint32_t acc = 0;
#pragma unroll 1
            for (int s = 0; s < 8; ++s) {
                const uint32_t koff = (s >> 2) * kSlabBytes + (s & 3) * 32;
                const uint64_t a1 = umma_desc(a_addr + koff), a2 = umma_desc(a_addr + kTermBytes + koff),
                               a3 = umma_desc(a_addr + 2 * kTermBytes + koff);
                const uint64_t b1 = umma_desc(b_addr + koff), b2 = umma_desc(b_addr + kTermBytes + koff),
                               b3 = umma_desc(b_addr + 2 * kTermBytes + koff);
                umma_bf16(s_tmem, a1, b3, acc);
                umma_bf16(s_tmem, a3, b1, 1);
                umma_bf16(s_tmem, a2, b2, 1);
                umma_bf16(s_tmem, a1, b2, 1);
                umma_bf16(s_tmem, a2, b1, 1);
                umma_bf16(s_tmem, a1, b1, 1);
                acc = 1;
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar_mma)
                         : "memory");
        }
    };
    auto gemm_wait = [&]() {
        if (!mbar_wait(bar_mma, mma_phase)) timed_out = true;
        mma_phase ^= 1;
        __syncwarp();  // thread 0 took the issue path; tcgen05.ld is warp-collective
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    };

    if (tid < 16) {
        s_bnd[tid] = a.bounds[tid];
        if (QJL) {
            __nv_bfloat16 c1, c2, c3;
            split3(a.centers[tid], c1, c2, c3);
            s_cen3[tid] = make_uint2((uint32_t)__bfloat16_as_ushort(c1) | ((uint32_t)__bfloat16_as_ushort(c2) << 16),
                                     (uint32_t)__bfloat16_as_ushort(c3));
        }
    }
    if (warp == 0) {  // TMEM: 128 columns of fp32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)),
                     "r"(128));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
    }
    if (tid == 0) {
        mbar_init(bar_b, 1);
        mbar_init(bar_mma, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        if ((int)blockIdx.x < a.n_tiles) load_b(a.b_image);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = s_tmem;
    const uint32_t row_tmem = tmem + ((uint32_t)((warp & 3) * 32) << 16);  // column 0 of this thread's lane
    const uint32_t my_tmem = row_tmem + 32 * hsel;                          // its quarter of the columns

    const int64_t n_vec = (int64_t)a.B * a.H * a.S;
    struct RowRef {
        const T *src;
        int64_t row;
        bool valid;
    };
    auto locate = [&](int tile) {  // this thread's vector of a tile: where it comes from, where it goes
        const int64_t vid = (int64_t)tile * kTile + vrow;
        RowRef r;
        r.valid = vid < n_vec;
        const int64_t v2 = r.valid ? vid : 0;
        const int t = (int)(v2 % a.S);
        const int h = (int)((v2 / a.S) % a.H);
        const int b = (int)(v2 / ((int64_t)a.S * a.H));
        r.src = reinterpret_cast<const T *>(a.x) + b * a.sb + h * a.sh + (int64_t)t * a.st;
        r.row = b * a.cache_sb + h * a.cache_sh + a.pos0 + t;
        return r;
    };
    float x[32];  // this thread's quarter of the vector
    float ss = 0.f;
    auto fetch = [&](const RowRef &r) {  // load the quarter, start its squared norm
        ss = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float v[8];
            RowLoader<T>::load8(r.src + 32 * hsel + 8 * c, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[8 * c + i] = v[i], ss = fmaf(v[i], v[i], ss);
        }
    };
    RowRef cur = locate(blockIdx.x);
    if ((int)blockIdx.x < a.n_tiles) fetch(cur);
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
        // ---------------- stage 1: normalise, split, store swizzled.  The rows were loaded while the
        // previous tile's last GEMM ran.
        const bool valid = cur.valid;
        const int64_t row = cur.row;
        const bool more = tile + (int)gridDim.x < a.n_tiles;
        RowRef nxt = cur;
        s_sq[hsel][vrow] = ss;
        __syncthreads();
        const float nrm = sqrtf((s_sq[0][vrow] + s_sq[1][vrow]) + (s_sq[2][vrow] + s_sq[3][vrow]));
        const float safe = nrm > 0.0f ? nrm : 1.0f;
        // x * (1 / n) instead of x / n: at most one ulp from the quotient, i.e. 1e-8 on a unit
        // vector's coordinate, two orders below the 1e-6 band in which a code may differ at all
        const float inv = valid ? 1.0f / safe : 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            __align__(16) uint32_t t1[4], t2[4], t3[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) split3x2(x[8 * c + 2 * i] * inv, x[8 * c + 2 * i + 1] * inv, t1[i], t2[i], t3[i]);
            const int off = operand_offset(vrow, 32 * hsel + 8 * c);
            *reinterpret_cast<uint4 *>(a_tiles + off) = *reinterpret_cast<const uint4 *>(t1);
            *reinterpret_cast<uint4 *>(a_tiles + kTermBytes + off) = *reinterpret_cast<const uint4 *>(t2);
            *reinterpret_cast<uint4 *>(a_tiles + 2 * kTermBytes + off) = *reinterpret_cast<const uint4 *>(t3);
        }
        gemm_issue();
        if (!QJL && more) {  // the row is split and stored: fetch the next tile's under the MMAs
            nxt = locate(tile + (int)gridDim.x);
            fetch(nxt);
        }
        gemm_wait();
        if (QJL && tid == 0) load_b(a.b_image2);  // (a plain Q_mse encode keeps its one operand resident)

        // ---------------- epilogue 1: this thread's accumulator row -> codes
        uint32_t words[BITS + 1];  // this quarter's 32 codes
#pragma unroll
        for (int w = 0; w <= BITS; ++w) words[w] = 0;
        {
            uint32_t r[32];
            tmem_ld32(my_tmem, r);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float z = __uint_as_float(r[i]);
                uint32_t idx = 0;  // number of boundaries strictly below z
#pragma unroll
                for (int stepw = 1 << (BITS - 1); stepw > 0; stepw >>= 1)
                    if (s_bnd[idx + stepw - 1] < z) idx += stepw;
                const int bit = i * BITS, w = bit >> 5, sh = bit & 31;
                words[w] |= idx << sh;
                if (sh + BITS > 32) words[w + 1] |= idx >> (32 - sh);
            }
        }
        const uint16_t nh = tq_float_to_half_bits(safe);
        if (valid) {
            uint32_t *dst = reinterpret_cast<uint32_t *>(a.codes + row * (int64_t)(16 * BITS) + hsel * (4 * BITS));
#pragma unroll
            for (int w = 0; w < BITS; ++w) dst[w] = words[w];
            if (hsel == 0) a.norms[row] = nh;
        }

        if (QJL) {
            // ---------------- stage 2: A = centres[codes] (three bf16 terms from a 2^BITS-entry table)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                __align__(16) uint32_t t1[4], t2[4], t3[4];
                auto code = [&](int e) {  // code of the thread's element e
                    const int bit = e * BITS, w = bit >> 5, sh = bit & 31;
                    uint32_t idx = words[w] >> sh;
                    if (sh + BITS > 32) idx |= words[w + 1] << (32 - sh);
                    return idx & ((1u << BITS) - 1u);
                };
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint2 e0 = s_cen3[code(8 * c + 2 * i)], e1 = s_cen3[code(8 * c + 2 * i + 1)];
                    t1[i] = prmt_lo_lo(e0.x, e1.x), t2[i] = prmt_hi_hi(e0.x, e1.x), t3[i] = prmt_lo_lo(e0.y, e1.y);
                }
                const int off = operand_offset(vrow, 32 * hsel + 8 * c);
                *reinterpret_cast<uint4 *>(a_tiles + off) = *reinterpret_cast<const uint4 *>(t1);
                *reinterpret_cast<uint4 *>(a_tiles + kTermBytes + off) = *reinterpret_cast<const uint4 *>(t2);
                *reinterpret_cast<uint4 *>(a_tiles + 2 * kTermBytes + off) = *reinterpret_cast<const uint4 *>(t3);
            }
            gemm_issue();
            gemm_wait();
            if (tid == 0) load_b(a.b_image3);

            // ---------------- epilogue 2: residual against the dtype-rounded reconstruction
            const float nf = tq_half_bits_to_float(nh);
            float rs = 0.f;
            {
                uint32_t r[32];
                tmem_ld32(my_tmem, r);
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float r0 = __uint_as_float(r[i]) * nf, r1 = __uint_as_float(r[i + 1]) * nf;
                    round_through2<T>(r0, r1);
                    x[i] -= r0, x[i + 1] -= r1;  // x becomes the residual
                    rs = fmaf(x[i], x[i], rs);
                    rs = fmaf(x[i + 1], x[i + 1], rs);
                }
            }
            s_sq[hsel][vrow] = rs;  // (its last readers passed the barrier inside the first GEMM)
            __syncthreads();
            const float rn = sqrtf((s_sq[0][vrow] + s_sq[1][vrow]) + (s_sq[2][vrow] + s_sq[3][vrow]));
            const float rsafe = rn > 0.0f ? rn : 1.0f;
            const float rinv = valid ? 1.0f / rsafe : 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                __align__(16) uint32_t t1[4], t2[4], t3[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) split3x2(x[8 * c + 2 * i] * rinv, x[8 * c + 2 * i + 1] * rinv, t1[i], t2[i], t3[i]);
                const int off = operand_offset(vrow, 32 * hsel + 8 * c);
                *reinterpret_cast<uint4 *>(a_tiles + off) = *reinterpret_cast<const uint4 *>(t1);
                *reinterpret_cast<uint4 *>(a_tiles + kTermBytes + off) = *reinterpret_cast<const uint4 *>(t2);
                *reinterpret_cast<uint4 *>(a_tiles + 2 * kTermBytes + off) = *reinterpret_cast<const uint4 *>(t3);
            }
            // ---------------- stage 3: projection, sign bits
            gemm_issue();
            if (more) {  // the residual is split and stored: fetch the next tile's rows under the MMAs
                nxt = locate(tile + (int)gridDim.x);
                fetch(nxt);
            }
            gemm_wait();
            if (tid == 0 && more) load_b(a.b_image);
            uint32_t sg = 0u;
            {
                uint32_t r[32];
                tmem_ld32(my_tmem, r);
#pragma unroll
                for (int i = 0; i < 32; ++i) sg |= (__uint_as_float(r[i]) >= 0.0f ? 1u : 0u) << i;
            }
            if (valid) {
                *reinterpret_cast<uint32_t *>(a.signs + row * 16 + 4 * hsel) = sg;
                if (hsel == 0) a.rnorms[row] = tq_float_to_half_bits(rsafe);
            }
        }
        cur = nxt;
        // every accumulator row is read before the next GEMM overwrites the columns
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();
    }
    if (timed_out) atomicExch(a.error_flag, 3);
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(128));
    }
}

inline uint16_t host_bf16_rn(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    const uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}
inline float host_bf16_to_float(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float v;
    memcpy(&v, &u, 4);
    return v;
}

}  // namespace

// Host: the 96 KB shared-memory image of a [128 x 128] K-major operand `m[row][k]` split into
// three bf16 terms, each stored as two 64-wide slabs with the 128-byte swizzle.
void tq_build_operand_image(const float *m, uint16_t *image) {
    for (int row = 0; row < TQ_D; ++row)
        for (int k = 0; k < TQ_D; ++k) {
            const float v = m[(size_t)row * TQ_D + k];
            const uint16_t t1 = host_bf16_rn(v);
            const float r1 = v - host_bf16_to_float(t1);
            const uint16_t t2 = host_bf16_rn(r1);
            const uint16_t t3 = host_bf16_rn(r1 - host_bf16_to_float(t2));
            const int off = operand_offset(row, k) / 2;
            image[off] = t1;
            image[kTermBytes / 2 + off] = t2;
            image[2 * (kTermBytes / 2) + off] = t3;
        }
}

template <typename T, int BITS, bool QJL>
static cudaError_t launch_tc(const PackTcArgs &a, int grid, int device, cudaStream_t stream) {
    const int smem = 6 * kTermBytes + 1024;
    // the attribute belongs to the (kernel, device) pair: one flag per device of this instantiation
    static bool configured[TQ_MAX_DEVICES] = {};
    if (device < 0 || device >= TQ_MAX_DEVICES) return cudaErrorInvalidDevice;
    if (!configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(tq_pack_tc_kernel<T, BITS, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured[device] = true;
    }
    tq_pack_tc_kernel<T, BITS, QJL><<<grid, kThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

// Encode one dense tensor on the tensor cores: values (which == 1, Q_mse) or keys (which == 0,
// Q_mse or, when the context uses QJL, Q_prod with sign sketch and residual norms).  Returns
// TQ_ERR_UNSUPPORTED when the tensor's alignment rules it out.
int32_t tq_launch_pack_tc(tq_ctx *ctx, const tq_dense_desc *x, int which, int32_t n_tokens,
                          const tq_cache_desc *cache, int32_t pos0, cudaStream_t stream) {
    const int esize = x->dtype == TQ_DTYPE_F32 ? 4 : 2;
    if (((uintptr_t)x->data & 15) || ((x->stride_b * esize) & 15) || ((x->stride_h * esize) & 15) ||
        ((x->stride_t * esize) & 15))
        return TQ_ERR_UNSUPPORTED;
    PackTcArgs a;
    a.x = x->data, a.sb = x->stride_b, a.sh = x->stride_h, a.st = x->stride_t;
    a.B = cache->batch, a.H = cache->kv_heads, a.S = n_tokens, a.pos0 = pos0;
    a.codes = which == 0 ? cache->k_codes : cache->v_codes;
    a.norms = which == 0 ? cache->k_norms : cache->v_norms;
    a.cache_sb = cache->stride_b, a.cache_sh = cache->stride_h;
    a.b_image = which == 0 ? ctx->img_rot_k : ctx->img_rot_v;
    a.bounds = which == 0 ? ctx->bounds_k : ctx->bounds_v;
    a.error_flag = ctx->error_flag;
    a.b_image2 = ctx->img_rot_kt, a.b_image3 = ctx->img_qjl;
    a.centers = ctx->centers_k;
    a.signs = cache->k_signs, a.rnorms = cache->k_rnorms;
    const bool qjl = which == 0 && ctx->use_qjl;
    const int bits = which == 0 ? ctx->key_bits : ctx->bits;
    const int64_t n_vec = (int64_t)a.B * a.H * a.S;
    a.n_tiles = (int)((n_vec + kTile - 1) / kTile);
    const int grid = a.n_tiles < ctx->sm_count ? a.n_tiles : ctx->sm_count;
    cudaError_t e = cudaErrorInvalidValue;
#define TQ_TC_CASE(T)                                                                                     \
    switch (bits) {                                                                                       \
        case 1: e = qjl ? launch_tc<T, 1, true>(a, grid, ctx->device, stream) : cudaErrorInvalidValue; break;          \
        case 2: e = qjl ? launch_tc<T, 2, true>(a, grid, ctx->device, stream) : launch_tc<T, 2, false>(a, grid, ctx->device, stream); break; \
        case 3: e = qjl ? launch_tc<T, 3, true>(a, grid, ctx->device, stream) : launch_tc<T, 3, false>(a, grid, ctx->device, stream); break; \
        case 4: e = qjl ? cudaErrorInvalidValue : launch_tc<T, 4, false>(a, grid, ctx->device, stream); break;         \
        default: return TQ_ERR_UNSUPPORTED;                                                               \
    }
    if (x->dtype == TQ_DTYPE_F32) {
        TQ_TC_CASE(float)
    } else if (x->dtype == TQ_DTYPE_F16) {
        TQ_TC_CASE(__half)
    } else {
        TQ_TC_CASE(__nv_bfloat16)
    }
#undef TQ_TC_CASE
    tq_prof_count(ctx, 1);
    TQ_CUDA_CHECK(e);
    return TQ_OK;
}
