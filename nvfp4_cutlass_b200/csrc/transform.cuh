// Algorithm 1 on the device: one BF16 block of 16 elements -> a most-significant
// NVFP4 pass (q0, s0) and a x8 residual NVFP4 pass (q1, s1), bit-exact with the
// reference's CPU emulation (tests/python/reference/dual_nvfp4.py:123-158 there),
// plus the shared-memory addressing of everything the transform reads and writes.
//
// Exactness.  The emulation divides: u = x / s0 in FP32, q0 = RNE_e2m1(u),
// q1 = RNE_e2m1((u - q0) * 8).  A single multiply by a rounded reciprocal breaks
// exact ties (x = midpoint * s0), which are common because BF16 inputs and E4M3
// scales carry few significant bits.  Here the reciprocal is carried as an
// unevaluated sum r_hi + r_lo (r_lo = r_hi * (1 - s0 * r_hi), the residual formed
// exactly by one FMA) and u = fma(x, r_hi, x * r_lo).  The pre-rounding error is
// ~2^-46 relative while a quotient of an 8-bit by a 4-bit significand is either
// exactly representable or at least 2^-17 away from any rounding threshold, so u
// rounds like the true quotient wherever a code depends on it.  This holds for any
// r_hi within a few ulp of 1/s0 (checked exhaustively over all BF16 x and all E4M3
// s0, with r_hi perturbed by +-2 ulp), so the approximate reciprocal is enough.
#pragma once
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace nvfp4::xform {

// The reference kernel's four activation scale policies (include/nvfp4_gemm/transform/dual_nvfp4.cuh:31-61 there).
enum ScalePolicy : int { kDerivedDiv8 = 0, kResidualAmax = 1, kDerivedDiv4 = 2, kDiv4Radix8 = 3 };

// ---- shared-memory addressing ----------------------------------------------------
// BF16 activation tile as TMA lands it: boxes of 64 columns (128 B rows) x kRows,
// 128-byte swizzle: 16-byte chunk index ^= row % 8.
template <uint32_t kRows>
NVFP4_DEVICE uint32_t a_bf16_offset(uint32_t row, uint32_t k)   // byte offset of element (row, k), k % 8 == 0
{
    const uint32_t box = k >> 6;
    const uint32_t chunk = ((k & 63u) >> 3) ^ (row & 7u);
    return box * (kRows * 128u) + row * 128u + (chunk << 4);
}
// Packed-FP4 operand tile, K-major, one swizzle span per row: 64-byte rows (128 K
// elements) under the 64-byte swizzle, 16-byte chunk index ^= (row / 2) % 4; 128-byte
// rows (256 K elements) under the 128-byte swizzle, chunk index ^= row % 8.  The same
// function serves the TMA-written weights and the A0 / A1 tiles the transform writes,
// which is what the MMA descriptors assume.
template <uint32_t kBK, uint32_t kSubRows = 0>
NVFP4_DEVICE uint32_t fp4_offset(uint32_t row, uint32_t k)   // byte offset of element (row, k), k % 32 == 0
{
    static_assert(kBK == 128 || kBK == 256 || kBK == 512, "one or two swizzle spans per row");
    if constexpr (kBK == 128) return row * 64u + (((k >> 5) ^ ((row >> 1) & 3u)) << 4);
    else if constexpr (kBK == 256) return row * 128u + (((k >> 5) ^ (row & 7u)) << 4);
    else {
        // 512 K elements = two 128-byte-swizzled sub-tiles of kSubRows rows each, side by side along K
        static_assert(kSubRows > 0, "sub-tile height");
        return (k >> 8) * (kSubRows * 128u) + row * 128u + ((((k & 255u) >> 5) ^ (row & 7u)) << 4);
    }
}
NVFP4_DEVICE uint32_t fp4_sw64_offset(uint32_t row, uint32_t k) { return fp4_offset<128>(row, k); }
// Scale-factor atom (128 rows x four 16-blocks = 64 K elements) in the order the
// 32x128b.warpx4 tensor-memory copy wants: row r at word (r % 32) * 4 + r / 32,
// byte j of the word = 16-block j.
NVFP4_DEVICE uint32_t sf_word_offset(uint32_t row) { return (((row & 31u) << 2) + (row >> 5)) << 2; }
// Byte offset of the scale word of (64-K atom, row) in a run of 512-byte atoms.  An operand
// of R <= 128 rows uses only kCols = ceil(R / 32) of the four words of each 16-byte unit,
// so 4 / kCols consecutive K atoms are packed side by side into one 512-byte atom: one
// tensor-memory copy then brings the scales of several K atoms at once, and the MMA of K
// atom a reads them at column (a / per) * 4 + (a % per) * kCols of the scale region.
template <uint32_t kCols>
NVFP4_DEVICE uint32_t sf_atom_offset(uint32_t atom, uint32_t row)
{
    static_assert(kCols == 1 || kCols == 2 || kCols == 4, "columns per K atom");
    constexpr uint32_t per = 4u / kCols;
    return (atom / per) * 512u + ((row & 31u) << 4) + (((atom % per) * kCols + (row >> 5)) << 2);
}

// ---- Algorithm 1 on one 16-element block -------------------------------------------
struct Block16 {
    uint32_t q0[2];   // 16 E2M1 codes, element 0 in the lowest nibble of q0[0]
    uint32_t q1[2];
    uint32_t s0;      // E4M3 byte
    uint32_t s1;
};

// E4M3 byte -> FP32, subnormals included (only the residual_amax policy can produce them)
NVFP4_DEVICE float e4m3_to_f32(uint32_t c)
{
    return c < 8u ? static_cast<float>(c) * 0.001953125f : __uint_as_float((c << 20) + 0x3C000000u);
}

// kPolicy 0 = derived_div8: s1 = Q_e4m3(s0 / 8), q1 = Q((u - q0) * 8), s0 floored at 2^-6.
// kPolicy 1 = residual_amax: r = x - q0 * s0 (exact in FP32), s1 = Q_e4m3(max(amax(r) / 6, 2^-9)), q1 = Q(r / s1),
//             s0 floored at 2^-9 (tests/python/reference/dual_nvfp4.py:131-152 of the reference).
// kPolicy 2 = derived_div4: as 0 with radix 4 (s1 = Q_e4m3(s0 / 4), q1 = Q((u - q0) * 4)): the residual never clips.
// kPolicy 3 = div4_radix8: s0 = Q_e4m3(max(amax / 4, 2^-6)) so that q0 stays on the |u| <= 4 half of the E2M1 grid,
//             radix 8 (include/nvfp4_gemm/transform/dual_nvfp4.cuh:31-61 of the reference; these two exist only in
//             its kernel, so the CPU statement they are checked against follows the emulation's operation order with
//             these constants).
template <bool kResidual, int kPolicy = 0>
NVFP4_DEVICE void decompose_block16(const uint32_t (&w)[8], Block16& out)
{
    static_assert(kPolicy >= 0 && kPolicy <= 3, "scale policy");
    constexpr bool kAmax2 = kPolicy == 1;                     // second amax over the residual
    constexpr float kS0Mul = kPolicy == 3 ? 0.25f : 0.16666667163372040f;
    constexpr float kS1Mul = kPolicy == 2 ? 0.25f : 0.125f;
    constexpr float kRadix = kPolicy == 2 ? 4.0f : 8.0f;
    constexpr unsigned short kNegRadixF16 = kPolicy == 2 ? 0xC400u : 0xC800u;
    // block amax over 16 BF16 values (pairs packed low = even element)
    uint32_t m0 = ptx::max_abs_bf16x2(w[0], w[1]);
    uint32_t m1 = ptx::max_abs_bf16x2(w[2], w[3]);
    uint32_t m2 = ptx::max_abs_bf16x2(w[4], w[5]);
    uint32_t m3 = ptx::max_abs_bf16x2(w[6], w[7]);
    m0 = ptx::max_abs_bf16x2(m0, m1);
    m2 = ptx::max_abs_bf16x2(m2, m3);
    m0 = ptx::max_abs_bf16x2(m0, m2);
    m0 = ptx::max_abs_bf16x2(m0, m0 >> 16);
    const float amax = __uint_as_float((m0 & 0x7fffu) << 16);

    // s0 = Q_e4m3(max(amax * fl(1/6), floor)); with the 2^-6 floor always a normal E4M3 value
    const float s0_pre = fmaxf(__fmul_rn(amax, kS0Mul), kAmax2 ? 0.001953125f : 0.015625f);
    const uint32_t s0c = ptx::cvt_e4m3(s0_pre);
    const float s0 = kAmax2 ? e4m3_to_f32(s0c) : __uint_as_float((s0c << 20) + 0x3C000000u);
    out.s0 = s0c;
    out.s1 = kAmax2 ? 0u : ptx::cvt_e4m3(__fmul_rn(s0, kS1Mul));

    // u = x / s0 as the correctly rounded quotient: r_hi ~ 1 / s0, r_lo = its error term formed exactly by one FMA
    const float r_hi = ptx::rcp_approx(s0);
    const float r_lo = __fmul_rn(__fmaf_rn(-s0, r_hi, 1.0f), r_hi);

    float u[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float x0 = __uint_as_float(w[i] << 16);
        const float x1 = __uint_as_float(w[i] & 0xffff0000u);
        u[2 * i] = __fmaf_rn(x0, r_hi, __fmul_rn(x0, r_lo));
        u[2 * i + 1] = __fmaf_rn(x1, r_hi, __fmul_rn(x1, r_lo));
    }
    out.q0[0] = ptx::cvt_e2m1x8(u[0], u[1], u[2], u[3], u[4], u[5], u[6], u[7]);
    out.q0[1] = ptx::cvt_e2m1x8(u[8], u[9], u[10], u[11], u[12], u[13], u[14], u[15]);

    if constexpr (kResidual && kAmax2) {
        // r = x - dec(q0) * s0: the product has at most 7 significant bits and x has 8, so the FMA is exact;
        // dec(q0) comes back as FP16 and s0 (>= 2^-9) is an FP16 value too
        const unsigned short neg_s0 = __half_as_ushort(__float2half_rn(-s0));
        float r[16];
        float rmax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t byte = (out.q0[i >> 2] >> (8 * (i & 3))) & 0xffu;
            const uint32_t d = ptx::cvt_e2m1x2_to_f16x2(byte);
            r[2 * i] = ptx::fma_f32_f16(static_cast<unsigned short>(d & 0xffffu), neg_s0, __uint_as_float(w[i] << 16));
            r[2 * i + 1] = ptx::fma_f32_f16(static_cast<unsigned short>(d >> 16), neg_s0, __uint_as_float(w[i] & 0xffff0000u));
            rmax = fmaxf(rmax, fmaxf(fabsf(r[2 * i]), fabsf(r[2 * i + 1])));
        }
        const uint32_t s1c = ptx::cvt_e4m3(fmaxf(__fmul_rn(rmax, 0.16666667163372040f), 0.001953125f));
        const float s1 = e4m3_to_f32(s1c);
        out.s1 = s1c;
        // q1 = Q(r / s1), the quotient correctly rounded as for u
        const float t_hi = ptx::rcp_approx(s1);
        const float t_lo = __fmul_rn(__fmaf_rn(-s1, t_hi, 1.0f), t_hi);
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = __fmaf_rn(r[i], t_hi, __fmul_rn(r[i], t_lo));
        out.q1[0] = ptx::cvt_e2m1x8(r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7]);
        out.q1[1] = ptx::cvt_e2m1x8(r[8], r[9], r[10], r[11], r[12], r[13], r[14], r[15]);
    } else if constexpr (kResidual) {
        // r = (u - dec(q0)) * radix = radix * u + dec(q0) * (-radix): exact, the decode comes back as FP16
        float r[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t byte = (out.q0[i >> 2] >> (8 * (i & 3))) & 0xffu;
            const uint32_t d = ptx::cvt_e2m1x2_to_f16x2(byte);
            r[2 * i] = ptx::fma_f32_f16(static_cast<unsigned short>(d & 0xffffu), kNegRadixF16, __fmul_rn(u[2 * i], kRadix));
            r[2 * i + 1] = ptx::fma_f32_f16(static_cast<unsigned short>(d >> 16), kNegRadixF16, __fmul_rn(u[2 * i + 1], kRadix));
        }
        out.q1[0] = ptx::cvt_e2m1x8(r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7]);
        out.q1[1] = ptx::cvt_e2m1x8(r[8], r[9], r[10], r[11], r[12], r[13], r[14], r[15]);
    } else {
        out.q1[0] = out.q1[1] = 0u;
    }
}

// ---- one activation tile ------------------------------------------------------------
// kRows x kBK BF16 -> A0 / A1 (packed FP4, one swizzle span per row) and the SFA0 / SFA1
// atoms (one 512-byte atom per 64 K elements; rows past kRows of an atom are left
// untouched).  kThreads threads cooperate, t = 0..kThreads-1.  Thread t owns row
// t % kRows and a run of consecutive 16-blocks in it: lanes walk consecutive rows, which
// keeps the 128-bit shared-memory accesses free of bank conflicts under both swizzles and
// makes every thread's global read one contiguous run of whole cache lines.
//
// The work is split in two so that callers can overlap: `load_*` brings a thread's share
// into registers (from a TMA-landed shared-memory tile, or straight from global memory),
// `emit_tile` runs Algorithm 1 on the registers and writes the products.
template <uint32_t kRows, uint32_t kBK, uint32_t kThreads>
struct TileShare {
    static constexpr uint32_t kBlocks = kRows * (kBK / 16u);
    static constexpr uint32_t kActive = kThreads < kBlocks ? kThreads : kBlocks;   // surplus threads idle
    static constexpr uint32_t kBlocksPerThread = kBlocks / kActive;
    static_assert(kBlocksPerThread * kActive == kBlocks, "threads must tile the blocks");
    static_assert(kBlocksPerThread == 1 || kBlocksPerThread == 2 || kBlocksPerThread == 4 || kBlocksPerThread == 8,
                  "unsupported split");
    static_assert(kRows % 16 == 0 && kRows <= 128 && kActive % kRows == 0, "row count");
    uint32_t w[kBlocksPerThread][8];
};

// From the tile as TMA landed it at `a_smem` (boxes of 64 columns, 128-byte swizzle).
template <uint32_t kRows, uint32_t kBK, uint32_t kThreads>
NVFP4_DEVICE void load_tile_smem(TileShare<kRows, kBK, kThreads>& s, uint32_t a_smem, uint32_t t)
{
    using S = TileShare<kRows, kBK, kThreads>;
    if (t >= S::kActive) return;
    const uint32_t row = t % kRows, first_block = (t / kRows) * S::kBlocksPerThread;
#pragma unroll
    for (uint32_t j = 0; j < S::kBlocksPerThread; ++j) {
        const uint32_t k = (first_block + j) * 16u;
        const uint4 lo = ptx::lds128(a_smem + a_bf16_offset<kRows>(row, k));
        const uint4 hi = ptx::lds128(a_smem + a_bf16_offset<kRows>(row, k + 8));
        s.w[j][0] = lo.x; s.w[j][1] = lo.y; s.w[j][2] = lo.z; s.w[j][3] = lo.w;
        s.w[j][4] = hi.x; s.w[j][5] = hi.y; s.w[j][6] = hi.z; s.w[j][7] = hi.w;
    }
}

// Straight from global memory: `tile` points at element (first row of the tile, first K of
// the block); rows are `lda` elements apart.  Read-only, streaming (no L1 allocation: the
// reuse of an activation tile is across CTAs, through L2).
template <uint32_t kRows, uint32_t kBK, uint32_t kThreads>
NVFP4_DEVICE void load_tile_global(TileShare<kRows, kBK, kThreads>& s, const void* tile, int64_t lda, uint32_t t)
{
    using S = TileShare<kRows, kBK, kThreads>;
    if (t >= S::kActive) return;
    const uint32_t row = t % kRows, first_block = (t / kRows) * S::kBlocksPerThread;
    const char* src = static_cast<const char*>(tile) + (static_cast<int64_t>(row) * lda + first_block * 16) * 2;
#pragma unroll
    for (uint32_t j = 0; j < S::kBlocksPerThread; ++j) {
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h)
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(s.w[j][4 * h]), "=r"(s.w[j][4 * h + 1]), "=r"(s.w[j][4 * h + 2]), "=r"(s.w[j][4 * h + 3])
                         : "l"(src + j * 32 + h * 16));
    }
}

template <uint32_t kRows, uint32_t kBK, uint32_t kThreads, bool kResidual, uint32_t kSfCols = 4, uint32_t kSubRows = 0,
          int kPolicy = 0>
NVFP4_DEVICE void emit_tile(const TileShare<kRows, kBK, kThreads>& s, uint32_t a0_smem, uint32_t a1_smem,
                            uint32_t sfa0_smem, uint32_t sfa1_smem, uint32_t t)
{
    using S = TileShare<kRows, kBK, kThreads>;
    constexpr uint32_t kBlocksPerThread = S::kBlocksPerThread;
    if (t >= S::kActive) return;
    const uint32_t row = t % kRows, first_block = (t / kRows) * kBlocksPerThread;

    if constexpr (kBlocksPerThread == 1) {
        Block16 blk;
        decompose_block16<kResidual, kPolicy>(s.w[0], blk);
        const uint32_t off = fp4_offset<kBK, kSubRows>(row, (first_block * 16u) & ~31u) + ((first_block & 1u) << 3);
        ptx::sts64(a0_smem + off, blk.q0[0], blk.q0[1]);
        if constexpr (kResidual) ptx::sts64(a1_smem + off, blk.q1[0], blk.q1[1]);
        const uint32_t addr = sf_atom_offset<kSfCols>(first_block >> 2, row) + (first_block & 3u);
        ptx::sts8(sfa0_smem + addr, blk.s0);
        if constexpr (kResidual) ptx::sts8(sfa1_smem + addr, blk.s1);
    } else {
        uint32_t sf0 = 0, sf1 = 0;
#pragma unroll
        for (uint32_t pair = 0; pair < kBlocksPerThread / 2; ++pair) {
            Block16 blk[2];
            decompose_block16<kResidual, kPolicy>(s.w[pair * 2], blk[0]);
            decompose_block16<kResidual, kPolicy>(s.w[pair * 2 + 1], blk[1]);
            // two blocks = 32 elements = one 16-byte chunk of each packed row
            const uint32_t off = fp4_offset<kBK, kSubRows>(row, (first_block + pair * 2) * 16u);
            ptx::sts128(a0_smem + off, blk[0].q0[0], blk[0].q0[1], blk[1].q0[0], blk[1].q0[1]);
            if constexpr (kResidual)
                ptx::sts128(a1_smem + off, blk[0].q1[0], blk[0].q1[1], blk[1].q1[0], blk[1].q1[1]);
            const uint32_t shift = ((pair * 2) & 3u) * 8u;
            sf0 |= (blk[0].s0 | (blk[1].s0 << 8)) << shift;
            sf1 |= (blk[0].s1 | (blk[1].s1 << 8)) << shift;
            // flush a scale word (or half word) whenever this thread's share of a K atom is complete
            if constexpr (kBlocksPerThread == 2) {
                const uint32_t addr = sf_atom_offset<kSfCols>(first_block >> 2, row) + (first_block & 2u);
                ptx::sts16(sfa0_smem + addr, sf0);
                if constexpr (kResidual) ptx::sts16(sfa1_smem + addr, sf1);
            } else if ((pair & 1u) == 1u) {
                const uint32_t addr = sf_atom_offset<kSfCols>((first_block + pair * 2) >> 2, row);
                ptx::sts32(sfa0_smem + addr, sf0);
                if constexpr (kResidual) ptx::sts32(sfa1_smem + addr, sf1);
                sf0 = sf1 = 0;
            }
        }
    }
}

// Shared-memory tile in, products out; `on_loaded()` runs between the reads and the
// arithmetic (the caller releases the BF16 slot there).
template <uint32_t kRows, uint32_t kBK, uint32_t kThreads, bool kResidual, uint32_t kSfCols = 4, uint32_t kSubRows = 0,
          int kPolicy = 0, typename OnLoaded>
NVFP4_DEVICE void transform_tile(uint32_t a_smem, uint32_t a0_smem, uint32_t a1_smem, uint32_t sfa0_smem,
                                 uint32_t sfa1_smem, uint32_t t, OnLoaded&& on_loaded)
{
    TileShare<kRows, kBK, kThreads> s;
    load_tile_smem(s, a_smem, t);
    on_loaded();
    emit_tile<kRows, kBK, kThreads, kResidual, kSfCols, kSubRows, kPolicy>(s, a0_smem, a1_smem, sfa0_smem, sfa1_smem, t);
}

}  // namespace nvfp4::xform
