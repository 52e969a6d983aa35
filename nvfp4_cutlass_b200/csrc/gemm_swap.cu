// Grouped dual-NVFP4 GEMM, decode orientation ("swap-AB"): 128 weight rows on the
// MMA M axis, a small token tile (16 / 32 / 64 rows) on the MMA N axis.
//
// In this regime every expert sees a handful of tokens, so the job is to stream
// each active expert's FP4 weights from HBM exactly once at full bandwidth: a deep
// TMA ring of weight tiles (128 rows x 256 K = 16 KB + 2 KB of scales per slot) feeds
// tiny MMAs, while the token tile of the same K block is transformed by Algorithm 1
// into the MMA's B operand.  Two accumulator stages in tensor memory let the
// epilogue of one tile overlap the mainloop of the next.
//
//   W ring  (FP4 weights + their scales)   TMA warp        -> scale warps, MMA warp
//   A ring  (BF16 token rows)              TMA warp        -> transform warps
//   P ring  (A0, A1, SFT0, SFT1)           transform warps -> scale warps, MMA warp
//
// Scale factors go from shared to tensor memory through tcgen05.st issued by four scale warps, not
// through tensor-memory copies issued by the MMA thread.
//
// Counterpart in the reference: include/nvfp4_gemm/impls/sm100_bf16_dual_nvfp4_gemm_swap_ab.cuh,
// epilogue/sm100_store_cd_swap_ab.cuh, src/kernels/sm100_bf16_dual_nvfp4_gemm.hpp:489-632.
#include <cuda_bf16.h>

#include "host_common.hpp"
#include "launchers.hpp"
#include "transform.cuh"

namespace nvfp4 {
namespace {

constexpr uint32_t BW = 128;                         // weight rows per tile (MMA M)
constexpr uint32_t kWarpTma = 0, kWarpMma = 1, kWarpTmaA = 3, kWarpEpi0 = 4, kNumEpiWarps = 4, kWarpXform0 = 8;
constexpr uint32_t kXformWarps = 8, kXformThreads = kXformWarps * 32;
constexpr uint32_t kWarpSf0 = kWarpXform0 + kXformWarps, kNumSfWarps = 4;      // one scale warp per TMEM lane quadrant
constexpr uint32_t kThreads = (kWarpSf0 + kNumSfWarps) * 32;                 // 640
constexpr uint32_t kSmemBudget = 232448 - 1024;      // opt-in maximum minus alignment slack

// With the residual pass on, A0 and A1 of a token tile are stacked along the MMA N axis
// (rows [0, T) = A0, rows [T, 2T) = A1, scales likewise in one atom): one MMA of N = 2T
// per 64-K atom computes both passes into two column groups that the epilogue adds.  An
// MMA of N <= 128 costs the same issue time whatever N is, and the stacked scales need one
// tensor-memory copy instead of two, so the per-K-block issue cost almost halves.
template <uint32_t T, uint32_t BK, bool kResidual>
struct Cfg {
    static constexpr uint32_t kAtoms = BK / 64;
    static constexpr uint32_t kRowsP = kResidual ? 2 * T : T;             // rows of the stacked operand tile
    static constexpr uint32_t kRowBytes = BK >= 256 ? 128 : BK / 2;       // one swizzle span; BK = 512 is two sub-tiles
    static constexpr uint32_t kSubW = BW * kRowBytes, kSubP = kRowsP * kRowBytes;   // bytes of one sub-tile
    static constexpr uint32_t kSlotW = BW * BK / 2, kSlotSFW = kAtoms * 512;
    static constexpr uint32_t kSlotA = T * BK * 2;
    static constexpr uint32_t kSlotP = (kRowsP * BK / 2 + 1023u) & ~1023u;
    // token scales: one 512-byte atom and one tensor-memory copy per K atom.  (Packing the scales of several
    // K atoms side by side into one atom, with the MMA reading them at a column that is not a multiple of
    // four, raised a CUDA error on B200: the scale address of the MMA has to stay 4-column aligned.)
    static constexpr uint32_t kSfCols = 4, kAtomsPerCp = 4 / kSfCols;
    static constexpr uint32_t kNumSftCp = (kAtoms + kAtomsPerCp - 1) / kAtomsPerCp, kSlotSFT = kNumSftCp * 512;
    static constexpr uint32_t kA1Bytes = T * kRowBytes;                    // A1 rows start T rows below A0 (in every sub-tile)
    static constexpr uint32_t kSF1Bytes = T == 16 ? 256 : (T / 32) * 4;    // scale word of row T + r relative to row r
    static constexpr uint32_t kDepthA = BK == 512 ? (T == 16 ? 3 : 2) : (T >= 64 ? 3 : (T == 32 ? 5 : 6));   // covers the TMA latency
    static constexpr uint32_t kDepthP = BK == 512 ? 2 : 3;
    static constexpr uint32_t kFixed = kDepthA * kSlotA + kDepthP * (kSlotP + kSlotSFT) + 512;
    static constexpr uint32_t kDepthWRaw = (kSmemBudget - kFixed) / (kSlotW + kSlotSFW);
    static constexpr uint32_t kDepthW = kDepthWRaw > 12 ? 12 : kDepthWRaw;
    static constexpr uint32_t kOffW = 0;
    static constexpr uint32_t kOffA = kOffW + kDepthW * kSlotW;
    static constexpr uint32_t kOffP = kOffA + kDepthA * kSlotA;
    static constexpr uint32_t kOffSFW = kOffP + kDepthP * kSlotP;
    static constexpr uint32_t kOffSFT = kOffSFW + kDepthW * kSlotSFW;
    static constexpr uint32_t kOffBars = kOffSFT + kDepthP * kSlotSFT;
    static constexpr uint32_t kNumBars = 2 * kDepthW + 2 * kDepthA + kDepthP + 4 + 2;
    static constexpr uint32_t kSmemAlloc = kOffBars + kNumBars * 8 + 16 + 1024;
    static_assert(kDepthW >= 3, "weight ring too shallow");
    static_assert(kSmemAlloc <= 232448, "shared memory budget");
    // tensor memory: two accumulator stages of kRowsP columns, then the two scale groups
    static constexpr uint32_t kAccStride = kRowsP < 32 ? 32 : kRowsP;
    // then two alternating buffers of scale columns: weight scales (4 per K atom), token scales (4 per K atom)
    static constexpr uint32_t kColSF = 2 * kAccStride, kSfBufCols = 8 * kAtoms, kSfW = 0, kSfT = 4 * kAtoms;
    static constexpr uint32_t kColsUsed = kColSF + 2 * kSfBufCols;
    static constexpr uint32_t kTmemCols = kColsUsed <= 64 ? 64 : (kColsUsed <= 128 ? 128 : (kColsUsed <= 256 ? 256 : 512));
    static constexpr uint64_t kSwizzle = BK >= 256 ? ptx::kSwizzle128B : ptx::kSwizzle64B;
    static constexpr uint32_t kSBO = 8 * kRowBytes;  // eight rows of one swizzle span
};

struct Params {
    const float* gw;
    const int32_t* m_indices;
    __nv_bfloat16* d;
    int64_t ldd;
    uint32_t m, n, k;
    int32_t* status;
};

struct Ring {
    uint32_t slot = 0, phase = 0;
    template <uint32_t kDepth>
    __device__ __forceinline__ void advance()
    {
        if (++slot == kDepth) { slot = 0; phase ^= 1; }
    }
};

template <uint32_t T, uint32_t BK, bool kResidual, int kPolicy>
__global__ void __launch_bounds__(kThreads, 1)
gemm_swap_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                 const __grid_constant__ CUtensorMap tm_sfw, const Params p)
{
    using C = Cfg<T, BK, kResidual>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem - ptx::smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kOffBars);
    uint64_t* w_full = bars;
    uint64_t* w_empty = w_full + C::kDepthW;
    uint64_t* a_full = w_empty + C::kDepthW;
    uint64_t* a_empty = a_full + C::kDepthA;
    uint64_t* p_full = a_empty + C::kDepthA;
    uint64_t* sf_full = p_full + C::kDepthP;         // [2]: scales of a K block are in tensor memory
    uint64_t* tmem_full = sf_full + 2;               // [2]
    uint64_t* tmem_empty = tmem_full + 2;            // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < C::kDepthW; ++i) {
            ptx::mbar_init(w_full + i, 1);
            ptx::mbar_init(w_empty + i, 1);
        }
        for (uint32_t i = 0; i < C::kDepthA; ++i) { ptx::mbar_init(a_full + i, 1); ptx::mbar_init(a_empty + i, kXformWarps); }
        for (uint32_t i = 0; i < C::kDepthP; ++i) ptx::mbar_init(p_full + i, kXformWarps);
        for (uint32_t i = 0; i < 2; ++i) {
            ptx::mbar_init(tmem_full + i, 1);
            ptx::mbar_init(tmem_empty + i, kNumEpiWarps);
            ptx::mbar_init(sf_full + i, kNumSfWarps);
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tm_a);
        ptx::prefetch_tensormap(&tm_w);
        ptx::prefetch_tensormap(&tm_sfw);
    }
    if (warp == kWarpMma) ptx::tmem_alloc<C::kTmemCols>(tmem_slot);
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // launched with programmatic stream serialisation, the prologue above overlapped the tail of the previous
    // kernel of the stream; its results are visible from here on
    ptx::grid_dependency_wait();

    // tiles: all weight-row blocks of one token block are neighbours, so the CTAs of a
    // wave share that token block's activations through L2 while streaming disjoint weights
    const long long probe_start = ptx::probe_clock();
    const uint32_t num_n = p.n / BW, num_kb = p.k / BK;
    const uint32_t num_tiles = (p.m / T) * num_n;
    bool ok = true;
    ptx::ProbeAcc pa;
    auto give_up = [&](uint32_t code) {
        *abort_flag = 1;
        if (p.status != nullptr) atomicOr(p.status, static_cast<int32_t>(code));
        ok = false;
    };

    if (warp == kWarpTma) {
        // weight producer: runs ahead by the full depth of the W ring, whatever the transform does
        if (lane == 0) {
            Ring rw;
            const uint64_t stream_once = ptx::l2_policy_evict_first();
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const uint32_t m_blk = tile / num_n, n_blk = tile % num_n;
                const int32_t e = max(0, __ldg(p.m_indices + m_blk * T));
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(w_empty + rw.slot, rw.phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
                    ptx::mbar_arrive_expect_tx(w_full + rw.slot, C::kSlotW + C::kSlotSFW);
#pragma unroll
                    for (uint32_t sub = 0; sub < (BK / 2) / C::kRowBytes; ++sub)
                        ptx::tma_load_2d_hint(smem_gen + C::kOffW + rw.slot * C::kSlotW + sub * C::kSubW, &tm_w, w_full + rw.slot,
                                              kb * (BK / 2) + sub * C::kRowBytes, e * p.n + n_blk * BW, stream_once);
                    ptx::tma_load_2d_hint(smem_gen + C::kOffSFW + rw.slot * C::kSlotSFW, &tm_sfw, w_full + rw.slot,
                                          n_blk * BW, e * (p.k / 64) + kb * C::kAtoms, stream_once);
                    rw.advance<C::kDepthW>();
                }
            }
            ptx::grid_launch_dependents();          // the last loads are on their way: the next kernel may start its prologue
        }
    } else if (warp == kWarpTmaA) {
        // activation producer (a separate thread, so a full A ring never holds the weights back)
        if (lane == 0) {
            Ring ra;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const uint32_t m_blk = tile / num_n;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(a_empty + ra.slot, ra.phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
                    ptx::mbar_arrive_expect_tx(a_full + ra.slot, C::kSlotA);
#pragma unroll
                    for (uint32_t box = 0; box < BK / 64; ++box)
                        ptx::tma_load_2d(smem_gen + C::kOffA + ra.slot * C::kSlotA + box * (T * 128), &tm_a,
                                         a_full + ra.slot, kb * BK + box * 64, m_blk * T);
                    ra.advance<C::kDepthA>();
                }
            }
        }
    } else if (warp == kWarpMma) {
        Ring rw, rp;
        uint32_t it = 0, cnt = 0;
        constexpr uint32_t idesc = ptx::make_idesc_nvf4(BW, C::kRowsP);
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            if (!ptx::mbar_wait(tmem_empty + acc, acc_phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t tmem_acc = tmem_base + acc * C::kAccStride;
            for (uint32_t kb = 0; kb < num_kb; ++kb, ++cnt) {
                const uint32_t buf = cnt & 1u;
                if (!ptx::mbar_wait(p_full + rp.slot, rp.phase, abort_flag, pa, 1) ||
                    !ptx::mbar_wait(w_full + rw.slot, rw.phase, abort_flag, pa, 2) ||
                    !ptx::mbar_wait(sf_full + buf, (cnt >> 1) & 1u, abort_flag, pa, 3)) { give_up(1); break; }
                ptx::tcgen05_fence_after_sync();
                if (lane == 0) {
                    // the scales are already in tensor memory (scale warps, tcgen05.st): a tensor-memory copy per
                    // scale atom cost this thread as much issue time as an MMA, and there were two per K atom
                    const uint32_t w = smem + C::kOffW + rw.slot * C::kSlotW;
                    const uint32_t pt = smem + C::kOffP + rp.slot * C::kSlotP;
                    const uint32_t sf = tmem_base + C::kColSF + buf * C::kSfBufCols;
#pragma unroll
                    for (uint32_t a = 0; a < C::kAtoms; ++a)
                        ptx::tcgen05_mma_nvf4(tmem_acc,
                                              ptx::make_smem_desc(w + (a / 4) * C::kSubW + (a % 4) * 32, C::kSBO, C::kSwizzle),
                                              ptx::make_smem_desc(pt + (a / 4) * C::kSubP + (a % 4) * 32, C::kSBO, C::kSwizzle), idesc,
                                              sf + C::kSfW + 4 * a, sf + C::kSfT + 4 * a, (kb | a) != 0 ? 1u : 0u);
                    // one commit per K block: the weight producer, the scale warps and the transform warps all
                    // read "the MMAs of K block i have retired" from this barrier
                    ptx::tcgen05_commit(w_empty + rw.slot);
                    if (kb == num_kb - 1) ptx::tcgen05_commit(tmem_full + acc);
                }
                __syncwarp();
                rp.advance<C::kDepthP>();
                rw.advance<C::kDepthW>();
            }
        }
    } else if (warp >= kWarpSf0) {
        // scale warps: shared -> tensor memory with tcgen05.st, one warp per 32-lane quadrant (the MMA wants a
        // copy in each).  Lane r gets the scale words of rows r, r + 32, r + 64, r + 96 of an atom in four
        // consecutive columns: for the weight scales straight from the row-major words TMA landed (the
        // transposition a tensor-memory copy would have needed comes for free), for the token scales from the
        // atoms the transform wrote.  Two column buffers alternate; a buffer is rewritten once the MMAs of two K
        // blocks earlier have retired (their commit on the W-empty barrier).
        const uint32_t quad = warp & 3;
        Ring rw, rp;
        uint32_t cnt = 0;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (uint32_t kb = 0; kb < num_kb; ++kb, ++cnt) {
                const uint32_t buf = cnt & 1u;
                const uint32_t sf = tmem_base + ((quad * 32) << 16) + C::kColSF + buf * C::kSfBufCols;
                if (!ptx::mbar_wait(w_full + rw.slot, rw.phase, abort_flag, pa, 0) ||
                    !ptx::mbar_wait(p_full + rp.slot, rp.phase, abort_flag, pa, 1)) { give_up(1); break; }
                if (cnt >= 2 && !ptx::mbar_wait(w_empty + (cnt - 2) % C::kDepthW, ((cnt - 2) / C::kDepthW) & 1u, abort_flag, pa, 2)) {
                    give_up(1);
                    break;
                }
                ptx::tcgen05_fence_after_sync();
                const uint32_t sfw = smem + C::kOffSFW + rw.slot * C::kSlotSFW + lane * 4;
                const uint32_t sft = smem + C::kOffSFT + rp.slot * C::kSlotSFT + lane * 16;
#pragma unroll
                for (uint32_t a = 0; a < C::kAtoms; ++a) {
                    ptx::tmem_st_32x32b_x4(sf + C::kSfW + 4 * a, ptx::lds32(sfw + a * 512), ptx::lds32(sfw + a * 512 + 128),
                                           ptx::lds32(sfw + a * 512 + 256), ptx::lds32(sfw + a * 512 + 384));
                    const uint4 v = ptx::lds128(sft + a * 512);
                    ptx::tmem_st_32x32b_x4(sf + C::kSfT + 4 * a, v.x, v.y, v.z, v.w);
                }
                ptx::tmem_st_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(sf_full + buf);
                rw.advance<C::kDepthW>();
                rp.advance<C::kDepthP>();
            }
        }
    } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + kNumEpiWarps) {
        // accumulator lane = weight row n, column = token t: D[m0 + t, n0 + lane] -- for a
        // fixed token the 32 lanes of a warp write 32 consecutive BF16
        const uint32_t quad = warp & 3;
        uint32_t it = 0;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            const uint32_t m_blk = tile / num_n, n_blk = tile % num_n;
            const int32_t e = max(0, __ldg(p.m_indices + m_blk * T));
            const float g = __ldg(p.gw + e);
            if (!ptx::mbar_wait(tmem_full + acc, acc_phase, abort_flag, pa, 0)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            __nv_bfloat16* dcol = p.d + static_cast<int64_t>(m_blk * T) * p.ldd + n_blk * BW + quad * 32 + lane;
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + acc * C::kAccStride;
            // token t of the tile: columns t (pass 0) and T + t (pass 1, when present)
            auto release = [&] {
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tmem_empty + acc);
            };
            if constexpr (T == 16) {
                uint32_t v[32];
                if constexpr (kResidual) {
                    ptx::tmem_ld_32x32b_x32(taddr, v);
                } else {
                    uint32_t h[16];
                    ptx::tmem_ld_32x32b_x16(taddr, h);
#pragma unroll
                    for (uint32_t t = 0; t < 16; ++t) { v[t] = h[t]; v[16 + t] = 0u; }
                }
                ptx::tmem_ld_wait();
                release();
#pragma unroll
                for (uint32_t t = 0; t < 16; ++t)
                    dcol[static_cast<int64_t>(t) * p.ldd] =
                        __float2bfloat16_rn((__uint_as_float(v[t]) + __uint_as_float(v[16 + t])) * g);
            } else {
#pragma unroll 1
                for (uint32_t c = 0; c < T; c += 32) {
                    uint32_t v[32], r[32];
                    ptx::tmem_ld_32x32b_x32(taddr + c, v);
                    if constexpr (kResidual) ptx::tmem_ld_32x32b_x32(taddr + T + c, r);
                    ptx::tmem_ld_wait();
                    if (c + 32 == T) release();
#pragma unroll
                    for (uint32_t t = 0; t < 32; ++t) {
                        float x = __uint_as_float(v[t]);
                        if constexpr (kResidual) x += __uint_as_float(r[t]);
                        dcol[static_cast<int64_t>(c + t) * p.ldd] = __float2bfloat16_rn(x * g);
                    }
                }
            }
        }
    } else if (warp >= kWarpXform0 && warp < kWarpSf0) {
        const uint32_t t = threadIdx.x - kWarpXform0 * 32;
        Ring ra, rp;
        uint32_t cnt = 0;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (uint32_t kb = 0; kb < num_kb; ++kb, ++cnt) {
                if (!ptx::mbar_wait(a_full + ra.slot, ra.phase, abort_flag, pa, 0)) { give_up(1); break; }
                bool p_ok = true;
                xform::transform_tile<T, BK, kXformThreads, kResidual, C::kSfCols, C::kRowsP, kPolicy>(
                    smem + C::kOffA + ra.slot * C::kSlotA, smem + C::kOffP + rp.slot * C::kSlotP,
                    smem + C::kOffP + rp.slot * C::kSlotP + C::kA1Bytes, smem + C::kOffSFT + rp.slot * C::kSlotSFT,
                    smem + C::kOffSFT + rp.slot * C::kSlotSFT + C::kSF1Bytes, t, [&] {
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(a_empty + ra.slot);
                        // the slot is free once the MMAs of kDepthP K blocks ago have retired
                        p_ok = cnt < C::kDepthP ||
                               ptx::mbar_wait(w_empty + (cnt - C::kDepthP) % C::kDepthW, ((cnt - C::kDepthP) / C::kDepthW) & 1u,
                                              abort_flag, pa, 1);
                    });
                if (!p_ok) { give_up(1); break; }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(p_full + rp.slot);
                ra.advance<C::kDepthA>();
                rp.advance<C::kDepthP>();
            }
        }
    }

    ptx::probe_add(32 + (warp < 8 ? warp : 8), ptx::probe_clock() - probe_start);
    if (warp == 0) ptx::probe_flush(pa, 0);
    else if (warp == 3) ptx::probe_flush(pa, 1);
    else if (warp == 1) ptx::probe_flush(pa, 2, 3, 4, 5);
    else if (warp < 8) ptx::probe_flush(pa, 9);
    else if (warp < kWarpSf0) ptx::probe_flush(pa, 11, 12);
    else ptx::probe_flush(pa, 7, 8, 10);
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kWarpMma) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc<C::kTmemCols>(tmem_base);
    }
}

template <uint32_t T, uint32_t BK, bool kResidual, int kPolicy = 0>
int launch_variant(const void* a, int64_t lda, const void* b, const void* sfb, int M, int N, int K, int E,
                   const Params& p, bool pdl, int num_sms, cudaStream_t stream)
{
    using C = Cfg<T, BK, kResidual>;
    CUtensorMap tm_a, tm_w, tm_sfw;
    int rc = host::encode_tensor_map_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, K, M, lda * 2, 64, T,
                                        CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = host::encode_tensor_map_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, K / 2, static_cast<uint64_t>(E) * N,
                                    K / 2, C::kRowBytes, BW, BK >= 256 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    rc = host::encode_tensor_map_2d(&tm_sfw, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, sfb, N,
                                    static_cast<uint64_t>(E) * (K / 64), static_cast<uint64_t>(N) * 4, BW, C::kAtoms,
                                    CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    auto kernel = gemm_swap_kernel<T, BK, kResidual, kPolicy>;
    static bool attr_set[host::kMaxDevices] = {};
    int dev = 0;
    NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev]) {
        NVFP4_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemAlloc));
        attr_set[dev] = true;
    }
    const int num_tiles = (M / static_cast<int>(T)) * (N / static_cast<int>(BW));
    const int grid = num_tiles < num_sms ? num_tiles : num_sms;
    return host::launch_kernel(kernel, dim3(grid), dim3(kThreads), C::kSmemAlloc, stream, pdl, tm_a, tm_w, tm_sfw, p);
}

template <uint32_t T>
int launch_for_tile(const void* a, int64_t lda, const void* b, const void* sfb, int M, int N, int K, int E,
                    const Params& p, bool residual, int block_k, int policy, bool pdl, int num_sms, cudaStream_t stream)
{
    if (policy != 0)      // the other scale policies: the default K-block choice only
        return host::with_policy(policy, [&](auto pol) {
            constexpr int kP = decltype(pol)::value;
            if constexpr (T <= 32) {
                if (K % 512 == 0)
                    return residual ? launch_variant<T, 512, true, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                                    : launch_variant<T, 512, false, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
            }
            if (K % 256 == 0)
                return residual ? launch_variant<T, 256, true, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                                : launch_variant<T, 256, false, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
            return residual ? launch_variant<T, 128, true, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                            : launch_variant<T, 128, false, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
        });
    // K blocks of 512 halve the per-block barrier traffic and commits; a 64-token tile has no room for them
    if constexpr (T <= 32) {
        if (K % 512 == 0 && (block_k == 0 || block_k == 512))
            return residual ? launch_variant<T, 512, true>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                            : launch_variant<T, 512, false>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
    }
    if (K % 256 == 0 && block_k != 128)
        return residual ? launch_variant<T, 256, true>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                        : launch_variant<T, 256, false>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
    return residual ? launch_variant<T, 128, true>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                    : launch_variant<T, 128, false>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
}

}  // namespace

// token_tile: rows per tile (16, 32 or 64); every expert's row range must start on a
// multiple of it, which the caller guarantees through m_alignment % token_tile == 0.
int launch_gemm_swap(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                     int64_t ldd, const int32_t* m_indices, int M, int N, int K, int E, bool residual,
                     int token_tile, int block_k, int policy, bool pdl, int num_sms, int32_t* status, cudaStream_t stream)
{
    Params p;
    p.gw = gw;
    p.m_indices = m_indices;
    p.d = static_cast<__nv_bfloat16*>(d);
    p.ldd = ldd;
    p.m = M; p.n = N; p.k = K;
    p.status = status;
    switch (token_tile) {
        case 16: return launch_for_tile<16>(a, lda, b, sfb, M, N, K, E, p, residual, block_k, policy, pdl, num_sms, stream);
        case 32: return launch_for_tile<32>(a, lda, b, sfb, M, N, K, E, p, residual, block_k, policy, pdl, num_sms, stream);
        case 64: return launch_for_tile<64>(a, lda, b, sfb, M, N, K, E, p, residual, block_k, policy, pdl, num_sms, stream);
        default: return host::fail(NVFP4_E_INVALID_ARGUMENT, "token tile %d is not 16, 32 or 64", token_tile);
    }
}

#ifdef NVFP4_PROBE
extern "C" __attribute__((visibility("default"))) int nvfp4_probe_read_swap(unsigned long long* out64, int reset)
{
    cudaMemcpyFromSymbol(out64, ptx::g_probe, sizeof(unsigned long long) * 64);
    if (reset) { unsigned long long z[64] = {}; cudaMemcpyToSymbol(ptx::g_probe, z, sizeof z); }
    return 0;
}
#endif

}  // namespace nvfp4
