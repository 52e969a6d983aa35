// Grouped dual-NVFP4 GEMM, normal orientation: token rows on the MMA M axis.
//
//   d[m, n] = bf16( gw[e(m)] * sum_k (q0*s0 + q1*s1)[m, k] * (dec(W)*S)[e(m), n, k] )
//
// One persistent CTA per SM works through 128 x 256 output tiles.  Per 128-wide K
// block the roles hand data along rings of shared-memory slots:
//
//   P ring  (A0, A1, SFA0, SFA1, 18 KB/slot)  transform warps -> MMA warp
//   B ring  (FP4 weights + SFB, 18 KB/slot)   TMA warp        -> SFB-transpose warp, MMA warp
//
//   A ring  (BF16 activations, 32 KB/slot)    TMA warp        -> transform warps
//
// A second variant (tune_direct_a = 1) skips the A ring: each transform thread reads its 128
// contiguous bytes of the next K block straight from global memory into registers while it
// runs Algorithm 1 on the current one.  It saves a 32 KB write and a 32 KB read of shared
// memory per K block but measured 1.8x slower on B200 (a warp's 16-byte loads touch 32
// different lines per instruction), so TMA staging stays the default.
//
// and the accumulator (128 lanes x 256 FP32 columns of tensor memory) goes from
// the MMA warp to the epilogue warps.  Each ring has its own full / empty
// mbarriers and its own depth, so a shallow ring never throttles a deep one.  The
// quantised activations live only in shared memory.
//
// Counterpart in the reference: include/nvfp4_gemm/impls/sm100_bf16_dual_nvfp4_gemm.cuh
// (kernel), scheduler/grouped_gemm.cuh (tile order), epilogue/sm100_store_cd.cuh
// (G_W epilogue), src/kernels/sm100_bf16_dual_nvfp4_gemm.hpp:226-480 (launcher).
#include <cuda_bf16.h>

#include "gemm_common.cuh"
#include "host_common.hpp"
#include "launchers.hpp"
#include "transform.cuh"

namespace nvfp4 {

namespace {

constexpr uint32_t BM = 128, BK = 128;
constexpr uint32_t kKAtoms = BK / 64;               // MMA K = 64: one scale atom per instruction
constexpr uint32_t kSlotA = BM * BK * 2;            // 32768
constexpr uint32_t kSlotA0 = BM * BK / 2;           // 8192
constexpr uint32_t kSlotSFA = kKAtoms * 512;        // 1024

// BN = 256 output columns per tile whenever N allows it (one transformed activation tile
// then feeds twice the tensor work); BN = 128 serves N that is an odd multiple of 128.
template <uint32_t BN, bool kDirectA>
struct Cfg {
    static constexpr uint32_t kSlotB = BN * BK / 2;                      // 16384 at BN = 256
    static constexpr uint32_t kSlotSFB = kKAtoms * (BN / 128) * 512;     // 2048
    static constexpr uint32_t kDepthA = kDirectA ? 0 : 3, kDepthP = kDirectA ? 3 : 2;
    static constexpr uint32_t kDepthB = kDirectA ? (BN == 256 ? 7 : 10) : (BN == 256 ? 4 : 6);
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffA0 = kOffA + kDepthA * kSlotA;
    static constexpr uint32_t kOffA1 = kOffA0 + kDepthP * kSlotA0;
    static constexpr uint32_t kOffB = kOffA1 + kDepthP * kSlotA0;
    static constexpr uint32_t kOffSFA0 = kOffB + kDepthB * kSlotB;
    static constexpr uint32_t kOffSFA1 = kOffSFA0 + kDepthP * kSlotSFA;
    static constexpr uint32_t kOffSFB = kOffSFA1 + kDepthP * kSlotSFA;
    static constexpr uint32_t kOffStage = kOffSFB + kDepthB * kSlotSFB;     // epilogue staging (gemm::store_rows_staged)
    static constexpr uint32_t kOffBars = kOffStage + 4 * gemm::kStageWarp;
    static constexpr uint32_t kNumBars = 2 * 3 + 2 * kDepthP + 3 * kDepthB + 2;
    static constexpr uint32_t kSmemBytes = kOffBars + kNumBars * 8 + 16;
    static constexpr uint32_t kSmemAlloc = kSmemBytes + 1024;            // slack to align the base to 1024 B
    static_assert(kSmemAlloc <= 232448, "shared memory budget");
};

// tensor-memory columns
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColAcc = 0, kColSFA0 = 256, kColSFA1 = kColSFA0 + 4 * kKAtoms, kColSFB = kColSFA1 + 4 * kKAtoms;

// warp roles
constexpr uint32_t kWarpTma = 0, kWarpMma = 1, kWarpSfb = 2, kWarpTmaA = 3, kWarpEpi0 = 4, kNumEpiWarps = 4, kWarpXform0 = 8;

struct Params {
    const __nv_bfloat16* a;    // activations and their row stride (the direct-read variant)
    int64_t lda;
    const float* gw;
    const int32_t* m_indices;
    __nv_bfloat16* d;
    int64_t ldd;
    uint32_t m, n, k, num_experts;
    uint32_t group_m;          // m-blocks per scheduling group
    int32_t* status;           // may be null
};

using gemm::Ring;
using gemm::tile_coords;

template <uint32_t BN, uint32_t kXformWarps, bool kResidual, bool kDirectA, int kPolicy>
__global__ void __launch_bounds__((kWarpXform0 + kXformWarps) * 32, 1)
gemm_normal_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const __grid_constant__ CUtensorMap tm_sfb, const Params p)
{
    using C = Cfg<BN, kDirectA>;
    constexpr uint32_t kSlotB = C::kSlotB, kSlotSFB = C::kSlotSFB, kDepthB = C::kDepthB, kDepthP = C::kDepthP;
    constexpr uint32_t kDepthA = kDirectA ? 3 : C::kDepthA;   // barrier slots exist either way
    constexpr uint32_t kOffA = C::kOffA, kOffA0 = C::kOffA0, kOffA1 = C::kOffA1, kOffB = C::kOffB, kOffSFA0 = C::kOffSFA0,
                       kOffSFA1 = C::kOffSFA1, kOffSFB = C::kOffSFB, kOffBars = C::kOffBars;
    constexpr uint32_t kXformThreads = kXformWarps * 32;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem - ptx::smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + kOffBars);
    uint64_t* a_full = bars;
    uint64_t* a_empty = a_full + kDepthA;
    uint64_t* p_full = a_empty + kDepthA;
    uint64_t* p_empty = p_full + kDepthP;
    uint64_t* b_full = p_empty + kDepthP;
    uint64_t* b_ready = b_full + kDepthB;
    uint64_t* b_empty = b_ready + kDepthB;
    uint64_t* tmem_full = b_empty + kDepthB;
    uint64_t* tmem_empty = tmem_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < kDepthA; ++i) { ptx::mbar_init(a_full + i, 1); ptx::mbar_init(a_empty + i, kXformWarps); }
        for (uint32_t i = 0; i < kDepthP; ++i) { ptx::mbar_init(p_full + i, kXformWarps); ptx::mbar_init(p_empty + i, 1); }
        for (uint32_t i = 0; i < kDepthB; ++i) {
            ptx::mbar_init(b_full + i, 1);
            ptx::mbar_init(b_ready + i, 1);
            ptx::mbar_init(b_empty + i, 1);
        }
        ptx::mbar_init(tmem_full, 1);
        ptx::mbar_init(tmem_empty, kNumEpiWarps);
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tm_a);
        ptx::prefetch_tensormap(&tm_b);
        ptx::prefetch_tensormap(&tm_sfb);
    }
    if (warp == kWarpMma) ptx::tmem_alloc<kTmemCols>(tmem_slot);
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // launched with programmatic stream serialisation, the prologue above overlapped the tail of the previous
    // kernel of the stream; its results are visible from here on
    ptx::grid_dependency_wait();

    const long long probe_start = ptx::probe_clock();
    const uint32_t num_m = p.m / BM, num_n = p.n / BN, num_kb = p.k / BK;
    const uint32_t num_tiles = num_m * num_n;
    bool ok = true;
    ptx::ProbeAcc pa;
    auto give_up = [&](uint32_t code) {
        *abort_flag = 1;
        if (p.status != nullptr) atomicOr(p.status, static_cast<int32_t>(code));
        ok = false;
    };

    if (warp == kWarpTma) {
        // ================= weight producer (one lane) =================
        if (lane == 0) {
            Ring rb;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                uint32_t m_blk, n_blk;
                tile_coords(tile, num_m, num_n, p.group_m, m_blk, n_blk);
                const int32_t e = max(0, __ldg(p.m_indices + m_blk * BM));
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(b_empty + rb.slot, rb.phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
                    ptx::mbar_arrive_expect_tx(b_full + rb.slot, kSlotB + kSlotSFB);
                    ptx::tma_load_2d(smem_gen + kOffB + rb.slot * kSlotB, &tm_b, b_full + rb.slot, kb * (BK / 2),
                                     e * p.n + n_blk * BN);
                    ptx::tma_load_2d(smem_gen + kOffSFB + rb.slot * kSlotSFB, &tm_sfb, b_full + rb.slot, n_blk * BN,
                                     e * (p.k / 64) + kb * kKAtoms);
                    rb.advance<kDepthB>();
                }
            }
            ptx::grid_launch_dependents();          // the last loads are on their way: the next kernel may start its prologue
        }
    } else if (warp == kWarpTmaA) {
        // ================= activation producer of the staged variant (its own lane) =====
        if (!kDirectA && lane == 0) {
            Ring ra;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                uint32_t m_blk, n_blk;
                tile_coords(tile, num_m, num_n, p.group_m, m_blk, n_blk);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(a_empty + ra.slot, ra.phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
#ifdef NVFP4_ABLATE_A_TMA   // timing experiments only (wrong results); never defined in the shipped build
                    ptx::mbar_arrive(a_full + ra.slot);
#else
                    ptx::mbar_arrive_expect_tx(a_full + ra.slot, kSlotA);
                    const uint32_t a_dst = kOffA + ra.slot * kSlotA;
                    ptx::tma_load_2d(smem_gen + a_dst, &tm_a, a_full + ra.slot, kb * BK, m_blk * BM);
                    ptx::tma_load_2d(smem_gen + a_dst + kSlotA / 2, &tm_a, a_full + ra.slot, kb * BK + 64, m_blk * BM);
#endif
                    ra.advance<kDepthA>();
                }
            }
        }
    } else if (warp == kWarpMma) {
        // ================= MMA issue (one lane) =================
        Ring rp, rb;
        uint32_t acc_phase = 0;
        constexpr uint32_t idesc = ptx::make_idesc_nvf4(BM, BN);
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            if (!ptx::mbar_wait(tmem_empty, acc_phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!ptx::mbar_wait(p_full + rp.slot, rp.phase, abort_flag, pa, 1) ||
                    !ptx::mbar_wait(b_ready + rb.slot, rb.phase, abort_flag, pa, 2) ||
                    !ptx::mbar_wait(b_full + rb.slot, rb.phase, abort_flag, pa, 3)) { give_up(1); break; }
                ptx::tcgen05_fence_after_sync();
                if (lane == 0) {
                    const uint32_t sfa0 = smem + kOffSFA0 + rp.slot * kSlotSFA;
                    const uint32_t sfa1 = smem + kOffSFA1 + rp.slot * kSlotSFA;
                    const uint32_t sfb = smem + kOffSFB + rb.slot * kSlotSFB;
#pragma unroll
                    for (uint32_t a = 0; a < kKAtoms; ++a) {
                        ptx::tcgen05_cp_32x128b_warpx4(tmem_base + kColSFA0 + 4 * a,
                                                       ptx::make_smem_desc(sfa0 + a * 512, 128, ptx::kSwizzleNone));
                        if constexpr (kResidual)
                            ptx::tcgen05_cp_32x128b_warpx4(tmem_base + kColSFA1 + 4 * a,
                                                           ptx::make_smem_desc(sfa1 + a * 512, 128, ptx::kSwizzleNone));
#pragma unroll
                        for (uint32_t i = 0; i < BN / 128; ++i)
                            ptx::tcgen05_cp_32x128b_warpx4(
                                tmem_base + kColSFB + 4 * (a * (BN / 128) + i),
                                ptx::make_smem_desc(sfb + (a * (BN / 128) + i) * 512, 128, ptx::kSwizzleNone));
                    }
                    const uint32_t a0 = smem + kOffA0 + rp.slot * kSlotA0;
                    const uint32_t a1 = smem + kOffA1 + rp.slot * kSlotA0;
                    const uint32_t b = smem + kOffB + rb.slot * kSlotB;
#pragma unroll
                    for (uint32_t a = 0; a < kKAtoms; ++a) {
                        // 64 K elements = 32 bytes further along each 64-byte swizzled row
                        const uint64_t desc_b = ptx::make_smem_desc(b + a * 32, 512, ptx::kSwizzle64B);
                        ptx::tcgen05_mma_nvf4(tmem_base + kColAcc, ptx::make_smem_desc(a0 + a * 32, 512, ptx::kSwizzle64B),
                                              desc_b, idesc, tmem_base + kColSFA0 + 4 * a,
                                              tmem_base + kColSFB + 4 * a * (BN / 128), (kb | a) != 0 ? 1u : 0u);
                        if constexpr (kResidual)
                            ptx::tcgen05_mma_nvf4(tmem_base + kColAcc,
                                                  ptx::make_smem_desc(a1 + a * 32, 512, ptx::kSwizzle64B), desc_b, idesc,
                                                  tmem_base + kColSFA1 + 4 * a,
                                                  tmem_base + kColSFB + 4 * a * (BN / 128), 1u);
                    }
                    ptx::tcgen05_commit(p_empty + rp.slot);
                    ptx::tcgen05_commit(b_empty + rb.slot);
                    if (kb == num_kb - 1) ptx::tcgen05_commit(tmem_full);
                }
                __syncwarp();
                rp.advance<kDepthP>();
                rb.advance<kDepthB>();
            }
            acc_phase ^= 1;
        }
    } else if (warp == kWarpSfb) {
        // ================= SFB transpose into tensor-memory-copy order =================
        // TMA lands each 128-row atom as 128 consecutive words (row r at word r); the
        // copy wants row r at word (r % 32) * 4 + r / 32.
        Ring rb;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!ptx::mbar_wait(b_full + rb.slot, rb.phase, abort_flag, pa, 0)) { give_up(1); break; }
                const uint32_t base = smem + kOffSFB + rb.slot * kSlotSFB;
#pragma unroll
                for (uint32_t i = 0; i < kKAtoms * (BN / 128); ++i) {
                    const uint32_t atom = base + i * 512;
                    const uint32_t v0 = ptx::lds32(atom + (lane) * 4);
                    const uint32_t v1 = ptx::lds32(atom + (32 + lane) * 4);
                    const uint32_t v2 = ptx::lds32(atom + (64 + lane) * 4);
                    const uint32_t v3 = ptx::lds32(atom + (96 + lane) * 4);
                    __syncwarp();
                    ptx::sts128(atom + lane * 16, v0, v1, v2, v3);
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(b_ready + rb.slot);
                rb.advance<kDepthB>();
            }
        }
    } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + kNumEpiWarps) {
        // ================= epilogue: TMEM -> x G_W -> BF16 -> global =================
        const uint32_t quad = warp & 3;                  // TMEM lane quadrant of this warp
        uint32_t acc_phase = 0;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            uint32_t m_blk, n_blk;
            tile_coords(tile, num_m, num_n, p.group_m, m_blk, n_blk);
            const int32_t e = max(0, __ldg(p.m_indices + m_blk * BM));
            const float g = __ldg(p.gw + e);
            if (!ptx::mbar_wait(tmem_full, acc_phase, abort_flag, pa, 0)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            // 64 columns at a time: tensor memory -> registers -> x G_W -> BF16 -> four whole 128-byte lines per store
            // instruction through the warp's staging area; the accumulator goes back to the MMA warp as soon as this
            // warp's last columns are in registers, so the stores of the tail run under the next tile's main loop
            const uint32_t stage = smem + C::kOffStage + (warp - kWarpEpi0) * gemm::kStageWarp;
            __nv_bfloat16* d_lane = p.d + static_cast<int64_t>(m_blk * BM + quad * 32 + (lane >> 3)) * p.ldd + n_blk * BN + (lane & 7u) * 8;
#pragma unroll 1
            for (uint32_t c = 0; c < BN; c += 64) {
                uint32_t o[32];
                {
                    uint32_t va[32], vb[32];
                    ptx::tmem_ld_32x32b_x32(tmem_base + ((quad * 32) << 16) + kColAcc + c, va);
                    ptx::tmem_ld_32x32b_x32(tmem_base + ((quad * 32) << 16) + kColAcc + c + 32, vb);
                    ptx::tmem_ld_wait();
                    if (c + 64 == BN) {
                        ptx::tcgen05_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(tmem_empty);
                    }
                    gemm::scale_pack_bf16(va, g, o);
                    gemm::scale_pack_bf16(vb, g, o + 16);
                }
                gemm::store_rows_staged(o, stage, d_lane + c, p.ldd, lane);
            }
            acc_phase ^= 1;
        }
    } else if (warp >= kWarpXform0) {
        // ================= transform: Algorithm 1 on every activation tile =================
        const uint32_t t = threadIdx.x - kWarpXform0 * 32;
        Ring ra, rp;
        if constexpr (kDirectA) {
            // registers <- global for K block i + 1 while Algorithm 1 runs on K block i
            using Share = xform::TileShare<BM, BK, kXformThreads>;
            Share bufs[2];
            uint32_t tile = blockIdx.x, kb = 0, m_blk = 0, n_blk = 0;
            auto tile_ptr = [&](uint32_t mb, uint32_t k_block) {
                return p.a + static_cast<int64_t>(mb) * BM * p.lda + k_block * BK;
            };
            if (tile < num_tiles) {
                tile_coords(tile, num_m, num_n, p.group_m, m_blk, n_blk);
                xform::load_tile_global(bufs[0], tile_ptr(m_blk, 0), p.lda, t);
            }
            auto one_block = [&](Share& cur, Share& nxt) {
                uint32_t ntile = tile, nkb = kb + 1, nm = m_blk;
                if (nkb == num_kb) {
                    nkb = 0;
                    ntile += gridDim.x;
                    if (ntile < num_tiles) tile_coords(ntile, num_m, num_n, p.group_m, nm, n_blk);
                }
                if (ntile < num_tiles) xform::load_tile_global(nxt, tile_ptr(nm, nkb), p.lda, t);
                if (!ptx::mbar_wait(p_empty + rp.slot, rp.phase ^ 1, abort_flag, pa, 1)) { give_up(1); return; }
                xform::emit_tile<BM, BK, kXformThreads, kResidual, 4, 0, kPolicy>(
                    cur, smem + kOffA0 + rp.slot * kSlotA0, smem + kOffA1 + rp.slot * kSlotA0,
                    smem + kOffSFA0 + rp.slot * kSlotSFA, smem + kOffSFA1 + rp.slot * kSlotSFA, t);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(p_full + rp.slot);
                rp.advance<kDepthP>();
                tile = ntile; kb = nkb; m_blk = nm;
            };
            while (tile < num_tiles && ok) {
                one_block(bufs[0], bufs[1]);
                if (!(tile < num_tiles && ok)) break;
                one_block(bufs[1], bufs[0]);
            }
        } else {
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(a_full + ra.slot, ra.phase, abort_flag, pa, 0)) { give_up(1); break; }
                    bool p_ok = true;
                    xform::transform_tile<BM, BK, kXformThreads, kResidual, 4, 0, kPolicy>(
                        smem + kOffA + ra.slot * kSlotA, smem + kOffA0 + rp.slot * kSlotA0, smem + kOffA1 + rp.slot * kSlotA0,
                        smem + kOffSFA0 + rp.slot * kSlotSFA, smem + kOffSFA1 + rp.slot * kSlotSFA, t, [&] {
                            // the tile now lives in registers: hand the BF16 slot back before the arithmetic
                            __syncwarp();
                            if (lane == 0) ptx::mbar_arrive(a_empty + ra.slot);
                            p_ok = ptx::mbar_wait(p_empty + rp.slot, rp.phase ^ 1, abort_flag, pa, 1);
                        });
                    if (!p_ok) { give_up(1); break; }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(p_full + rp.slot);
                    ra.advance<kDepthA>();
                    rp.advance<kDepthP>();
                }
            }
        }
    }

    ptx::probe_add(32 + (warp < 8 ? warp : 8), ptx::probe_clock() - probe_start);
    if (warp == 0) ptx::probe_flush(pa, 0);
    else if (warp == 3) ptx::probe_flush(pa, 1);
    else if (warp == 1) ptx::probe_flush(pa, 2, 3, 4, 5);
    else if (warp == 2) ptx::probe_flush(pa, 7);
    else if (warp < 8) ptx::probe_flush(pa, 9);
    else ptx::probe_flush(pa, 11, 12);
    // teardown: everyone meets here, on the normal path and after a timeout alike
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kWarpMma) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc<kTmemCols>(tmem_base);
    }
}

template <uint32_t BN, uint32_t kXformWarps, bool kResidual, bool kDirectA, int kPolicy = 0>
int launch_variant(const void* a, int64_t lda, const void* b, const void* sfb, int M, int N, int K, int E,
                   const Params& p, bool pdl, int num_sms, cudaStream_t stream)
{
    using C = Cfg<BN, kDirectA>;
    CUtensorMap tm_a, tm_b, tm_sfb;
    int rc = host::encode_tensor_map_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, K, M, lda * 2, 64, BM,
                                        CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = host::encode_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, K / 2, static_cast<uint64_t>(E) * N,
                                    K / 2, BK / 2, BN, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    rc = host::encode_tensor_map_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, sfb, N,
                                    static_cast<uint64_t>(E) * (K / 64), static_cast<uint64_t>(N) * 4, BN, kKAtoms,
                                    CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    auto kernel = gemm_normal_kernel<BN, kXformWarps, kResidual, kDirectA, kPolicy>;
    static bool attr_set[host::kMaxDevices] = {};
    int dev = 0;
    NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev]) {
        NVFP4_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemAlloc));
        attr_set[dev] = true;
    }
    const int num_tiles = (M / static_cast<int>(BM)) * (N / static_cast<int>(BN));
    const int grid = num_tiles < num_sms ? num_tiles : num_sms;
    return host::launch_kernel(kernel, dim3(grid), dim3((kWarpXform0 + kXformWarps) * 32), C::kSmemAlloc, stream, pdl, tm_a, tm_b,
                               tm_sfb, p);
}

template <uint32_t BN>
int launch_for_bn(const void* a, int64_t lda, const void* b, const void* sfb, int M, int N, int K, int E,
                  const Params& p, bool residual, int xform_warps, bool direct_a, int policy, bool pdl, int num_sms, cudaStream_t stream)
{
    if (policy != 0)      // the other scale policies: the TMA-staged kernel with eight transform warps only
        return host::with_policy(policy, [&](auto pol) {
            constexpr int kP = decltype(pol)::value;
            return residual ? launch_variant<BN, 8, true, false, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                            : launch_variant<BN, 8, false, false, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
        });
    if (!direct_a) {
        if (xform_warps == 16)
            return residual ? launch_variant<BN, 16, true, false>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                            : launch_variant<BN, 16, false, false>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
        return residual ? launch_variant<BN, 8, true, false>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                        : launch_variant<BN, 8, false, false>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
    }
    return residual ? launch_variant<BN, 8, true, true>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                    : launch_variant<BN, 8, false, true>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
}

}  // namespace

// Validated arguments in, launch out.  See nvfp4_grouped_gemm_contiguous for meanings.
int launch_gemm_normal(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                       int64_t ldd, const int32_t* m_indices, int M, int N, int K, int E, bool residual,
                       int xform_warps, int group_m, bool direct_a, int policy, bool pdl, int num_sms, int32_t* status,
                       cudaStream_t stream)
{
    Params p;
    p.a = static_cast<const __nv_bfloat16*>(a);
    p.lda = lda;
    p.gw = gw;
    p.m_indices = m_indices;
    p.d = static_cast<__nv_bfloat16*>(d);
    p.ldd = ldd;
    p.m = M; p.n = N; p.k = K; p.num_experts = E;
    p.group_m = group_m > 0 ? group_m : 8;
    p.status = status;
    if (N % 256 == 0) return launch_for_bn<256>(a, lda, b, sfb, M, N, K, E, p, residual, xform_warps, direct_a, policy, pdl, num_sms, stream);
    return launch_for_bn<128>(a, lda, b, sfb, M, N, K, E, p, residual, xform_warps, direct_a, policy, pdl, num_sms, stream);
}

#ifdef NVFP4_PROBE
extern "C" __attribute__((visibility("default"))) int nvfp4_probe_read_normal(unsigned long long* out64, int reset)
{
    cudaMemcpyFromSymbol(out64, ptx::g_probe, sizeof(unsigned long long) * 64);
    if (reset) { unsigned long long z[64] = {}; cudaMemcpyToSymbol(ptx::g_probe, z, sizeof z); }
    return 0;
}
#endif

}  // namespace nvfp4
