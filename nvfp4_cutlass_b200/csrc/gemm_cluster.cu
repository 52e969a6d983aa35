// Grouped dual-NVFP4 GEMM, normal orientation, Algorithm 1 inside the main loop, with the activation
// transform shared by the CTAs of a thread-block cluster (four, or two).
//
// The CTAs of a cluster work on the same 128 token rows and on neighbouring 256-column weight tiles.  The
// quantised activation tile (A0, A1 and their scales) is the same for all of them, so each CTA loads and
// transforms only its 128 / CL rows, writes the products into its own shared memory and a push warp sends the
// finished share to every peer with TWO bulk shared-to-shared copies (cp.async.bulk shared::cta ->
// shared::cluster, completing bytes on the peer's P-full barrier): one for the packed codes of both passes, one
// for the scales.  Per CTA and K block that divides the Algorithm-1 arithmetic -- which saturates the issue slots
// of a single-CTA kernel -- by CL, while the tensor work per CTA is unchanged.  Nothing quantised is ever written
// to global memory.
//
// The share of a CTA is contiguous because of how a P slot is laid out.  Row m of the MMA tile is token row m and
// the CTA of rank c owns rows [c * 128 / CL, (c + 1) * 128 / CL).  The packed codes of the two passes are
// interleaved by 8-row group -- [A0 rows 0-7][A1 rows 0-7][A0 rows 8-15]... (512 bytes each) -- which the MMA
// descriptors express as a stride of 1024 bytes between row groups, so the rows of one CTA, both passes, are one
// run of bytes.  The scale words are kept per source CTA, pass and K atom, [c][pass][atom][row] (this staging
// layout is read only by the scale warps, which carry the words to tensor memory with tcgen05.st).
// Measured on B200 (E=8 x 512 rows, N=28672, K=4096): twelve small copies per peer and K block (an earlier
// layout with strided shares) ran at ~6 B/clk per CTA and set the pace of the kernel at 0.78 ms; transform
// threads storing straight into the peers' shared memory (st.shared::cluster + a releasing remote arrive) were
// slower still, 1.65 ms for pairs and 1.78 ms for quads: every transform warp then sits out the round trip, and a
// cluster-scope releasing arrive alone costs ~1500 cycles on this GPU (measured later, in the split path's pair kernel).
//
// The scale factors reach tensor memory through tcgen05.st issued by the (otherwise idle) epilogue warps, not
// through tensor-memory copies issued by the MMA thread; see the MMA role below.
//
// Barriers: P-full of a CTA counts its own eight transform warps, the push warp's announcement of the bytes the
// peers will send, and those bytes; P-empty counts one tcgen05.commit per CTA, delivered to all CTAs by the
// commit's cluster mask, so a slot is rewritten (locally or by a peer's copy) only after every tensor core has
// read it.  The P ring, the weight ring and the scale columns in tensor memory have the same depth and advance
// together, so that one commit per K block frees all three, and the MMA thread waits on a single barrier per K
// block (scales-in-tensor-memory, which the scale warps signal only after they have seen P-full and B-full
// themselves).  No load in this file is a multicast: the cross-CTA traffic is the bulk copies, mbarrier
// signalling and the commit mask.
//
// Counterpart in the reference: include/nvfp4_gemm/impls/sm100_bf16_dual_nvfp4_gemm.cuh (single-CTA kernel;
// the reference measured cluster co-scheduling only, without sharing the transform).
#include <cuda_bf16.h>

#include "gemm_common.cuh"
#include "host_common.hpp"
#include "launchers.hpp"
#include "transform.cuh"

namespace nvfp4 {
namespace {

using gemm::Ring;

constexpr uint32_t BM = 128, BN = 256, BK = 128, kKAtoms = 2;
constexpr uint32_t kSlotB = BN * BK / 2, kSlotSFB = kKAtoms * 2 * 512;
// 32 warps (scale and epilogue warps sit on warp ids whose low two bits are their tensor-memory quadrant): four
// single-thread roles, eight scale warps (per tensor-memory quadrant one for the weight scales and one
// for the activation scales), eight epilogue warps (two per quadrant, 128 accumulator columns each), twelve transform
// warps.  The scale warps do nothing else: an event trace showed one warp per quadrant carrying both kinds of scales
// to be the slowest stage of the pipeline (it shares its scheduler with seven other warps), and scale warps that double
// as epilogue warps stall the first K blocks of the next tile.
constexpr uint32_t kWarpTma = 0, kWarpMma = 1, kWarpTmaA = 2, kWarpPush = 3, kWarpSf0 = 4, kNumSfWarps = 8, kWarpEpi0 = 12,
                   kNumEpiWarps = 8, kWarpXform0 = 20, kXW = 12;
constexpr uint32_t kEpiCols = BN / (kNumEpiWarps / 4);          // accumulator columns per epilogue warp
constexpr uint32_t kThreads = (kWarpXform0 + kXW) * 32;        // 1024
// tensor memory: 256 accumulator columns, then one buffer of 32 scale columns (SFA0 8, SFA1 8, SFB 16) per
// slot of the operand rings
constexpr uint32_t kTmemCols = 512, kColAcc = 0, kColSF = 256, kSfBufCols = 32, kSfA0 = 0, kSfA1 = 8, kSfB = 16;

// Twelve transform warps.  Algorithm 1 on a 16-block is a long dependent chain (~600 cycles for a warp that does one
// block, ~1000 for two interleaved), so what the transform needs is K blocks in flight: a thread always takes two
// adjacent blocks, four warps cover the 256 blocks of a quad's K block and the three groups of four take K blocks in
// turn; the 512 blocks of a pair's K block need eight warps, one group (the other four warps idle).
template <uint32_t CL, bool kResidual>
struct Cfg {
    static_assert(CL == 2 || CL == 4, "cluster of two or four CTAs");
    static constexpr uint32_t kPass = kResidual ? 2 : 1;
    // packed codes: 8-row groups of the passes interleaved (see the top of the file)
    static constexpr uint32_t kGroupStride = 512 * kPass, kPassOffset = 512;
    static constexpr uint32_t kSlotCodes = BM * (BK / 2) * kPass;             // 16 KB (8 KB single pass)
    static constexpr uint32_t kSlotScales = kPass * kKAtoms * BM * 4;         // 2 KB (1 KB)
    static constexpr uint32_t kRows = BM / CL;                  // rows this CTA loads and transforms
    static constexpr uint32_t kSlotA = kRows * BK * 2;          // 16 KB (pairs), 8 KB (quads)
    static constexpr uint32_t kBlocks = kRows * (BK / 16);      // 16-blocks per K block and CTA: 512 (pairs), 256 (quads)
    static constexpr uint32_t kBpt = 2;                         // 16-blocks per transform thread
    static constexpr uint32_t kGroupWarps = kBlocks / (kBpt * 32);   // warps that share one K block: 8 (pairs), 4 (quads)
    static constexpr uint32_t kGroups = kXW / kGroupWarps;      // groups taking K blocks in turn: 1 (pairs), 3 (quads)
    static_assert(kGroups >= 1 && kGroups <= 4, "transform split");
    // P, B and scale columns move together.  A quad has room for five ring positions (its BF16 slots are 8 KB); the loop
    // transform -> copy to the peers -> scale warps -> MMA -> commit back to every CTA is longer than four K blocks of
    // tensor work, so with four positions the tensor pipe idles a quarter of the time.
    static constexpr uint32_t kDepthP = CL == 4 ? 5 : 4, kDepthB = kDepthP, kDepthA = CL == 4 ? 5 : 4;
    static_assert(kColSF + kDepthP * kSfBufCols <= kTmemCols, "scale columns");
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffCodes = kOffA + kDepthA * kSlotA;
    static constexpr uint32_t kOffB = kOffCodes + kDepthP * kSlotCodes;
    static constexpr uint32_t kOffScales = kOffB + kDepthB * kSlotB;
    static constexpr uint32_t kOffSFB = kOffScales + kDepthP * kSlotScales;
    static constexpr uint32_t kOffStage = kOffSFB + kDepthB * kSlotSFB;
    static constexpr uint32_t kOffBars = kOffStage + kNumEpiWarps * gemm::kStageWarp;
    static constexpr uint32_t kNumBars = 2 * kDepthA + 4 * kDepthP + kDepthB + 2;
    // what one CTA sends to one peer per K block: its rows of the packed codes, its block of scale words
    static constexpr uint32_t kShareCodes = kSlotCodes / CL, kShareScales = kSlotScales / CL;
    static constexpr uint32_t kSmemAlloc = kOffBars + kNumBars * 8 + 16 + 1024;
    static_assert(kSmemAlloc <= 232448, "shared memory budget");
};

#ifdef NVFP4_PROBE
// event trace of CTA 0 (timing studies): g_ctrace[point][K block] = clock64 at the event
__device__ long long g_ctrace[16][96];
#define NVFP4_CTRACE(point, kbi) do { if (blockIdx.x == 0 && (kbi) < 96 && (threadIdx.x & 31u) == 0) g_ctrace[point][kbi] = clock64(); } while (0)
#else
#define NVFP4_CTRACE(point, kbi) do { } while (0)
#endif

struct Params {
    const float* gw;
    const int32_t* m_indices;
    __nv_bfloat16* d;
    int64_t ldd;
    uint32_t m, n, k;
    uint32_t group_m;
    int32_t* status;
};

template <uint32_t CL, bool kResidual, int kPolicy>
__global__ void __launch_bounds__(kThreads, 1)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_sfb, const Params p)
{
    using C = Cfg<CL, kResidual>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem - ptx::smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kOffBars);
    uint64_t* a_full = bars;
    uint64_t* a_empty = a_full + C::kDepthA;
    uint64_t* p_full = a_empty + C::kDepthA;         // the whole slot is written: own share + the bytes of the peers' copies
    uint64_t* p_empty = p_full + C::kDepthP;         // every CTA's tensor core has read this slot
    uint64_t* b_full = p_empty + C::kDepthP;
    uint64_t* share_full = b_full + C::kDepthB;      // [kDepthP]: this CTA's share of a slot is written
    uint64_t* sf_full = share_full + C::kDepthP;     // [kDepthP]: scales of a K block are in tensor memory
    uint64_t* tmem_full = sf_full + C::kDepthP;
    uint64_t* tmem_empty = tmem_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_cta_rank();

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < C::kDepthA; ++i) { ptx::mbar_init(a_full + i, 1); ptx::mbar_init(a_empty + i, C::kGroupWarps); }
        for (uint32_t i = 0; i < C::kDepthP; ++i) {
            ptx::mbar_init(p_full + i, C::kGroupWarps + 1);     // own transform warps + the push warp; peers' shares arrive as bytes
            ptx::mbar_init(share_full + i, C::kGroupWarps);
            ptx::mbar_init(p_empty + i, CL);                    // one commit per CTA of the cluster
            ptx::mbar_init(sf_full + i, kNumSfWarps);
        }
        for (uint32_t i = 0; i < C::kDepthB; ++i) ptx::mbar_init(b_full + i, 1);
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
    ptx::cluster_sync();                                         // every CTA's barriers exist before any remote arrival
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // launched with programmatic stream serialisation, everything above overlapped the tail of the previous
    // kernel in the stream; its results are visible from here on
    ptx::grid_dependency_wait();

    const uint32_t num_m = p.m / BM, num_ns = p.n / (BN * CL), num_kb = p.k / BK;
    const uint32_t num_super = num_m * num_ns;
    const uint32_t cid = ptx::cluster_id_x(), ncl = ptx::num_clusters_x();
    bool ok = true;
    ptx::ProbeAcc pa;                                // per-site wait accounting of timing studies; empty in the shipped build
    const long long probe_start = ptx::probe_clock();
    auto give_up = [&](uint32_t code) {
        *abort_flag = 1;
        if (p.status != nullptr) atomicOr(p.status, static_cast<int32_t>(code));
        ok = false;
    };

    if (warp == kWarpTma) {
        // ================= weight producer =================
        if (lane == 0) {
            Ring rb;
            for (uint32_t st = cid; st < num_super && ok; st += ncl) {
                uint32_t m_blk, ns;
                gemm::tile_coords(st, num_m, num_ns, p.group_m, m_blk, ns);
                const uint32_t n_blk = ns * CL + rank;
                const int32_t e = max(0, __ldg(p.m_indices + m_blk * BM));
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    // slot i of the weight ring is free when slot i of the P ring is: one commit covers both
                    if (!ptx::mbar_wait_sleep<true>(p_empty + rb.slot, rb.phase ^ 1, abort_flag, 64, pa, 0)) { give_up(1); break; }
                    ptx::mbar_arrive_expect_tx(b_full + rb.slot, kSlotB + kSlotSFB);
                    ptx::tma_load_2d(smem_gen + C::kOffB + rb.slot * kSlotB, &tm_b, b_full + rb.slot, kb * (BK / 2),
                                     e * p.n + n_blk * BN);
                    ptx::tma_load_2d(smem_gen + C::kOffSFB + rb.slot * kSlotSFB, &tm_sfb, b_full + rb.slot, n_blk * BN,
                                     e * (p.k / 64) + kb * kKAtoms);
                    rb.advance<C::kDepthB>();
                }
            }
            ptx::grid_launch_dependents();          // the last loads are on their way: the next kernel may start its prologue
        }
    } else if (warp == kWarpTmaA) {
        // ================= activation producer: this CTA's share of the rows =================
        if (lane == 0) {
            Ring ra;
            for (uint32_t st = cid; st < num_super && ok; st += ncl) {
                uint32_t m_blk, ns;
                gemm::tile_coords(st, num_m, num_ns, p.group_m, m_blk, ns);
                const uint32_t row0 = m_blk * BM + rank * C::kRows;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait_sleep<false>(a_empty + ra.slot, ra.phase ^ 1, abort_flag, 64, pa, 0)) { give_up(1); break; }
                    ptx::mbar_arrive_expect_tx(a_full + ra.slot, C::kSlotA);
                    const uint32_t a_dst = C::kOffA + ra.slot * C::kSlotA;
                    ptx::tma_load_2d(smem_gen + a_dst, &tm_a, a_full + ra.slot, kb * BK, row0);
                    ptx::tma_load_2d(smem_gen + a_dst + C::kSlotA / 2, &tm_a, a_full + ra.slot, kb * BK + 64, row0);
                    ra.advance<C::kDepthA>();
                }
            }
        }
    } else if (warp == kWarpMma) {
        // ================= MMA issue =================
        // The scale factors are already in tensor memory when a K block is issued (the scale warps
        // put them there with tcgen05.st), so a K block costs this thread four MMAs and its commits:
        // a tensor-memory copy of one scale atom costs as much issue time as an MMA of N <= 128, and
        // eight of them per K block were the larger half of the tensor-side time.
        // One thread runs the whole role.  A round takes the next K block and, if its scales are already up, the one
        // after it too: the fixed cost of a round (barrier round trips, loop) is then paid once per eight MMAs.
        if (lane == 0) {
            Ring rp;
            uint32_t acc_phase = 0;
            int32_t pending = -1;                   // ring position whose commit is still to be issued
            constexpr uint32_t idesc = ptx::make_idesc_nvf4(BM, BN);
            constexpr uint16_t kAllCtas = static_cast<uint16_t>((1u << CL) - 1u);
            for (uint32_t st = cid; st < num_super && ok; st += ncl) {
                if (!ptx::mbar_wait(tmem_empty, acc_phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
                ptx::tcgen05_fence_after_sync();
                uint32_t kb = 0;
                while (kb < num_kb) {
                    // the scale warps arrive here only after they have seen this slot's P-full (acquired at cluster
                    // scope) and B-full complete, so this one wait also covers the operand tiles in shared memory
                    NVFP4_CTRACE(12, (st - cid) / ncl * num_kb + kb);
                    if (!ptx::mbar_wait(sf_full + rp.slot, rp.phase, abort_flag, pa, 3)) { give_up(1); break; }
                    NVFP4_CTRACE(10, (st - cid) / ncl * num_kb + kb);
                    Ring r2 = rp;
                    r2.advance<C::kDepthP>();
                    const uint32_t blocks = (kb + 1 < num_kb && ptx::mbar_try_wait(sf_full + r2.slot, r2.phase)) ? 2u : 1u;
                    ptx::tcgen05_fence_after_sync();
                    for (uint32_t u = 0; u < blocks; ++u, ++kb) {
                        // the 8-row groups of the two passes alternate: the stride between the row groups of one pass
                        // is kGroupStride and the second pass starts kPassOffset into the slot
                        const uint32_t a0 = smem + C::kOffCodes + rp.slot * C::kSlotCodes;
                        const uint32_t a1 = a0 + C::kPassOffset;
                        const uint32_t b = smem + C::kOffB + rp.slot * kSlotB;
                        const uint32_t sf = tmem_base + kColSF + rp.slot * kSfBufCols;
#pragma unroll
                        for (uint32_t a = 0; a < kKAtoms; ++a) {
                            const uint64_t desc_b = ptx::make_smem_desc(b + a * 32, 512, ptx::kSwizzle64B);
                            ptx::tcgen05_mma_nvf4(tmem_base + kColAcc, ptx::make_smem_desc(a0 + a * 32, C::kGroupStride, ptx::kSwizzle64B),
                                                  desc_b, idesc, sf + kSfA0 + 4 * a, sf + kSfB + 8 * a, (kb | a) != 0 ? 1u : 0u);
                            // One commit per K block, to every CTA of the cluster: it frees the P slot, the weight slot
                            // and the scale columns of a ring position.  A commit holds this thread until the MMAs before
                            // it have been handed to the tensor pipe; issued at the end of its own K block it leaves the
                            // pipe with nothing queued while this thread finds the next K block, so it goes out after the
                            // first MMA of the NEXT block.
                            if (a == 0 && pending >= 0) ptx::tcgen05_commit_cluster(p_empty + pending, kAllCtas);
                            if constexpr (kResidual)
                                ptx::tcgen05_mma_nvf4(tmem_base + kColAcc, ptx::make_smem_desc(a1 + a * 32, C::kGroupStride, ptx::kSwizzle64B),
                                                      desc_b, idesc, sf + kSfA1 + 4 * a, sf + kSfB + 8 * a, 1u);
                        }
                        if (kb == num_kb - 1) {              // nothing follows in this tile: commit now
                            ptx::tcgen05_commit_cluster(p_empty + rp.slot, kAllCtas);
                            ptx::tcgen05_commit(tmem_full);
                        }
                        pending = kb == num_kb - 1 ? -1 : static_cast<int32_t>(rp.slot);
                        NVFP4_CTRACE(11, (st - cid) / ncl * num_kb + kb);
                        rp.advance<C::kDepthP>();
                    }
                }
                acc_phase ^= 1;
            }
        }
    } else if (warp == kWarpPush) {
        // ================= push: this CTA's finished share to every peer =================
        // Two bulk shared-to-shared copies per peer and K block (codes of both passes, scale words), to the same
        // offsets in the peer's slot; the bytes complete on the peer's P-full barrier.  The lanes of the warp issue
        // one copy each, so the transform warps never wait for copy issue or for the round trip.
        constexpr uint32_t kCopies = (CL - 1) * 2;
        constexpr uint32_t kPeerBytes = (CL - 1) * (C::kShareCodes + C::kShareScales);
        Ring rp;
        for (uint32_t st = cid; st < num_super && ok; st += ncl) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!ptx::mbar_wait(share_full + rp.slot, rp.phase, abort_flag, pa, 0)) { give_up(1); break; }
                NVFP4_CTRACE(4, (st - cid) / ncl * num_kb + kb);
                if (lane < kCopies) {
                    const uint32_t peer = (rank + 1 + lane / 2) % CL;
                    const bool scales = (lane & 1u) != 0;
                    const uint32_t off = scales ? C::kOffScales + rp.slot * C::kSlotScales + rank * C::kShareScales
                                                : C::kOffCodes + rp.slot * C::kSlotCodes + rank * C::kShareCodes;
                    ptx::bulk_copy_to_cta(ptx::map_to_cta(smem + off, peer), smem + off, scales ? C::kShareScales : C::kShareCodes,
                                          ptx::map_to_cta(ptx::smem_u32(p_full + rp.slot), peer));
                }
                if (lane == 0) ptx::mbar_arrive_expect_tx(p_full + rp.slot, kPeerBytes);
                NVFP4_CTRACE(5, (st - cid) / ncl * num_kb + kb);
                __syncwarp();
                rp.advance<C::kDepthP>();
            }
        }
    } else if (warp >= kWarpSf0 && warp < kWarpSf0 + kNumSfWarps) {
        // ================= scale warps =================
        // The scale factors go from shared to tensor memory with tcgen05.st (a warp reaches only its own quadrant of
        // lanes, and the MMA wants each quadrant to hold a copy): lane r of each quadrant gets the scale words of rows
        // r, r + 32, r + 64, r + 96 in four consecutive columns.  Warps 4-7 take the weight scales straight from the
        // rows TMA landed (which also does the transposition a tensor-memory copy would have needed) and run ahead of
        // the transform; warps 8-11 take the activation scales of both passes from the staging layout the transform
        // warps and the peers' copies fill.  There is one set of scale columns per ring position; it is rewritten once
        // the MMAs that used it have retired (the P-empty barrier).
        const uint32_t quad = warp & 3, kind = (warp - kWarpSf0) >> 2;      // 0: weight scales, 1: activation scales
        Ring rp;
        for (uint32_t st = cid; st < num_super && ok; st += ncl) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                const uint32_t sf = tmem_base + ((quad * 32) << 16) + kColSF + rp.slot * kSfBufCols;
                // the columns of this ring position are free once its previous MMAs have retired
                if (!ptx::mbar_wait_sleep<true>(p_empty + rp.slot, rp.phase ^ 1, abort_flag, 32, pa, 2)) { give_up(1); break; }
                if (warp == kWarpSf0 + 4) NVFP4_CTRACE(6, (st - cid) / ncl * num_kb + kb);
                if (kind == 0) {
                    if (!ptx::mbar_wait_sleep<false>(b_full + rp.slot, rp.phase, abort_flag, 32, pa, 1)) { give_up(1); break; }
                    if (warp == kWarpSf0) NVFP4_CTRACE(7, (st - cid) / ncl * num_kb + kb);
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t sfb = smem + C::kOffSFB + rp.slot * kSlotSFB + lane * 4;
                    uint32_t v[16];
#pragma unroll
                    for (uint32_t i = 0; i < kKAtoms * 2; ++i)
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) v[4 * i + j] = ptx::lds32(sfb + i * 512 + j * 128);
                    ptx::tmem_st_32x32b(sf + kSfB, v);
                } else {
                    if (!ptx::mbar_wait_cluster(p_full + rp.slot, rp.phase, abort_flag, pa, 1)) { give_up(1); break; }
                    if (warp == kWarpSf0 + 4) NVFP4_CTRACE(8, (st - cid) / ncl * num_kb + kb);
                    ptx::tcgen05_fence_after_sync();
                    // staging layout [source CTA][pass][K atom][row of that CTA]; lane r wants rows r, r + 32, r + 64, r + 96
                    uint32_t v[kResidual ? 16 : 8];
                    const uint32_t sc = smem + C::kOffScales + rp.slot * C::kSlotScales;
#pragma unroll
                    for (uint32_t ps = 0; ps < C::kPass; ++ps)
#pragma unroll
                        for (uint32_t a = 0; a < kKAtoms; ++a)
#pragma unroll
                            for (uint32_t j = 0; j < 4; ++j) {
                                const uint32_t m = 32 * j + lane;
                                v[8 * ps + 4 * a + j] = ptx::lds32(sc + (((m / C::kRows) * C::kPass + ps) * kKAtoms + a) * (C::kRows * 4) +
                                                                   (m % C::kRows) * 4);
                            }
                    ptx::tmem_st_32x32b(sf + kSfA0, v);          // SFA0 columns 0-7, SFA1 columns 8-15
                }
                ptx::tmem_st_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(sf_full + rp.slot);
                if (warp == kWarpSf0 + 4) NVFP4_CTRACE(9, (st - cid) / ncl * num_kb + kb);
                if (warp == kWarpSf0) NVFP4_CTRACE(13, (st - cid) / ncl * num_kb + kb);
                if (warp == kWarpSf0 + 7) NVFP4_CTRACE(14, (st - cid) / ncl * num_kb + kb);
                if (warp == kWarpSf0 + 3) NVFP4_CTRACE(15, (st - cid) / ncl * num_kb + kb);
                rp.advance<C::kDepthP>();
            }
        }
    } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + kNumEpiWarps) {
        // ================= epilogue: TMEM -> x G_W -> BF16 -> global =================
        // Two (or four) warps per quadrant of tensor memory, 128 (64) accumulator columns each, taken out 32 at a time and
        // stored 64 at a time (1024 threads leave 64 registers each); the accumulator goes back to the MMA warp as soon
        // as its last column has left tensor memory, before the last 64 columns are stored.
        const uint32_t quad = warp & 3, part = (warp - kWarpEpi0) >> 2;
        uint32_t acc_phase = 0;
        for (uint32_t st = cid; st < num_super && ok; st += ncl) {
            uint32_t m_blk, ns;
            gemm::tile_coords(st, num_m, num_ns, p.group_m, m_blk, ns);
            const uint32_t n_blk = ns * CL + rank;
            const int32_t e = max(0, __ldg(p.m_indices + m_blk * BM));
            const float g = __ldg(p.gw + e);
            if (!ptx::mbar_wait_relaxed(tmem_full, acc_phase, abort_flag, 100)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            const long long epi0 = ptx::probe_clock();
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + kColAcc + part * kEpiCols;
            const uint32_t stage = smem + C::kOffStage + (warp - kWarpEpi0) * gemm::kStageWarp;
            __nv_bfloat16* d_lane = p.d + static_cast<int64_t>(m_blk * BM + quad * 32 + (lane >> 3)) * p.ldd + n_blk * BN +
                                    part * kEpiCols + (lane & 7u) * 8;
#pragma unroll
            for (uint32_t hh = 0; hh < kEpiCols / 64; ++hh) {
                uint32_t o[32];
                {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(taddr + hh * 64, v);
                    ptx::tmem_ld_wait();
                    gemm::scale_pack_bf16(v, g, o);
                }
                {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(taddr + hh * 64 + 32, v);
                    ptx::tmem_ld_wait();
                    if (hh == kEpiCols / 64 - 1) {
                        ptx::tcgen05_fence_before_sync();         // everything has left tensor memory
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(tmem_empty);
                        ptx::probe_count(pa, 3, ptx::probe_clock() - epi0);
                    }
                    gemm::scale_pack_bf16(v, g, o + 16);
                }
                gemm::store_rows_staged(o, stage, d_lane + hh * 64, p.ldd, lane);
            }
            acc_phase ^= 1;
        }
    } else if (warp >= kWarpXform0) {
        // ================= transform: this CTA's rows into its own P slot =================
        // Thread t owns one row of this CTA's share and one (quads) or two adjacent (pairs) 16-blocks of it: the
        // 8 (4) threads of a row are neighbours in a warp, so a warp's stores of packed codes cover whole 64-byte
        // rows and the scale bytes of a K atom are gathered into one word with two shuffles.
        const uint32_t gid = (warp - kWarpXform0) / C::kGroupWarps;                // which of the alternating groups
        const uint32_t t = threadIdx.x - (kWarpXform0 + gid * C::kGroupWarps) * 32;   // thread inside the group
        constexpr uint32_t kPerRow = 8 / C::kBpt;                                  // threads per row
        const uint32_t lrow = t / kPerRow, piece = t % kPerRow;                    // row inside this CTA's share
        const uint32_t mrow = rank * C::kRows + lrow;                              // its row in the MMA tile
        const uint32_t first_block = piece * C::kBpt;
        // where this thread's products go, relative to a slot: 8-row group, pass, row in the group, swizzled chunk
        const uint32_t chunk = ((first_block >> 1) ^ ((mrow >> 1) & 3u)) << 4;
        const uint32_t code_off = (mrow >> 3) * C::kGroupStride + (mrow & 7u) * 64 + chunk + (C::kBpt == 1 ? ((first_block & 1u) << 3) : 0u);
        const uint32_t sf_off = ((rank * C::kPass) * kKAtoms + (first_block >> 2)) * (C::kRows * 4) + lrow * 4;
        const bool sf_writer = (first_block & 3u) == 0;                           // the thread that holds a K atom's scale word
        uint32_t it = 0;                                                           // K blocks of this CTA so far, over all tiles
        // (a pair has work for one group of eight warps only: the surplus warps have no K blocks and must not touch a barrier)
        for (uint32_t st = cid; st < num_super && ok && gid < C::kGroups; st += ncl) {
            for (uint32_t kb = 0; kb < num_kb; ++kb, ++it) {
                if (C::kGroups > 1 && it % C::kGroups != gid) continue;            // another group's K block
                const Ring ra{it % C::kDepthA, (it / C::kDepthA) & 1u}, rp{it % C::kDepthP, (it / C::kDepthP) & 1u};
                if (!ptx::mbar_wait_sleep<false>(a_full + ra.slot, ra.phase, abort_flag, 32, pa, 0)) { give_up(1); break; }
                const long long xt0 = ptx::probe_clock();
                const bool leader = (warp - kWarpXform0) % C::kGroupWarps == 0;
                if (leader) NVFP4_CTRACE(0, it);
                const uint32_t a_smem = smem + C::kOffA + ra.slot * C::kSlotA;
                uint32_t w[C::kBpt][8];
#pragma unroll
                for (uint32_t j = 0; j < C::kBpt; ++j) {
                    const uint32_t k = (first_block + j) * 16u;
                    const uint4 lo = ptx::lds128(a_smem + xform::a_bf16_offset<C::kRows>(lrow, k));
                    const uint4 hi = ptx::lds128(a_smem + xform::a_bf16_offset<C::kRows>(lrow, k + 8));
                    w[j][0] = lo.x; w[j][1] = lo.y; w[j][2] = lo.z; w[j][3] = lo.w;
                    w[j][4] = hi.x; w[j][5] = hi.y; w[j][6] = hi.z; w[j][7] = hi.w;
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(a_empty + ra.slot);   // the tile now lives in registers
                const long long xt1 = ptx::probe_clock();
                ptx::probe_count(pa, 2, xt1 - xt0);
                xform::Block16 blk[C::kBpt];
#pragma unroll
                for (uint32_t j = 0; j < C::kBpt; ++j) xform::decompose_block16<kResidual, kPolicy>(w[j], blk[j]);
                // the scale bytes of one K atom (four 16-blocks of a row) -> one word, held by the atom's first thread
                uint32_t s0w, s1w;
                if constexpr (C::kBpt == 1) {
                    const uint32_t sh = (first_block & 3u) * 8u;
                    s0w = blk[0].s0 << sh; s1w = blk[0].s1 << sh;
                    s0w |= __shfl_xor_sync(0xffffffffu, s0w, 1); s0w |= __shfl_xor_sync(0xffffffffu, s0w, 2);
                    if constexpr (kResidual) { s1w |= __shfl_xor_sync(0xffffffffu, s1w, 1); s1w |= __shfl_xor_sync(0xffffffffu, s1w, 2); }
                } else {
                    const uint32_t sh = (first_block & 2u) * 8u;
                    s0w = (blk[0].s0 | (blk[1].s0 << 8)) << sh; s1w = (blk[0].s1 | (blk[1].s1 << 8)) << sh;
                    s0w |= __shfl_xor_sync(0xffffffffu, s0w, 1);
                    if constexpr (kResidual) s1w |= __shfl_xor_sync(0xffffffffu, s1w, 1);
                }
                const long long xt2 = ptx::probe_clock();
                ptx::probe_count(pa, 3, xt2 - xt1);
                if (leader) NVFP4_CTRACE(1, it);
                // every tensor core of the cluster must be done with this slot before anyone rewrites it
                if (!ptx::mbar_wait_sleep<true>(p_empty + rp.slot, rp.phase ^ 1, abort_flag, 32, pa, 1)) { give_up(1); break; }
                const long long xt3 = ptx::probe_clock();
                if (leader) NVFP4_CTRACE(2, it);
                const uint32_t codes = smem + C::kOffCodes + rp.slot * C::kSlotCodes + code_off;
                const uint32_t scales = smem + C::kOffScales + rp.slot * C::kSlotScales + sf_off;
                if constexpr (C::kBpt == 1) {
                    ptx::sts64(codes, blk[0].q0[0], blk[0].q0[1]);
                    if constexpr (kResidual) ptx::sts64(codes + C::kPassOffset, blk[0].q1[0], blk[0].q1[1]);
                } else {
                    ptx::sts128(codes, blk[0].q0[0], blk[0].q0[1], blk[1].q0[0], blk[1].q0[1]);
                    if constexpr (kResidual) ptx::sts128(codes + C::kPassOffset, blk[0].q1[0], blk[0].q1[1], blk[1].q1[0], blk[1].q1[1]);
                }
                if (sf_writer) {
                    ptx::sts32(scales, s0w);
                    if constexpr (kResidual) ptx::sts32(scales + kKAtoms * C::kRows * 4, s1w);
                }
                ptx::fence_proxy_async_smem();                   // own stores -> async proxy (MMA reads, bulk-copy reads)
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(p_full + rp.slot);
                    ptx::mbar_arrive(share_full + rp.slot);      // the push warp takes it from here
                }
                ptx::probe_count(pa, 4, ptx::probe_clock() - xt3);
                if (leader) NVFP4_CTRACE(3, it);
            }
        }
    }

    ptx::probe_add(32 + (warp < 4 ? warp : (warp < kWarpXform0 ? 4 : 8)), ptx::probe_clock() - probe_start);
    if (warp == kWarpTma) ptx::probe_flush(pa, 15);
    else if (warp == kWarpTmaA) ptx::probe_flush(pa, 16);
    else if (warp == kWarpPush) ptx::probe_flush(pa, 14);
    else if (warp == kWarpMma) ptx::probe_flush(pa, 2, -1, -1, 5);
    else if (warp < kWarpEpi0) ptx::probe_flush(pa, -1, 10, 13);
    else if (warp < kWarpXform0) ptx::probe_flush(pa, -1, -1, -1, 17);
    else ptx::probe_flush(pa, 11, 12, 18, 19, 20);
    // teardown: nobody leaves while a peer may still write into its shared memory or signal its barriers
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == kWarpMma) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc<kTmemCols>(tmem_base);
    }
}

template <uint32_t CL, bool kResidual, int kPolicy>
int launch_variant(const void* a, int64_t lda, const void* b, const void* sfb, int M, int N, int K, int E,
                   const Params& p, bool pdl, int num_sms, cudaStream_t stream)
{
    using C = Cfg<CL, kResidual>;
    CUtensorMap tm_a, tm_b, tm_sfb;
    int rc = host::encode_tensor_map_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, K, M, lda * 2, 64, C::kRows,
                                        CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = host::encode_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, K / 2, static_cast<uint64_t>(E) * N,
                                    K / 2, BK / 2, BN, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    rc = host::encode_tensor_map_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, sfb, N,
                                    static_cast<uint64_t>(E) * (K / 64), static_cast<uint64_t>(N) * 4, BN, kKAtoms,
                                    CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    auto kernel = gemm_cluster_kernel<CL, kResidual, kPolicy>;
    static int max_clusters[host::kMaxDevices] = {};
    int dev = 0;
    NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemAlloc;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (max_clusters[dev] == 0) {
        NVFP4_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemAlloc));
        cfg.gridDim = dim3(static_cast<unsigned>(num_sms / CL * CL));
        int n = 0;
        NVFP4_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
        if (n <= 0) return host::fail(NVFP4_E_CUDA, "no cluster of %u CTAs fits on this device", CL);
        max_clusters[dev] = n;
    }
    const int num_super = (M / static_cast<int>(BM)) * (N / static_cast<int>(BN * CL));
    int clusters = max_clusters[dev] < num_sms / static_cast<int>(CL) ? max_clusters[dev] : num_sms / static_cast<int>(CL);
    if (clusters > num_super) clusters = num_super;
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * CL));
    cfg.numAttrs = pdl ? 2 : 1;
    NVFP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, tm_sfb, p));
    return NVFP4_OK;
}

}  // namespace

// cluster = 2 or 4 CTAs per activation tile; N must be a multiple of 256 * cluster.
int launch_gemm_cluster(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                        int64_t ldd, const int32_t* m_indices, int M, int N, int K, int E, bool residual,
                        int cluster, int policy, int group_m, bool pdl, int num_sms, int32_t* status, cudaStream_t stream)
{
    Params p;
    p.gw = gw;
    p.m_indices = m_indices;
    p.d = static_cast<__nv_bfloat16*>(d);
    p.ldd = ldd;
    p.m = M; p.n = N; p.k = K;
    p.group_m = group_m > 0 ? group_m : 8;
    p.status = status;
    return host::with_policy(policy, [&](auto pol) {
        constexpr int kP = decltype(pol)::value;
        if (cluster == 4)
            return residual ? launch_variant<4, true, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                            : launch_variant<4, false, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
        return residual ? launch_variant<2, true, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream)
                        : launch_variant<2, false, kP>(a, lda, b, sfb, M, N, K, E, p, pdl, num_sms, stream);
    });
}

#ifdef NVFP4_PROBE
extern "C" __attribute__((visibility("default"))) int nvfp4_probe_read_cluster(unsigned long long* out64, int reset)
{
    cudaMemcpyFromSymbol(out64, ptx::g_probe, sizeof(unsigned long long) * 64);
    if (reset) { unsigned long long z[64] = {}; cudaMemcpyToSymbol(ptx::g_probe, z, sizeof z); }
    return 0;
}
extern "C" __attribute__((visibility("default"))) int nvfp4_probe_read_ctrace(long long* out)
{
    cudaMemcpyFromSymbol(out, g_ctrace, sizeof(long long) * 16 * 96);
    return 0;
}
#endif

}  // namespace nvfp4
