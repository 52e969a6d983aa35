// Grouped dual-NVFP4 GEMM, normal orientation, Algorithm 1 inside the main loop, with the activation
// transform shared by the CTAs of a thread-block cluster (four, or two).
//
// The CTAs of a cluster work on the same 128 token rows and on neighbouring 256-column weight tiles.  The
// quantised activation tile (A0, A1 and their scales) is the same for all of them, so each CTA loads and
// transforms only its 128 / CL rows and its transform threads write the products straight into the P slot of
// EVERY CTA of the cluster: ordinary stores into the own shared memory, `st.shared::cluster` stores into the
// peers' (distributed shared memory).  A warp's stores cover whole rows of the packed tile (256 contiguous
// bytes per instruction), and one `mbarrier.arrive.release.cluster` per warp and destination hands them over.
// Per CTA and K block that divides the Algorithm-1 arithmetic -- which saturates the issue slots of a
// single-CTA kernel -- by CL, while the tensor work per CTA is unchanged.  Nothing quantised is ever written
// to global memory.
//
// An earlier form of this kernel pushed each CTA's finished share to its peers with shared-to-shared bulk
// copies issued by a warp of their own; those copies were measured at ~6 B/clk per CTA and the extra hop
// (transform -> push warp -> copy -> peer) set the pace of the whole kernel.
//
// The scale factors reach tensor memory through tcgen05.st issued by the (otherwise idle) epilogue warps, not
// through tensor-memory copies issued by the MMA thread; see the MMA role below.
//
// Barriers: P-full of a CTA counts one arrival per transform warp of every CTA of the cluster; P-empty counts
// one tcgen05.commit per CTA, delivered to all CTAs by the commit's cluster mask, so a slot is rewritten
// (locally or by a peer) only after every tensor core has read it.  The P ring, the weight ring and the scale
// columns in tensor memory have the same depth and advance together, so that one commit per K block frees
// all three, and the MMA thread waits on a single barrier per K block (scales-in-tensor-memory, which the
// scale warps signal only after they have seen P-full and B-full themselves).  No load in this file is a
// multicast: the cross-CTA traffic is plain stores, mbarrier signalling and the commit mask.
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
constexpr uint32_t kSlotP0 = BM * BK / 2;                       // 8192: one packed pass
constexpr uint32_t kSlotSFA = kKAtoms * 512;                    // 1024
constexpr uint32_t kSlotB = BN * BK / 2, kSlotSFB = kKAtoms * 2 * 512;
// warp 3 has no role; it keeps the epilogue warps on warp ids whose low two bits are their tensor-memory quadrant
constexpr uint32_t kWarpTma = 0, kWarpMma = 1, kWarpTmaA = 2, kWarpEpi0 = 4, kNumEpiWarps = 8, kWarpXform0 = 12, kXformWarps = 8;
constexpr uint32_t kThreads = (kWarpXform0 + kXformWarps) * 32;   // 640
// tensor memory: 256 accumulator columns, then one buffer of 32 scale columns (SFA0 8, SFA1 8, SFB 16) per
// slot of the operand rings
constexpr uint32_t kTmemCols = 512, kColAcc = 0, kColSF = 256, kSfBufCols = 32, kSfA0 = 0, kSfA1 = 8, kSfB = 16;

template <uint32_t CL>
struct Cfg {
    static_assert(CL == 2 || CL == 4, "cluster of two or four CTAs");
    static constexpr uint32_t kRows = BM / CL;                  // rows this CTA loads and transforms
    static constexpr uint32_t kSlotA = kRows * BK * 2;          // 16 KB (pairs), 8 KB (quads)
    static constexpr uint32_t kBpt = kRows * (BK / 16) / (kXformWarps * 32);   // 16-blocks per transform thread: 2 or 1
    static_assert(kBpt == 1 || kBpt == 2, "one or two 16-blocks per thread");
    static constexpr uint32_t kDepthA = CL == 4 ? 6 : 4, kDepthP = 4, kDepthB = kDepthP;   // P, B and scale columns move together
    static_assert(kColSF + kDepthP * kSfBufCols <= kTmemCols, "scale columns");
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffA0 = kOffA + kDepthA * kSlotA;
    static constexpr uint32_t kOffA1 = kOffA0 + kDepthP * kSlotP0;
    static constexpr uint32_t kOffB = kOffA1 + kDepthP * kSlotP0;
    static constexpr uint32_t kOffSFA0 = kOffB + kDepthB * kSlotB;
    static constexpr uint32_t kOffSFA1 = kOffSFA0 + kDepthP * kSlotSFA;
    static constexpr uint32_t kOffSFB = kOffSFA1 + kDepthP * kSlotSFA;
    static constexpr uint32_t kOffStage = kOffSFB + kDepthB * kSlotSFB;
    static constexpr uint32_t kOffBars = kOffStage + kNumEpiWarps * gemm::kStageWarp;
    static constexpr uint32_t kNumBars = 2 * kDepthA + 3 * kDepthP + kDepthB + 2;
    static constexpr uint32_t kSmemAlloc = kOffBars + kNumBars * 8 + 16 + 1024;
    static_assert(kSmemAlloc <= 232448, "shared memory budget");
};

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
    using C = Cfg<CL>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem - ptx::smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kOffBars);
    uint64_t* a_full = bars;
    uint64_t* a_empty = a_full + C::kDepthA;
    uint64_t* p_full = a_empty + C::kDepthA;         // every CTA's transform warps have written their rows of this slot
    uint64_t* p_empty = p_full + C::kDepthP;         // every CTA's tensor core has read this slot
    uint64_t* b_full = p_empty + C::kDepthP;
    uint64_t* sf_full = b_full + C::kDepthB;         // [kDepthP]: scales of a K block are in tensor memory
    uint64_t* tmem_full = sf_full + C::kDepthP;
    uint64_t* tmem_empty = tmem_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_cta_rank();

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < C::kDepthA; ++i) { ptx::mbar_init(a_full + i, 1); ptx::mbar_init(a_empty + i, kXformWarps); }
        for (uint32_t i = 0; i < C::kDepthP; ++i) {
            ptx::mbar_init(p_full + i, kXformWarps * CL);       // one arrival per transform warp of every CTA
            ptx::mbar_init(p_empty + i, CL);                    // one commit per CTA of the cluster
            ptx::mbar_init(sf_full + i, kNumEpiWarps);
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
    ptx::ProbeAcc pa;
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
                    if (!ptx::mbar_wait_cluster(p_empty + rb.slot, rb.phase ^ 1, abort_flag)) { give_up(1); break; }
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
                    if (!ptx::mbar_wait_impl(a_empty + ra.slot, ra.phase ^ 1, abort_flag)) { give_up(1); break; }
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
        Ring rp;
        uint32_t acc_phase = 0;
        constexpr uint32_t idesc = ptx::make_idesc_nvf4(BM, BN);
        constexpr uint16_t kAllCtas = static_cast<uint16_t>((1u << CL) - 1u);
        for (uint32_t st = cid; st < num_super && ok; st += ncl) {
            if (!ptx::mbar_wait(tmem_empty, acc_phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                // the scale warps arrive here only after they have seen this slot's P-full (acquired at cluster
                // scope) and B-full complete, so this one wait also covers the operand tiles in shared memory
                if (!ptx::mbar_wait(sf_full + rp.slot, rp.phase, abort_flag, pa, 3)) { give_up(1); break; }
                ptx::tcgen05_fence_after_sync();
                if (lane == 0) {
                    const uint32_t a0 = smem + C::kOffA0 + rp.slot * kSlotP0;
                    const uint32_t a1 = smem + C::kOffA1 + rp.slot * kSlotP0;
                    const uint32_t b = smem + C::kOffB + rp.slot * kSlotB;
                    const uint32_t sf = tmem_base + kColSF + rp.slot * kSfBufCols;
#pragma unroll
                    for (uint32_t a = 0; a < kKAtoms; ++a) {
                        const uint64_t desc_b = ptx::make_smem_desc(b + a * 32, 512, ptx::kSwizzle64B);
                        ptx::tcgen05_mma_nvf4(tmem_base + kColAcc, ptx::make_smem_desc(a0 + a * 32, 512, ptx::kSwizzle64B), desc_b,
                                              idesc, sf + kSfA0 + 4 * a, sf + kSfB + 8 * a, (kb | a) != 0 ? 1u : 0u);
                        if constexpr (kResidual)
                            ptx::tcgen05_mma_nvf4(tmem_base + kColAcc, ptx::make_smem_desc(a1 + a * 32, 512, ptx::kSwizzle64B),
                                                  desc_b, idesc, sf + kSfA1 + 4 * a, sf + kSfB + 8 * a, 1u);
                    }
                    // one commit per K block, to every CTA of the cluster: it frees the P slot, the weight slot and
                    // the scale columns of this ring position
                    ptx::tcgen05_commit_cluster(p_empty + rp.slot, kAllCtas);
                    if (kb == num_kb - 1) ptx::tcgen05_commit(tmem_full);
                }
                __syncwarp();
                rp.advance<C::kDepthP>();
            }
            acc_phase ^= 1;
        }
    } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + kNumEpiWarps) {
        // ================= scale warps during the main loop, epilogue at the end of a tile =================
        // Eight warps: two per 32-lane quadrant of tensor memory.  During the main loop they carry the scale
        // factors from shared to tensor memory with tcgen05.st (a warp reaches only its own quadrant of lanes,
        // and the MMA wants each quadrant to hold a copy): lane r of each quadrant gets the scale words of rows
        // r, r + 32, r + 64, r + 96 in four consecutive columns.  Warps 4-7 take the weight scales straight from
        // the rows TMA landed (which also does the transposition a tensor-memory copy would have needed), warps
        // 8-11 the activation scales of both passes.  There is one set of scale columns per ring position; it is
        // rewritten once the MMAs that used it have retired (the P-empty barrier).
        // At the end of a tile each warp drains 128 of the 256 accumulator columns, 64 at a time, and hands the
        // accumulator back as soon as its last column has left tensor memory, before that half is stored.
        const uint32_t quad = warp & 3, half = (warp - kWarpEpi0) >> 2;
        uint32_t acc_phase = 0;
        Ring rp;
        for (uint32_t st = cid; st < num_super && ok; st += ncl) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                const uint32_t sf = tmem_base + ((quad * 32) << 16) + kColSF + rp.slot * kSfBufCols;
                const bool src_ok = half == 0 ? ptx::mbar_wait(b_full + rp.slot, rp.phase, abort_flag, pa, 1)
                                              : ptx::mbar_wait_cluster(p_full + rp.slot, rp.phase, abort_flag, pa, 1);
                if (!src_ok) { give_up(1); break; }
                // the columns of this ring position are free once its previous MMAs have retired
                if (!ptx::mbar_wait_cluster(p_empty + rp.slot, rp.phase ^ 1, abort_flag, pa, 2)) { give_up(1); break; }
                ptx::tcgen05_fence_after_sync();
                if (half == 0) {
                    const uint32_t sfb = smem + C::kOffSFB + rp.slot * kSlotSFB + lane * 4;
                    uint32_t v[16];
#pragma unroll
                    for (uint32_t i = 0; i < kKAtoms * 2; ++i)
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) v[4 * i + j] = ptx::lds32(sfb + i * 512 + j * 128);
                    ptx::tmem_st_32x32b(sf + kSfB, v);
                } else {
                    uint32_t v[kResidual ? 16 : 8];
#pragma unroll
                    for (uint32_t a = 0; a < kKAtoms; ++a) {
                        const uint4 q = ptx::lds128(smem + C::kOffSFA0 + rp.slot * kSlotSFA + a * 512 + lane * 16);
                        v[4 * a] = q.x; v[4 * a + 1] = q.y; v[4 * a + 2] = q.z; v[4 * a + 3] = q.w;
                        if constexpr (kResidual) {
                            const uint4 r = ptx::lds128(smem + C::kOffSFA1 + rp.slot * kSlotSFA + a * 512 + lane * 16);
                            v[8 + 4 * a] = r.x; v[8 + 4 * a + 1] = r.y; v[8 + 4 * a + 2] = r.z; v[8 + 4 * a + 3] = r.w;
                        }
                    }
                    ptx::tmem_st_32x32b(sf + kSfA0, v);          // SFA0 columns 0-7, SFA1 columns 8-15
                }
                ptx::tmem_st_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(sf_full + rp.slot);
                rp.advance<C::kDepthP>();
            }
            if (!ok) break;
            uint32_t m_blk, ns;
            gemm::tile_coords(st, num_m, num_ns, p.group_m, m_blk, ns);
            const uint32_t n_blk = ns * CL + rank;
            const int32_t e = max(0, __ldg(p.m_indices + m_blk * BM));
            const float g = __ldg(p.gw + e);
            if (!ptx::mbar_wait_impl(tmem_full, acc_phase, abort_flag)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + kColAcc + half * (BN / 2);
            const uint32_t stage = smem + C::kOffStage + (warp - kWarpEpi0) * gemm::kStageWarp;
            __nv_bfloat16* d_lane = p.d + static_cast<int64_t>(m_blk * BM + quad * 32 + (lane >> 3)) * p.ldd + n_blk * BN +
                                    half * (BN / 2) + (lane & 7u) * 8;
            // 128 columns in three rounds (64, 32, 32) so that at most 64 FP32 values are live beside the packed ones
            uint32_t o[32], o2[32];
            {
                uint32_t va[32], vb[32];
                ptx::tmem_ld_32x32b_x32(taddr, va);
                ptx::tmem_ld_32x32b_x32(taddr + 32, vb);
                ptx::tmem_ld_wait();
                gemm::scale_pack_bf16(va, g, o);
                gemm::scale_pack_bf16(vb, g, o + 16);
            }
            {
                uint32_t vc[32];
                ptx::tmem_ld_32x32b_x32(taddr + 64, vc);
                ptx::tmem_ld_wait();
                gemm::scale_pack_bf16(vc, g, o2);
            }
            {
                uint32_t vd[32];
                ptx::tmem_ld_32x32b_x32(taddr + 96, vd);
                ptx::tmem_ld_wait();
                ptx::tcgen05_fence_before_sync();                 // everything has left tensor memory
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tmem_empty);
                gemm::scale_pack_bf16(vd, g, o2 + 16);
            }
            gemm::store_rows_staged(o, stage, d_lane, p.ldd, lane);
            gemm::store_rows_staged(o2, stage, d_lane + 64, p.ldd, lane);
            acc_phase ^= 1;
        }
    } else if (warp >= kWarpXform0) {
        // ================= transform: this CTA's rows into the P slot of every CTA of the cluster =================
        // Thread t owns one row of this CTA's share and one (quads) or two adjacent (pairs) 16-blocks of it: the
        // 8 (4) threads of a row are neighbours in a warp, so a warp's stores of packed codes cover 4 (8) whole
        // 64-byte rows -- contiguous bytes, which is what the path to a peer's shared memory wants -- and the
        // scale bytes of a K atom are gathered into one word with two shuffles.  Row m of the MMA tile is token
        // row m: the CTA of rank c owns rows [c * kRows, (c + 1) * kRows).
        const uint32_t t = threadIdx.x - kWarpXform0 * 32;
        constexpr uint32_t kPerRow = 8 / C::kBpt;                                  // threads per row
        const uint32_t lrow = t / kPerRow, piece = t % kPerRow;                    // row inside this CTA's share
        const uint32_t mrow = rank * C::kRows + lrow;                              // its row in the MMA tile
        const uint32_t first_block = piece * C::kBpt;
        uint32_t peer_base[CL];                                                    // shared::cluster address of every CTA's window
#pragma unroll
        for (uint32_t c = 0; c < CL; ++c) peer_base[c] = ptx::map_to_cta(smem, c);
        // where this thread's products go, relative to a slot (the same in every CTA)
        const uint32_t code_off = xform::fp4_offset<BK>(mrow, (first_block * 16u) & ~31u) + (C::kBpt == 1 ? ((first_block & 1u) << 3) : 0u);
        const uint32_t sf_off = (first_block >> 2) * 512u + xform::sf_word_offset(mrow);
        const bool sf_writer = (first_block & 3u) == 0;                           // the thread that holds a K atom's scale word
        Ring ra, rp;
        for (uint32_t st = cid; st < num_super && ok; st += ncl) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!ptx::mbar_wait(a_full + ra.slot, ra.phase, abort_flag, pa, 0)) { give_up(1); break; }
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
                // every tensor core of the cluster must be done with this slot before anyone rewrites it
                if (!ptx::mbar_wait_cluster(p_empty + rp.slot, rp.phase ^ 1, abort_flag, pa, 1)) { give_up(1); break; }
                const uint32_t off_a0 = C::kOffA0 + rp.slot * kSlotP0 + code_off, off_a1 = C::kOffA1 + rp.slot * kSlotP0 + code_off;
                const uint32_t off_s0 = C::kOffSFA0 + rp.slot * kSlotSFA + sf_off, off_s1 = C::kOffSFA1 + rp.slot * kSlotSFA + sf_off;
#pragma unroll
                for (uint32_t c = 0; c < CL; ++c) {
                    const uint32_t base = peer_base[c];          // c == rank: the own window, reached the same way
                    if constexpr (C::kBpt == 1) {
                        ptx::st_cluster64(base + off_a0, blk[0].q0[0], blk[0].q0[1]);
                        if constexpr (kResidual) ptx::st_cluster64(base + off_a1, blk[0].q1[0], blk[0].q1[1]);
                    } else {
                        ptx::st_cluster128(base + off_a0, blk[0].q0[0], blk[0].q0[1], blk[1].q0[0], blk[1].q0[1]);
                        if constexpr (kResidual) ptx::st_cluster128(base + off_a1, blk[0].q1[0], blk[0].q1[1], blk[1].q1[0], blk[1].q1[1]);
                    }
                    if (sf_writer) {
                        ptx::st_cluster32(base + off_s0, s0w);
                        if constexpr (kResidual) ptx::st_cluster32(base + off_s1, s1w);
                    }
                }
                // generic-proxy stores (own and remote shared memory) -> async proxy (the tensor cores' operand reads),
                // then one releasing arrival per destination CTA for the whole warp
                ptx::fence_proxy_async_all();
                __syncwarp();
                if (lane < CL) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(p_full + rp.slot), lane));
                ra.advance<C::kDepthA>();
                rp.advance<C::kDepthP>();
            }
        }
    }

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
    using C = Cfg<CL>;
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

}  // namespace nvfp4
