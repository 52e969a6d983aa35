// Grouped dual-NVFP4 GEMM, normal orientation, with the activation transform shared by
// the CTAs of a thread-block cluster (two, or four: the text below describes pairs; with four
// CTAs every share is half as large and goes to three peers).
//
// Both CTAs work on the same 128 token rows and on two neighbouring 256-column weight
// tiles.  The quantised activation tile (A0, A1 and their scales) is the same for both, so
// each CTA loads and transforms only 64 of the rows, writes its products into its own
// shared memory and then pushes the finished share to its peer with a handful of bulk
// shared-to-shared copies (cp.async.bulk, shared::cta -> shared::cluster, completing bytes on
// the peer's P-full barrier).  Per CTA and K block that halves the Algorithm-1 arithmetic,
// which saturates the integer/convert pipe of the single-CTA kernel, and the BF16 bytes
// coming in; the tensor work per CTA is unchanged.
//
// For the pushed share to be a few contiguous runs, MMA row m of the tile is token row
// 64 * ((m % 32) / 16) + 16 * (m / 32) + m % 16: the CTA of rank c owns the MMA rows whose
// m % 32 lies in [16c, 16c + 16) -- four runs of 16 packed rows (1 KB each) and one run of
// 256 bytes inside every 512-byte scale atom.  The epilogue applies the same map to the
// accumulator lanes.
//
// The scale factors reach tensor memory through tcgen05.st issued by the (otherwise idle) epilogue
// warps, not through tensor-memory copies issued by the MMA thread; see the MMA role below.
//
// Barriers: P-full of a CTA counts its own eight transform warps plus the bytes of the
// peer's copies; P-empty counts one tcgen05.commit per CTA, delivered to both CTAs by the
// commit's cluster mask, so a slot is rewritten (locally or by the peer's copies) only after
// both tensor cores have read it.  The P ring, the weight ring and the scale columns in tensor
// memory have the same depth and advance together, so that one commit per K block frees all
// three, and the MMA thread waits on a single barrier per K block (scales-in-tensor-memory, which
// the scale warps signal only after they have seen P-full and B-full themselves).  No load in
// this file is a multicast: the cross-CTA traffic is the bulk copies, mbarrier signalling and
// the commit mask.
#include <cuda_bf16.h>

#include "host_common.hpp"
#include "launchers.hpp"
#include "transform.cuh"

namespace nvfp4 {
namespace {

constexpr uint32_t BM = 128, BN = 256, BK = 128, kKAtoms = 2;
constexpr uint32_t kSlotP0 = BM * BK / 2;                       // 8192: one packed pass
constexpr uint32_t kSlotSFA = kKAtoms * 512;                    // 1024
constexpr uint32_t kSlotB = BN * BK / 2, kSlotSFB = kKAtoms * 2 * 512;
constexpr uint32_t kWarpTma = 0, kWarpMma = 1, kWarpPush = 2, kWarpTmaA = 3, kWarpEpi0 = 4, kNumEpiWarps = 8, kWarpXform0 = 12;
constexpr uint32_t kThreadsFor(uint32_t xform_warps) { return (kWarpXform0 + xform_warps) * 32; }   // 640 or 896
// tensor memory: 256 accumulator columns, then one buffer of 32 scale columns (SFA0 8, SFA1 8, SFB 16) per
// slot of the operand rings
constexpr uint32_t kTmemCols = 512, kColAcc = 0, kColSF = 256, kSfBufCols = 32, kSfA0 = 0, kSfA1 = 8, kSfB = 16;

template <uint32_t CL, uint32_t kXW>
struct Cfg {
    static_assert(CL == 2 || CL == 4, "cluster of two or four CTAs");
    static_assert(kXW == 8 || kXW == 16, "transform warps");
    static constexpr uint32_t kRows = BM / CL;                  // rows this CTA loads and transforms
    static constexpr uint32_t kRun = 32 / CL;                   // consecutive MMA rows it owns in every group of 32
    static constexpr uint32_t kSlotA = kRows * BK * 2;          // 16 KB (pairs), 8 KB (quads)
    static constexpr uint32_t kActiveWarps = kXW;               // every transform warp takes part
    static constexpr uint32_t kBpt = kRows * (BK / 16) / (kXW * 32);   // 16-blocks per transform thread: 1 or 2
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
    // epilogue staging: per warp four output rows of 64 BF16 (128 bytes, padded to 144 against bank conflicts)
    static constexpr uint32_t kStageRow = 144, kStageWarp = 4 * kStageRow;
    static constexpr uint32_t kOffStage = kOffSFB + kDepthB * kSlotSFB;
    static constexpr uint32_t kOffBars = kOffStage + kNumEpiWarps * kStageWarp;
    static constexpr uint32_t kNumBars = 2 * kDepthA + 4 * kDepthP + kDepthB + 2;
    static constexpr uint32_t kSmemAlloc = kOffBars + kNumBars * 8 + 16 + 1024;
    static_assert(kSmemAlloc <= 232448, "shared memory budget");
    // what one CTA pushes to one peer per K block and pass: four runs of kRun packed rows, one run per scale atom
    static constexpr uint32_t kRunBytes = kRun * 64, kSfRunBytes = kRun * 16;
    static constexpr uint32_t kBytesPerPass = 4 * kRunBytes + kKAtoms * kSfRunBytes;
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

struct Ring {
    uint32_t slot = 0, phase = 0;
    template <uint32_t kDepth>
    __device__ __forceinline__ void advance()
    {
        if (++slot == kDepth) { slot = 0; phase ^= 1; }
    }
};

__device__ __forceinline__ void super_tile_coords(uint32_t st, uint32_t num_m, uint32_t num_ns, uint32_t group_m,
                                                  uint32_t& m_blk, uint32_t& ns)
{
    const uint32_t per_group = group_m * num_ns;
    const uint32_t g = st / per_group, r = st % per_group;
    const uint32_t first = g * group_m;
    const uint32_t rows = min(group_m, num_m - first);
    m_blk = first + r % rows;
    ns = r / rows;
}

template <uint32_t CL, bool kResidual, uint32_t kXW>
__global__ void __launch_bounds__(kThreadsFor(kXW), 1)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_sfb, const Params p)
{
    using C = Cfg<CL, kXW>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem - ptx::smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kOffBars);
    uint64_t* a_full = bars;
    uint64_t* a_empty = a_full + C::kDepthA;
    uint64_t* p_full = a_empty + C::kDepthA;
    uint64_t* p_empty = p_full + C::kDepthP;
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
        for (uint32_t i = 0; i < C::kDepthA; ++i) { ptx::mbar_init(a_full + i, 1); ptx::mbar_init(a_empty + i, C::kActiveWarps); }
        for (uint32_t i = 0; i < C::kDepthP; ++i) {
            ptx::mbar_init(p_full + i, C::kActiveWarps + 1);    // own transform warps + the push warp; peers' shares arrive as bytes
            ptx::mbar_init(share_full + i, C::kActiveWarps);
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

    const uint32_t num_m = p.m / BM, num_ns = p.n / (BN * CL), num_kb = p.k / BK;
    const uint32_t num_super = num_m * num_ns;
    const uint32_t cid = ptx::cluster_id_x(), ncl = ptx::num_clusters_x();
    bool ok = true;
    ptx::ProbeAcc pa;
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
                super_tile_coords(st, num_m, num_ns, p.group_m, m_blk, ns);
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
        }
    } else if (warp == kWarpTmaA) {
        // ================= activation producer: this CTA's share of the rows =================
        if (lane == 0) {
            Ring ra;
            for (uint32_t st = cid; st < num_super && ok; st += ncl) {
                uint32_t m_blk, ns;
                super_tile_coords(st, num_m, num_ns, p.group_m, m_blk, ns);
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
                // the scale warps arrive here only after they have seen this slot's P-full and B-full complete, so
                // this one wait also covers the operand tiles in shared memory
                if (!ptx::mbar_wait(sf_full + rp.slot, rp.phase, abort_flag, pa, 3)) { give_up(1); break; }
                ptx::tcgen05_fence_after_sync();
                const long long pt1 = ptx::probe_clock();
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
                    const long long pt2 = ptx::probe_clock();
                    ptx::probe_count(pa, 5, pt2 - pt1);
                    // one commit per K block, to every CTA of the cluster: it frees the P slot, the weight slot and
                    // the scale columns of this ring position
                    ptx::tcgen05_commit_cluster(p_empty + rp.slot, kAllCtas);
                    if (kb == num_kb - 1) ptx::tcgen05_commit(tmem_full);
                    ptx::probe_count(pa, 6, ptx::probe_clock() - pt2);
                }
                __syncwarp();
                rp.advance<C::kDepthP>();
            }
            acc_phase ^= 1;
        }
    } else if (warp == kWarpPush) {
        // ================= push: this CTA's finished share to every peer =================
        // One bulk shared-to-shared copy per contiguous run, to the same offsets in the peer's slot; the bytes
        // complete on the peer's P-full barrier.  The lanes of the warp issue one copy each, so the transform
        // warps never wait for copy issue and the list costs one instruction slot per 32 copies.
        constexpr uint32_t kPerPeer = (kResidual ? 2u : 1u) * (4u + kKAtoms);
        constexpr uint32_t kCopies = (CL - 1) * kPerPeer;
        constexpr uint32_t kPeerBytes = (CL - 1) * (kResidual ? 2u : 1u) * C::kBytesPerPass;
        Ring rp;
        for (uint32_t st = cid; st < num_super && ok; st += ncl) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!ptx::mbar_wait_impl(share_full + rp.slot, rp.phase, abort_flag)) { give_up(1); break; }
                const uint32_t off_a0 = C::kOffA0 + rp.slot * kSlotP0, off_a1 = C::kOffA1 + rp.slot * kSlotP0;
                const uint32_t off_s0 = C::kOffSFA0 + rp.slot * kSlotSFA, off_s1 = C::kOffSFA1 + rp.slot * kSlotSFA;
                for (uint32_t i = lane; i < kCopies; i += 32) {
                    const uint32_t peer = (rank + 1 + i / kPerPeer) % CL;
                    uint32_t j = i % kPerPeer, off, bytes;
                    const bool second = j >= 4 + kKAtoms;        // second pass (A1 / SFA1)
                    if (second) j -= 4 + kKAtoms;
                    if (j < 4) {
                        off = (second ? off_a1 : off_a0) + (32 * j + C::kRun * rank) * 64;
                        bytes = C::kRunBytes;
                    } else {
                        off = (second ? off_s1 : off_s0) + (j - 4) * 512 + C::kRun * rank * 16;
                        bytes = C::kSfRunBytes;
                    }
                    ptx::bulk_copy_to_cta(ptx::map_to_cta(smem + off, peer), smem + off, bytes,
                                          ptx::map_to_cta(ptx::smem_u32(p_full + rp.slot), peer));
                }
                if (lane == 0) ptx::mbar_arrive_expect_tx(p_full + rp.slot, kPeerBytes);
                __syncwarp();
                rp.advance<C::kDepthP>();
            }
        }
    } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + kNumEpiWarps) {
        // ================= epilogue: TMEM -> x G_W -> BF16 -> global =================
        // Eight warps: two per 32-lane quadrant of tensor memory, each draining 128 of the 256 columns in
        // chunks of 16, with the load of the next chunk in flight while the current one is scaled, packed
        // and stored.  The accumulator is handed back to the MMA warp as soon as its last chunk has left
        // tensor memory, before that chunk is stored.
        //
        // During the mainloop the same warps carry the scale factors from shared to tensor memory with
        // tcgen05.st (a warp reaches only its own quadrant of lanes, and the MMA wants each quadrant to hold
        // a copy): lane r of each quadrant gets the scale words of rows r, r + 32, r + 64, r + 96 in four
        // consecutive columns.  Warps 4-7 take the weight scales straight from the rows TMA landed (which also
        // does the transposition a tensor-memory copy would have needed), warps 8-11 the activation scales of
        // both passes.  There is one set of scale columns per ring position; it is rewritten once the MMAs
        // that used it have retired (the P-empty barrier).
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
#pragma unroll
                    for (uint32_t i = 0; i < kKAtoms * 2; ++i)
                        ptx::tmem_st_32x32b_x4(sf + kSfB + 4 * i, ptx::lds32(sfb + i * 512), ptx::lds32(sfb + i * 512 + 128),
                                               ptx::lds32(sfb + i * 512 + 256), ptx::lds32(sfb + i * 512 + 384));
                } else {
#pragma unroll
                    for (uint32_t a = 0; a < kKAtoms; ++a) {
                        const uint4 v0 = ptx::lds128(smem + C::kOffSFA0 + rp.slot * kSlotSFA + a * 512 + lane * 16);
                        ptx::tmem_st_32x32b_x4(sf + kSfA0 + 4 * a, v0.x, v0.y, v0.z, v0.w);
                        if constexpr (kResidual) {
                            const uint4 v1 = ptx::lds128(smem + C::kOffSFA1 + rp.slot * kSlotSFA + a * 512 + lane * 16);
                            ptx::tmem_st_32x32b_x4(sf + kSfA1 + 4 * a, v1.x, v1.y, v1.z, v1.w);
                        }
                    }
                }
                ptx::tmem_st_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(sf_full + rp.slot);
                rp.advance<C::kDepthP>();
            }
            if (!ok) break;
            uint32_t m_blk, ns;
            super_tile_coords(st, num_m, num_ns, p.group_m, m_blk, ns);
            const uint32_t n_blk = ns * CL + rank;
            const int32_t e = max(0, __ldg(p.m_indices + m_blk * BM));
            const float g = __ldg(p.gw + e);
            if (!ptx::mbar_wait_impl(tmem_full, acc_phase, abort_flag)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            // Accumulator lane m = 32 * quad + lane holds token row kRows * (lane / kRun) + kRun * quad + lane % kRun.
            // A store instruction should write whole 128-byte lines, but in tensor memory a lane is a row: so 64
            // columns at a time are packed to BF16 in registers and go, four rows per pass, through a 576-byte
            // staging area (four lanes write their 128 bytes, the warp reads 16 bytes per lane and stores four
            // full lines).  One 16-byte store per lane and row cost thousands of partial-line requests per tile
            // and held up the loads and MMAs of the next tile.
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + kColAcc + half * (BN / 2);
            const uint32_t stage = smem + C::kOffStage + (warp - kWarpEpi0) * C::kStageWarp;
            const uint32_t rd = stage + (lane >> 3) * C::kStageRow + (lane & 7u) * 16;
#pragma unroll
            for (uint32_t hh = 0; hh < 2; ++hh) {
                uint32_t o[32];
#pragma unroll
                for (uint32_t q = 0; q < 2; ++q) {
                    uint32_t va[16], vb[16];
                    ptx::tmem_ld_32x32b_x16(taddr + hh * 64 + q * 32, va);
                    ptx::tmem_ld_32x32b_x16(taddr + hh * 64 + q * 32 + 16, vb);
                    ptx::tmem_ld_wait();
                    if (hh == 1 && q == 1) {
                        ptx::tcgen05_fence_before_sync();         // everything has left tensor memory
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(tmem_empty);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(va[2 * i]) * g, __uint_as_float(va[2 * i + 1]) * g);
                        const __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(vb[2 * i]) * g, __uint_as_float(vb[2 * i + 1]) * g);
                        o[16 * q + i] = *reinterpret_cast<const uint32_t*>(&h0);
                        o[16 * q + 8 + i] = *reinterpret_cast<const uint32_t*>(&h1);
                    }
                }
#pragma unroll 1
                for (uint32_t pass = 0; pass < 8; ++pass) {
                    if ((lane >> 2) == pass) {
                        const uint32_t wr = stage + (lane & 3u) * C::kStageRow;
#pragma unroll
                        for (uint32_t c = 0; c < 8; ++c) ptx::sts128(wr + c * 16, o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
                    }
                    __syncwarp();
                    const uint4 v = ptx::lds128(rd);
                    const uint32_t sl = 4 * pass + (lane >> 3);   // the lane whose row this thread stores a piece of
                    const uint32_t row = m_blk * BM + C::kRows * (sl / C::kRun) + C::kRun * quad + sl % C::kRun;
                    *reinterpret_cast<uint4*>(p.d + static_cast<int64_t>(row) * p.ldd + n_blk * BN + half * (BN / 2) + hh * 64 +
                                              (lane & 7u) * 8) = v;
                    __syncwarp();
                }
            }
            acc_phase ^= 1;
        }
    } else if (warp >= kWarpXform0) {
        // ================= transform: this CTA's rows into its own P slot =================
        const uint32_t t = threadIdx.x - kWarpXform0 * 32;
        const uint32_t lrow = t % C::kRows;                                                      // row inside this CTA's share
        const uint32_t mrow = 32 * (lrow / C::kRun) + C::kRun * rank + lrow % C::kRun;           // its row in the MMA tile
        const uint32_t first_block = (t / C::kRows) * C::kBpt;
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
                // every tensor core of the cluster must be done with this slot before anyone rewrites it
                if (!ptx::mbar_wait_cluster(p_empty + rp.slot, rp.phase ^ 1, abort_flag, pa, 1)) { give_up(1); break; }
                const uint32_t off_a0 = C::kOffA0 + rp.slot * kSlotP0, off_a1 = C::kOffA1 + rp.slot * kSlotP0;
                const uint32_t off_s0 = C::kOffSFA0 + rp.slot * kSlotSFA, off_s1 = C::kOffSFA1 + rp.slot * kSlotSFA;
                const uint32_t sf_base = (first_block >> 2) * 512u + xform::sf_word_offset(mrow);
                if constexpr (C::kBpt == 2) {
                    xform::Block16 blk[2];
                    xform::decompose_block16<kResidual>(w[0], blk[0]);
                    xform::decompose_block16<kResidual>(w[1], blk[1]);
                    const uint32_t off = xform::fp4_offset<BK>(mrow, first_block * 16u);
                    ptx::sts128(smem + off_a0 + off, blk[0].q0[0], blk[0].q0[1], blk[1].q0[0], blk[1].q0[1]);
                    if constexpr (kResidual)
                        ptx::sts128(smem + off_a1 + off, blk[0].q1[0], blk[0].q1[1], blk[1].q1[0], blk[1].q1[1]);
                    const uint32_t sf_addr = sf_base + (first_block & 2u);
                    ptx::sts16(smem + off_s0 + sf_addr, blk[0].s0 | (blk[1].s0 << 8));
                    if constexpr (kResidual) ptx::sts16(smem + off_s1 + sf_addr, blk[0].s1 | (blk[1].s1 << 8));
                } else {
                    xform::Block16 blk;
                    xform::decompose_block16<kResidual>(w[0], blk);
                    const uint32_t off = xform::fp4_offset<BK>(mrow, (first_block * 16u) & ~31u) + ((first_block & 1u) << 3);
                    ptx::sts64(smem + off_a0 + off, blk.q0[0], blk.q0[1]);
                    if constexpr (kResidual) ptx::sts64(smem + off_a1 + off, blk.q1[0], blk.q1[1]);
                    const uint32_t sf_addr = sf_base + (first_block & 3u);
                    ptx::sts8(smem + off_s0 + sf_addr, blk.s0);
                    if constexpr (kResidual) ptx::sts8(smem + off_s1 + sf_addr, blk.s1);
                }
                ptx::fence_proxy_async_smem();                   // own stores -> async proxy (MMA reads, bulk-copy reads)
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(p_full + rp.slot);
                    ptx::mbar_arrive(share_full + rp.slot);      // the push warp takes it from here
                }
                ra.advance<C::kDepthA>();
                rp.advance<C::kDepthP>();
            }
        }
    }

    ptx::probe_add(32 + (warp < 4 ? warp : (warp < kWarpXform0 ? 4 : 8)), ptx::probe_clock() - probe_start);
    if (warp == 1) ptx::probe_flush(pa, 2, 3, 4, 5, 20, 21, 22);
    else if (warp >= kWarpEpi0 && warp < kWarpXform0) ptx::probe_flush(pa, 9, 10, 13);
    else if (warp >= kWarpXform0) ptx::probe_flush(pa, 11, 12);
    // teardown: nobody leaves while a peer may still write into its shared memory
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == kWarpMma) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc<kTmemCols>(tmem_base);
    }
}

template <uint32_t CL, bool kResidual, uint32_t kXW>
int launch_variant(const void* a, int64_t lda, const void* b, const void* sfb, int M, int N, int K, int E,
                   const Params& p, int num_sms, cudaStream_t stream)
{
    using C = Cfg<CL, kXW>;
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
    auto kernel = gemm_cluster_kernel<CL, kResidual, kXW>;
    static int max_clusters[host::kMaxDevices] = {};
    int dev = 0;
    NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreadsFor(kXW));
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
    NVFP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, tm_sfb, p));
    return NVFP4_OK;
}

}  // namespace

// cluster = 2 or 4 CTAs per activation tile; N must be a multiple of 256 * cluster.
int launch_gemm_cluster(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                        int64_t ldd, const int32_t* m_indices, int M, int N, int K, int E, bool residual,
                        int cluster, int xform_warps, int group_m, int num_sms, int32_t* status, cudaStream_t stream)
{
    Params p;
    p.gw = gw;
    p.m_indices = m_indices;
    p.d = static_cast<__nv_bfloat16*>(d);
    p.ldd = ldd;
    p.m = M; p.n = N; p.k = K;
    p.group_m = group_m > 0 ? group_m : 8;
    p.status = status;
    // transform warps: 8 unless the caller asks for 16 (pairs only; measured equally fast, and 8 leave the
    // epilogue its registers)
    if (cluster == 4)
        return residual ? launch_variant<4, true, 8>(a, lda, b, sfb, M, N, K, E, p, num_sms, stream)
                        : launch_variant<4, false, 8>(a, lda, b, sfb, M, N, K, E, p, num_sms, stream);
    if (xform_warps == 16)
        return residual ? launch_variant<2, true, 16>(a, lda, b, sfb, M, N, K, E, p, num_sms, stream)
                        : launch_variant<2, false, 16>(a, lda, b, sfb, M, N, K, E, p, num_sms, stream);
    return residual ? launch_variant<2, true, 8>(a, lda, b, sfb, M, N, K, E, p, num_sms, stream)
                    : launch_variant<2, false, 8>(a, lda, b, sfb, M, N, K, E, p, num_sms, stream);
}

#ifdef NVFP4_PROBE
extern "C" __attribute__((visibility("default"))) int nvfp4_probe_read_cluster(unsigned long long* out64, int reset)
{
    cudaMemcpyFromSymbol(out64, ptx::g_probe, sizeof(unsigned long long) * 64);
    if (reset) { unsigned long long z[64] = {}; cudaMemcpyToSymbol(ptx::g_probe, z, sizeof z); }
    return 0;
}
#endif

}  // namespace nvfp4
