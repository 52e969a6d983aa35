// Grouped dual-NVFP4 GEMM, normal orientation, with the activation decomposition done once, ahead of
// the GEMM, instead of once per weight-column tile inside it.
//
// The fused kernels (gemm_normal.cu, gemm_cluster.cu) run Algorithm 1 on a 128-row activation tile every
// time a CTA visits it, i.e. N / 256 (or N / 512) times per element; on wide layers that arithmetic, not
// the tensor pipe, sets the pace.  Here a first, bandwidth-bound kernel quantises every activation element
// exactly once into a workspace in global memory -- A0 and A1 packed row-major, their block scales already
// in the 512-byte atoms the tensor core reads -- at a cost of 1.125 bytes written (and later re-read through
// L2) per BF16 element.  The second kernel is then a plain block-scaled FP4 GEMM with two MMAs per K atom:
// every operand arrives by TMA / bulk copy, no warp does arithmetic in the main loop, and the MMA thread
// issues back to back.  The two launches are chained with programmatic dependent launch, so that the
// prologue of the GEMM (barriers, tensor-memory allocation, descriptor prefetch) overlaps the first kernel.
//
// The codes and scales are produced by the same device function as in the fused kernels
// (xform::decompose_block16), so the result is the same bit for bit up to FP32 summation order.
#include <cuda_bf16.h>

#include <type_traits>

#include "gemm_common.cuh"
#include "host_common.hpp"
#include "launchers.hpp"
#include "transform.cuh"

namespace nvfp4 {
namespace {

using gemm::Ring;

constexpr uint32_t BM = 128, BN = 256;
// Eight scale warps (two per tensor-memory quadrant: weight scales, activation scales) and sixteen epilogue warps
// (four per quadrant, 64 accumulator columns each).  They are separate so that the scale factors of the next
// tile's first K blocks go up while the epilogue of the current tile is still storing.
constexpr uint32_t kWarpTma = 0, kWarpMma = 1, kWarpSf0 = 2, kNumSfWarps = 8, kWarpEpi0 = kWarpSf0 + kNumSfWarps,
                   kNumEpiWarps = 16;
constexpr uint32_t kThreads = (kWarpEpi0 + kNumEpiWarps) * 32;   // 832
constexpr uint32_t kSmemBudget = 232448 - 1024;

// ---------------------------------------------------------------------------------------------------
// Kernel 1: BF16 activations -> workspace.
//   a0, a1  (M, K/2) bytes, two E2M1 codes per byte, even element in the low nibble
//   sfa     (M/128, K/64, passes, 512) bytes: one scale atom per 128 rows x 64 K x pass; inside an atom the
//           four scale bytes of row r sit at (r % 32) * 16 + (r / 32) * 4 (the tensor-memory image)
// One thread per 16-element block; the four threads of a 64-K atom row combine their scale bytes into one
// 32-bit store.
// ---------------------------------------------------------------------------------------------------
// With kSwiglu the activation is not read but made: `a` is the (M, 2 K) output of a fused gate+up projection and
// element (row, j) is bf16(silu(a[row, j]) * a[row, K + j]) -- the same arithmetic and the same BF16 rounding as
// the stand-alone SwiGLU kernel (moe_glue.cu), so the codes are those of the unfused sequence, bit for bit.
// Masked layout (masked_m != nullptr): the rows are `m / max_m` groups of max_m rows of which only the first
// masked_m[g], rounded up to the 128-row tile, are quantised; the others are never read by the GEMM.
template <bool kResidual, int kPolicy, bool kSwiglu = false>
__global__ void __launch_bounds__(256)
quantize_activation_kernel(const __nv_bfloat16* __restrict__ a, int64_t lda, uint32_t m, uint32_t k,
                           uint8_t* __restrict__ a0, uint8_t* __restrict__ a1, uint8_t* __restrict__ sfa,
                           const int32_t* __restrict__ masked_m, uint32_t max_m)
{
    constexpr uint32_t kPass = kResidual ? 2 : 1;
    const uint32_t k16 = k / 16;
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t total = static_cast<uint64_t>(m) * k16;
    // the activations (and the row counts) may be the previous kernel's output
    ptx::grid_dependency_wait();
    // the grid is padded to whole warps of valid work: m * k16 is a multiple of 128 * 4
    if (idx >= total) { ptx::grid_launch_dependents(); return; }
    const uint32_t row = static_cast<uint32_t>(idx / k16), blk16 = static_cast<uint32_t>(idx % k16);
    if (masked_m != nullptr) {      // whole warps leave together: a 128-row tile is 128 * k16 blocks, a multiple of 32, so
                                    // the 32 blocks of a warp never straddle a tile boundary
        const uint32_t rows = min(static_cast<uint32_t>(max(0, __ldg(masked_m + row / max_m))), max_m);
        if (row % max_m >= (rows + BM - 1) / BM * BM) { ptx::grid_launch_dependents(); return; }
    }
    const uint4* src = reinterpret_cast<const uint4*>(a + static_cast<int64_t>(row) * lda + blk16 * 16);
    uint32_t w[8];
    {
        uint4 lo, hi;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w) : "l"(src));
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "l"(src + 1));
        w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w;
        w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
    }
    if constexpr (kSwiglu) {
        const uint4* up = reinterpret_cast<const uint4*>(a + static_cast<int64_t>(row) * lda + k + blk16 * 16);
        uint4 lo, hi;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w) : "l"(up));
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "l"(up + 1));
        const uint32_t u[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[i]));
            const __nv_bfloat162 p = __floats2bfloat162_rn(gf.x / (1.0f + __expf(-gf.x)) * uf.x, gf.y / (1.0f + __expf(-gf.y)) * uf.y);
            w[i] = *reinterpret_cast<const uint32_t*>(&p);
        }
    }
    xform::Block16 out;
    xform::decompose_block16<kResidual, kPolicy>(w, out);
    const uint64_t code_off = static_cast<uint64_t>(row) * (k / 2) + blk16 * 8;
    *reinterpret_cast<uint2*>(a0 + code_off) = make_uint2(out.q0[0], out.q0[1]);
    if constexpr (kResidual) *reinterpret_cast<uint2*>(a1 + code_off) = make_uint2(out.q1[0], out.q1[1]);
    // scale bytes of the four blocks of a K atom -> one word (the four threads are neighbours in a warp)
    const uint32_t sh = (threadIdx.x & 3u) * 8u;
    uint32_t s0 = static_cast<uint32_t>(out.s0) << sh, s1 = static_cast<uint32_t>(out.s1) << sh;
    s0 |= __shfl_xor_sync(0xffffffffu, s0, 1); s0 |= __shfl_xor_sync(0xffffffffu, s0, 2);
    if constexpr (kResidual) { s1 |= __shfl_xor_sync(0xffffffffu, s1, 1); s1 |= __shfl_xor_sync(0xffffffffu, s1, 2); }
    if ((threadIdx.x & 3u) == 0) {
        const uint32_t r = row % BM;
        const uint64_t atom = (static_cast<uint64_t>(row / BM) * (k / 64) + blk16 / 4) * kPass;
        uint8_t* dst = sfa + atom * 512 + (r % 32) * 16 + (r / 32) * 4;
        *reinterpret_cast<uint32_t*>(dst) = s0;
        if constexpr (kResidual) *reinterpret_cast<uint32_t*>(dst + 512) = s1;
    }
    // the GEMM may be scheduled once every block has come this far (its prologue then overlaps our tail; it waits
    // for the completion of this grid before it reads the workspace)
    ptx::grid_launch_dependents();
}

// ---------------------------------------------------------------------------------------------------
// Kernel 2: block-scaled FP4 GEMM over the workspace.
// ---------------------------------------------------------------------------------------------------
// kGroup ring positions share one "free again" barrier and one commit: the operands of a group are requested
// together but land, and are consumed, one K block at a time, so the first MMAs of a group start while the rest
// of its bytes are still in flight.
template <uint32_t BK, bool kResidual, uint32_t kGroup = 1>
struct Cfg {
    static_assert(BK == 128 || BK == 256, "K block");
    static constexpr uint32_t kAtoms = BK / 64, kPass = kResidual ? 2 : 1;
    static constexpr uint32_t kRowBytes = BK / 2;                             // 64 or 128: one swizzle span per row
    static constexpr uint64_t kSwizzle = BK == 256 ? ptx::kSwizzle128B : ptx::kSwizzle64B;
    static constexpr uint32_t kSBO = 8 * kRowBytes;
    static constexpr uint32_t kSlotA = BM * kRowBytes;                         // one pass
    static constexpr uint32_t kSlotB = BN * kRowBytes;
    static constexpr uint32_t kSlotSFA = kAtoms * kPass * 512, kSlotSFB = kAtoms * 2 * 512;
    static constexpr uint32_t kStage = kPass * kSlotA + kSlotB + kSlotSFA + kSlotSFB;
    // tensor memory: 256 accumulator columns, then per ring position SFA (4 columns per atom and pass) and SFB
    // (8 columns per atom: two 128-row groups)
    static constexpr uint32_t kTmemCols = 512, kColAcc = 0, kColSF = 256;
    static constexpr uint32_t kSfA = 0, kSfB = 4 * kAtoms * kPass, kSfCols = kSfB + 8 * kAtoms;
    static constexpr uint32_t kDepthSmem = (kSmemBudget - 1024 - kNumEpiWarps * 4 * 144) / kStage, kDepthTmem = (kTmemCols - kColSF) / kSfCols;
    static constexpr uint32_t kDepthRaw = kDepthSmem < kDepthTmem ? kDepthSmem : kDepthTmem;
    static constexpr uint32_t kDepthCap = kDepthRaw > 8 ? 8 : kDepthRaw;
    static constexpr uint32_t kDepth = kDepthCap / kGroup * kGroup;           // whole groups
    static constexpr uint32_t kNumGroups = kDepth / kGroup;
    static_assert(kDepth >= 3 && kNumGroups >= 2, "ring too shallow");
    static constexpr uint32_t kOffA = 0;                                       // [kDepth][kPass][kSlotA]
    static constexpr uint32_t kOffB = kOffA + kDepth * kPass * kSlotA;
    static constexpr uint32_t kOffSFA = kOffB + kDepth * kSlotB;
    static constexpr uint32_t kOffSFB = kOffSFA + kDepth * kSlotSFA;
    // epilogue staging: per warp four output rows of 64 BF16 (gemm::store_rows_staged)
    static constexpr uint32_t kOffStage = kOffSFB + kDepth * kSlotSFB;
    static constexpr uint32_t kOffBars = kOffStage + kNumEpiWarps * gemm::kStageWarp;
    static constexpr uint32_t kNumBars = 4 * kDepth + 2;
    static constexpr uint32_t kSmemAlloc = kOffBars + kNumBars * 8 + 16 + 1024;
    static_assert(kSmemAlloc <= 232448, "shared memory budget");
};

struct Params {
    const float* gw;
    const int32_t* layout;     // contiguous: m_indices (expert of every row); masked: real rows of every group
    const uint8_t* sfa;
    __nv_bfloat16* d;
    int64_t ldd;
    uint32_t m, n, k;          // m: all rows of a / d (masked: groups * max_m)
    uint32_t group_m;
    uint32_t groups, max_m;    // masked layout only
    // SwiGLU-quantised output (kSwigluOut kernels): the workspace of the NEXT GEMM, whose K is n / 2
    uint8_t* out_a0;
    uint8_t* out_a1;
    uint8_t* out_sf;
    int32_t* status;
};


// Epilogue of an up-projection whose weight rows were interleaved in runs of 32 (gate rows, then the matching up rows):
// the 64 accumulator columns a lane holds for its row are 32 gate values and their 32 up values.  The activation
// silu(gate) * up is formed exactly as the stand-alone kernels form it -- both factors rounded to BF16 first, the product
// rounded to BF16 -- and decomposed on the spot (two 16-blocks per lane), so what leaves the kernel is the quantised
// workspace of the down-projection: 8 + 8 code bytes per block and pass, and the blocks' scale bytes in their
// tensor-memory atoms.  The (rows, 2 I) BF16 intermediate is never written and never read back.
//   o[0..15]: gate columns as BF16 pairs, o[16..31]: up columns; row: row of a / d; pcol: first of the 32 product columns
__device__ __forceinline__ void store_swiglu_quantized(const uint32_t (&o)[32], const Params& p, uint32_t row, uint32_t pcol)
{
    const uint32_t k_out = p.n / 2;
    uint32_t pw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o[i]));
        const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o[16 + i]));
        const __nv_bfloat162 pr = __floats2bfloat162_rn(gf.x / (1.0f + __expf(-gf.x)) * uf.x, gf.y / (1.0f + __expf(-gf.y)) * uf.y);
        pw[i] = *reinterpret_cast<const uint32_t*>(&pr);
    }
    const uint32_t w0[8] = {pw[0], pw[1], pw[2], pw[3], pw[4], pw[5], pw[6], pw[7]};
    const uint32_t w1[8] = {pw[8], pw[9], pw[10], pw[11], pw[12], pw[13], pw[14], pw[15]};
    xform::Block16 b0, b1;
    xform::decompose_block16<true, 0>(w0, b0);
    xform::decompose_block16<true, 0>(w1, b1);
    const uint64_t code_off = static_cast<uint64_t>(row) * (k_out / 2) + pcol / 2;
    *reinterpret_cast<uint4*>(p.out_a0 + code_off) = make_uint4(b0.q0[0], b0.q0[1], b1.q0[0], b1.q0[1]);
    *reinterpret_cast<uint4*>(p.out_a1 + code_off) = make_uint4(b0.q1[0], b0.q1[1], b1.q1[0], b1.q1[1]);
    // the two blocks are bytes (pcol / 16) % 4 and + 1 of the row's word in the atom of K atom pcol / 64
    const uint32_t r = row % BM;
    uint8_t* word = p.out_sf + ((static_cast<uint64_t>(row / BM) * (k_out / 64) + pcol / 64) * 2) * 512 + (r % 32) * 16 + (r / 32) * 4 +
                    (pcol / 16) % 4;
    *reinterpret_cast<uint16_t*>(word) = static_cast<uint16_t>(b0.s0 | (b1.s0 << 8));
    *reinterpret_cast<uint16_t*>(word + 512) = static_cast<uint16_t>(b0.s1 | (b1.s1 << 8));
}

#ifdef NVFP4_PROBE
// event trace of block 0 (timing studies): g_trace[point][stage] = clock64 at the event
__device__ long long g_trace[10][64];
#define NVFP4_TRACE(point, stage) do { if (blockIdx.x == 0 && (stage) < 64 && (threadIdx.x & 31u) == 0) g_trace[point][stage] = clock64(); } while (0)
#else
#define NVFP4_TRACE(point, stage) do { } while (0)
#endif

template <uint32_t BK, bool kResidual, uint32_t kGroup, bool kMasked, bool kSwigluOut = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_split_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
                  const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_sfb, const Params p)
{
    using C = Cfg<BK, kResidual, kGroup>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem - ptx::smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kOffBars);
    uint64_t* full = bars;                           // operand tiles of a K block have landed (one arrive + bytes)
    uint64_t* empty = full + C::kDepth;              // [kNumGroups] the MMAs that read a group of ring positions have retired
    uint64_t* sf_in = empty + C::kDepth;             // the scale factors of a K block have landed (they are requested
                                                     // first and are small, so the scale warps finish their copy
                                                     // while the operand tiles are still arriving)
    uint64_t* sf_full = sf_in + C::kDepth;           // its scales are in tensor memory (the eight scale warps)
    uint64_t* tmem_full = sf_full + C::kDepth;
    uint64_t* tmem_empty = tmem_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < C::kDepth; ++i) {
            ptx::mbar_init(full + i, 1);
            if (i < C::kNumGroups) ptx::mbar_init(empty + i, 1);
            ptx::mbar_init(sf_in + i, 1);
            ptx::mbar_init(sf_full + i, kNumSfWarps);
        }
        ptx::mbar_init(tmem_full, 1);
        ptx::mbar_init(tmem_empty, kNumEpiWarps);
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tm_a0);
        if constexpr (kResidual) ptx::prefetch_tensormap(&tm_a1);
        ptx::prefetch_tensormap(&tm_b);
        ptx::prefetch_tensormap(&tm_sfb);
    }
    if (warp == kWarpMma) ptx::tmem_alloc<C::kTmemCols>(tmem_slot);
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // everything above overlapped the quantisation kernel; its stores are visible from here on
    ptx::grid_dependency_wait();

    const uint32_t num_kb = p.k / BK;
    // every role walks the same sequence of tiles (static stride over the CTAs; masked layout: row blocks from the
    // device-side row counts)
    gemm::TileWalker<BM, kMasked> walk(p.layout, p.m, p.n, BN, p.group_m, p.groups, p.max_m);
    gemm::Tile t;
    bool ok = true;
    ptx::ProbeAcc pa;
    const long long probe_start = ptx::probe_clock();
    auto give_up = [&](uint32_t code) {
        *abort_flag = 1;
        if (p.status != nullptr) atomicOr(p.status, static_cast<int32_t>(code));
        ok = false;
    };

    if (warp == kWarpTma) {
        // ================= producer: every operand of a K block on one barrier =================
        if (lane == 0) {
            Ring r;
            for (uint32_t tile = blockIdx.x; ok && walk.next(tile, t); tile += gridDim.x) {
                const uint32_t n_blk = t.n_blk;
                const int32_t e = t.expert;
                const uint8_t* sfa_row = p.sfa + static_cast<uint64_t>(t.row0 / BM) * (p.k / 64) * (C::kPass * 512);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (r.slot % kGroup == 0 &&
                        !ptx::mbar_wait(empty + r.slot / kGroup, r.phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
                    NVFP4_TRACE(0, (tile - blockIdx.x) / gridDim.x * num_kb + kb);
                    ptx::mbar_arrive_expect_tx(sf_in + r.slot, C::kSlotSFA + C::kSlotSFB);
                    ptx::tma_load_2d(smem_gen + C::kOffSFB + r.slot * C::kSlotSFB, &tm_sfb, sf_in + r.slot, n_blk * BN,
                                     e * (p.k / 64) + kb * C::kAtoms);
                    ptx::bulk_load(smem_gen + C::kOffSFA + r.slot * C::kSlotSFA,
                                   sfa_row + static_cast<uint64_t>(kb) * C::kSlotSFA, C::kSlotSFA, sf_in + r.slot);
                    ptx::mbar_arrive_expect_tx(full + r.slot, C::kPass * C::kSlotA + C::kSlotB);
                    uint8_t* a_dst = smem_gen + C::kOffA + r.slot * C::kPass * C::kSlotA;
                    ptx::tma_load_2d(a_dst, &tm_a0, full + r.slot, kb * C::kRowBytes, t.row0);
                    if constexpr (kResidual)
                        ptx::tma_load_2d(a_dst + C::kSlotA, &tm_a1, full + r.slot, kb * C::kRowBytes, t.row0);
                    ptx::tma_load_2d(smem_gen + C::kOffB + r.slot * C::kSlotB, &tm_b, full + r.slot, kb * C::kRowBytes,
                                     e * p.n + n_blk * BN);
                    r.advance<C::kDepth>();
                }
            }
            ptx::grid_launch_dependents();          // the last loads are on their way: the next kernel may start its prologue
        }
    } else if (warp == kWarpMma) {
        // ================= MMA issue: one wait, 2 x kAtoms (x passes) MMAs, one commit per K block =================
        Ring r;
        uint32_t acc_phase = 0;
        int32_t pending = -1;                       // group whose commit is still to be issued
        constexpr uint32_t idesc = ptx::make_idesc_nvf4(BM, BN);
        for (uint32_t tile = blockIdx.x; ok && walk.next(tile, t); tile += gridDim.x) {
            if (!ptx::mbar_wait(tmem_empty, acc_phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
            ptx::tcgen05_fence_after_sync();
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!ptx::mbar_wait(sf_full + r.slot, r.phase, abort_flag, pa, 1) ||
                    !ptx::mbar_wait(full + r.slot, r.phase, abort_flag, pa, 2)) { give_up(1); break; }
                NVFP4_TRACE(3, (tile - blockIdx.x) / gridDim.x * num_kb + kb);
                ptx::tcgen05_fence_after_sync();
                const long long pt1 = ptx::probe_clock();
                if (lane == 0) {
                    const uint32_t a0 = smem + C::kOffA + r.slot * C::kPass * C::kSlotA, a1 = a0 + C::kSlotA;
                    const uint32_t b = smem + C::kOffB + r.slot * C::kSlotB;
                    const uint32_t sf = tmem_base + C::kColSF + r.slot * C::kSfCols;
#pragma unroll
                    for (uint32_t a = 0; a < C::kAtoms; ++a) {
                        const uint64_t desc_b = ptx::make_smem_desc(b + a * 32, C::kSBO, C::kSwizzle);
                        ptx::tcgen05_mma_nvf4(tmem_base + C::kColAcc, ptx::make_smem_desc(a0 + a * 32, C::kSBO, C::kSwizzle),
                                              desc_b, idesc, sf + C::kSfA + 4 * (a * C::kPass), sf + C::kSfB + 8 * a,
                                              (kb | a) != 0 ? 1u : 0u);
                        if constexpr (kResidual)
                            ptx::tcgen05_mma_nvf4(tmem_base + C::kColAcc, ptx::make_smem_desc(a1 + a * 32, C::kSBO, C::kSwizzle),
                                                  desc_b, idesc, sf + C::kSfA + 4 * (a * C::kPass + 1), sf + C::kSfB + 8 * a, 1u);
                        // A commit holds this thread until the MMAs before it have been handed to the tensor pipe.
                        // Issued at the end of a K block it would leave the pipe with nothing queued while this
                        // thread finds the next K block; issued after the first atom of the NEXT block it costs the
                        // ring positions a few hundred cycles but the pipe keeps its queue.
                        if (a == 0 && pending >= 0) ptx::tcgen05_commit(empty + pending);
                    }
                    const long long pt2 = ptx::probe_clock();
                    ptx::probe_count(pa, 5, pt2 - pt1);
                    if (kb == num_kb - 1) {
                        if (r.slot % kGroup == kGroup - 1) ptx::tcgen05_commit(empty + r.slot / kGroup);
                        ptx::tcgen05_commit(tmem_full);
                    }
                    ptx::probe_count(pa, 6, ptx::probe_clock() - pt2);
                }
                // a group is complete with its last ring position; at a tile end it has been committed above
                pending = (r.slot % kGroup == kGroup - 1 && kb != num_kb - 1) ? static_cast<int32_t>(r.slot / kGroup) : -1;
                NVFP4_TRACE(4, (tile - blockIdx.x) / gridDim.x * num_kb + kb);
                __syncwarp();
                r.advance<C::kDepth>();
            }
            acc_phase ^= 1;
        }
    } else if (warp >= kWarpSf0 && warp < kWarpEpi0) {
        // ================= scale warps =================
        // Scales go from shared to tensor memory with tcgen05.st: a warp reaches only its own quadrant of lanes and
        // the MMA wants a copy in each, so four warps (one per quadrant) carry the weight scales and four the
        // activation scales.  Lane r of a quadrant gets the scale words of rows r, r + 32, r + 64, r + 96 of an
        // atom in four consecutive columns: for the weights straight from the row-major words TMA landed, for the
        // activations from the atoms the quantisation kernel laid out in that order.  All the columns of a K block
        // go up in one store.
        const uint32_t quad = warp & 3, group = (warp - kWarpSf0) >> 2;     // group 0: weight scales, 1: activation scales
        Ring r;
        for (uint32_t tile = blockIdx.x; ok && walk.next(tile, t); tile += gridDim.x) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                // the scales of this phase were requested after the producer had seen the ring position free, so the
                // MMAs that used its scale columns have retired
                if (!ptx::mbar_wait(sf_in + r.slot, r.phase, abort_flag, pa, 2)) { give_up(1); break; }
                if (warp == kWarpSf0) NVFP4_TRACE(1, (tile - blockIdx.x) / gridDim.x * num_kb + kb);
                const uint32_t sf = tmem_base + ((quad * 32) << 16) + C::kColSF + r.slot * C::kSfCols;
                const long long duty0 = ptx::probe_clock();
                if (group == 0) {
                    // word i * 4 + j = row 32 j + lane of 128-row group i (two groups per K atom)
                    const uint32_t sfb = smem + C::kOffSFB + r.slot * C::kSlotSFB + lane * 4;
                    uint32_t v[8 * C::kAtoms];
#pragma unroll
                    for (uint32_t i = 0; i < C::kAtoms * 2; ++i)
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) v[4 * i + j] = ptx::lds32(sfb + i * 512 + j * 128);
                    ptx::tmem_st_32x32b(sf + C::kSfB, v);
                } else {
                    const uint32_t sfa = smem + C::kOffSFA + r.slot * C::kSlotSFA + lane * 16;
                    uint32_t v[4 * C::kAtoms * C::kPass];
#pragma unroll
                    for (uint32_t i = 0; i < C::kAtoms * C::kPass; ++i) {
                        const uint4 q = ptx::lds128(sfa + i * 512);
                        v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
                    }
                    ptx::tmem_st_32x32b(sf + C::kSfA, v);
                }
                ptx::tmem_st_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(sf_full + r.slot);
                ptx::probe_count(pa, 4, ptx::probe_clock() - duty0);
                if (warp == kWarpSf0) NVFP4_TRACE(2, (tile - blockIdx.x) / gridDim.x * num_kb + kb);
                r.advance<C::kDepth>();
            }
        }
    } else if (warp >= kWarpEpi0) {
        // ================= epilogue: TMEM -> x G_W -> BF16 -> global =================
        // The warp's 32 lanes x 64 columns leave tensor memory in one go and the accumulator goes straight back to
        // the MMA warp; scaling, packing and the stores then run under the next tile's main loop.
        const uint32_t quad = warp & 3, group = (warp - kWarpEpi0) >> 2;
        uint32_t acc_phase = 0;
        for (uint32_t tile = blockIdx.x; ok && walk.next(tile, t); tile += gridDim.x) {
            const float g = __ldg(p.gw + t.expert);
            if (!ptx::mbar_wait_relaxed(tmem_full, acc_phase, abort_flag, 100)) { give_up(1); break; }
            if (warp == kWarpEpi0) NVFP4_TRACE(5, (tile - blockIdx.x) / gridDim.x);
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + C::kColAcc + group * 64;
            uint32_t o[32];                                    // this lane's row, 64 columns as BF16 pairs
            {
                uint32_t va[32], vb[32];
                ptx::tmem_ld_32x32b_x32(taddr, va);
                ptx::tmem_ld_32x32b_x32(taddr + 32, vb);
                ptx::tmem_ld_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tmem_empty);
                if (warp == kWarpEpi0) NVFP4_TRACE(6, (tile - blockIdx.x) / gridDim.x);
                gemm::scale_pack_bf16(va, g, o);
                gemm::scale_pack_bf16(vb, g, o + 16);
            }
            if constexpr (kSwigluOut) {
                store_swiglu_quantized(o, p, t.row0 + quad * 32 + lane, t.n_blk * (BN / 2) + group * 32);
            } else {
                const uint32_t stage = smem + C::kOffStage + (warp - kWarpEpi0) * gemm::kStageWarp;
                __nv_bfloat16* d_lane = p.d + static_cast<int64_t>(t.row0 + quad * 32 + (lane >> 3)) * p.ldd + t.n_blk * BN +
                                        group * 64 + (lane & 7u) * 8;
                gemm::store_rows_staged(o, stage, d_lane, p.ldd, lane);
            }
            if (warp == kWarpEpi0) NVFP4_TRACE(8, (tile - blockIdx.x) / gridDim.x);
            acc_phase ^= 1;
        }
    }

    ptx::probe_add(32 + (warp < 2 ? warp : (warp < kWarpEpi0 ? 2 : 4)), ptx::probe_clock() - probe_start);
    if (warp == kWarpTma) ptx::probe_flush(pa, 0);
    else if (warp == kWarpMma) ptx::probe_flush(pa, 2, 3, -1, -1, -1, 21, 22);
    else if (warp >= kWarpSf0) ptx::probe_flush(pa, -1, -1, 10, 13, 14);
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kWarpMma) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc<C::kTmemCols>(tmem_base);
    }
}


// ---------------------------------------------------------------------------------------------------
// Kernel 2, CTA-pair form: two CTAs of a cluster on 256 token rows x 256 weight columns.
// ---------------------------------------------------------------------------------------------------
// One tcgen05.mma.cta_group::2 drives both tensor cores: each CTA contributes its own 128 rows of A0 / A1 (and their
// scales) and HALF of the weight tile's rows; the hardware shows each tensor core the other half out of the peer's
// shared memory.  Per K block a CTA therefore takes in 16 KB of weights instead of 32 KB, and the tensor core reads
// each weight row from shared memory once per 256 token rows instead of once per 128 -- the single-CTA kernel's
// shared-memory pipe (TMA writes + operand reads, ~115 of 128 B/clk) is what stretches its MMAs.
//
// Who signals whom.  The MMA thread exists only in the pair's even CTA (the leader).  Its barriers `full` (operands of
// both CTAs: the peer's loads complete their bytes on the leader's barrier), `sf_full` (scale warps of both CTAs) and
// `tmem_empty` (epilogue warps of both) live in the leader; `empty`, `sf_in`, `tmem_full` are local to each CTA and
// the leader's commits reach both through the commit's CTA mask.
//
// A pair tile cannot straddle two experts (one weight tile per MMA), so the rows are cut into units: two
// consecutive row blocks of the same expert, or a single left-over block (then the odd CTA repeats the even CTA's
// rows and stores nothing).  Masked layout: units follow from the per-group row counts.  Contiguous layout: a table
// of units is built in shared memory from m_indices at kernel start (prefix scan over the row blocks by one warp).
constexpr uint32_t kMaxUnitBlocks = 4096;   // row blocks the unit table covers (contiguous layout)

// Shared and tensor memory of the pair kernel.  What limits the operand ring is the time a tile needs to arrive
// (~2200 cycles for the 48 KB of a K block, measured) against the MMA time of the positions in flight, so the operands
// get as many positions as fit -- four of 48 KB at BK = 256 -- and the scale factors, which the scale warps lift into
// tensor memory as soon as they land, go through a ring of their own that is half as deep.
// (Tried: scale factors from global memory through registers, with no shared-memory stage at all.  The four warps of
// a group need the same words, and four trips through L1 cost more than one TMA write and four shared-memory reads:
// 0.42 ms against 0.38 ms on E=8 x 512 rows, N=28672, K=4096.)
template <uint32_t BK, bool kResidual>
struct PairCfg {
    static_assert(BK == 128 || BK == 256, "K block");
    static constexpr uint32_t kAtoms = BK / 64, kPass = kResidual ? 2 : 1;
    static constexpr uint32_t kRowBytes = BK / 2;
    static constexpr uint64_t kSwizzle = BK == 256 ? ptx::kSwizzle128B : ptx::kSwizzle64B;
    static constexpr uint32_t kSBO = 8 * kRowBytes;
    static constexpr uint32_t kSlotA = BM * kRowBytes;                         // one pass, this CTA's 128 rows
    static constexpr uint32_t kSlotB = BN / 2 * kRowBytes;                     // this CTA's half of the weight tile's rows
    static constexpr uint32_t kStage = kPass * kSlotA + kSlotB;
    static constexpr uint32_t kSlotSFA = kAtoms * kPass * 512, kSlotSFB = kAtoms * 2 * 512, kSfStage = kSlotSFA + kSlotSFB;
    static constexpr uint32_t kTmemCols = 512, kColAcc = 0, kColSF = 256;
    static constexpr uint32_t kSfA = 0, kSfB = 4 * kAtoms * kPass, kSfCols = 4 * kAtoms * 2 + 8 * kAtoms;
    static constexpr uint32_t kDepth = 1024 / BK, kDepthSf = kDepth / 2;       // 4 + 2 (BK = 256), 8 + 4 (BK = 128)
    static_assert(kColSF + kDepth * kSfCols <= kTmemCols, "scale columns");
    static constexpr uint32_t kOffA = 0;                                       // [kDepth][A0, A1, B]
    static constexpr uint32_t kOffSf = kDepth * kStage;                        // [kDepthSf][SFA, SFB]
    static constexpr uint32_t kOffStage = kOffSf + kDepthSf * kSfStage;
    static constexpr uint32_t kOffUnits = kOffStage + kNumEpiWarps * gemm::kStageWarp;
    static constexpr uint32_t kOffBars = kOffUnits + kMaxUnitBlocks * 2;
    static constexpr uint32_t kNumBars = 3 * kDepth + 2 * kDepthSf + 2;
    static constexpr uint32_t kSmemAlloc = kOffBars + kNumBars * 8 + 16 + 1024;
    static_assert(kSmemAlloc <= 232448, "shared memory budget");
    static_assert(kDepth * kStage >= kMaxUnitBlocks * 4, "the expert table of the unit builder borrows the ring");
};

// nanoseconds between barrier polls of the roles that run ahead (producer, scale warps)
constexpr uint32_t PAIR_SLEEP_TMA = 64, PAIR_SLEEP_SF = 32;

struct PairTile {
    uint32_t row0;     // first row of the unit
    uint32_t n_blk;
    int32_t expert;
    bool pair;         // two row blocks (else one)
};

template <bool kMasked>
struct PairWalker {
    const int32_t* layout;
    const uint16_t* units;
    uint32_t num_units, num_n, group_m, groups, max_m;
    uint32_t g = 0, units_before = 0, blocks_here = 0;
    bool primed = false;

    __device__ __forceinline__ uint32_t blocks_of(uint32_t group) const
    {
        const uint32_t rows = min(static_cast<uint32_t>(max(0, __ldg(layout + group))), max_m);
        return (rows + BM - 1) / BM;
    }
    __device__ __forceinline__ bool next(uint32_t linear, PairTile& t)
    {
        uint32_t unit;
        if constexpr (!kMasked) {
            if (linear >= num_units * num_n) return false;
            gemm::tile_coords(linear, num_units, num_n, group_m, unit, t.n_blk);
            const uint32_t w = units[unit];
            t.row0 = (w & 0x7fffu) * BM;
            t.pair = (w >> 15) != 0;
            t.expert = max(0, __ldg(layout + t.row0));
            return true;
        } else {
            if (!primed) { blocks_here = groups ? blocks_of(0) : 0; primed = true; }
            for (;;) {
                if (g >= groups) return false;
                if (linear < (units_before + (blocks_here + 1) / 2) * num_n) break;
                units_before += (blocks_here + 1) / 2;
                if (++g < groups) blocks_here = blocks_of(g);
            }
            gemm::tile_coords(linear - units_before * num_n, (blocks_here + 1) / 2, num_n, group_m, unit, t.n_blk);
            t.row0 = g * max_m + unit * 2 * BM;
            t.pair = unit * 2 + 1 < blocks_here;
            t.expert = static_cast<int32_t>(g);
            return true;
        }
    }
};

// Contiguous layout: cut the num_m row blocks into units.  Block i starts a unit when it sits an even number of blocks
// after the start of its run of equal expert ids; the unit is a pair when block i + 1 belongs to the same run.  Every
// thread of the CTA calls this; `experts` is scratch for num_m words; the table and *num_units are valid on return.
__device__ __forceinline__ void build_units(const int32_t* m_indices, uint32_t num_m, int32_t* experts, uint16_t* units,
                                            uint32_t* num_units)
{
    for (uint32_t i = threadIdx.x; i < num_m; i += blockDim.x) experts[i] = max(0, __ldg(m_indices + static_cast<uint64_t>(i) * BM));
    __syncthreads();
    if (threadIdx.x < 32) {                          // one warp: three short walks over the table and two shuffle scans
        const uint32_t lane = threadIdx.x, per = (num_m + 31) / 32;
        const uint32_t lo = min(lane * per, num_m), hi = min(lo + per, num_m);
        // effect of this lane's chunk on the parity p = (distance from the run start) & 1: p_out = reset ? val : p_in ^ val
        bool reset = false;
        uint32_t val = 0;
        for (uint32_t i = lo; i < hi; ++i) {
            if (i == 0 || experts[i] != experts[i - 1]) { reset = true; val = 0; } else val ^= 1;
        }
        // inclusive scan of the chunk effects over the lanes, then shift by one lane
        bool r = reset;
        uint32_t v = val;
        for (uint32_t d = 1; d < 32; d <<= 1) {
            const bool r_up = __shfl_up_sync(0xffffffffu, r ? 1u : 0u, d) != 0;
            const uint32_t v_up = __shfl_up_sync(0xffffffffu, v, d);
            if (lane >= d && !r) { r = r_up; v ^= v_up; }
        }
        // Block 0 starts a run, so every non-empty prefix ends in a known parity: lane L now holds the parity of the last
        // block before its successor's chunk.
        const uint32_t v_prev = __shfl_up_sync(0xffffffffu, v, 1);
        const uint32_t p = lane == 0 ? 0u : v_prev;
        // count the unit starts of the chunk
        uint32_t count = 0, q = p;
        for (uint32_t i = lo; i < hi; ++i) {
            q = (i == 0 || experts[i] != experts[i - 1]) ? 0u : (q ^ 1u);
            count += q == 0;
        }
        uint32_t incl = count;
        for (uint32_t d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        uint32_t at = incl - count;
        q = p;
        for (uint32_t i = lo; i < hi; ++i) {
            q = (i == 0 || experts[i] != experts[i - 1]) ? 0u : (q ^ 1u);
            if (q == 0) {
                const bool pair = i + 1 < num_m && experts[i + 1] == experts[i];
                units[at++] = static_cast<uint16_t>(i | (pair ? 0x8000u : 0u));
            }
        }
        if (lane == 31) *num_units = incl;
    }
    ptx::fence_proxy_async_smem();                   // the scratch is about to be overwritten by bulk copies
    __syncthreads();
}


template <uint32_t BK, bool kResidual, bool kMasked, bool kSwigluOut = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_split_pair_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
                       const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_sfb, const Params p)
{
    using C = PairCfg<BK, kResidual>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem - ptx::smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kOffBars);
    uint64_t* full = bars;                           // LEADER: the operand tiles of both CTAs have landed
    uint64_t* empty = full + C::kDepth;              // each CTA: the pair MMAs that read a ring position have retired
    uint64_t* sf_full = empty + C::kDepth;           // LEADER: the scales of both CTAs are in their tensor memories
    uint64_t* sf_in = sf_full + C::kDepth;           // each CTA, scale ring: its scale factors have landed
    uint64_t* sf_free = sf_in + C::kDepthSf;         // each CTA, scale ring: the scale warps have lifted them out
    uint64_t* tmem_full = sf_free + C::kDepthSf;     // each CTA: the accumulator is complete
    uint64_t* tmem_empty = tmem_full + 1;            // LEADER: the epilogue warps of both CTAs have drained theirs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* num_units_slot = tmem_slot + 2;
    uint16_t* units = reinterpret_cast<uint16_t*>(smem_gen + C::kOffUnits);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_cta_rank();   // 0: leader (issues the MMAs), 1: peer
    const uint32_t pair_id = ptx::cluster_id_x(), num_pairs = ptx::num_clusters_x();
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < C::kDepth; ++i) {
            ptx::mbar_init(full + i, 1);
            ptx::mbar_init(empty + i, 1);
            ptx::mbar_init(sf_full + i, 2 * kNumSfWarps);
            if (i < C::kDepthSf) {
                ptx::mbar_init(sf_in + i, 1);
                ptx::mbar_init(sf_free + i, kNumSfWarps);
            }
        }
        ptx::mbar_init(tmem_full, 1);
        ptx::mbar_init(tmem_empty, 2 * kNumEpiWarps);
        *abort_flag = 0;
        *num_units_slot = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tm_a0);
        if constexpr (kResidual) ptx::prefetch_tensormap(&tm_a1);
        ptx::prefetch_tensormap(&tm_b);
        ptx::prefetch_tensormap(&tm_sfb);
    }
    if (warp == kWarpMma) ptx::tmem_alloc_pair<C::kTmemCols>(tmem_slot);
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_sync();                             // the peer's barriers exist before anything signals them
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // everything above overlapped the quantisation kernel; its stores (and the routing index) are visible from here on
    ptx::grid_dependency_wait();
    if constexpr (!kMasked)
        build_units(p.layout, p.m / BM, reinterpret_cast<int32_t*>(smem_gen + C::kOffA), units, num_units_slot);

    const uint32_t num_kb = p.k / BK;
    PairWalker<kMasked> walk{p.layout, units, *num_units_slot, p.n / BN, p.group_m, p.groups, p.max_m};
    PairTile t;
    bool ok = true;
    ptx::ProbeAcc pa;
    auto give_up = [&](uint32_t code) {
        *abort_flag = 1;
        if (p.status != nullptr) atomicOr(p.status, static_cast<int32_t>(code));
        ok = false;
    };
    // rows of this CTA inside a unit: the odd CTA of a single-block unit repeats the even CTA's rows
    auto my_row0 = [&](const PairTile& pt) { return pt.row0 + (pt.pair ? rank * BM : 0u); };

    if (warp == kWarpTma) {
        // ================= producer =================
        if (lane == 0) {
            Ring r, rs;
            const uint32_t full_leader = ptx::map_to_cta(ptx::smem_u32(full), 0);
            for (uint32_t tile = pair_id; ok && walk.next(tile, t); tile += num_pairs) {
                const uint32_t row0 = my_row0(t);
                const uint8_t* sfa_row = p.sfa + static_cast<uint64_t>(row0 / BM) * (p.k / 64) * (C::kPass * 512);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    // the roles that run ahead sleep between polls: every poll is an instruction of the shared-memory pipe
                    if (!ptx::mbar_wait_sleep<false>(empty + r.slot, r.phase ^ 1, abort_flag, PAIR_SLEEP_TMA, pa, 0)) { give_up(1); break; }
                    if (!ptx::mbar_wait_sleep<false>(sf_free + rs.slot, rs.phase ^ 1, abort_flag, PAIR_SLEEP_TMA, pa, 0)) { give_up(1); break; }
                    NVFP4_TRACE(0, (tile - pair_id) / num_pairs * num_kb + kb);
                    uint8_t* sf_dst = smem_gen + C::kOffSf + rs.slot * C::kSfStage;
                    ptx::mbar_arrive_expect_tx(sf_in + rs.slot, C::kSfStage);
                    ptx::tma_load_2d(sf_dst + C::kSlotSFA, &tm_sfb, sf_in + rs.slot, t.n_blk * BN,
                                     t.expert * (p.k / 64) + kb * C::kAtoms);
                    ptx::bulk_load(sf_dst, sfa_row + static_cast<uint64_t>(kb) * C::kSlotSFA, C::kSlotSFA, sf_in + rs.slot);
                    // the leader announces the operand bytes of both CTAs; the peer's bytes complete on the leader's barrier
                    if (rank == 0) ptx::mbar_arrive_expect_tx(full + r.slot, 2 * (C::kPass * C::kSlotA + C::kSlotB));
                    const uint32_t bar = full_leader + r.slot * 8;
                    uint8_t* a_dst = smem_gen + C::kOffA + r.slot * C::kStage;
                    ptx::tma_load_2d_pair(a_dst, &tm_a0, bar, kb * C::kRowBytes, row0);
                    if constexpr (kResidual) ptx::tma_load_2d_pair(a_dst + C::kSlotA, &tm_a1, bar, kb * C::kRowBytes, row0);
                    ptx::tma_load_2d_pair(a_dst + C::kPass * C::kSlotA, &tm_b, bar, kb * C::kRowBytes,
                                          t.expert * p.n + t.n_blk * BN + rank * (BN / 2));
                    r.advance<C::kDepth>();
                    rs.advance<C::kDepthSf>();
                }
            }
            ptx::grid_launch_dependents();
        }
    } else if (warp == kWarpMma) {
        // ================= MMA issue (leader only) =================
        if (rank == 0) {
            Ring r;
            uint32_t acc_phase = 0;
            int32_t pending = -1;                   // ring position whose commit is still to be issued
            constexpr uint32_t idesc = ptx::make_idesc_nvf4(2 * BM, BN);
            constexpr uint16_t kBoth = 3;
            for (uint32_t tile = pair_id; ok && walk.next(tile, t); tile += num_pairs) {
                if (!ptx::mbar_wait(tmem_empty, acc_phase ^ 1, abort_flag, pa, 0)) { give_up(1); break; }
                ptx::tcgen05_fence_after_sync();
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(sf_full + r.slot, r.phase, abort_flag, pa, 1) ||
                        !ptx::mbar_wait(full + r.slot, r.phase, abort_flag, pa, 2)) { give_up(1); break; }
                    NVFP4_TRACE(3, (tile - pair_id) / num_pairs * num_kb + kb);
                    ptx::tcgen05_fence_after_sync();
                    if (lane == 0) {
                        const uint32_t a0 = smem + C::kOffA + r.slot * C::kStage, a1 = a0 + C::kSlotA;
                        const uint32_t b = a0 + C::kPass * C::kSlotA;
                        const uint32_t sf = tmem_base + C::kColSF + r.slot * C::kSfCols;
#pragma unroll
                        for (uint32_t a = 0; a < C::kAtoms; ++a) {
                            const uint64_t desc_b = ptx::make_smem_desc(b + a * 32, C::kSBO, C::kSwizzle);
                            ptx::tcgen05_mma_nvf4_pair(tmem_base + C::kColAcc, ptx::make_smem_desc(a0 + a * 32, C::kSBO, C::kSwizzle),
                                                       desc_b, idesc, sf + C::kSfA + 4 * (a * C::kPass), sf + C::kSfB + 8 * a,
                                                       (kb | a) != 0 ? 1u : 0u);
                            if constexpr (kResidual)
                                ptx::tcgen05_mma_nvf4_pair(tmem_base + C::kColAcc,
                                                           ptx::make_smem_desc(a1 + a * 32, C::kSBO, C::kSwizzle), desc_b, idesc,
                                                           sf + C::kSfA + 4 * (a * C::kPass + 1), sf + C::kSfB + 8 * a, 1u);
                            // as in the single-CTA kernel: the commit of a K block goes out after the first atom of the next
                            if (a == 0 && pending >= 0) ptx::tcgen05_commit_pair(empty + pending, kBoth);
                        }
                        if (kb == num_kb - 1) {
                            ptx::tcgen05_commit_pair(empty + r.slot, kBoth);
                            ptx::tcgen05_commit_pair(tmem_full, kBoth);
                        }
                    }
                    pending = kb != num_kb - 1 ? static_cast<int32_t>(r.slot) : -1;
                    NVFP4_TRACE(4, (tile - pair_id) / num_pairs * num_kb + kb);
                    __syncwarp();
                    r.advance<C::kDepth>();
                }
                acc_phase ^= 1;
            }
        }
    } else if (warp >= kWarpSf0 && warp < kWarpEpi0) {
        // ================= scale warps: as in the single-CTA kernel, signalling the leader =================
        const uint32_t quad = warp & 3, group = (warp - kWarpSf0) >> 2;     // group 0: weight scales, 1: activation scales
        const uint32_t sf_full_leader = ptx::map_to_cta(ptx::smem_u32(sf_full), 0);
        Ring r, rs;
        for (uint32_t tile = pair_id; ok && walk.next(tile, t); tile += num_pairs) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                // the scale columns of ring position r are free: the producer requested these scales only after it had
                // seen the position's MMAs retire
                if (!ptx::mbar_wait_sleep<false>(sf_in + rs.slot, rs.phase, abort_flag, PAIR_SLEEP_SF, pa, 2)) { give_up(1); break; }
                if (warp == kWarpSf0) NVFP4_TRACE(1, (tile - pair_id) / num_pairs * num_kb + kb);
                const uint32_t sf = tmem_base + ((quad * 32) << 16) + C::kColSF + r.slot * C::kSfCols;
                if (group == 0) {
                    const uint32_t sfb = smem + C::kOffSf + rs.slot * C::kSfStage + C::kSlotSFA + lane * 4;
                    uint32_t v[8 * C::kAtoms];
#pragma unroll
                    for (uint32_t i = 0; i < C::kAtoms * 2; ++i)
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) v[4 * i + j] = ptx::lds32(sfb + i * 512 + j * 128);
                    ptx::tmem_st_32x32b(sf + C::kSfB, v);
                } else {
                    const uint32_t sfa = smem + C::kOffSf + rs.slot * C::kSfStage + lane * 16;
                    uint32_t v[4 * C::kAtoms * C::kPass];
#pragma unroll
                    for (uint32_t i = 0; i < C::kAtoms * C::kPass; ++i) {
                        const uint4 q = ptx::lds128(sfa + i * 512);
                        v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
                    }
                    ptx::tmem_st_32x32b(sf + C::kSfA, v);
                }
                ptx::tmem_st_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                // A cluster-scope releasing arrive (mbarrier.arrive.release.cluster) was measured to cost ~1500 cycles here
                // and to set the pace of the whole kernel (0.52 ms against 0.38 ms).  The scales went to tensor memory,
                // which the tcgen05 fences order, so the plain form is enough.
                if (lane == 0) {
                    ptx::mbar_arrive_remote(sf_full_leader + r.slot * 8);
                    ptx::mbar_arrive(sf_free + rs.slot);      // the words are in tensor memory: the slot may be refilled
                }
                if (warp == kWarpSf0) NVFP4_TRACE(2, (tile - pair_id) / num_pairs * num_kb + kb);
                r.advance<C::kDepth>();
                rs.advance<C::kDepthSf>();
            }
        }
    } else if (warp >= kWarpEpi0) {
        // ================= epilogue: each CTA drains and stores its own 128 rows =================
        const uint32_t quad = warp & 3, group = (warp - kWarpEpi0) >> 2;
        const uint32_t tmem_empty_leader = ptx::map_to_cta(ptx::smem_u32(tmem_empty), 0);
        uint32_t acc_phase = 0;
        for (uint32_t tile = pair_id; ok && walk.next(tile, t); tile += num_pairs) {
            const float g = __ldg(p.gw + t.expert);
            if (!ptx::mbar_wait_relaxed(tmem_full, acc_phase, abort_flag, 100)) { give_up(1); break; }
            if (warp == kWarpEpi0) NVFP4_TRACE(5, (tile - pair_id) / num_pairs);
            ptx::tcgen05_fence_after_sync();
            acc_phase ^= 1;
            if (!t.pair && rank != 0) {             // nothing of ours in this unit
                if (lane == 0) ptx::mbar_arrive_remote(tmem_empty_leader);
                continue;
            }
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + C::kColAcc + group * 64;
            uint32_t o[32];
            {
                uint32_t va[32], vb[32];
                ptx::tmem_ld_32x32b_x32(taddr, va);
                ptx::tmem_ld_32x32b_x32(taddr + 32, vb);
                ptx::tmem_ld_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_remote(tmem_empty_leader);
                if (warp == kWarpEpi0) NVFP4_TRACE(6, (tile - pair_id) / num_pairs);
                gemm::scale_pack_bf16(va, g, o);
                gemm::scale_pack_bf16(vb, g, o + 16);
            }
            if constexpr (kSwigluOut) {
                store_swiglu_quantized(o, p, my_row0(t) + quad * 32 + lane, t.n_blk * (BN / 2) + group * 32);
            } else {
                const uint32_t stage = smem + C::kOffStage + (warp - kWarpEpi0) * gemm::kStageWarp;
                __nv_bfloat16* d_lane = p.d + static_cast<int64_t>(my_row0(t) + quad * 32 + (lane >> 3)) * p.ldd + t.n_blk * BN +
                                        group * 64 + (lane & 7u) * 8;
                gemm::store_rows_staged(o, stage, d_lane, p.ldd, lane);
            }
            if (warp == kWarpEpi0) NVFP4_TRACE(8, (tile - pair_id) / num_pairs);
        }
    }

    // neither CTA may leave (or give up its tensor memory) while the other can still signal it or read its operands
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_sync();
    if (warp == kWarpMma) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc_pair<C::kTmemCols>(tmem_base);
    }
}

// What a call of the split path is made of, after validation.
struct Call {
    const void* a; int64_t lda;             // activations (SwiGLU-folded form: the (M, 2 K) gate+up output)
    const void* b; const void* sfb;
    int M, N, K, E;
    bool pdl, swiglu;
    int policy;
    const int32_t* masked_m; int max_m;     // masked layout: device-side row counts, rows reserved per group
    int num_sms;
    bool pair;                              // CTA-pair GEMM kernel
    cudaStream_t stream;
    // activations that arrive quantised (the expert-parallel layer's quantised dispatch): the caller's a0, a1
    // (M, K/2) and scale atoms (M/128, K/64, passes, 512) stand in for the workspace and kernel 1 is skipped
    const uint8_t* ext_a0 = nullptr; const uint8_t* ext_a1 = nullptr; const uint8_t* ext_sfa = nullptr;
    // SwiGLU-quantised output instead of BF16 rows (see store_swiglu_quantized): the next GEMM's a0, a1, scale atoms
    uint8_t* out_a0 = nullptr; uint8_t* out_a1 = nullptr; uint8_t* out_sf = nullptr;
};

// Kernel 1 into the given workspace pieces.
template <bool kResidual>
int launch_quantize(const Call& c, uint8_t* a0, uint8_t* a1, uint8_t* sfa)
{
    auto quantize = quantize_activation_kernel<kResidual, 0, true>;
    if (!c.swiglu)
        host::with_policy(c.policy, [&](auto pol) {
            quantize = quantize_activation_kernel<kResidual, decltype(pol)::value, false>;
            return 0;
        });
    const uint64_t blocks16 = static_cast<uint64_t>(c.M) * (c.K / 16);
    return host::launch_kernel(quantize, dim3(static_cast<unsigned>((blocks16 + 255) / 256)), dim3(256), 0, c.stream, c.pdl,
                               static_cast<const __nv_bfloat16*>(c.a), c.lda, static_cast<uint32_t>(c.M),
                               static_cast<uint32_t>(c.K), a0, a1, sfa, c.masked_m, static_cast<uint32_t>(c.max_m > 0 ? c.max_m : 1));
}

template <uint32_t BK, bool kResidual, uint32_t kGroup, bool kMasked, bool kPair = false, bool kSwigluOut = false>
int launch_variant(const Call& c, Params p)
{
    using C = std::conditional_t<kPair, PairCfg<BK, kResidual>, Cfg<BK, kResidual, kGroup>>;
    const int M = c.M, N = c.N, K = c.K;
    int dev = 0;
    NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
    const size_t code_bytes = static_cast<size_t>(M) * (K / 2);
    const size_t sf_bytes = static_cast<size_t>(M) * (K / 16) * C::kPass;
    const bool ext = c.ext_a0 != nullptr;
    uint8_t* ws = nullptr;
    uint8_t *a0, *a1, *sfa;
    if (ext) {
        a0 = const_cast<uint8_t*>(c.ext_a0);
        a1 = const_cast<uint8_t*>(kResidual ? c.ext_a1 : c.ext_a0);
        sfa = const_cast<uint8_t*>(c.ext_sfa);
    } else {
        cudaMemPool_t pool;
        if (int rc = host::workspace_pool(dev, &pool)) return rc;
        NVFP4_CUDA_CHECK(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&ws), C::kPass * code_bytes + sf_bytes, pool, c.stream));
        a0 = ws;
        a1 = kResidual ? ws + code_bytes : ws;
        sfa = ws + C::kPass * code_bytes;
    }
    p.sfa = sfa;

    auto release = [&](int rc) {
        if (ws != nullptr) cudaFreeAsync(ws, c.stream);
        return rc;
    };
    CUtensorMap tm_a0, tm_a1, tm_b, tm_sfb;
    const CUtensorMapSwizzle sw = BK == 256 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    int rc = host::encode_tensor_map_2d(&tm_a0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a0, K / 2, M, K / 2, C::kRowBytes, BM, sw);
    if (rc) return release(rc);
    rc = host::encode_tensor_map_2d(&tm_a1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a1, K / 2, M, K / 2, C::kRowBytes, BM, sw);
    if (rc) return release(rc);
    rc = host::encode_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, c.b, K / 2, static_cast<uint64_t>(c.E) * N, K / 2,
                                    C::kRowBytes, BN / (kPair ? 2 : 1), sw);
    if (rc) return release(rc);
    rc = host::encode_tensor_map_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, c.sfb, N, static_cast<uint64_t>(c.E) * (K / 64),
                                    static_cast<uint64_t>(N) * 4, BN, C::kAtoms, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return release(rc);

    if (!ext)
        if (int qrc = launch_quantize<kResidual>(c, a0, a1, sfa)) return release(qrc);

    auto kernel = [] {
        if constexpr (kPair) return gemm_split_pair_kernel<BK, kResidual, kMasked, kSwigluOut>;
        else return gemm_split_kernel<BK, kResidual, kGroup, kMasked, kSwigluOut>;
    }();
    static bool attr_set[host::kMaxDevices] = {};
    if (!attr_set[dev]) {
        if (cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemAlloc);
            err != cudaSuccess)
            return release(host::fail(NVFP4_E_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(err)));
        attr_set[dev] = true;
    }
    // masked layout: the number of tiles is only known on the device; surplus CTAs find no tile and leave
    const int num_tiles = (M / static_cast<int>(BM)) * (N / static_cast<int>(BN));
    if constexpr (kPair) {
        // one cluster of two CTAs per pair of SMs; a unit is at most two row blocks, so there are at least num_tiles / 2
        // and at most num_tiles pair tiles
        int pairs = c.num_sms / 2;
        if (pairs > num_tiles) pairs = num_tiles;
        if (pairs < 1) pairs = 1;
        return release(host::launch_kernel_cluster(kernel, dim3(static_cast<unsigned>(2 * pairs)), dim3(kThreads), C::kSmemAlloc,
                                                   c.stream, c.pdl, 2u, tm_a0, tm_a1, tm_b, tm_sfb, p));
    } else {
        const int grid = num_tiles < c.num_sms ? num_tiles : c.num_sms;
        return release(host::launch_kernel(kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), C::kSmemAlloc, c.stream,
                                           c.pdl, tm_a0, tm_a1, tm_b, tm_sfb, p));
    }
}

template <bool kMasked>
int launch_for_layout(const Call& c, const Params& p, bool residual, int block_k)
{
    // block_k: 0 = the library's choice, 256 = one 256-wide K block per ring position, 128 = 128-wide with a commit
    // per position, 130 = 128-wide in groups of two (requested and freed together, consumed one by one)
    if constexpr (kMasked) {
        if (c.out_a0 != nullptr) {          // SwiGLU-quantised output: built for the masked layout with both passes
            if (!residual) return host::fail(NVFP4_E_UNSUPPORTED, "the SwiGLU-quantised output needs the residual pass");
            const bool wide = c.K % 256 == 0 && block_k != 128;
            if (c.pair) return wide ? launch_variant<256, true, 1, true, true, true>(c, p) : launch_variant<128, true, 1, true, true, true>(c, p);
            return wide ? launch_variant<256, true, 1, true, false, true>(c, p) : launch_variant<128, true, 1, true, false, true>(c, p);
        }
    }
    if (!kMasked && block_k == 130)
        return residual ? launch_variant<128, true, 2, false>(c, p) : launch_variant<128, false, 2, false>(c, p);
    if (c.pair) {
        if (c.K % 256 == 0 && block_k != 128)
            return residual ? launch_variant<256, true, 1, kMasked, true>(c, p) : launch_variant<256, false, 1, kMasked, true>(c, p);
        return residual ? launch_variant<128, true, 1, kMasked, true>(c, p) : launch_variant<128, false, 1, kMasked, true>(c, p);
    }
    if (c.K % 256 == 0 && block_k != 128)
        return residual ? launch_variant<256, true, 1, kMasked>(c, p) : launch_variant<256, false, 1, kMasked>(c, p);
    return residual ? launch_variant<128, true, 1, kMasked>(c, p) : launch_variant<128, false, 1, kMasked>(c, p);
}

}  // namespace

// Two launches: activations -> NVFP4 workspace, then the block-scaled GEMM over it.  N % 256 == 0.
// masked_m == nullptr: contiguous layout (layout = m_indices, M rows).  Otherwise the masked layout: E groups of
// max_m rows (M = E * max_m), masked_m[g] of them real.
int launch_gemm_split(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                      int64_t ldd, const int32_t* m_indices, const int32_t* masked_m, int max_m, int M, int N, int K, int E,
                      bool residual, int block_k, int group_m, bool pdl, int policy, bool swiglu, int num_sms, bool pair,
                      int32_t* status, cudaStream_t stream)
{
    Params p;
    p.gw = gw;
    p.layout = masked_m != nullptr ? masked_m : m_indices;
    p.sfa = nullptr;
    p.d = static_cast<__nv_bfloat16*>(d);
    p.ldd = ldd;
    p.m = M; p.n = N; p.k = K;
    p.group_m = group_m > 0 ? group_m : 8;
    p.groups = E; p.max_m = max_m > 0 ? max_m : 1;
    p.out_a0 = p.out_a1 = p.out_sf = nullptr;
    p.status = status;
    // the pair kernel's unit table covers kMaxUnitBlocks row blocks of the contiguous layout
    const bool use_pair = pair && num_sms >= 2 && (masked_m != nullptr || M / static_cast<int>(BM) <= static_cast<int>(kMaxUnitBlocks));
    const Call c{a, lda, b, sfb, M, N, K, E, pdl, swiglu, policy, masked_m, max_m, num_sms, use_pair, stream};
    return masked_m != nullptr ? launch_for_layout<true>(c, p, residual, block_k) : launch_for_layout<false>(c, p, residual, block_k);
}

// The GEMM alone over activations the caller holds quantised (masked layout: E groups of max_m rows).
int launch_gemm_split_quantized(const void* a0, const void* a1, const void* sfa, const void* b, const void* sfb, const float* gw,
                                void* d, int64_t ldd, const int32_t* masked_m, int max_m, int N, int K, int E, bool residual,
                                int block_k, int group_m, bool pdl, int num_sms, bool pair, void* out_a0, void* out_a1, void* out_sf,
                                int32_t* status, cudaStream_t stream)
{
    Params p;
    p.gw = gw;
    p.layout = masked_m;
    p.sfa = nullptr;
    p.d = static_cast<__nv_bfloat16*>(d);
    p.ldd = ldd;
    p.m = E * max_m; p.n = N; p.k = K;
    p.group_m = group_m > 0 ? group_m : 8;
    p.groups = E; p.max_m = max_m > 0 ? max_m : 1;
    p.out_a0 = p.out_a1 = p.out_sf = nullptr;
    p.status = status;
    Call c{nullptr, 0, b, sfb, E * max_m, N, K, E, pdl, false, 0, masked_m, max_m, num_sms, pair && num_sms >= 2, stream};
    c.ext_a0 = static_cast<const uint8_t*>(a0);
    c.ext_a1 = static_cast<const uint8_t*>(a1);
    c.ext_sfa = static_cast<const uint8_t*>(sfa);
    c.out_a0 = static_cast<uint8_t*>(out_a0);
    c.out_a1 = static_cast<uint8_t*>(out_a1);
    c.out_sf = static_cast<uint8_t*>(out_sf);
    p.out_a0 = c.out_a0; p.out_a1 = c.out_a1; p.out_sf = c.out_sf;
    return launch_for_layout<true>(c, p, residual, block_k);
}

// Test hook: kernel 1 alone, into buffers of the caller (a0, a1: (M, K/2) bytes; sfa: (M/128, K/64, passes, 512) bytes).
int launch_debug_split_workspace(const void* a, int64_t lda, int M, int K, int policy, bool residual, bool swiglu, void* a0,
                                 void* a1, void* sfa, cudaStream_t stream)
{
    const Call c{a, lda, nullptr, nullptr, M, 0, K, 0, false, swiglu, policy, nullptr, 0, 0, false, stream};
    return residual ? launch_quantize<true>(c, static_cast<uint8_t*>(a0), static_cast<uint8_t*>(a1), static_cast<uint8_t*>(sfa))
                    : launch_quantize<false>(c, static_cast<uint8_t*>(a0), static_cast<uint8_t*>(a1), static_cast<uint8_t*>(sfa));
}

#ifdef NVFP4_PROBE
extern "C" __attribute__((visibility("default"))) int nvfp4_probe_read_split(unsigned long long* out64, int reset)
{
    cudaMemcpyFromSymbol(out64, ptx::g_probe, sizeof(unsigned long long) * 64);
    if (reset) { unsigned long long z[64] = {}; cudaMemcpyToSymbol(ptx::g_probe, z, sizeof z); }
    return 0;
}
extern "C" __attribute__((visibility("default"))) int nvfp4_probe_read_trace(long long* out)
{
    cudaMemcpyFromSymbol(out, g_trace, sizeof(long long) * 10 * 64);
    return 0;
}
#endif

}  // namespace nvfp4
