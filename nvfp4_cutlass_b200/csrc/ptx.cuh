// Raw PTX for sm_100a: mbarrier, TMA (non-multicast only), tcgen05 (TMEM
// allocation, block-scaled FP4 MMA, scale-factor copy, commit, load), proxy
// fences and the FP4 / E4M3 converts.  Nothing here depends on CUTLASS or CuTe.
//
// Every wait in this file is bounded: a waiter that runs out of time reports it
// and the caller unwinds, so a protocol bug ends as an error status, never as a
// hung GPU.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace nvfp4::ptx {

#define NVFP4_DEVICE __device__ __forceinline__

NVFP4_DEVICE uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }


// ---- mbarrier ---------------------------------------------------------------
NVFP4_DEVICE void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
NVFP4_DEVICE void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
NVFP4_DEVICE void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
NVFP4_DEVICE void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
NVFP4_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Clock budget of one wait (about a second at B200 clocks).  Legitimate waits
// in these kernels last microseconds.
constexpr long long kWaitBudgetCycles = 2000000000ll;

// Returns false if the phase did not complete within `budget` clock cycles, or if another
// thread of the CTA already gave up (`*abort_flag != 0`).
NVFP4_DEVICE bool mbar_wait_budget(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, long long budget)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag != 0 || clock64() - t0 > budget) return false;
    }
}
NVFP4_DEVICE bool mbar_wait_impl(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag)
{
    return mbar_wait_budget(bar, parity, abort_flag, kWaitBudgetCycles);
}

// The same bounded wait for roles that wait long and need not react within cycles (an epilogue warp waiting
// for a whole tile): it sleeps between polls, which leaves issue slots and power to the warps that work.
NVFP4_DEVICE bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t sleep_ns)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) {
            __nanosleep(sleep_ns);
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (*abort_flag != 0 || clock64() - t0 > kWaitBudgetCycles) return false;
    }
}

// Optional per-site wait accounting for timing studies (NVFP4_PROBE is never defined in
// the shipped build): waits add their duration to a thread-local counter that the role
// flushes once, when it leaves its loop.
struct ProbeAcc {
#ifdef NVFP4_PROBE
    long long v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
};
#ifdef NVFP4_PROBE
static __device__ unsigned long long g_probe[64];
NVFP4_DEVICE void probe_flush(const ProbeAcc& a, int s0, int s1 = -1, int s2 = -1, int s3 = -1, int s4 = -1, int s5 = -1,
                              int s6 = -1, int s7 = -1)
{
    if ((threadIdx.x & 31u) != 0) return;
    const int sites[8] = {s0, s1, s2, s3, s4, s5, s6, s7};
    for (int i = 0; i < 8; ++i)
        if (sites[i] >= 0) atomicAdd(&g_probe[sites[i]], static_cast<unsigned long long>(a.v[i]));
}
NVFP4_DEVICE void probe_add(int site, long long cycles)
{
    if ((threadIdx.x & 31u) == 0) atomicAdd(&g_probe[site], static_cast<unsigned long long>(cycles));
}
NVFP4_DEVICE long long probe_clock() { return clock64(); }
NVFP4_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, ProbeAcc& acc, int idx)
{
    const long long t0 = clock64();
    const bool ok = mbar_wait_impl(bar, parity, abort_flag);
    acc.v[idx] += clock64() - t0;
    return ok;
}
NVFP4_DEVICE void probe_count(ProbeAcc& acc, int idx, long long cycles) { acc.v[idx] += cycles; }
#else
NVFP4_DEVICE void probe_count(ProbeAcc&, int, long long) {}
NVFP4_DEVICE void probe_flush(const ProbeAcc&, int, int = -1, int = -1, int = -1, int = -1, int = -1, int = -1, int = -1) {}
NVFP4_DEVICE void probe_add(int, long long) {}
NVFP4_DEVICE long long probe_clock() { return 0; }
NVFP4_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, ProbeAcc&, int)
{
    return mbar_wait_impl(bar, parity, abort_flag);
}
#endif

// ---- proxy fences -------------------------------------------------------------
// Generic-proxy shared-memory writes must be made visible to the async proxy
// (TMA stores, tcgen05.mma / tcgen05.cp operand reads) before the hand-off.
NVFP4_DEVICE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- TMA (cp.async.bulk.tensor, never multicast) -------------------------------
NVFP4_DEVICE void prefetch_tensormap(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
NVFP4_DEVICE void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
// Untiled bulk copy global -> this CTA's shared memory (both addresses 16-byte aligned, size a multiple of
// 16); the bytes complete on `bar`.
NVFP4_DEVICE void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
NVFP4_DEVICE void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1,
                                   uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "l"(policy)
        : "memory");
}

NVFP4_DEVICE uint64_t l2_policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ---- programmatic dependent launch -----------------------------------------------
NVFP4_DEVICE void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
NVFP4_DEVICE void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- tensor memory -----------------------------------------------------------------
// TMEM address: lane in bits [31:16], column in bits [15:0].
template <uint32_t kCols>
NVFP4_DEVICE void tmem_alloc(uint32_t* smem_result)
{
    static_assert(kCols >= 32 && kCols <= 512 && (kCols & (kCols - 1)) == 0, "TMEM columns: power of two in [32, 512]");
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "n"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <uint32_t kCols>
NVFP4_DEVICE void tmem_dealloc(uint32_t taddr)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(kCols) : "memory");
}
NVFP4_DEVICE void tcgen05_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
NVFP4_DEVICE void tcgen05_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// All earlier tcgen05.mma / tcgen05.cp of this thread arrive (once) on `bar` when they retire.
NVFP4_DEVICE void tcgen05_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 rows x 128 bit from shared memory, replicated into the four 32-lane
// quadrants: one 128-row x 4-byte scale-factor atom into 4 TMEM columns.
NVFP4_DEVICE void tcgen05_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with per-16-element E4M3 block scales read from TMEM.
// E2M1 operands, K = 64 per instruction.
NVFP4_DEVICE void tcgen05_mma_nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                   uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
        : "memory");
}

// Instruction descriptor of kind::mxf4nvf4: E2M1 x E2M1, UE4M3 scales, both operands K-major.
//   [4,6) B scale id  [7,10) A format (1 = E2M1)  [10,13) B format  [15] A major  [16] B major
//   [17,23) N >> 3  [23] scale format (0 = UE4M3)  [24,29) M >> 4  [29,31) A scale id  [31] K size (0 = 64)
__host__ __device__ constexpr uint32_t make_idesc_nvf4(uint32_t m, uint32_t n)
{
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Shared-memory matrix descriptor (K-major):
//   [0,14) address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) version (1 on sm_100)   [61,64) swizzle: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B
enum : uint64_t { kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6 };
NVFP4_DEVICE uint64_t make_smem_desc(uint32_t smem_addr, uint32_t stride_bytes, uint64_t swizzle)
{
    return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(stride_bytes >> 4) << 32) |
           (1ull << 46) | (swizzle << 61);
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets row (lane base + i), columns [c, c + 32).
NVFP4_DEVICE void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
NVFP4_DEVICE void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 4 columns of 32-bit: thread i of the warp writes its four words to lane (base + i).
NVFP4_DEVICE void tmem_st_32x32b_x4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}
// 32 lanes x N columns of 32-bit in one instruction: thread i of the warp writes v[0..N) to lane (base + i),
// columns [c, c + N).
template <uint32_t N>
NVFP4_DEVICE void tmem_st_32x32b(uint32_t taddr, const uint32_t (&v)[N])
{
    static_assert(N == 4 || N == 8 || N == 16 || N == 32, "column count");
    if constexpr (N == 4) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
                     ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
    } else if constexpr (N == 8) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
    } else if constexpr (N == 16) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                     ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
    } else {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                     ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
    }
}
NVFP4_DEVICE void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
NVFP4_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- shared-memory vector access -------------------------------------------------------
NVFP4_DEVICE uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
NVFP4_DEVICE void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
NVFP4_DEVICE void sts64(uint32_t addr, uint32_t a, uint32_t b)
{
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
NVFP4_DEVICE void sts32(uint32_t addr, uint32_t a) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(a) : "memory"); }
NVFP4_DEVICE void sts16(uint32_t addr, uint32_t a)
{
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(static_cast<unsigned short>(a)) : "memory");
}
NVFP4_DEVICE void sts8(uint32_t addr, uint32_t a)
{
    asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(a) : "memory");
}
NVFP4_DEVICE uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// ---- number-format converts ---------------------------------------------------------------
// Eight FP32 -> eight E2M1 codes in one word (RNE, saturating); element 0 in the lowest nibble.
NVFP4_DEVICE uint32_t cvt_e2m1x8(float f0, float f1, float f2, float f3, float f4, float f5, float f6, float f7)
{
    uint32_t r;
    asm("{\n"
        " .reg .b8 t0, t1, t2, t3;\n"
        " cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n"
        " cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n"
        " cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n"
        " cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n"
        " mov.b32 %0, {t0, t1, t2, t3};\n"
        "}\n"
        : "=r"(r)
        : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
    return r;
}
// One byte holding two E2M1 codes -> two FP16 values (low nibble in the low half).
NVFP4_DEVICE uint32_t cvt_e2m1x2_to_f16x2(uint32_t byte)
{
    uint32_t r;
    asm("{\n .reg .b8 t;\n cvt.u8.u32 t, %1;\n cvt.rn.f16x2.e2m1x2 %0, t;\n}" : "=r"(r) : "r"(byte));
    return r;
}
// FP32 -> E4M3 byte (RNE, saturating to 448).
NVFP4_DEVICE uint32_t cvt_e4m3(float x)
{
    unsigned short s;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(s) : "f"(0.0f), "f"(x));
    return static_cast<uint32_t>(s) & 0xffu;
}
// d = a * b + c with a, b FP16 and c, d FP32 (one rounding).
NVFP4_DEVICE float fma_f32_f16(unsigned short a, unsigned short b, float c)
{
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
// max(|a|, |b|) per BF16 lane; the sign of the result is the xor of the signs.
NVFP4_DEVICE uint32_t max_abs_bf16x2(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
NVFP4_DEVICE float rcp_approx(float x)
{
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

}  // namespace nvfp4::ptx

// ---- thread-block clusters: distributed shared memory and cluster-scope barriers --------
namespace nvfp4::ptx {

NVFP4_DEVICE uint32_t cluster_cta_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
NVFP4_DEVICE uint32_t cluster_id_x() { uint32_t r; asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r)); return r; }
NVFP4_DEVICE uint32_t num_clusters_x() { uint32_t r; asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r)); return r; }

// Address of the same shared-memory location in CTA `rank` of the cluster.
NVFP4_DEVICE uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
NVFP4_DEVICE void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier of another CTA of the cluster (address from map_to_cta) with the default, CTA-scope release:
// enough when what the waiter consumes was not written by this thread's generic-proxy stores (tensor-memory traffic is
// ordered by the tcgen05 fences around the barrier).  The cluster-scope releasing form (mbarrier.arrive.release.cluster)
// was measured at ~1500 cycles per arrive on B200.
NVFP4_DEVICE void mbar_arrive_remote(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
NVFP4_DEVICE bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait that acquires at cluster scope (the data was written by other CTAs).
NVFP4_DEVICE bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag)
{
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*abort_flag != 0 || clock64() - t0 > kWaitBudgetCycles) return false;
    }
}
NVFP4_DEVICE bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, ProbeAcc& acc, int idx)
{
    const long long t0 = probe_clock();
    const bool ok = mbar_wait_cluster(bar, parity, abort_flag);
    probe_count(acc, idx, probe_clock() - t0);
    return ok;
}
// Bounded waits that sleep between polls, at CTA or cluster scope: for roles that run ahead and wait long (producers
// waiting for ring space, transform warps waiting for a slot).  Every poll of an mbarrier is an instruction of the
// shared-memory pipe, which the latency-critical roles (MMA issue, scale warps) need for their own barriers and loads:
// a dozen warps polling without pause were measured to stretch a completed-barrier check of the MMA thread to ~350 cycles.
template <bool kCluster>
NVFP4_DEVICE bool mbar_wait_sleep(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t sleep_ns, ProbeAcc& acc,
                                  int idx)
{
    auto poll = [&] { return kCluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity); };
    if (poll()) return true;
    const long long t0 = clock64();
    bool ok = false;
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16 && !ok; ++i) {
            __nanosleep(sleep_ns);
            ok = poll();
        }
        if (ok || *abort_flag != 0 || clock64() - t0 > kWaitBudgetCycles) break;
    }
    probe_count(acc, idx, clock64() - t0);
    return ok;
}
// All earlier tcgen05 operations of this thread arrive, when they retire, on the barrier at
// this offset in every CTA of the cluster named by `cta_mask`.
NVFP4_DEVICE void tcgen05_commit_cluster(uint64_t* bar, uint16_t cta_mask)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(cta_mask)
                 : "memory");
}
// Bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned) from this CTA's shared
// memory to the shared memory of another CTA of the cluster; the bytes complete on `dst_bar`,
// an mbarrier of the destination CTA.  Addresses of the destination come from map_to_cta.
NVFP4_DEVICE void bulk_copy_to_cta(uint32_t dst_cluster_addr, uint32_t src_cta_addr, uint32_t bytes, uint32_t dst_bar)
{
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_cluster_addr), "r"(src_cta_addr), "r"(bytes), "r"(dst_bar)
                 : "memory");
}
// ---- CTA pairs (cta_group::2): one MMA instruction drives the tensor cores of two SMs ----------------
// Tensor memory of both CTAs of a pair at once; one warp of EACH CTA executes it, with the same arguments.
template <uint32_t kCols>
NVFP4_DEVICE void tmem_alloc_pair(uint32_t* smem_result)
{
    static_assert(kCols >= 32 && kCols <= 512 && (kCols & (kCols - 1)) == 0, "TMEM columns: power of two in [32, 512]");
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "n"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <uint32_t kCols>
NVFP4_DEVICE void tmem_dealloc_pair(uint32_t taddr)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(kCols) : "memory");
}
// Tiled load into this CTA's shared memory whose bytes complete on an mbarrier that may live in the other CTA
// of the pair (`bar_cluster_addr` from map_to_cta).  Not a multicast: every CTA fetches its own tile.
NVFP4_DEVICE void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int32_t c0, int32_t c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
// D[tmem of both CTAs] (+)= A * B over a CTA pair: M = 256 (each CTA its own 128 rows of A, from its own shared
// memory at the descriptor's offset), N up to 256 (each CTA holds half of the rows of B), block scales from each
// CTA's own tensor memory (SFA of its rows, SFB of all N).  Issued by one thread of the pair's even CTA.
NVFP4_DEVICE void tcgen05_mma_nvf4_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
        : "memory");
}
// All earlier pair MMAs of this thread arrive, when they retire, on the barrier at this offset in the CTAs of
// the cluster named by `cta_mask`.
NVFP4_DEVICE void tcgen05_commit_pair(uint64_t* bar, uint16_t cta_mask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(cta_mask)
                 : "memory");
}

}  // namespace nvfp4::ptx
