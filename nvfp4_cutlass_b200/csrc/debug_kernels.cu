// Test and measurement hooks behind nvfp4_debug_decompose and nvfp4_debug_mma_peak.
// They run the same device functions as the GEMM kernels, so what they show is
// what the GEMM computes.
#include <cuda_bf16.h>

#include "host_common.hpp"
#include "launchers.hpp"
#include "transform.cuh"

namespace nvfp4 {
namespace {

// One CTA per 128 x 128 activation tile: stage the tile in shared memory exactly
// where TMA would put it, run the GEMM's transform, then copy the products out
// through the same addressing functions the MMA descriptors assume.
// Counterpart in the reference: tests/standalone/test_transform.cu:50-132.
template <uint32_t kThreads, int kPolicy>
__global__ void __launch_bounds__(kThreads) decompose_dump_kernel(const __nv_bfloat16* __restrict__ a, int64_t lda, int K,
                                                                  uint8_t* __restrict__ q0, uint8_t* __restrict__ q1,
                                                                  uint8_t* __restrict__ s0, uint8_t* __restrict__ s1)
{
    extern __shared__ uint8_t dump_smem_raw[];
    uint8_t* tile = dump_smem_raw + ((1024u - (ptx::smem_u32(dump_smem_raw) & 1023u)) & 1023u);
    uint8_t* a0 = tile + 32768;
    uint8_t* a1 = a0 + 8192;
    uint8_t* sfa0 = a1 + 8192;
    uint8_t* sfa1 = sfa0 + 1024;
    const uint32_t kb = blockIdx.x, mb = blockIdx.y, t = threadIdx.x;
    for (uint32_t c = t; c < 128 * 16; c += kThreads) {          // 16-byte chunks: 128 rows x 16 per row
        const uint32_t row = c >> 4, k = (c & 15u) * 8u;
        const uint4 v = *reinterpret_cast<const uint4*>(a + (static_cast<int64_t>(mb) * 128 + row) * lda + kb * 128 + k);
        *reinterpret_cast<uint4*>(tile + xform::a_bf16_offset<128>(row, k)) = v;
    }
    __syncthreads();
    xform::transform_tile<128, 128, kThreads, true, 4, 0, kPolicy>(ptx::smem_u32(tile), ptx::smem_u32(a0), ptx::smem_u32(a1),
                                               ptx::smem_u32(sfa0), ptx::smem_u32(sfa1), t, [] {});
    __syncthreads();
    for (uint32_t c = t; c < 128 * 4; c += kThreads) {           // 16-byte chunks of packed codes: 4 per row
        const uint32_t row = c >> 2, k = (c & 3u) * 32u;
        const int64_t dst = (static_cast<int64_t>(mb) * 128 + row) * (K / 2) + (kb * 128 + k) / 2;
        *reinterpret_cast<uint4*>(q0 + dst) = *reinterpret_cast<const uint4*>(a0 + xform::fp4_sw64_offset(row, k));
        *reinterpret_cast<uint4*>(q1 + dst) = *reinterpret_cast<const uint4*>(a1 + xform::fp4_sw64_offset(row, k));
    }
    for (uint32_t c = t; c < 128 * 2; c += kThreads) {           // one scale word per row and K atom
        const uint32_t row = c >> 1, atom = c & 1u;
        const int64_t dst = (static_cast<int64_t>(mb) * 128 + row) * (K / 16) + kb * 8 + atom * 4;
        *reinterpret_cast<uint32_t*>(s0 + dst) = *reinterpret_cast<const uint32_t*>(sfa0 + atom * 512 + xform::sf_word_offset(row));
        *reinterpret_cast<uint32_t*>(s1 + dst) = *reinterpret_cast<const uint32_t*>(sfa1 + atom * 512 + xform::sf_word_offset(row));
    }
}

// A bounded wait that runs out: one thread waits, with a budget of `budget` clock cycles, on an mbarrier nobody
// arrives on, while the CTA holds tensor memory like a GEMM CTA does.  On expiry it takes the same way out as
// the GEMM kernels: abort flag, status bit 0, every thread meets at the closing barrier, tensor memory is freed.
// Nothing faults and nothing hangs; this exists so that the unwind path can be tested.
__global__ void __launch_bounds__(64, 1) wait_timeout_kernel(long long budget, int32_t* status)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot, abort_word;
    volatile uint32_t* abort_flag = &abort_word;
    const uint32_t warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { ptx::mbar_init(&bar, 1); *abort_flag = 0; ptx::fence_mbar_init(); }
    if (warp == 1) ptx::tmem_alloc<32>(&tmem_slot);
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0) {
        if (!ptx::mbar_wait_budget(&bar, 0, abort_flag, budget)) {
            *abort_flag = 1;
            atomicOr(status, 1);
        }
    } else if (warp == 1) {
        // a second role that would wait for the first: it sees the abort flag and gives up at once
        while (*abort_flag == 0 && !ptx::mbar_try_wait(&bar, 0)) { __nanosleep(200); }
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc<32>(tmem);
    }
}

// Resident-operand tensor-pipe study: every CTA issues `iters` rounds of `num_cp`
// scale-factor copies (tcgen05.cp 32x128b.warpx4) followed by `num_mma` block-scaled FP4
// MMAs of 128 x mma_n x 64 on operands that never leave shared / tensor memory.  With
// num_cp = 0, num_mma = 8, mma_n = 256 this is the tensor-pipe ceiling.  `alt_cols`
// alternates the scale columns between two sets from round to round.
template <uint32_t kN>
__global__ void __launch_bounds__(128, 1) mma_pattern_kernel(int iters, int num_cp, int num_mma, int alt_cols, int32_t* status)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (smem - ptx::smem_u32(smem_raw));
    constexpr uint32_t kA = 0, kB = 8192, kSF = kB + 16384, kBar = kSF + 2048;
    uint64_t* bar = reinterpret_cast<uint64_t*>(gen + kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + kBar + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    for (uint32_t i = threadIdx.x; i < (kSF) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(gen)[i] = 0x9e3779b9u * (i + 1u + blockIdx.x);       // arbitrary FP4 codes
    for (uint32_t i = threadIdx.x; i < 2048 / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(gen + kSF)[i] = 0x38383838u;                         // scales of 1.0
    if (threadIdx.x == 0) { ptx::mbar_init(bar, 1); *abort_flag = 0; ptx::fence_mbar_init(); }
    if (threadIdx.x < 32) ptx::tmem_alloc<512>(tmem_slot);
    ptx::fence_proxy_async_smem();
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < 16; ++i)
            ptx::tcgen05_cp_32x128b_warpx4(tmem + 256 + 4 * i, ptx::make_smem_desc(smem + kSF + (i & 3) * 512, 128, ptx::kSwizzleNone));
        constexpr uint32_t idesc = ptx::make_idesc_nvf4(128, kN);
        for (int it = 0; it < iters; ++it) {
            const uint32_t col = 256 + ((alt_cols && (it & 1)) ? 32 : 0);
            for (int j = 0; j < num_cp; ++j)
                ptx::tcgen05_cp_32x128b_warpx4(tmem + col + 4 * (j & 7), ptx::make_smem_desc(smem + kSF + (j & 3) * 512, 128, ptx::kSwizzleNone));
            for (int j = 0; j < num_mma; ++j)
                ptx::tcgen05_mma_nvf4(tmem, ptx::make_smem_desc(smem + kA + (j & 1u) * 32, 512, ptx::kSwizzle64B),
                                      ptx::make_smem_desc(smem + kB + (j & 1u) * 32, 512, ptx::kSwizzle64B), idesc,
                                      tmem + col, tmem + col + 8, (it | j) != 0 ? 1u : 0u);
        }
        ptx::tcgen05_commit(bar);
        if (!ptx::mbar_wait_impl(bar, 0, abort_flag) && status != nullptr) atomicOr(status, 1);
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) { ptx::tcgen05_fence_after_sync(); ptx::tmem_dealloc<512>(tmem); }
}


// The same ceiling for CTA pairs: one thread of the even CTA of every 2-CTA cluster issues 256 x 256 x 64 MMAs
// (tcgen05.mma.cta_group::2) on operands resident in the two CTAs' shared memories (each holds its 128 rows of A and
// 128 of the 256 rows of B) and scales resident in their tensor memories.
__global__ void __launch_bounds__(128, 1) mma_pair_peak_kernel(int iters, int num_mma, int32_t* status)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (smem - ptx::smem_u32(smem_raw));
    constexpr uint32_t kA = 0, kB = 8192, kBar = kB + 8192;
    uint64_t* bar = reinterpret_cast<uint64_t*>(gen + kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + kBar + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    for (uint32_t i = threadIdx.x; i < kBar / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(gen)[i] = 0x9e3779b9u * (i + 1u + blockIdx.x);       // arbitrary FP4 codes
    if (threadIdx.x == 0) { ptx::mbar_init(bar, 1); *abort_flag = 0; ptx::fence_mbar_init(); }
    if (threadIdx.x < 32) ptx::tmem_alloc_pair<512>(tmem_slot);
    ptx::fence_proxy_async_smem();
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_sync();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    {
        uint32_t ones[32];                                                              // scales of 1.0 in 32 columns
#pragma unroll
        for (int i = 0; i < 32; ++i) ones[i] = 0x38383838u;
        ptx::tmem_st_32x32b(tmem + (((threadIdx.x >> 5) * 32) << 16) + 256, ones);
        ptx::tmem_st_wait();
    }
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_sync();
    ptx::tcgen05_fence_after_sync();
    if (threadIdx.x == 0 && ptx::cluster_cta_rank() == 0) {
        constexpr uint32_t idesc = ptx::make_idesc_nvf4(256, 256);
        for (int it = 0; it < iters; ++it)
            for (int j = 0; j < num_mma; ++j)
                ptx::tcgen05_mma_nvf4_pair(tmem, ptx::make_smem_desc(smem + kA + (j & 1u) * 32, 512, ptx::kSwizzle64B),
                                           ptx::make_smem_desc(smem + kB + (j & 1u) * 32, 512, ptx::kSwizzle64B), idesc,
                                           tmem + 256, tmem + 264, (it | j) != 0 ? 1u : 0u);
        ptx::tcgen05_commit_pair(bar, 3);
    }
    if (threadIdx.x == 0 && !ptx::mbar_wait_impl(bar, 0, abort_flag) && status != nullptr) atomicOr(status, 1);
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_sync();
    if (threadIdx.x < 32) { ptx::tcgen05_fence_after_sync(); ptx::tmem_dealloc_pair<512>(tmem); }
}

}  // namespace

int launch_debug_decompose(const void* a, int64_t lda, int M, int K, int policy, void* q0, void* q1, void* s0, void* s1,
                           cudaStream_t stream)
{
    if (M == 0 || K == 0) return NVFP4_OK;
    constexpr int kDumpSmem = 32768 + 2 * 8192 + 2 * 1024 + 1024;
    return host::with_policy(policy, [&](auto pol) {
        auto kernel = decompose_dump_kernel<256, decltype(pol)::value>;
        NVFP4_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDumpSmem));
        kernel<<<dim3(K / 128, M / 128), 256, kDumpSmem, stream>>>(
            static_cast<const __nv_bfloat16*>(a), lda, K, static_cast<uint8_t*>(q0), static_cast<uint8_t*>(q1),
            static_cast<uint8_t*>(s0), static_cast<uint8_t*>(s1));
        NVFP4_CUDA_CHECK(cudaGetLastError());
        return static_cast<int>(NVFP4_OK);
    });
}

int launch_debug_wait_timeout(int64_t budget_cycles, int32_t* status, cudaStream_t stream)
{
    wait_timeout_kernel<<<1, 64, 0, stream>>>(static_cast<long long>(budget_cycles), status);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_mma_pattern(int iters, int num_cp, int num_mma, int mma_n, int alt_cols, int num_sms, double* flops_per_launch,
                       cudaStream_t stream)
{
    constexpr int kSmem = 8192 + 16384 + 2048 + 64 + 1024;
    void (*kernel)(int, int, int, int, int32_t*) = nullptr;
    switch (mma_n) {
        case 16: kernel = mma_pattern_kernel<16>; break;
        case 32: kernel = mma_pattern_kernel<32>; break;
        case 64: kernel = mma_pattern_kernel<64>; break;
        case 128: kernel = mma_pattern_kernel<128>; break;
        case 256: kernel = mma_pattern_kernel<256>; break;
        default: return host::fail(NVFP4_E_INVALID_ARGUMENT, "mma_n %d not in {16, 32, 64, 128, 256}", mma_n);
    }
    NVFP4_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    kernel<<<num_sms, 128, kSmem, stream>>>(iters, num_cp, num_mma, alt_cols, nullptr);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    if (flops_per_launch) *flops_per_launch = 2.0 * 128 * mma_n * 64 * static_cast<double>(num_mma) * iters * num_sms;
    return NVFP4_OK;
}

int launch_mma_peak_pair(int iters, int num_sms, double* flops_per_launch, cudaStream_t stream)
{
    constexpr int kSmem = 8192 + 8192 + 64 + 1024;
    const int pairs = num_sms / 2;
    if (pairs < 1) return host::fail(NVFP4_E_UNSUPPORTED, "a CTA pair needs two SMs");
    NVFP4_CUDA_CHECK(cudaFuncSetAttribute(mma_pair_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    if (int rc = host::launch_kernel_cluster(mma_pair_peak_kernel, dim3(static_cast<unsigned>(2 * pairs)), dim3(128), kSmem, stream,
                                             false, 2u, iters, 8, static_cast<int32_t*>(nullptr)))
        return rc;
    if (flops_per_launch) *flops_per_launch = 2.0 * 256 * 256 * 64 * 8.0 * iters * pairs;
    return NVFP4_OK;
}

int launch_mma_peak(int iters, int num_sms, double* flops_per_launch, cudaStream_t stream)
{
    return launch_mma_pattern(iters, 0, 8, 256, 0, num_sms, flops_per_launch, stream);
}

}  // namespace nvfp4
