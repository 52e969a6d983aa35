// Offline NVFP4 weight quantisation on the GPU: w ~= dec(q) * S * G with one FP32 G
// per expert, one E4M3 S per 16 elements and E2M1 codes, written straight into the
// physical layouts the GEMM's tensor maps describe.  Bit-exact with the reference's
// torch implementation (python/nvfp4_gemm/layout.py:68-127): the same three true
// FP32 divisions, the same clamps, RNE everywhere.
//
// HBM-bound: 2 or 4 bytes read per element, 9/16 byte written.  One thread owns one
// 64-element scale atom of one weight row (a 128-byte line of BF16 input, a 32-byte
// sector of packed output); consecutive threads take consecutive rows, so the scale
// words, which the kernel wants transposed to (K/64, N), are written coalesced.
#include <cuda_bf16.h>

#include <mutex>

#include "host_common.hpp"
#include "launchers.hpp"
#include "ptx.cuh"

namespace nvfp4 {
namespace {

template <typename T> __device__ __forceinline__ float load_f32(const T* p);
template <> __device__ __forceinline__ float load_f32<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float load_f32<__nv_bfloat16>(const __nv_bfloat16* p)
{
    return __uint_as_float(static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(p))) << 16);
}

template <typename T>
__global__ void expert_amax_kernel(const T* __restrict__ w, int64_t per_expert, uint32_t* __restrict__ amax_bits)
{
    const int e = blockIdx.y;
    const T* we = w + static_cast<int64_t>(e) * per_expert;
    float m = 0.0f;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < per_expert;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        m = fmaxf(m, fabsf(load_f32(we + i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits + e, __float_as_uint(m));   // non-negative floats order as integers
}

__device__ __forceinline__ float e4m3_to_f32(uint32_t code)
{
    uint32_t h2;
    asm("{\n .reg .b16 t;\n cvt.u16.u32 t, %1;\n cvt.rn.f16x2.e4m3x2 %0, t;\n}" : "=r"(h2) : "r"(code & 0xffu));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

template <typename T>
__global__ void quantize_weight_kernel(const T* __restrict__ w, int N, int K, const uint32_t* __restrict__ amax_bits,
                                       uint8_t* __restrict__ b, int32_t* __restrict__ sfb, float* __restrict__ gw)
{
    const int atoms = K / 64;
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int at = blockIdx.y, e = blockIdx.z;
    const float tiny = 1.17549435e-38f;
    const float g = fmaxf(__fdiv_rn(__uint_as_float(amax_bits[e]), 2688.0f), tiny);
    if (n == 0 && at == 0) gw[e] = g;
    if (n >= N) return;
    const T* src = w + (static_cast<int64_t>(e) * N + n) * K + at * 64;
    uint32_t word = 0;
    uint32_t packed[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float x[16];
        float bmax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) { x[i] = load_f32(src + j * 16 + i); bmax = fmaxf(bmax, fabsf(x[i])); }
        const float s_pre = fmaxf(__fdiv_rn(__fdiv_rn(bmax, 6.0f), g), 0.001953125f);
        const uint32_t sc = ptx::cvt_e4m3(s_pre);
        word |= sc << (8 * j);
        const float denom = fmaxf(__fmul_rn(e4m3_to_f32(sc), g), tiny);
        float q[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) q[i] = __fdiv_rn(x[i], denom);
        packed[2 * j] = ptx::cvt_e2m1x8(q[0], q[1], q[2], q[3], q[4], q[5], q[6], q[7]);
        packed[2 * j + 1] = ptx::cvt_e2m1x8(q[8], q[9], q[10], q[11], q[12], q[13], q[14], q[15]);
    }
    uint4* dst = reinterpret_cast<uint4*>(b + (static_cast<int64_t>(e) * N + n) * (K / 2) + at * 32);
    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    sfb[(static_cast<int64_t>(e) * atoms + at) * N + n] = static_cast<int32_t>(word);
}

// The two kernels (G needs the whole expert's maximum first) with the per-expert maxima staged in `amax_bits`,
// E words the caller provides; they are cleared here, on the call's stream.
int run_quantize_weight(const void* w, int w_dtype, int E, int N, int K, void* b, void* sfb, float* gw, uint32_t* amax_bits,
                        cudaStream_t stream)
{
    NVFP4_CUDA_CHECK(cudaMemsetAsync(amax_bits, 0, sizeof(uint32_t) * E, stream));
    const int64_t per_expert = static_cast<int64_t>(N) * K;
    int blocks = static_cast<int>((per_expert + 256 * 16 - 1) / (256 * 16));
    blocks = blocks < 1 ? 1 : (blocks > 1024 ? 1024 : blocks);
    const dim3 qgrid((N + 127) / 128, K / 64, E);
    if (w_dtype == NVFP4_DTYPE_BF16) {
        auto* wt = static_cast<const __nv_bfloat16*>(w);
        expert_amax_kernel<<<dim3(blocks, E), 256, 0, stream>>>(wt, per_expert, amax_bits);
        quantize_weight_kernel<<<qgrid, 128, 0, stream>>>(wt, N, K, amax_bits, static_cast<uint8_t*>(b),
                                                          static_cast<int32_t*>(sfb), gw);
    } else {
        auto* wt = static_cast<const float*>(w);
        expert_amax_kernel<<<dim3(blocks, E), 256, 0, stream>>>(wt, per_expert, amax_bits);
        quantize_weight_kernel<<<qgrid, 128, 0, stream>>>(wt, N, K, amax_bits, static_cast<uint8_t*>(b),
                                                          static_cast<int32_t*>(sfb), gw);
    }
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

}  // namespace

// The per-expert maxima live in a stream-ordered allocation from the library's memory pool: calls on
// different streams never share it, nothing synchronises the device, and after the first call it is a pool look-up.
int launch_quantize_weight(const void* w, int w_dtype, int E, int N, int K, void* b, void* sfb, float* gw,
                           cudaStream_t stream)
{
    if (E == 0 || N == 0 || K == 0) return NVFP4_OK;
    int dev = 0;
    NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    if (int rc = host::workspace_pool(dev, &pool)) return rc;
    uint32_t* amax_bits = nullptr;
    NVFP4_CUDA_CHECK(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&amax_bits), sizeof(uint32_t) * E, pool, stream));
    const int rc = run_quantize_weight(w, w_dtype, E, N, K, b, sfb, gw, amax_bits, stream);
    cudaFreeAsync(amax_bits, stream);
    return rc;
}

// ---- allocation-free variant ----------------------------------------------------------
// Same two kernels, but the per-expert maxima are staged in a fixed array that is part of
// the library image instead of an allocation.  Every process that loads the library holds
// NVFP4_STATIC_MAX_EXPERTS words of it on every GPU it uses, until it exits.
namespace {
static __device__ __align__(256) uint32_t g_static_amax[NVFP4_STATIC_MAX_EXPERTS];
std::mutex g_static_mutex;
}  // namespace

// In host code `g_static_amax` is only the host-side handle of the symbol, not an address
// a kernel can dereference.  The device address comes from cudaGetSymbolAddress, asked once
// per device with that device current -- here on the first call made on that device.
int launch_quantize_weight_static(const void* w, int w_dtype, int E, int N, int K, void* b, void* sfb, float* gw,
                                  cudaStream_t stream)
{
    if (E == 0 || N == 0 || K == 0) return NVFP4_OK;
    static uint32_t* scratch_addr[host::kMaxDevices] = {};
    int dev = 0;
    NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= host::kMaxDevices) return host::fail(NVFP4_E_INVALID_ARGUMENT, "device %d out of range", dev);
    uint32_t* amax_bits = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (scratch_addr[dev] == nullptr) {
            void* addr = nullptr;
            NVFP4_CUDA_CHECK(cudaGetSymbolAddress(&addr, g_static_amax));
            if (addr == nullptr) return host::fail(NVFP4_E_CUDA, "cudaGetSymbolAddress gave no address for the scratch array");
            scratch_addr[dev] = static_cast<uint32_t*>(addr);
        }
        amax_bits = scratch_addr[dev];
    }
    // the array keeps whatever the previous call left in it: run_quantize_weight clears the maxima first
    return run_quantize_weight(w, w_dtype, E, N, K, b, sfb, gw, amax_bits, stream);
}

}  // namespace nvfp4
