// Host-side plumbing shared by the launchers: thread-local error text, CUDA
// call checking, a per-device runtime record (SM count, kernel attributes set
// once) and the tensor-map encoder.
// Counterpart in the reference: src/runtime/{device,tma_desc,exception}.hpp.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <type_traits>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/nvfp4_b200.h"

namespace nvfp4::host {

// Sets the calling thread's error text and returns `code` (so callers can `return fail(...)`).
int fail(int code, const char* fmt, ...);
void clear_error();

#define NVFP4_CUDA_CHECK(expr)                                                                        \
    do {                                                                                              \
        cudaError_t err__ = (expr);                                                                   \
        if (err__ != cudaSuccess)                                                                     \
            return ::nvfp4::host::fail(NVFP4_E_CUDA, "%s failed: %s (%s:%d)", #expr,                  \
                                       cudaGetErrorString(err__), __FILE__, __LINE__);                \
    } while (0)

#define NVFP4_REQUIRE(cond, ...)                                                                      \
    do {                                                                                              \
        if (!(cond)) return ::nvfp4::host::fail(NVFP4_E_INVALID_ARGUMENT, __VA_ARGS__);               \
    } while (0)

constexpr int kMaxDevices = 64;

// Calls f(std::integral_constant<int, policy>{}) for an activation scale policy code (NVFP4_POLICY_*), so that
// launchers can pick the kernel instantiation of a policy without a ladder of their own.
template <typename F>
int with_policy(int policy, F&& f)
{
    switch (policy) {
        case NVFP4_POLICY_DERIVED_DIV8: return f(std::integral_constant<int, 0>{});
        case NVFP4_POLICY_RESIDUAL_AMAX: return f(std::integral_constant<int, 1>{});
        case NVFP4_POLICY_DERIVED_DIV4: return f(std::integral_constant<int, 2>{});
        case NVFP4_POLICY_DIV4_RADIX8: return f(std::integral_constant<int, 3>{});
        default: return fail(NVFP4_E_INVALID_ARGUMENT, "unknown scale policy %d", policy);
    }
}

struct DeviceInfo {
    bool known = false;
    int hw_sms = 0;       // multiProcessorCount
    int num_sms = 0;      // what the persistent grids use (set_num_sms)
    int cc_major = 0, cc_minor = 0;
    int max_smem_optin = 0;
};

// Launch with, optionally, the programmatic-stream-serialisation attribute (programmatic dependent launch): the
// kernel may then be scheduled while the previous kernel of the stream is still draining; it must execute
// griddepcontrol.wait before it touches anything that kernel wrote.
// Counterpart in the reference: src/jit/launch.hpp:63-96.
template <typename... Params, typename... Args>
int launch_kernel_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                          unsigned cluster_x, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = n;
    if (cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...); err != cudaSuccess)
        return fail(NVFP4_E_CUDA, "kernel launch failed: %s", cudaGetErrorString(err));
    return NVFP4_OK;
}
template <typename... Params, typename... Args>
int launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, Args&&... args)
{
    return launch_kernel_cluster(kernel, grid, block, smem, stream, pdl, 1u, static_cast<Args&&>(args)...);
}

// Properties of `device` (< 0: current), cached per device (not per process).
int device_info(int device, DeviceInfo** out);

// Stream-ordered workspace: a private memory pool per device that keeps what it has been given, so that after
// the first call an allocation is a pool look-up ordered on the caller's stream (no device synchronisation,
// safe with concurrent streams, legal during stream capture).
int workspace_pool(int dev, cudaMemPool_t* out);

// 2-D tiled tensor map.  dims/box: innermost first, in elements; row_stride_bytes
// is the stride of dimension 1.  Returns NVFP4_E_CUDA with the driver's code on failure.
int encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                         uint64_t dim0, uint64_t dim1, uint64_t row_stride_bytes, uint32_t box0, uint32_t box1,
                         CUtensorMapSwizzle swizzle);

}  // namespace nvfp4::host
