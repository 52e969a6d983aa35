// Host-side plumbing shared by the launchers: thread-local error text, CUDA
// call checking, a per-device runtime record (SM count, kernel attributes set
// once) and the tensor-map encoder.
// Counterpart in the reference: src/runtime/{device,tma_desc,exception}.hpp.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
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

struct DeviceInfo {
    bool known = false;
    int hw_sms = 0;       // multiProcessorCount
    int num_sms = 0;      // what the persistent grids use (set_num_sms)
    int cc_major = 0, cc_minor = 0;
    int max_smem_optin = 0;
};

// Properties of `device` (< 0: current), cached per device (not per process).
int device_info(int device, DeviceInfo** out);

// 2-D tiled tensor map.  dims/box: innermost first, in elements; row_stride_bytes
// is the stride of dimension 1.  Returns NVFP4_E_CUDA with the driver's code on failure.
int encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                         uint64_t dim0, uint64_t dim1, uint64_t row_stride_bytes, uint32_t box0, uint32_t box1,
                         CUtensorMapSwizzle swizzle);

}  // namespace nvfp4::host
