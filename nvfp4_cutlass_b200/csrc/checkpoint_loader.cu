// NVFP4 checkpoint layout -> the layout the grouped GEMM reads.
//
// Checkpoints store each projection of an expert on its own: packed E2M1 codes `weight_packed` (N_p, K/2),
// E4M3 block scales `weight_scale` (N_p, K/16) row-major, and ONE FP32 `weight_global_scale` per projection and
// expert.  The GEMM wants the projections that share an activation fused along N (gate and up -> N = N_gate +
// N_up), the scales transposed into (E * K/64, N) words of four bytes, and ONE global scale gw per expert,
// applied in its epilogue.  Fusing projections with different global scales therefore means re-folding: with
// the shared gw'[e] = max over the parts of their own global multiplier G_p[e], every block scale becomes
// S' = Q_e4m3(S * (G_p / gw')) (ratio <= 1, so nothing overflows; a non-zero scale that would round to zero is
// held at the smallest subnormal).  A single part re-folds with ratio 1 and comes through bit for bit.
// The codes are copied unchanged.  (The reference describes this step and leaves it to the weight loader:
// docs/bf16-dual-nvfp4-algorithm.html:235-244; layouts: python/nvfp4_gemm/layout.py:108-127.)
//
// HBM-bound, load-time: 9/16 byte read and written per weight element.
#include <cuda_fp16.h>

#include "host_common.hpp"
#include "launchers.hpp"
#include "ptx.cuh"

namespace nvfp4 {
namespace {

constexpr int kMaxParts = NVFP4_MAX_CHECKPOINT_PARTS;

struct Parts {
    const uint8_t* packed[kMaxParts];     // (E, rows[p], K/2)
    const uint8_t* scale[kMaxParts];      // (E, rows[p], K/16) E4M3 bytes
    const float* global[kMaxParts];       // (E,)
    int rows[kMaxParts];
    int first_row[kMaxParts];             // row of the fused N axis where the part starts
    int num;
};

// the multiplier form of a part's global scale: w = dec(q) * dec(S) * G
__device__ __forceinline__ float multiplier(float global, bool divisor) { return divisor ? __fdiv_rn(1.0f, global) : global; }

__global__ void shared_gw_kernel(Parts parts, bool divisor, int E, float* __restrict__ gw)
{
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    float g = 0.0f;
    for (int p = 0; p < parts.num; ++p) g = fmaxf(g, multiplier(__ldg(parts.global[p] + e), divisor));
    gw[e] = g;
}

__device__ __forceinline__ float e4m3_to_f32(uint32_t code)
{
    uint32_t h2;
    asm("{\n .reg .b16 t;\n cvt.u16.u32 t, %1;\n cvt.rn.f16x2.e4m3x2 %0, t;\n}" : "=r"(h2) : "r"(code & 0xffu));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

// One thread per (row of the fused N axis, 64-element K atom): 32 bytes of codes copied, one scale word
// re-folded and written transposed; consecutive threads take consecutive rows, so the scale words are coalesced.
__global__ void repack_checkpoint_kernel(Parts parts, bool divisor, int K, int n_total, const float* __restrict__ gw,
                                         uint8_t* __restrict__ b, int32_t* __restrict__ sfb)
{
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int at = blockIdx.y, e = blockIdx.z;
    if (n >= n_total) return;
    int p = 0;
#pragma unroll
    for (int i = 1; i < kMaxParts; ++i)
        if (i < parts.num && n >= parts.first_row[i]) p = i;
    const int row = n - parts.first_row[p];
    const int64_t src_row = static_cast<int64_t>(e) * parts.rows[p] + row;
    const uint4* src = reinterpret_cast<const uint4*>(parts.packed[p] + src_row * (K / 2) + at * 32);
    uint4* dst = reinterpret_cast<uint4*>(b + (static_cast<int64_t>(e) * n_total + n) * (K / 2) + at * 32);
    const uint4 c0 = __ldg(src), c1 = __ldg(src + 1);
    dst[0] = c0;
    dst[1] = c1;
    const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(parts.scale[p] + src_row * (K / 16) + at * 4));
    const float ratio = __fdiv_rn(multiplier(__ldg(parts.global[p] + e), divisor), gw[e]);
    uint32_t out = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t sc = (word >> (8 * j)) & 0xffu;
        uint32_t folded = ptx::cvt_e4m3(__fmul_rn(e4m3_to_f32(sc & 0x7fu), ratio));
        if (folded == 0 && (sc & 0x7fu) != 0) folded = 1;        // a live block keeps a non-zero scale
        out |= folded << (8 * j);
    }
    sfb[(static_cast<int64_t>(e) * (K / 64) + at) * n_total + n] = static_cast<int32_t>(out);
}

}  // namespace

int launch_load_checkpoint(int num_parts, const void* const* packed, const void* const* scale, const float* const* global_scale,
                           const int32_t* part_rows, bool divisor, int E, int K, int n_total, void* b, void* sfb, float* gw,
                           cudaStream_t stream)
{
    Parts parts = {};
    parts.num = num_parts;
    int first = 0;
    for (int i = 0; i < num_parts; ++i) {
        parts.packed[i] = static_cast<const uint8_t*>(packed[i]);
        parts.scale[i] = static_cast<const uint8_t*>(scale[i]);
        parts.global[i] = global_scale[i];
        parts.rows[i] = part_rows[i];
        parts.first_row[i] = first;
        first += part_rows[i];
    }
    shared_gw_kernel<<<(E + 127) / 128, 128, 0, stream>>>(parts, divisor, E, gw);
    repack_checkpoint_kernel<<<dim3((n_total + 127) / 128, K / 64, E), 128, 0, stream>>>(
        parts, divisor, K, n_total, gw, static_cast<uint8_t*>(b), static_cast<int32_t*>(sfb));
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

}  // namespace nvfp4
