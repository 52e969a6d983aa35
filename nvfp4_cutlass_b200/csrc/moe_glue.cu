// Row movers and the activation function of the expert-parallel MoE layer around the grouped GEMM.
//
// The grouped GEMM wants its rows expert-major with every group padded to the tile height; tokens arrive
// token-major with k experts each.  Between the two sit a gather (token rows -> send order), a scatter
// (received rows -> padded expert-major buffer), SwiGLU between the two GEMMs, and the weighted sum of the k
// expert outputs of every token.  All four are plain HBM-bound passes over rows of a few KB: one block per
// row (grid-stride), 16-byte accesses, nothing staged in shared memory.  Written as kernels because the
// equivalent chains of framework index operations took four times as long as the two GEMMs between them.
// The reference project has no multi-GPU mode; these have no counterpart there.
#include <cuda_bf16.h>

#include <cstdint>

#include "host_common.hpp"
#include "launchers.hpp"
#include "transform.cuh"

namespace nvfp4 {
namespace {

// dst[dst_idx ? dst_idx[i] : i] = src[(src_idx ? src_idx[i] : i) / src_div], rows of row16 16-byte words
__global__ void __launch_bounds__(256)
permute_rows_kernel(const uint4* __restrict__ src, int64_t src_ld16, const int64_t* __restrict__ src_idx, int src_div,
                    const int64_t* __restrict__ dst_idx, int64_t n_rows, int row16, uint4* __restrict__ dst, int64_t dst_ld16)
{
    for (int64_t i = blockIdx.x; i < n_rows; i += gridDim.x) {
        const int64_t s = (src_idx ? src_idx[i] : i) / src_div;
        const int64_t d = dst_idx ? dst_idx[i] : i;
        const uint4* sp = src + s * src_ld16;
        uint4* dp = dst + d * dst_ld16;
        for (int c = threadIdx.x; c < row16; c += blockDim.x) dp[c] = __ldg(sp + c);
    }
}

__device__ __forceinline__ float silu(float g) { return g / (1.0f + __expf(-g)); }

// out[r, j] = silu(h[r, j]) * h[r, inter + j], BF16 in and out, products rounded once from FP32
__global__ void __launch_bounds__(256)
swiglu_kernel(const uint4* __restrict__ h, int64_t h_ld16, int64_t rows, int inter16, uint4* __restrict__ out, int64_t out_ld16)
{
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const uint4* gate = h + r * h_ld16;
        const uint4* up = gate + inter16;
        uint4* o = out + r * out_ld16;
        for (int c = threadIdx.x; c < inter16; c += blockDim.x) {
            const uint4 g = __ldg(gate + c), u = __ldg(up + c);
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
            uint32_t ow[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
                const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[i]));
                const __nv_bfloat162 p = __floats2bfloat162_rn(silu(gf.x) * uf.x, silu(gf.y) * uf.y);
                ow[i] = *reinterpret_cast<const uint32_t*>(&p);
            }
            o[c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
    }
}

// y[t] = sum_j w[t, j] * rows[pos[t * k + j]] in FP32, j ascending (deterministic), BF16 out
__global__ void __launch_bounds__(256)
combine_rows_kernel(const uint4* __restrict__ rows, int64_t rows_ld16, const int64_t* __restrict__ pos,
                    const float* __restrict__ w, int64_t tokens, int k, int row16, uint4* __restrict__ y, int64_t y_ld16)
{
    for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
        for (int c = threadIdx.x; c < row16; c += blockDim.x) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int j = 0; j < k; ++j) {
                const float wj = __ldg(w + t * k + j);
                const uint4 v = __ldg(rows + __ldg(pos + t * k + j) * rows_ld16 + c);
                const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vw[i]));
                    acc[2 * i] = fmaf(wj, f.x, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(wj, f.y, acc[2 * i + 1]);
                }
            }
            uint32_t ow[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                ow[i] = *reinterpret_cast<const uint32_t*>(&p);
            }
            y[t * y_ld16 + c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
    }
}

// Peer-memory variants for the expert-parallel layer on several GPUs of one NVLink domain.  `peers` holds, per
// rank, the base address of that rank's copy of a symmetric buffer as mapped into this process.
//
// dispatch: row i of the send order (token src_idx[i] / src_div) is stored straight into row dst_row[i] of rank
// dst_rank[i]'s expert-major buffer -- the gather, the all-to-all and the scatter in one pass, every byte
// crossing NVLink once as plain 16-byte stores.
// A pair whose rank or row is outside [0, world) x [0, rows_cap) is skipped (row -1 is how the plan marks a pair that
// does not fit its expert's capacity; anything else out of range also raises bit 3 of the status word).
//
// Both peer kernels run as a few FAT blocks -- 1024 threads, one warp per row, eight 16-byte accesses in flight per
// thread -- on as many SMs as the caller grants them (`sm_budget`; 0 = every SM).  A block fills its SM, so it never
// shares one with a GEMM block: with the micro-batches of a step on streams of their own and the GEMMs sized to the
// other SMs (nvfp4_set_num_sms), the NVLink traffic of one micro-batch runs beside the GEMMs of another whichever
// kernel is launched first.  (Slim blocks tucked into the registers a resident GEMM block leaves free were tried
// first: ~170 threads per SM cannot keep enough loads in flight for NVLink's latency.)  Sixteen SMs carry more than
// the ~0.7 TB/s an NVLink port takes.
constexpr int kPeerThreads = 1024;
__global__ void __launch_bounds__(kPeerThreads, 1)
dispatch_rows_peer_kernel(const uint4* __restrict__ src, int64_t src_ld16, const int64_t* __restrict__ src_idx, int src_div,
                          const int64_t* __restrict__ peers, const int64_t* __restrict__ dst_rank,
                          const int64_t* __restrict__ dst_row, int64_t n_rows, int row16, int64_t dst_ld16, int world,
                          int64_t rows_cap, int32_t* __restrict__ status)
{
    const int lane = threadIdx.x & 31, warps = kPeerThreads / 32;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * warps + (threadIdx.x >> 5); i < n_rows; i += static_cast<int64_t>(gridDim.x) * warps) {
        const int64_t r = dst_rank[i], row = dst_row[i];
        if (r < 0 || r >= world || row < 0 || row >= rows_cap) {
            if (row != -1 && lane == 0 && status != nullptr) atomicOr(status, 8);
            continue;
        }
        const uint4* sp = src + ((src_idx ? src_idx[i] : i) / src_div) * src_ld16;
        uint4* dp = reinterpret_cast<uint4*>(peers[r]) + row * dst_ld16;
        int c = lane;
        for (; c + 7 * 32 < row16; c += 8 * 32) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldg(sp + c + u * 32);
#pragma unroll
            for (int u = 0; u < 8; ++u) dp[c + u * 32] = v[u];
        }
        for (; c < row16; c += 32) dp[c] = __ldg(sp + c);
    }
}

// Dispatch of QUANTISED rows.  A token goes to k experts and every owner would run Algorithm 1 on its copy of the
// row: the same arithmetic k times, on BF16 rows that crossed NVLink at 2 bytes per element.  Here the sender
// decomposes each token once (xform::decompose_block16, the function every GEMM path uses, so the codes are the same
// bit for bit) and stores, for each of the k pairs, the two packed code rows (K/2 bytes each) and the two rows of
// block scales (K/16 bytes each) into the owner's buffers: 1.125 bytes per element instead of 2.  The owner's
// buffers are three planes of one symmetric allocation: a0 (rows, K/2), a1 (rows, K/2), scales (rows, 2, K/16) --
// the first two are what the split path's GEMM reads through its tensor maps; the scale rows are re-laid into
// 512-byte tensor-memory atoms by relayout_scales_kernel on the owner (scattering 4-byte words over NVLink instead
// would cost more than the BF16 rows did).
// One warp per token.  In step j lane l owns the block pair j * 32 + l (32 elements): its loads are 64-byte pieces of
// one row, its code stores 16 bytes next to its neighbours' (512 contiguous bytes per warp instruction).  Scale bytes
// are gathered by shuffles so that every lane stores 8 consecutive bytes per pass.  K % 1024 == 0.
template <int kRounds>
__global__ void __launch_bounds__(kPeerThreads, 1)
dispatch_quantized_peer_kernel(const uint4* __restrict__ x, int64_t x_ld16, int64_t tokens, int k,
                               const int64_t* __restrict__ peers, int64_t a1_off, int64_t sf_off,
                               const int64_t* __restrict__ dst_rank, const int64_t* __restrict__ dst_row, int world,
                               int64_t rows_cap, int32_t* __restrict__ status)
{
    constexpr int kMaxRounds = kRounds, rounds = kRounds, kdim = kRounds * 1024;
    const int lane = threadIdx.x & 31, warps = kPeerThreads / 32;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * warps + (threadIdx.x >> 5); t < tokens; t += static_cast<int64_t>(gridDim.x) * warps) {
        const uint4* row = x + t * x_ld16;
        uint4 q0[kMaxRounds], q1[kMaxRounds];
        uint32_t s0[kMaxRounds], s1[kMaxRounds];         // two scale bytes each
#pragma unroll
        for (int j = 0; j < kMaxRounds; ++j) {
            if (j >= rounds) break;
            const uint4* src = row + (j * 32 + lane) * 4;
            const uint4 v0 = __ldg(src), v1 = __ldg(src + 1), v2 = __ldg(src + 2), v3 = __ldg(src + 3);
            const uint32_t wa[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            const uint32_t wb[8] = {v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w};
            xform::Block16 a, b;
            xform::decompose_block16<true, 0>(wa, a);
            xform::decompose_block16<true, 0>(wb, b);
            q0[j] = make_uint4(a.q0[0], a.q0[1], b.q0[0], b.q0[1]);
            q1[j] = make_uint4(a.q1[0], a.q1[1], b.q1[0], b.q1[1]);
            s0[j] = static_cast<uint32_t>(a.s0) | (static_cast<uint32_t>(b.s0) << 8);
            s1[j] = static_cast<uint32_t>(a.s1) | (static_cast<uint32_t>(b.s1) << 8);
        }
        // scale bytes [8 l, 8 l + 8) of the row belong to round l / 8, lanes 4 (l % 8) ... + 3
        uint32_t s0w[2] = {0, 0}, s1w[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < kMaxRounds; ++j) {
            if (j >= rounds) break;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t g0 = __shfl_sync(0xffffffffu, s0[j], 4 * (lane & 7) + i);
                const uint32_t g1 = __shfl_sync(0xffffffffu, s1[j], 4 * (lane & 7) + i);
                if (j == (lane >> 3)) {
                    s0w[i >> 1] |= g0 << (16 * (i & 1));
                    s1w[i >> 1] |= g1 << (16 * (i & 1));
                }
            }
        }
        for (int c = 0; c < k; ++c) {
            const int64_t r = dst_rank[t * k + c], dr = dst_row[t * k + c];
            if (r < 0 || r >= world || dr < 0 || dr >= rows_cap) {
                if (dr != -1 && lane == 0 && status != nullptr) atomicOr(status, 8);
                continue;
            }
            uint8_t* base = reinterpret_cast<uint8_t*>(peers[r]);
            uint4* d0 = reinterpret_cast<uint4*>(base + dr * (kdim / 2));
            uint4* d1 = reinterpret_cast<uint4*>(base + a1_off + dr * (kdim / 2));
#pragma unroll
            for (int j = 0; j < kMaxRounds; ++j) {
                if (j >= rounds) break;
                d0[j * 32 + lane] = q0[j];
                d1[j * 32 + lane] = q1[j];
            }
            // a row's scale bytes: K / 16 per pass; the lanes of rounds that exist cover them 8 bytes each
            if (lane < rounds * 8) {
                uint2* ds = reinterpret_cast<uint2*>(base + sf_off + dr * (kdim / 8));
                ds[lane] = make_uint2(s0w[0], s0w[1]);
                ds[kdim / 128 + lane] = make_uint2(s1w[0], s1w[1]);
            }
        }
    }
}

// Scale rows (rows, 2, K/16) as the quantised dispatch delivers them -> the (rows/128, K/64, 2, 512) atoms the GEMM's
// scale warps read (inside an atom the four bytes of row r at (r % 32) * 16 + (r / 32) * 4).  One block per 128-row block,
// one warp per atom at a time: lane l gathers the words of rows l, l + 32, l + 64, l + 96 (a row's consecutive K atoms are
// consecutive words, so neighbouring warps share the sectors they read) and the warp writes the atom as 512 contiguous
// bytes per pass.  Masked layout: groups of max_m rows of which the first masked_m[g], rounded up to the 128-row tile,
// are converted.  Runs on the owner, on local memory.  (One thread per row and atom, with its two scattered 4-byte stores,
// took three times as long.)
__global__ void __launch_bounds__(256)
relayout_scales_kernel(const uint8_t* __restrict__ sf_rows, const int32_t* __restrict__ masked_m, uint32_t max_m, uint64_t rows,
                       uint32_t kdim, uint8_t* __restrict__ atoms)
{
    ptx::grid_dependency_wait();
    const uint32_t k64 = kdim / 64, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * 128;
    bool live = row0 < rows;
    if (live && masked_m != nullptr) {
        const uint32_t count = min(static_cast<uint32_t>(max(0, __ldg(masked_m + row0 / max_m))), max_m);
        live = row0 % max_m < (count + 127) / 128 * 128;
    }
    if (live) {
        const uint8_t* src = sf_rows + (row0 + lane) * (kdim / 8);
        const uint64_t row_step = static_cast<uint64_t>(32) * (kdim / 8);
        for (uint32_t katom = warp; katom < k64; katom += 8) {
            uint32_t w0[4], w1[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint8_t* p = src + j * row_step + katom * 4;
                w0[j] = *reinterpret_cast<const uint32_t*>(p);
                w1[j] = *reinterpret_cast<const uint32_t*>(p + kdim / 16);
            }
            uint4* dst = reinterpret_cast<uint4*>(atoms + ((row0 / 128) * k64 + katom) * 1024) + lane;
            dst[0] = make_uint4(w0[0], w0[1], w0[2], w0[3]);
            dst[32] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        }
    }
    ptx::grid_launch_dependents();
}

// combine: y[t] = sum_j w[t, j] * (row src_row[t, j] of rank src_rank[t, j]'s output buffer), read over NVLink
// with plain loads (the data was written by another GPU during this step: no read-only cache path).  One warp per
// token; for every 16-byte piece of the row the loads of up to eight experts go out together (a round trip over NVLink
// is a few microseconds) and are consumed in order, so the sum stays in ascending j.
__global__ void __launch_bounds__(kPeerThreads, 1)
combine_rows_peer_kernel(const int64_t* __restrict__ peers, int64_t rows_ld16, const int64_t* __restrict__ src_rank,
                         const int64_t* __restrict__ src_row, const float* __restrict__ w, int64_t tokens, int k, int row16,
                         uint4* __restrict__ y, int64_t y_ld16, int world, int64_t rows_cap)
{
    const int lane = threadIdx.x & 31, warps = kPeerThreads / 32;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * warps + (threadIdx.x >> 5); t < tokens; t += static_cast<int64_t>(gridDim.x) * warps) {
        for (int c = lane; c < row16; c += 32) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int j0 = 0; j0 < k; j0 += 8) {
                uint4 v[8];
                float wj[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int j = j0 + u < k ? j0 + u : k - 1;
                    const int64_t pr = src_rank[t * k + j], prow = src_row[t * k + j];
                    const bool valid = j0 + u < k && pr >= 0 && pr < world && prow >= 0 && prow < rows_cap;   // else: contributes nothing
                    wj[u] = valid ? w[t * k + j] : 0.0f;
                    v[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (valid) {
                        const uint4* row = reinterpret_cast<const uint4*>(peers[pr]) + prow * rows_ld16;
                        asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(row + c));
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (j0 + u >= k) break;
                    const uint32_t vw[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vw[i]));
                        acc[2 * i] = fmaf(wj[u], f.x, acc[2 * i]);
                        acc[2 * i + 1] = fmaf(wj[u], f.y, acc[2 * i + 1]);
                    }
                }
            }
            uint32_t ow[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                ow[i] = *reinterpret_cast<const uint32_t*>(&p);
            }
            y[t * y_ld16 + c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
    }
}

// The same combine with the rows fetched by bulk copies (cp.async.bulk global -> shared, completing on an mbarrier)
// instead of per-thread loads: a bulk copy is one request for a whole row, and a CTA can have its entire shared memory
// in flight, where a thread's loads over NVLink are bounded by what the SM's load path keeps outstanding (sixteen SMs of
// the kernel above pull ~250 GB/s, all 148 about 600).
// One CTA per granted SM.  Shared memory is a ring of slots, a slot = the k rows of one token.  Thread 0 walks the CTA's
// tokens, waits for a slot to be free and requests the rows of every valid pair; the other warps wait for the slot's
// bytes, form y[t] = sum_j w[t, j] * row_j in FP32 in ascending j (the order of the kernel above and of the all-to-all
// path: the same bits), store the BF16 row and free the slot.  No multicast; every wait is bounded.
// Measured (2 GPUs, 16384 tokens x 8 rows of 8 KB per rank): on the whole GPU 0.85 ms against 0.88 ms for the kernel
// above; on 8 SMs the eight arithmetic warps, not NVLink, set the pace (2.5 ms for half the tokens).
constexpr int kBulkThreads = 288;                       // warp 0: requests; warps 1-8: arithmetic
__global__ void __launch_bounds__(kBulkThreads, 1)
combine_rows_bulk_kernel(const int64_t* __restrict__ peers, int64_t rows_ld_bytes, const int64_t* __restrict__ src_rank,
                         const int64_t* __restrict__ src_row, const float* __restrict__ w, int64_t tokens, int k, int row_bytes,
                         uint4* __restrict__ y, int64_t y_ld16, int world, int64_t rows_cap, int slots, int32_t* __restrict__ status)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 127u) & ~127u;
    uint8_t* gen = smem_raw + (smem - ptx::smem_u32(smem_raw));
    const uint32_t slot_bytes = static_cast<uint32_t>(k) * row_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(gen + static_cast<size_t>(slots) * slot_bytes);
    uint64_t* empty = full + slots;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty + slots);
    constexpr int kWorkers = kBulkThreads / 32 - 1;
    if (threadIdx.x == 0) {
        for (int i = 0; i < slots; ++i) { ptx::mbar_init(full + i, 1); ptx::mbar_init(empty + i, kWorkers); }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto valid_pair = [&](int64_t p) {
        const int64_t pr = src_rank[p], prow = src_row[p];
        return pr >= 0 && pr < world && prow >= 0 && prow < rows_cap;
    };
    if (warp == 0) {
        if (lane == 0) {
            uint32_t slot = 0, phase = 0;
            for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
                if (!ptx::mbar_wait_impl(empty + slot, phase ^ 1, abort_flag)) {
                    *abort_flag = 1;
                    if (status != nullptr) atomicOr(status, 1);
                    break;
                }
                uint32_t bytes = 0;
                for (int j = 0; j < k; ++j) bytes += valid_pair(t * k + j) ? row_bytes : 0;
                ptx::mbar_arrive_expect_tx(full + slot, bytes);
                for (int j = 0; j < k; ++j) {
                    const int64_t p = t * k + j;
                    if (!valid_pair(p)) continue;
                    const uint8_t* row = reinterpret_cast<const uint8_t*>(peers[src_rank[p]]) + src_row[p] * rows_ld_bytes;
                    ptx::bulk_load(gen + static_cast<size_t>(slot) * slot_bytes + static_cast<size_t>(j) * row_bytes, row, row_bytes, full + slot);
                }
                if (++slot == static_cast<uint32_t>(slots)) { slot = 0; phase ^= 1; }
            }
        }
    } else {
        uint32_t slot = 0, phase = 0;
        const int worker = threadIdx.x - 32, row16 = row_bytes / 16;
        for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
            float wj[16];
            bool live[16];
            for (int j = 0; j < k; ++j) { live[j] = valid_pair(t * k + j); wj[j] = live[j] ? w[t * k + j] : 0.0f; }
            if (!ptx::mbar_wait_impl(full + slot, phase, abort_flag)) {
                *abort_flag = 1;
                if (status != nullptr) atomicOr(status, 1);
                break;
            }
            const uint32_t base = smem + slot * slot_bytes;
            for (int c = worker; c < row16; c += kWorkers * 32) {
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int j = 0; j < k; ++j) {
                    if (!live[j]) continue;                     // contributes nothing (its bytes were never requested)
                    const uint4 v = ptx::lds128(base + j * row_bytes + c * 16);
                    const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vw[i]));
                        acc[2 * i] = fmaf(wj[j], f.x, acc[2 * i]);
                        acc[2 * i + 1] = fmaf(wj[j], f.y, acc[2 * i + 1]);
                    }
                }
                uint32_t ow[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __nv_bfloat162 pk = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                    ow[i] = *reinterpret_cast<const uint32_t*>(&pk);
                }
                y[t * y_ld16 + c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(empty + slot);
            if (++slot == static_cast<uint32_t>(slots)) { slot = 0; phase ^= 1; }
        }
    }
}

// counts[e] += number of ids equal to e (counts zeroed by the caller); per-block histogram in shared memory first, so
// that the global atomics are one per expert and block instead of one per pair on a handful of addresses
__global__ void __launch_bounds__(1024)
expert_histogram_kernel(const int64_t* __restrict__ ids, int64_t n, int num_experts, unsigned long long* __restrict__ counts)
{
    extern __shared__ unsigned int hist[];
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < n; p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t e = ids[p];
        if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1u);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
        if (hist[e] != 0) atomicAdd(&counts[e], static_cast<unsigned long long>(hist[e]));
}

// Routing plan of the peer-memory path, from the gathered (source rank, expert) count matrix (plan_offsets_masked_kernel
// below gives base and limit): dst_row[p] = base[e] + (number of pairs p' < p routed to e), for every pair p routed to e
// -- a stable counting sort without the sort: pairs keep their order inside an expert's group.  With `limit`
// (fixed-capacity plan) a pair whose row would reach limit[e] does not fit and gets row -1.
// Two passes over the pairs, each block on its own chunk: plan_chunk_hist_kernel counts every chunk's pairs per expert;
// plan_rows_kernel starts each expert's counter at base[e] + (pairs of e in earlier chunks) and hands out rows chunk-locally:
// 1024 pairs at a time, the warps take turns in order (inside a warp __match_any_sync ranks the lanes of one expert), so
// the order of the pairs is kept.  (The first version gave every expert a block that scanned ALL pairs: 128 experts x
// 131072 pairs took 0.2 ms.)
constexpr int kPlanThreads = 1024;
__global__ void __launch_bounds__(kPlanThreads)
plan_chunk_hist_kernel(const int64_t* __restrict__ ids, int64_t n, int64_t chunk, int num_experts, int32_t* __restrict__ chunk_hist)
{
    extern __shared__ int hist_s[];
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist_s[e] = 0;
    __syncthreads();
    const int64_t lo = blockIdx.x * chunk, hi = min(lo + chunk, n);
    for (int64_t p = lo + threadIdx.x; p < hi; p += blockDim.x) {
        const int64_t e = ids[p];
        if (e >= 0 && e < num_experts) atomicAdd(&hist_s[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) chunk_hist[static_cast<int64_t>(blockIdx.x) * num_experts + e] = hist_s[e];
}

__global__ void __launch_bounds__(kPlanThreads)
plan_rows_kernel(const int64_t* __restrict__ ids, int64_t n, int64_t chunk, int num_experts, const int32_t* __restrict__ chunk_hist,
                 const int64_t* __restrict__ base, const int64_t* __restrict__ limit, int64_t* __restrict__ dst_row)
{
    extern __shared__ long long next_row[];          // [num_experts] next free row of every expert, for this chunk onwards
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        long long r = base[e];
        for (int c = 0; c < static_cast<int>(blockIdx.x); ++c) r += chunk_hist[static_cast<int64_t>(c) * num_experts + e];
        next_row[e] = r;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t lo = blockIdx.x * chunk, hi = min(lo + chunk, n);
    for (int64_t p0 = lo; p0 < hi; p0 += blockDim.x) {
        const int64_t p = p0 + threadIdx.x;
        const int64_t e = p < hi ? ids[p] : -1;
        const bool valid = e >= 0 && e < num_experts;
        // lanes of this warp with the same expert, and this lane's rank among them
        const unsigned same = __match_any_sync(0xffffffffu, valid ? static_cast<int>(e) : -1 - lane);
        const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
        const int leader = __ffs(same) - 1;
        for (int w = 0; w < kPlanThreads / 32; ++w) {
            if (w == wid) {
                long long first = 0;
                if (valid && lane == leader) {       // one lane per expert present in the warp; experts differ, no race
                    first = next_row[e];
                    next_row[e] = first + __popc(same);
                }
                first = __shfl_sync(0xffffffffu, first, leader);
                if (valid) {
                    const long long row = first + rank_in_warp;
                    dst_row[p] = (limit == nullptr || row < limit[e]) ? row : -1;
                }
            }
            __syncthreads();
        }
    }
}

// Fixed-capacity plan: every local expert owns `cap_m` rows of its rank's buffer (the masked layout of the GEMM),
// so a pair's row depends only on the gathered counts, never on a host-side prefix sum of padded group sizes.
//   base[e]  = (e % e_local) * cap_m + rows of e from lower ranks      limit[e] = (e % e_local + 1) * cap_m
//   masked_m[j] = min(rows of local expert j, cap_m)                   status |= 4 if some expert anywhere overflows
// Every rank sees the same gathered counts, hence the same overflow verdict.
__global__ void __launch_bounds__(1024)
plan_offsets_masked_kernel(const int64_t* __restrict__ all_counts, int world, int num_experts, int rank, int cap_m,
                           int64_t* __restrict__ base, int64_t* __restrict__ limit, int32_t* __restrict__ masked_m,
                           int32_t* __restrict__ status)
{
    const int e_local = num_experts / world;
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        int64_t total = 0, before = 0;
        for (int s = 0; s < world; ++s) {
            const int64_t c = all_counts[static_cast<int64_t>(s) * num_experts + e];
            if (s < rank) before += c;
            total += c;
        }
        const int64_t group = static_cast<int64_t>(e % e_local) * cap_m;
        base[e] = group + before;
        limit[e] = group + cap_m;
        if (e / e_local == rank) masked_m[e % e_local] = static_cast<int32_t>(total < cap_m ? total : cap_m);
        if (total > cap_m && status != nullptr) atomicOr(status, 4);
    }
}

// Barrier over the GPUs of one NVLink domain with a bounded wait.  `flag_peers[r]` is the address, in this process,
// of rank r's flag array (int64 [slots][world], symmetric, zero at start).  Thread p tells rank p "rank `rank` has
// reached `epoch`" with a releasing system-scope store into flags[slot][rank] over there, then waits until its own
// flags[slot][p] shows that rank p has reached it too.  Epochs only grow, so no reset is needed.  A wait that lasts
// longer than `budget` clock cycles gives up: bit 1 of the status word is set and the kernel returns -- nothing
// traps and nothing spins for ever, the host reads the word and raises.
__global__ void __launch_bounds__(64)
peer_barrier_kernel(const int64_t* __restrict__ flag_peers, int rank, int world, int slot, long long epoch, long long budget,
                    int32_t* __restrict__ status)
{
    const int p = threadIdx.x;
    if (p >= world) return;
    __threadfence_system();                      // everything this stream wrote before the barrier, peers' memory included
    long long* theirs = reinterpret_cast<long long*>(flag_peers[p]) + static_cast<int64_t>(slot) * world + rank;
    asm volatile("st.release.sys.global.s64 [%0], %1;" ::"l"(theirs), "l"(epoch) : "memory");
    const long long* mine = reinterpret_cast<const long long*>(flag_peers[rank]) + static_cast<int64_t>(slot) * world + p;
    const long long t0 = clock64();
    for (;;) {
        long long seen;
        asm volatile("ld.acquire.sys.global.s64 %0, [%1];" : "=l"(seen) : "l"(mine) : "memory");
        if (seen >= epoch) break;
        if (clock64() - t0 > budget) {
            if (status != nullptr) atomicOr(status, 2);
            break;
        }
        __nanosleep(100);
    }
}

unsigned grid_for(int64_t rows, int num_sms)
{
    const int64_t cap = static_cast<int64_t>(num_sms) * 8;
    return static_cast<unsigned>(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

}  // namespace

int launch_permute_rows(const void* src, int64_t src_ld_bytes, const int64_t* src_idx, int src_div, const int64_t* dst_idx,
                        int64_t n_rows, int row_bytes, void* dst, int64_t dst_ld_bytes, int num_sms, cudaStream_t stream)
{
    permute_rows_kernel<<<grid_for(n_rows, num_sms), 256, 0, stream>>>(
        static_cast<const uint4*>(src), src_ld_bytes / 16, src_idx, src_div, dst_idx, n_rows, row_bytes / 16,
        static_cast<uint4*>(dst), dst_ld_bytes / 16);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_swiglu(const void* h, int64_t h_ld_elems, int64_t rows, int inter, void* out, int64_t out_ld_elems, int num_sms,
                  cudaStream_t stream)
{
    swiglu_kernel<<<grid_for(rows, num_sms), 256, 0, stream>>>(static_cast<const uint4*>(h), h_ld_elems / 8, rows, inter / 8,
                                                                static_cast<uint4*>(out), out_ld_elems / 8);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_combine_rows(const void* rows, int64_t rows_ld_elems, const int64_t* pos, const float* w, int64_t tokens, int k,
                        int hidden, void* y, int64_t y_ld_elems, int num_sms, cudaStream_t stream)
{
    combine_rows_kernel<<<grid_for(tokens, num_sms), 256, 0, stream>>>(static_cast<const uint4*>(rows), rows_ld_elems / 8, pos, w,
                                                                        tokens, k, hidden / 8, static_cast<uint4*>(y),
                                                                        y_ld_elems / 8);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_expert_histogram(const int64_t* ids, int64_t n, int num_experts, int64_t* counts, cudaStream_t stream)
{
    NVFP4_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int64_t) * num_experts, stream));
    if (n == 0) return NVFP4_OK;
    const unsigned blocks = static_cast<unsigned>((n + 8191) / 8192 < 64 ? (n + 8191) / 8192 : 64);
    expert_histogram_kernel<<<blocks, 1024, num_experts * sizeof(unsigned int), stream>>>(
        ids, n, num_experts, reinterpret_cast<unsigned long long*>(counts));
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_plan_peer_masked(const int64_t* all_counts, int world, int num_experts, int rank, int cap_m, const int64_t* ids,
                            int64_t n, int64_t* base, int64_t* limit, int32_t* masked_m, int64_t* dst_row, int32_t* status,
                            cudaStream_t stream)
{
    plan_offsets_masked_kernel<<<1, 1024, 0, stream>>>(all_counts, world, num_experts, rank, cap_m, base, limit, masked_m, status);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    if (n == 0) return NVFP4_OK;
    // chunks of whole 1024-pair steps, at most 128 of them
    int64_t chunk = (n + 127) / 128;
    chunk = (chunk + kPlanThreads - 1) / kPlanThreads * kPlanThreads;
    const unsigned blocks = static_cast<unsigned>((n + chunk - 1) / chunk);
    int dev = 0;
    NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    if (int rc = host::workspace_pool(dev, &pool)) return rc;
    int32_t* chunk_hist = nullptr;
    NVFP4_CUDA_CHECK(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&chunk_hist), sizeof(int32_t) * blocks * num_experts, pool, stream));
    plan_chunk_hist_kernel<<<blocks, kPlanThreads, num_experts * sizeof(int), stream>>>(ids, n, chunk, num_experts, chunk_hist);
    plan_rows_kernel<<<blocks, kPlanThreads, num_experts * sizeof(long long), stream>>>(ids, n, chunk, num_experts, chunk_hist, base, limit,
                                                                                      dst_row);
    const cudaError_t err = cudaGetLastError();
    cudaFreeAsync(chunk_hist, stream);
    if (err != cudaSuccess) return host::fail(NVFP4_E_CUDA, "plan kernels failed to launch: %s", cudaGetErrorString(err));
    return NVFP4_OK;
}

int launch_peer_barrier(const int64_t* flag_peers, int rank, int world, int slot, int64_t epoch, int64_t budget_cycles,
                        int32_t* status, cudaStream_t stream)
{
    peer_barrier_kernel<<<1, 64, 0, stream>>>(flag_peers, rank, world, slot, static_cast<long long>(epoch),
                                              static_cast<long long>(budget_cycles), status);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_dispatch_rows_peer(const void* src, int64_t src_ld_bytes, const int64_t* src_idx, int src_div, const int64_t* peers,
                              const int64_t* dst_rank, const int64_t* dst_row, int64_t n_rows, int row_bytes,
                              int64_t dst_ld_bytes, int world, int64_t rows_cap, int32_t* status, int num_sms, cudaStream_t stream)
{
    dispatch_rows_peer_kernel<<<static_cast<unsigned>(num_sms), kPeerThreads, 0, stream>>>(
        static_cast<const uint4*>(src), src_ld_bytes / 16, src_idx, src_div, peers, dst_rank, dst_row, n_rows, row_bytes / 16,
        dst_ld_bytes / 16, world, rows_cap, status);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_combine_rows_peer(const int64_t* peers, int64_t rows_ld_elems, const int64_t* src_rank, const int64_t* src_row,
                             const float* w, int64_t tokens, int k, int hidden, void* y, int64_t y_ld_elems, int world,
                             int64_t rows_cap, int num_sms, bool bulk, int32_t* status, cudaStream_t stream)
{
    // bulk copies: a slot holds the k rows of a token; at least two slots must fit beside the barriers
    const size_t slot_bytes = static_cast<size_t>(k) * hidden * 2;
    constexpr size_t kSmemMax = 232448 - 1024;
    const int slots = slot_bytes ? static_cast<int>((kSmemMax - 256) / slot_bytes) : 0;
    if (bulk && slots >= 2 && k <= 16 && (hidden * 2) % 16 == 0) {
        const int use = slots > 8 ? 8 : slots;
        const size_t smem = use * slot_bytes + 2 * use * 8 + 16 + 128;
        static bool attr_set[host::kMaxDevices] = {};
        int dev = 0;
        NVFP4_CUDA_CHECK(cudaGetDevice(&dev));
        if (!attr_set[dev]) {
            NVFP4_CUDA_CHECK(cudaFuncSetAttribute(combine_rows_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemMax)));
            attr_set[dev] = true;
        }
        combine_rows_bulk_kernel<<<static_cast<unsigned>(num_sms), kBulkThreads, smem, stream>>>(
            peers, rows_ld_elems * 2, src_rank, src_row, w, tokens, k, hidden * 2, static_cast<uint4*>(y), y_ld_elems / 8, world, rows_cap,
            use, status);
        NVFP4_CUDA_CHECK(cudaGetLastError());
        return NVFP4_OK;
    }
    combine_rows_peer_kernel<<<static_cast<unsigned>(num_sms), kPeerThreads, 0, stream>>>(peers, rows_ld_elems / 8, src_rank, src_row, w, tokens,
                                                                             k, hidden / 8, static_cast<uint4*>(y), y_ld_elems / 8,
                                                                             world, rows_cap);
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_dispatch_quantized_peer(const void* x, int64_t x_ld_bytes, int64_t tokens, int k, int kdim, const int64_t* peers,
                                   int64_t a1_off, int64_t sf_off, const int64_t* dst_rank, const int64_t* dst_row, int world,
                                   int64_t rows_cap, int32_t* status, int num_sms, cudaStream_t stream)
{
    auto go = [&](auto kernel) {
        kernel<<<static_cast<unsigned>(num_sms), kPeerThreads, 0, stream>>>(static_cast<const uint4*>(x), x_ld_bytes / 16, tokens, k, peers,
                                                                           a1_off, sf_off, dst_rank, dst_row, world, rows_cap, status);
    };
    switch (kdim / 1024) {
        case 1: go(dispatch_quantized_peer_kernel<1>); break;
        case 2: go(dispatch_quantized_peer_kernel<2>); break;
        case 3: go(dispatch_quantized_peer_kernel<3>); break;
        case 4: go(dispatch_quantized_peer_kernel<4>); break;
        case 5: go(dispatch_quantized_peer_kernel<5>); break;
        case 6: go(dispatch_quantized_peer_kernel<6>); break;
        case 7: go(dispatch_quantized_peer_kernel<7>); break;
        case 8: go(dispatch_quantized_peer_kernel<8>); break;
        default: return host::fail(NVFP4_E_UNSUPPORTED, "quantised dispatch is built for K = 1024 ... 8192 in steps of 1024 (K=%d)", kdim);
    }
    NVFP4_CUDA_CHECK(cudaGetLastError());
    return NVFP4_OK;
}

int launch_relayout_scales(const void* sf_rows, const int32_t* masked_m, int max_m, int64_t rows, int kdim, void* atoms, bool pdl,
                           cudaStream_t stream)
{
    if (rows == 0) return NVFP4_OK;
    return host::launch_kernel(relayout_scales_kernel, dim3(static_cast<unsigned>((rows + 127) / 128)), dim3(256), 0, stream, pdl,
                               static_cast<const uint8_t*>(sf_rows), masked_m, static_cast<uint32_t>(max_m > 0 ? max_m : 1),
                               static_cast<uint64_t>(rows), static_cast<uint32_t>(kdim), static_cast<uint8_t*>(atoms));
}

}  // namespace nvfp4
