// Pieces shared by the GEMM kernels of the normal orientation: the ring cursor, the persistent tile order
// (contiguous and masked layouts) and the epilogue's staged, line-coalesced output stores.
#pragma once
#include <cuda_bf16.h>

#include "ptx.cuh"

namespace nvfp4::gemm {

// Cursor of a ring of `kDepth` slots; the phase bit flips on every wrap.
struct Ring {
    uint32_t slot = 0, phase = 0;
    template <uint32_t kDepth>
    __device__ __forceinline__ void advance()
    {
        if (++slot == kDepth) { slot = 0; phase ^= 1; }
    }
};

// Tiles are walked in groups of `group_m` row blocks: inside a group the row block changes fastest, so the
// CTAs running at the same time share a few weight tiles and a few activation tiles in L2.
// Counterpart in the reference: include/nvfp4_gemm/scheduler/grouped_gemm.cuh:86-99.
__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t num_m, uint32_t num_n, uint32_t group_m,
                                            uint32_t& m_blk, uint32_t& n_blk)
{
    const uint32_t per_group = group_m * num_n;
    const uint32_t g = tile / per_group, r = tile % per_group;
    const uint32_t first = g * group_m;
    const uint32_t rows = min(group_m, num_m - first);
    m_blk = first + r % rows;
    n_blk = r / rows;
}

// What a role needs to know about its next tile.
struct Tile {
    uint32_t row0;     // first row of the tile in a / d
    uint32_t n_blk;    // column block
    int32_t expert;    // whose weights
};

// Persistent static-stride tile order over either layout.
//   contiguous: rows grouped by expert, expert of a row block read from m_indices (negative ids read as 0)
//   masked:     `groups` experts with `max_m` rows reserved each, of which the first masked_m[g] (a device-side
//               count, clamped to max_m) are real; row blocks past the count do not exist
//               (counterpart in the reference: scheduler/grouped_gemm.cuh:139-156)
// Every role of a CTA owns a walker and calls next() with the same sequence of linear tile indices.
template <uint32_t kBM, bool kMasked>
struct TileWalker {
    const int32_t* layout;   // m_indices (contiguous) or masked_m (masked)
    uint32_t num_m, num_n, group_m, groups, max_m;
    uint32_t g = 0, blocks_before = 0, blocks_here = 0;
    bool primed = false;

    __device__ __forceinline__ TileWalker(const int32_t* layout_, uint32_t m_rows, uint32_t n_cols, uint32_t bn,
                                          uint32_t group_m_, uint32_t groups_, uint32_t max_m_)
        : layout(layout_), num_m(m_rows / kBM), num_n(n_cols / bn), group_m(group_m_), groups(groups_), max_m(max_m_)
    {
    }

    __device__ __forceinline__ uint32_t blocks_of(uint32_t group) const
    {
        const uint32_t rows = min(static_cast<uint32_t>(max(0, __ldg(layout + group))), max_m);
        return (rows + kBM - 1) / kBM;
    }

    // false when `linear` is past the last tile
    __device__ __forceinline__ bool next(uint32_t linear, Tile& t)
    {
        if constexpr (!kMasked) {
            if (linear >= num_m * num_n) return false;
            uint32_t m_blk;
            tile_coords(linear, num_m, num_n, group_m, m_blk, t.n_blk);
            t.row0 = m_blk * kBM;
            t.expert = max(0, __ldg(layout + t.row0));
            return true;
        } else {
            if (!primed) { blocks_here = groups ? blocks_of(0) : 0; primed = true; }
            for (;;) {
                if (g >= groups) return false;
                if (linear < (blocks_before + blocks_here) * num_n) break;
                blocks_before += blocks_here;
                if (++g < groups) blocks_here = blocks_of(g);
            }
            uint32_t m_blk;
            tile_coords(linear - blocks_before * num_n, blocks_here, num_n, group_m, m_blk, t.n_blk);
            t.row0 = g * max_m + m_blk * kBM;
            t.expert = static_cast<int32_t>(g);
            return true;
        }
    }
};

// Epilogue stores of one warp: `o` holds this lane's output row as 32 BF16 pairs (64 columns; in tensor memory
// a lane is a row).  A store instruction should write whole 128-byte lines, and with one row per lane every
// 16-byte store of the warp would land in a different line -- 4096 partial-line requests per 128 x 256 tile,
// measured to hold up the operand loads and the tensor pipe of the next tile for thousands of cycles.  So four
// rows at a time go through a 576-byte staging area (`stage`, this warp's own): four lanes write their 128
// bytes, then the whole warp reads 16 bytes per lane and stores four full lines.  `d_lane` points at the first
// of the eight 16-byte pieces this lane stores: row (lane / 8) of the warp's 32, column piece (lane % 8).
constexpr uint32_t kStageRow = 144, kStageWarp = 4 * kStageRow;   // 128-byte rows padded against bank conflicts
__device__ __forceinline__ void store_rows_staged(const uint32_t (&o)[32], uint32_t stage, __nv_bfloat16* d_lane, int64_t ldd,
                                                  uint32_t lane)
{
    const uint32_t rd = stage + (lane >> 3) * kStageRow + (lane & 7u) * 16;
#pragma unroll 1
    for (uint32_t pass = 0; pass < 8; ++pass) {
        if ((lane >> 2) == pass) {
            const uint32_t wr = stage + (lane & 3u) * kStageRow;
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) ptx::sts128(wr + c * 16, o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        }
        __syncwarp();
        const uint4 q = ptx::lds128(rd);
        *reinterpret_cast<uint4*>(d_lane + static_cast<int64_t>(pass * 4) * ldd) = q;
        __syncwarp();
    }
}

// 32 FP32 accumulator values x gw -> 16 BF16 pairs
__device__ __forceinline__ void scale_pack_bf16(const uint32_t (&v)[32], float g, uint32_t* out16)
{
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * i]) * g, __uint_as_float(v[2 * i + 1]) * g);
        out16[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
}

}  // namespace nvfp4::gemm
