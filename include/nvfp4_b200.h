/*
 * nvfp4_b200 -- C ABI of the B200 (sm_100a) grouped dual-NVFP4 GEMM.
 *
 * This is the drop-in boundary for the one hot path of the nvfp4-cutlass project:
 * the contiguous-layout grouped MoE GEMM with BF16 activations decomposed on chip
 * into two NVFP4 passes.  Plain pointers and sizes only; every pointer is a CUDA
 * device pointer on the current device unless said otherwise; `stream` is a
 * cudaStream_t / CUstream passed as void*.  Calls are asynchronous on `stream`.
 *
 * Every function returns 0 on success or one of the NVFP4_E_* codes; the text of the
 * last error of the calling thread is available from nvfp4_last_error().  Nothing
 * throws across this boundary and nothing here ever falls back to a CPU path.
 *
 * "Replaces" comments name the interface of the reference project that each entry
 * point stands in for (path within that project : lines).
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define NVFP4_API __attribute__((visibility("default")))
#else
#define NVFP4_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
    NVFP4_OK = 0,
    NVFP4_E_INVALID_ARGUMENT = 1,  /* bad pointer, dtype code, shape relation or alignment */
    NVFP4_E_UNSUPPORTED = 2,       /* well-formed request this build has no kernel for */
    NVFP4_E_CUDA = 3,              /* a CUDA runtime / driver call failed */
    NVFP4_E_DEVICE_TIMEOUT = 4     /* a bounded in-kernel wait expired (returned by nvfp4_read_status) */
};

/* activation scale policies (reference: src/api.hpp:106-112, include/nvfp4_gemm/transform/dual_nvfp4.cuh:31-61);
 * all four are built in every kernel family. */
enum { NVFP4_POLICY_DERIVED_DIV8 = 0, NVFP4_POLICY_RESIDUAL_AMAX = 1, NVFP4_POLICY_DERIVED_DIV4 = 2,
       NVFP4_POLICY_DIV4_RADIX8 = 3 };
/* operand orientation (reference: tune_swap_ab, src/api.hpp:84-104) */
enum { NVFP4_ORIENT_NORMAL = 0, NVFP4_ORIENT_SWAP_AB = 1 };
/* weight input dtypes of nvfp4_quantize_weight */
enum { NVFP4_DTYPE_BF16 = 0, NVFP4_DTYPE_F32 = 1 };

/* Text of the calling thread's last error ("" if none).  Never NULL. */
NVFP4_API const char* nvfp4_last_error(void);

/* Library / build identification, e.g. "nvfp4_b200 0.1 sm_100a". */
NVFP4_API const char* nvfp4_version(void);

/* SM count the persistent kernels size their grid with.
 * Replaces: _C.get_num_sms / _C.set_num_sms (src/api.hpp:150,156; src/runtime/device.hpp:38-54).
 * `device` < 0 means the current device.  set: 0 restores the hardware count; values
 * above 2x the hardware count are rejected. */
NVFP4_API int nvfp4_get_num_sms(int device, int* out);
NVFP4_API int nvfp4_set_num_sms(int device, int value);

/* Offline NVFP4 weight quantisation on the GPU, bit-exact with the reference's
 * torch implementation.
 * Replaces: nvfp4_gemm.quantize_weight_nvfp4 (python/nvfp4_gemm/layout.py:68-127).
 *   w    (E, N, K) row-major, BF16 or FP32 (w_dtype)
 *   b    (E*N, K/2) bytes, two E2M1 codes per byte, even element in the low nibble
 *   sfb  (E*K/64, N) int32, byte j = E4M3 scale of 16-block j of the 64-element atom
 *   gw   (E,) float
 * K must be a multiple of 64 (NVFP4_E_INVALID_ARGUMENT otherwise, where the
 * reference raises ValueError). */
NVFP4_API int nvfp4_quantize_weight(const void* w, int w_dtype, int E, int N, int K,
                          void* b, void* sfb, float* gw, void* stream);

/* nvfp4_quantize_weight for callers that must not allocate.  It has no counterpart in the
 * reference project.
 *
 * nvfp4_quantize_weight takes a small scratch buffer (one word per expert) from a stream-ordered
 * memory pool on every call; the pool grows with cudaMalloc-like driver work the first time and
 * whenever it needs more.  Some callers cannot afford that: code running while a stream is
 * being captured, latency-critical loops in which a cudaMalloc would synchronise the whole
 * device, processes whose device memory has been handed out completely to a pool of their
 * own.  This variant does the same work with its scratch in a fixed array inside the library
 * image: it calls no cudaMalloc, no cudaFree and no allocating library routine.
 *
 *   - At most NVFP4_STATIC_MAX_EXPERTS experts per call; more is NVFP4_E_INVALID_ARGUMENT.
 *   - The array (4 KB) exists once per GPU per process for as long as the library is loaded.
 *   - The first call made on a device looks the array's device address up (one
 *     cudaGetSymbolAddress); make that first call outside any stream capture.
 *   - All calls on a device share the array, which is cleared at the start of each call on
 *     the call's stream.  Two calls whose kernels may overlap on the GPU (different streams
 *     without an ordering between them) race on it; order them.
 * Arguments, layouts and results are those of nvfp4_quantize_weight, bit for bit. */
#define NVFP4_STATIC_MAX_EXPERTS 1024
NVFP4_API int nvfp4_quantize_weight_static(const void* w, int w_dtype, int E, int N, int K,
                                           void* b, void* sfb, float* gw, void* stream);

/* The hot path.  d[M,N] (BF16) = (A0 + A1) * W^T * gw[expert], experts by row group.
 * Replaces: _C.m_grouped_bf16_dual_nvfp4_gemm_contiguous (src/api.hpp:26-144,
 * kernels src/kernels/sm100_bf16_dual_nvfp4_gemm.hpp:226-480 and :489-632).
 *   a          (M, K) BF16, K contiguous, row stride lda_elems
 *   b, sfb, gw as produced by nvfp4_quantize_weight for E experts of shape (N, K)
 *   d          (M, N) BF16, row stride ldd_elems, written in place
 *   m_indices  (M,) int32 expert id of each row; each expert's rows start on an
 *              m_alignment boundary (128 normal, 16/32/64/128 swap-AB); only the
 *              first row of each aligned block is read, negative ids read as 0.  Normal
 *              orientation also takes m_alignment 256: a statement that every expert's rows
 *              are a multiple of 256, which lets the split path run its CTA-pair GEMM
 *              (two CTAs, one tcgen05.mma.cta_group::2 over 256 rows) without left-over blocks
 *   enable_residual_pass 0 = the single_nvfp4 variant (second pass skipped)
 *   tune       optional host array of 18 int32 in the order of the reference's
 *              tune_* keywords (src/api.hpp:166-203), or NULL; 0 = default.  Honoured: [0] block_n
 *              (swap-AB token tile 16/32/64), [1] transform_warps (8/16: single-CTA fused kernel),
 *              [5] block_k, [7] swap_ab is the `orientation` argument, [8] cluster (fused kernels: 1/2/4 CTAs share
 *              a transformed activation tile; split path: 2 = CTA-pair GEMM kernel, 1 = single-CTA), [9] direct_a, [11] no_pdl, [12] sched_group,
 *              [13] split_transform.  NOTE [13] means something else than in the reference (there:
 *              signal A0 early inside its one kernel): here 1 = quantise the activations once in a
 *              kernel of their own ahead of the GEMM, 2 = Algorithm 1 inside the GEMM main loop,
 *              0 = the library's choice.  All other knobs (epilogue_threads, num_stages,
 *              swizzle_cd, epilogue_stages, l2_pin_weights, timing_probe, tail_split,
 *              shallow_stages, produced_stages, a token tile of 128) are accepted and ignored.
 *   device_status optional device int32 the kernel ORs error bits into (bit 0 =
 *              a bounded wait expired); may be NULL
 * Constraints as in the reference (src/api.hpp:58-79): N % 128 == 0, K % 128 == 0,
 * M % m_alignment == 0; M == 0 or N == 0 returns NVFP4_OK without a launch. */
NVFP4_API int nvfp4_grouped_gemm_contiguous(const void* a, int64_t lda_elems, const void* b, const void* sfb,
                                  const float* gw, void* d, int64_t ldd_elems,
                                  const int32_t* m_indices, int M, int N, int K, int E,
                                  int scale_policy, int enable_residual_pass, int orientation,
                                  int m_alignment, const int32_t* tune, int32_t* device_status,
                                  void* stream);

/* The same GEMM over the masked layout: `E` groups (experts) with `max_m` rows reserved each in `a` and `d`
 * (row g * max_m + r; max_m % 128 == 0), of which the first masked_m[g] are real.  masked_m is a DEVICE array that
 * an earlier kernel of the stream may have written: the host never needs the row counts, so a routing step and the
 * GEMMs after it can be enqueued (or captured) without a read-back.  Row blocks past a group's count are skipped;
 * rows between the count and the end of its last 128-row block are computed like real rows (as in the contiguous
 * layout).  Counts are clamped to [0, max_m].
 * fold_swiglu != 0: `a` is the (E * max_m, 2 K) gate+up output and the activation is
 * Q(silu(a[:, :K]) * a[:, K:]) as in nvfp4_grouped_gemm_swiglu_contiguous (derived_div8 only).
 * Replaces: GemmType::MGroupedMasked of the reference's kernel (include/nvfp4_gemm/common/types.cuh:22-24,
 * scheduler/grouped_gemm.cuh:139-156, epilogue/sm100_store_cd.cuh:134), which its host API never exposes.
 * Normal orientation, N % 256 == 0, K % 128 == 0. */
NVFP4_API int nvfp4_grouped_gemm_masked(const void* a, int64_t lda_elems, const void* b, const void* sfb, const float* gw,
                                        void* d, int64_t ldd_elems, const int32_t* masked_m, int E, int max_m, int N, int K,
                                        int scale_policy, int enable_residual_pass, int fold_swiglu, const int32_t* tune,
                                        int32_t* device_status, void* stream);

/* NVFP4 checkpoint tensors -> (b, sfb, gw) as the GEMM reads them, on the GPU.
 * A checkpoint stores every projection of an expert separately: weight_packed (rows, K/2) two E2M1 codes per byte
 * (even element low), weight_scale (rows, K/16) E4M3 bytes row-major, and one FP32 weight_global_scale.  Here every
 * part p < num_parts is given stacked over the experts: weight_packed[p] (E, part_rows[p], K/2), weight_scale[p]
 * (E, part_rows[p], K/16), weight_global_scale[p] (E,); the arrays of pointers are HOST arrays of DEVICE pointers.
 * The parts are fused along N in the order given (gate then up for a fused gate+up projection; one part for a
 * down projection): b (E * N, K/2), sfb (E * K/64, N) int32, N = sum of part_rows.  gw[e] becomes the largest of
 * the parts' global multipliers and every block scale is re-folded to S' = Q_e4m3(S * (G_p / gw[e])), the step the
 * reference leaves to "the real weight loader" (docs/bf16-dual-nvfp4-algorithm.html:235-244).  With one part the
 * result is the checkpoint's own codes and scales bit for bit.
 * global_scale_is_divisor != 0: w = dec(q) * dec(S) / weight_global_scale (the convention of checkpoints that use
 * these tensor names); 0: w = dec(q) * dec(S) * weight_global_scale.  K % 64 == 0. */
#define NVFP4_MAX_CHECKPOINT_PARTS 4
NVFP4_API int nvfp4_load_checkpoint_weights(int num_parts, const void* const* weight_packed, const void* const* weight_scale,
                                            const float* const* weight_global_scale, const int32_t* part_rows,
                                            int global_scale_is_divisor, int E, int K, void* b, void* sfb, float* gw,
                                            void* stream);

/* Reads and clears a kernel status word: copies *device_status to the host on `stream`, resets it to 0, waits for the
 * stream, stores the value through host_value (may be NULL) and returns NVFP4_OK if it was 0, NVFP4_E_DEVICE_TIMEOUT
 * if a bounded in-kernel wait had expired (bit 0).  Synchronous; not for use during stream capture. */
NVFP4_API int nvfp4_read_status(int32_t* device_status, int32_t* host_value, void* stream);

/* The down-projection of a SwiGLU expert MLP with the activation folded into the activation-quantisation kernel:
 * d[M,N] = Q(silu(h[:, :K]) * h[:, K:]) * W^T * gw[expert], where h (M, 2 K) BF16 with row stride ldh_elems is the
 * output of the fused gate+up projection, Q is Algorithm 1 (derived_div8) on the BF16-rounded products, and the
 * other arguments are those of nvfp4_grouped_gemm_contiguous.  Same result, bit for bit, as nvfp4_swiglu followed
 * by nvfp4_grouped_gemm_contiguous on the split path, without writing and re-reading the (M, K) BF16 activation.
 * Normal orientation, N % 256 == 0, M % 128 == 0.  No counterpart in the reference (its benchmarks stop at the GEMM). */
NVFP4_API int nvfp4_grouped_gemm_swiglu_contiguous(const void* h, int64_t ldh_elems, const void* b, const void* sfb,
                                                   const float* gw, void* d, int64_t ldd_elems, const int32_t* m_indices,
                                                   int M, int N, int K, int E, int enable_residual_pass,
                                                   const int32_t* tune, int32_t* device_status, void* stream);

/* Row movers and activation of the expert-parallel MoE layer around the GEMM (dispatch, SwiGLU, combine).
 * They have no counterpart in the reference project, which has no multi-GPU mode; they exist because the
 * contiguous layout the GEMM wants (rows grouped by expert, groups padded to the tile height) has to be
 * produced from, and folded back into, token-major activations on every step.  All pointers are device
 * pointers, rows are BF16 with 16-byte-aligned starts and strides, index arrays are int64.
 *
 * nvfp4_permute_rows: dst[dst_idx ? dst_idx[i] : i] = src[(src_idx ? src_idx[i] : i) / src_div] for
 *   i < n_rows; row_bytes % 16 == 0.  src_div = k turns a (token, choice) pair index into its token.
 * nvfp4_swiglu: out[r, j] = silu(h[r, j]) * h[r, inter + j] for r < rows, j < inter (inter % 8 == 0),
 *   computed in FP32 and rounded once.
 * nvfp4_combine_rows: y[t] = sum over j < k of w[t * k + j] * rows[pos[t * k + j]], accumulated in FP32 in
 *   ascending j (deterministic), hidden % 8 == 0. */
NVFP4_API int nvfp4_permute_rows(const void* src, int64_t src_ld_bytes, const int64_t* src_idx, int src_div,
                                 const int64_t* dst_idx, int64_t n_rows, int row_bytes, void* dst,
                                 int64_t dst_ld_bytes, void* stream);
NVFP4_API int nvfp4_swiglu(const void* h, int64_t h_ld_elems, int64_t rows, int inter, void* out,
                           int64_t out_ld_elems, void* stream);
NVFP4_API int nvfp4_combine_rows(const void* rows, int64_t rows_ld_elems, const int64_t* pos, const float* w,
                                 int64_t tokens, int k, int hidden, void* y, int64_t y_ld_elems, void* stream);

/* Dispatch of QUANTISED rows over peer memory: every token row of `x` (tokens, K) BF16 is decomposed once (Algorithm 1,
 * derived_div8, both passes -- the codes the GEMM's own activation quantisation would produce, bit for bit) and stored
 * for each of its k (token, choice) pairs into row dst_row of rank dst_rank's buffer, which has three planes:
 * packed codes of the first pass (rows_cap, K/2) at offset 0, of the residual pass at a1_offset_bytes, and the block
 * scales (rows_cap, 2, K/16) at scale_offset_bytes.  1.125 bytes per element cross NVLink instead of 2, and Algorithm 1
 * runs once per token instead of once per pair.  K in 1024 ... 8192, a multiple of 1024.  Pairs out of range are
 * skipped as in nvfp4_dispatch_rows_peer.  No counterpart in the reference. */
NVFP4_API int nvfp4_dispatch_quantized_peer(const void* x, int64_t x_ld_elems, int64_t tokens, int k, int K, const int64_t* peers,
                                            int64_t a1_offset_bytes, int64_t scale_offset_bytes, const int64_t* dst_rank,
                                            const int64_t* dst_row, int world, int64_t rows_cap, int sm_budget,
                                            int32_t* device_status, void* stream);

/* Scale rows as the quantised dispatch delivers them, (E * max_m, 2, K/16) bytes, -> the (E * max_m / 128, K/64, 2, 512)
 * atoms nvfp4_grouped_gemm_masked_quantized reads.  masked_m (device, may be NULL = every row) limits the work to each
 * group's live row blocks. */
NVFP4_API int nvfp4_relayout_scales(const void* scale_rows, const int32_t* masked_m, int E, int max_m, int K, void* scale_atoms,
                                    void* stream);

/* nvfp4_grouped_gemm_masked over activations that are already quantised: a0, a1 (E * max_m, K/2) packed codes of the
 * two passes (a1 may be NULL when enable_residual_pass is 0), scale_atoms from nvfp4_relayout_scales.  One launch (the
 * GEMM kernel of the split path); same result as nvfp4_grouped_gemm_masked on the BF16 rows the codes came from. */
NVFP4_API int nvfp4_grouped_gemm_masked_quantized(const void* a0, const void* a1, const void* scale_atoms, const void* b,
                                                  const void* sfb, const float* gw, void* d, int64_t ldd_elems,
                                                  const int32_t* masked_m, int E, int max_m, int N, int K, int enable_residual_pass,
                                                  const int32_t* tune, int32_t* device_status, void* stream);

/* The up-projection of a SwiGLU expert MLP with the activation AND the next GEMM's activation quantisation folded into
 * its epilogue.  The weights (N = 2 I rows per expert) must be interleaved in runs of 32: rows [256 t + 64 g, +32) are gate
 * rows 128 t + 32 g ..., rows [256 t + 64 g + 32, +32) the matching up rows (I % 128 == 0), so that every 64 accumulator
 * columns a thread holds are 32 gate values and their 32 up values.  The epilogue forms bf16(silu(bf16 gate) * bf16 up) --
 * the arithmetic of nvfp4_swiglu -- runs Algorithm 1 (derived_div8, both passes) on it and writes the quantised workspace of
 * the down-projection: out_a0, out_a1 (E * max_m, I / 2) packed codes and out_scale_atoms (E * max_m / 128, I / 64, 2, 512),
 * ready for nvfp4_grouped_gemm_masked_quantized with K = I.  The (rows, 2 I) BF16 intermediate is never written.  Inputs as
 * nvfp4_grouped_gemm_masked_quantized.  No counterpart in the reference (its benchmarks stop at the GEMM). */
NVFP4_API int nvfp4_grouped_gemm_masked_quantized_swiglu(const void* a0, const void* a1, const void* scale_atoms, const void* b,
                                                         const void* sfb, const float* gw, void* out_a0, void* out_a1,
                                                         void* out_scale_atoms, const int32_t* masked_m, int E, int max_m, int N, int K,
                                                         const int32_t* tune, int32_t* device_status, void* stream);

/* The same two steps over peer memory, for ranks on the GPUs of one NVLink domain.  `peers` is a device array
 * with one int64 per rank: the address, in THIS process, of that rank's copy of a symmetric buffer (rows of
 * `row_bytes`, stride dst_ld_bytes / rows_ld_elems, the same on every rank).  No counterpart in the reference.
 *
 * nvfp4_dispatch_rows_peer: for i < n_rows, row src[(src_idx ? src_idx[i] : i) / src_div] is stored into row dst_row[i] of
 *   rank dst_rank[i]'s buffer (gather + all-to-all + scatter in one pass of plain stores).  The caller orders
 *   it after every rank has finished reading its buffer and tells the peers when the stores are complete.
 *   A pair with dst_rank outside [0, world) or dst_row outside [0, rows_cap) is skipped; row -1 is the plan's mark
 *   for "does not fit", anything else out of range also ORs bit 3 into *device_status (may be NULL).
 * nvfp4_combine_rows_peer: y[t] = sum over j < k of w[t*k+j] * (row src_row[t*k+j] of rank src_rank[t*k+j]'s
 *   buffer), read over NVLink: with per-thread loads (bulk_copies = 0), or with one bulk copy per row into shared memory
 *   (bulk_copies != 0; needs two tokens' rows, 2 * k * hidden * 2 bytes, to fit in shared memory, else the first form
 *   runs) -- a few SMs then saturate the NVLink port, where per-thread loads need most of the GPU.  Same summation order,
 *   same bits.  The caller orders it after every rank has written its buffer.  Pairs out of range (as above) contribute
 *   nothing.  device_status (may be NULL) receives bit 0 if a bounded wait of the bulk form expires.
 * sm_budget: the number of SMs the kernel may fill (one 1024-thread block each); 0 = all.  A caller that overlaps these
 *   kernels with GEMMs on another stream gives them a few SMs and sizes the GEMMs to the rest with nvfp4_set_num_sms.
 * Precondition of both plans: expert ids lie in [0, num_experts); ids outside are ignored by the histogram, get no
 *   row and are skipped by the two movers.
 *
 * nvfp4_expert_histogram: counts[e] = number of i < n with ids[i] == e, for e < num_experts <= 4096 (ids outside
 *   the range are ignored); what every rank all-gathers before the plan.
 *   (the routing plan built from the gathered histograms is nvfp4_plan_peer_masked below) */
NVFP4_API int nvfp4_expert_histogram(const int64_t* ids, int64_t n, int num_experts, int64_t* counts, void* stream);
NVFP4_API int nvfp4_dispatch_rows_peer(const void* src, int64_t src_ld_bytes, const int64_t* src_idx, int src_div,
                                       const int64_t* peers, const int64_t* dst_rank, const int64_t* dst_row,
                                       int64_t n_rows, int row_bytes, int64_t dst_ld_bytes, int world, int64_t rows_cap,
                                       int sm_budget, int32_t* device_status, void* stream);
NVFP4_API int nvfp4_combine_rows_peer(const int64_t* peers, int64_t rows_ld_elems, const int64_t* src_rank,
                                      const int64_t* src_row, const float* w, int64_t tokens, int k, int hidden,
                                      void* y, int64_t y_ld_elems, int world, int64_t rows_cap, int sm_budget, int bulk_copies,
                                      int32_t* device_status, void* stream);

/* The routing plan for the masked layout (nvfp4_grouped_gemm_masked): every local expert owns cap_m rows of its
 * rank's buffer, so nothing about the plan has to come back to the host.  all_counts[s * E + e] = pairs rank s routes
 * to expert e (the all-gathered histograms), ids[p] = expert of this rank's pair p (p = token * k + choice), n pairs,
 * E % world == 0, E <= 4096.  From these it writes
 *   base[e], limit[e] (E entries each: first row of this rank's pairs of expert e in the owner's buffer, end of that
 *   expert's cap_m rows), masked_m[j] (E / world int32: real rows of local expert j, clamped to cap_m -- the GEMM's
 *   row counts) and dst_row[p] (n entries; -1 for a pair that does not fit its expert's capacity).
 * If any expert of any rank receives more than cap_m rows, bit 2 of *device_status is set -- on every rank alike,
 * since all see the same histograms; the step's result is then incomplete and the caller repeats it another way.
 * cap_m % 128 == 0.  No counterpart in the reference.
 *
 * nvfp4_peer_barrier: a barrier over the ranks of one NVLink domain whose wait is bounded.  flag_peers[r] is the
 * address, in this process, of rank r's flag array: int64 [NVFP4_BARRIER_SLOTS][world] in symmetric memory, zero
 * before the first use.  Every rank calls it with the same slot and the same epoch, epochs growing by one per call
 * and slot.  A rank whose peers do not arrive within budget_cycles clock cycles ORs bit 1 into *device_status and
 * carries on: the kernel never traps and never spins for ever; the host reads the status word after the step. */
#define NVFP4_BARRIER_SLOTS 8
NVFP4_API int nvfp4_plan_peer_masked(const int64_t* all_counts, int world, int num_experts, int rank, int cap_m,
                                     const int64_t* ids, int64_t n, int64_t* base, int64_t* limit, int32_t* masked_m,
                                     int64_t* dst_row, int32_t* device_status, void* stream);
NVFP4_API int nvfp4_peer_barrier(const int64_t* flag_peers, int rank, int world, int slot, int64_t epoch,
                                 int64_t budget_cycles, int32_t* device_status, void* stream);

/* Test hook: Algorithm 1 exactly as the GEMM's transform warps run it (same device
 * code, same shared-memory layouts), with the codes copied out instead of being fed to
 * the tensor cores.  The GEMM itself never writes a quantised activation to global
 * memory; this exists so that q0/q1/s0/s1 can be compared bit for bit.
 * Counterpart in the reference: tests/standalone/test_transform.cu:50-132.
 *   a (M, K) BF16 row stride lda_elems; M % 128 == 0, K % 128 == 0
 *   q0, q1 (M, K/2) bytes (two codes per byte, even element low); s0, s1 (M, K/16) bytes */
NVFP4_API int nvfp4_debug_decompose(const void* a, int64_t lda_elems, int M, int K, int scale_policy,
                          void* q0, void* q1, void* s0, void* s1, void* stream);

/* Test hook: the first kernel of the two-kernel (split) path alone, into buffers of the caller, so that the
 * quantised activations the GEMM consumes can be compared byte for byte: a0, a1 (M, K/2) packed codes, sfa
 * (M/128, K/64, passes, 512) bytes, one tensor-memory-image scale atom per 128 rows x 64 K x pass (row r of an atom
 * at byte (r % 32) * 16 + (r / 32) * 4, byte j = 16-block j).  M % 128 == 0, K % 128 == 0. */
NVFP4_API int nvfp4_debug_split_workspace(const void* a, int64_t lda_elems, int M, int K, int scale_policy,
                                          int enable_residual_pass, int fold_swiglu, void* a0, void* a1, void* sfa,
                                          void* stream);

/* Test hook: launches one CTA in which a thread waits, for at most budget_cycles clock cycles, on a barrier nobody
 * signals, while the CTA holds tensor memory.  The wait runs out, the kernel ORs bit 0 into *device_status, unwinds
 * the way the GEMM kernels do (every role leaves, tensor memory is freed) and returns: the context stays usable. */
NVFP4_API int nvfp4_debug_wait_timeout(int64_t budget_cycles, int32_t* device_status, void* stream);

/* Measurement hook: issues `iters` rounds of resident-operand block-scaled FP4 MMAs
 * (128 x 256 x 64 each) per SM with no memory traffic and returns through
 * `flops_per_launch` the number of floating-point operations one launch performs.
 * Used to measure the tensor-pipe ceiling the roofline fractions are quoted against. */
NVFP4_API int nvfp4_debug_mma_peak(int iters, double* flops_per_launch, void* stream);

/* The same for CTA pairs: every two SMs run one thread-block cluster of two CTAs whose even CTA issues
 * 256 x 256 x 64 MMAs (tcgen05.mma.cta_group::2) over both tensor cores. */
NVFP4_API int nvfp4_debug_mma_peak_pair(int iters, double* flops_per_launch, void* stream);

/* Measurement hook: like nvfp4_debug_mma_peak, with the issue pattern of a K block made
 * explicit: per round `num_cp` scale-factor copies (tcgen05.cp 32x128b.warpx4) followed by
 * `num_mma` MMAs of 128 x mma_n x 64 (mma_n in {16, 32, 64, 128, 256}); alt_cols != 0
 * alternates the scale columns between two sets.  Used to size the per-K-block issue cost. */
NVFP4_API int nvfp4_debug_mma_pattern(int iters, int num_cp, int num_mma, int mma_n, int alt_cols,
                                      double* flops_per_launch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H_ */
