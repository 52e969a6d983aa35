// Internal launch functions behind the C ABI (arguments already validated).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace nvfp4 {

int launch_gemm_normal(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                       int64_t ldd, const int32_t* m_indices, int M, int N, int K, int E, bool residual,
                       int xform_warps, int group_m, bool direct_a, int policy, bool pdl, int num_sms, int32_t* status,
                       cudaStream_t stream);

// Cluster variant of the normal orientation (cluster = 2 or 4, N % (256 * cluster) == 0).
int launch_gemm_cluster(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                        int64_t ldd, const int32_t* m_indices, int M, int N, int K, int E, bool residual,
                        int cluster, int policy, int group_m, bool pdl, int num_sms, int32_t* status, cudaStream_t stream);

// masked_m == nullptr: contiguous layout.  Otherwise E groups of max_m rows each (M = E * max_m), masked_m[g] real.
int launch_gemm_split(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                      int64_t ldd, const int32_t* m_indices, const int32_t* masked_m, int max_m, int M, int N, int K, int E,
                      bool residual, int block_k, int group_m, bool pdl, int policy, bool swiglu, int num_sms, bool pair,
                      int32_t* status, cudaStream_t stream);

int launch_gemm_split_quantized(const void* a0, const void* a1, const void* sfa, const void* b, const void* sfb, const float* gw,
                                void* d, int64_t ldd, const int32_t* masked_m, int max_m, int N, int K, int E, bool residual,
                                int block_k, int group_m, bool pdl, int num_sms, bool pair, void* out_a0, void* out_a1, void* out_sf,
                                int32_t* status, cudaStream_t stream);

int launch_debug_split_workspace(const void* a, int64_t lda, int M, int K, int policy, bool residual, bool swiglu, void* a0,
                                 void* a1, void* sfa, cudaStream_t stream);

int launch_permute_rows(const void* src, int64_t src_ld_bytes, const int64_t* src_idx, int src_div, const int64_t* dst_idx,
                        int64_t n_rows, int row_bytes, void* dst, int64_t dst_ld_bytes, int num_sms, cudaStream_t stream);
int launch_swiglu(const void* h, int64_t h_ld_elems, int64_t rows, int inter, void* out, int64_t out_ld_elems, int num_sms,
                  cudaStream_t stream);
int launch_combine_rows(const void* rows, int64_t rows_ld_elems, const int64_t* pos, const float* w, int64_t tokens, int k,
                        int hidden, void* y, int64_t y_ld_elems, int num_sms, cudaStream_t stream);

int launch_expert_histogram(const int64_t* ids, int64_t n, int num_experts, int64_t* counts, cudaStream_t stream);
int launch_plan_peer_masked(const int64_t* all_counts, int world, int num_experts, int rank, int cap_m, const int64_t* ids,
                            int64_t n, int64_t* base, int64_t* limit, int32_t* masked_m, int64_t* dst_row, int32_t* status,
                            cudaStream_t stream);
int launch_peer_barrier(const int64_t* flag_peers, int rank, int world, int slot, int64_t epoch, int64_t budget_cycles,
                        int32_t* status, cudaStream_t stream);
int launch_dispatch_rows_peer(const void* src, int64_t src_ld_bytes, const int64_t* src_idx, int src_div, const int64_t* peers,
                              const int64_t* dst_rank, const int64_t* dst_row, int64_t n_rows, int row_bytes,
                              int64_t dst_ld_bytes, int world, int64_t rows_cap, int32_t* status, int num_sms, cudaStream_t stream);
int launch_dispatch_quantized_peer(const void* x, int64_t x_ld_bytes, int64_t tokens, int k, int kdim, const int64_t* peers,
                                   int64_t a1_off, int64_t sf_off, const int64_t* dst_rank, const int64_t* dst_row, int world,
                                   int64_t rows_cap, int32_t* status, int num_sms, cudaStream_t stream);
int launch_relayout_scales(const void* sf_rows, const int32_t* masked_m, int max_m, int64_t rows, int kdim, void* atoms, bool pdl,
                           cudaStream_t stream);
int launch_combine_rows_peer(const int64_t* peers, int64_t rows_ld_elems, const int64_t* src_rank, const int64_t* src_row,
                             const float* w, int64_t tokens, int k, int hidden, void* y, int64_t y_ld_elems, int world,
                             int64_t rows_cap, int num_sms, bool bulk, int32_t* status, cudaStream_t stream);

int launch_gemm_swap(const void* a, int64_t lda, const void* b, const void* sfb, const float* gw, void* d,
                     int64_t ldd, const int32_t* m_indices, int M, int N, int K, int E, bool residual,
                     int token_tile, int block_k, int policy, bool pdl, int num_sms, int32_t* status, cudaStream_t stream);

int launch_quantize_weight(const void* w, int w_dtype, int E, int N, int K, void* b, void* sfb, float* gw,
                           cudaStream_t stream);

int launch_quantize_weight_static(const void* w, int w_dtype, int E, int N, int K, void* b, void* sfb, float* gw,
                                  cudaStream_t stream);

int launch_debug_decompose(const void* a, int64_t lda, int M, int K, int policy, void* q0, void* q1, void* s0, void* s1,
                           cudaStream_t stream);

int launch_debug_wait_timeout(int64_t budget_cycles, int32_t* status, cudaStream_t stream);

// Checkpoint layout -> the GEMM's weight layout; see nvfp4_load_checkpoint_weights.
int launch_load_checkpoint(int num_parts, const void* const* packed, const void* const* scale, const float* const* global_scale,
                           const int32_t* part_rows, bool divisor, int E, int K, int n_total, void* b, void* sfb, float* gw,
                           cudaStream_t stream);

int launch_mma_peak(int iters, int num_sms, double* flops_per_launch, cudaStream_t stream);
int launch_mma_peak_pair(int iters, int num_sms, double* flops_per_launch, cudaStream_t stream);

int launch_mma_pattern(int iters, int num_cp, int num_mma, int mma_n, int alt_cols, int num_sms, double* flops_per_launch,
                       cudaStream_t stream);

}  // namespace nvfp4
