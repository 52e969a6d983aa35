// TEST INFRASTRUCTURE -- not product code.
//
// C-ABI shim around the reference's own C++ host twin of the dual-NVFP4
// algorithm (tests/standalone/reference.hpp in the reference project).  The
// header is included unmodified from where the reference is mounted; nothing
// of it is copied here.  The result (oracle/_ref/libref_twin.so) is the real
// reference arithmetic on the CPU: it validates the C restatement in
// dual_nvfp4_oracle.c and serves as the "reference" kind of CPU baseline.
//
// Built by oracle/Makefile with:  g++ -O2 -fopenmp -I$CUDA/include -DREF_HPP=...
#include REF_HPP

#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

// ref::decompose_block over every 16-element block of an (M, K) FP32 matrix.
// Codes one per byte; scales one E4M3 byte per block.
int ref_twin_decompose(const float* x, int64_t M, int64_t K, uint8_t* q0, uint8_t* q1,
                       uint8_t* s0, uint8_t* s1)
{
    if (K % ref::kBlockSize != 0) return -1;
    const int64_t nb = K / ref::kBlockSize;
#pragma omp parallel for
    for (int64_t m = 0; m < M; ++m)
        for (int64_t b = 0; b < nb; ++b)
            ref::decompose_block(x + m * K + b * ref::kBlockSize, q0 + m * K + b * ref::kBlockSize,
                                 q1 + m * K + b * ref::kBlockSize, s0[m * nb + b], s1[m * nb + b]);
    return 0;
}

// ref::quantize_weight: codes (E, N, K) one per byte, scales (E, N, K/16), g (E).
int ref_twin_quantize_weight(const float* w, int E, int N, int K, uint8_t* q, uint8_t* sf, float* g)
{
    std::vector<float> wv(w, w + static_cast<size_t>(E) * N * K);
    std::vector<uint8_t> qv, sv;
    std::vector<float> gv;
    ref::quantize_weight(wv, E, N, K, qv, sv, gv);
    std::memcpy(q, qv.data(), qv.size());
    std::memcpy(sf, sv.data(), sv.size());
    std::memcpy(g, gv.data(), gv.size() * sizeof(float));
    return 0;
}

// ref::dual_gemm on rows [0, M) and weight rows [0, N): the whole reference
// CPU chain (decompose, reconstruct, dequantise, FP32 dot products).
int ref_twin_dual_gemm(const float* a, const uint8_t* q, const uint8_t* sf, const float* g,
                       const int32_t* expert_of_row, int M, int N, int K, int E, float* out)
{
    std::vector<float> av(a, a + static_cast<size_t>(M) * K);
    std::vector<uint8_t> qv(q, q + static_cast<size_t>(E) * N * K);
    std::vector<uint8_t> sv(sf, sf + static_cast<size_t>(E) * N * (K / ref::kBlockSize));
    std::vector<float> gv(g, g + E);
    std::vector<int> ev(expert_of_row, expert_of_row + M);
    std::vector<float> r = ref::dual_gemm(av, qv, sv, gv, ev, M, N, K, E);
    std::memcpy(out, r.data(), r.size() * sizeof(float));
    return 0;
}

// The same chain on all host threads: the reference's function is serial, so row chunks
// of the input are handed to independent calls of it (each call runs the reference's
// own code start to end on its rows).
int ref_twin_dual_gemm_mt(const float* a, const uint8_t* q, const uint8_t* sf, const float* g,
                          const int32_t* expert_of_row, int M, int N, int K, int E, float* out, int threads)
{
    const int chunk = 8;
    const int nchunks = (M + chunk - 1) / chunk;
    std::vector<uint8_t> qv(q, q + static_cast<size_t>(E) * N * K);
    std::vector<uint8_t> sv(sf, sf + static_cast<size_t>(E) * N * (K / ref::kBlockSize));
    std::vector<float> gv(g, g + E);
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
    for (int c = 0; c < nchunks; ++c) {
        const int lo = c * chunk, hi = lo + chunk < M ? lo + chunk : M;
        std::vector<float> av(a + static_cast<size_t>(lo) * K, a + static_cast<size_t>(hi) * K);
        std::vector<int> ev(expert_of_row + lo, expert_of_row + hi);
        std::vector<float> r = ref::dual_gemm(av, qv, sv, gv, ev, hi - lo, N, K, E);
        std::memcpy(out + static_cast<size_t>(lo) * N, r.data(), r.size() * sizeof(float));
    }
    return 0;
}

}  // extern "C"
