// The C ABI (include/nvfp4_b200.h): argument validation, per-device runtime
// state, dispatch to the kernels.  Counterpart in the reference: src/api.hpp
// (validation + dispatch), src/runtime/device.hpp, src/runtime/exception.hpp.
#include <climits>
#include <cstring>
#include <mutex>

#include "host_common.hpp"
#include "launchers.hpp"

namespace nvfp4::host {

namespace {
thread_local char g_error[512] = "";
DeviceInfo g_devices[kMaxDevices];
std::mutex g_mutex;
}  // namespace

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}
void clear_error() { g_error[0] = '\0'; }

int device_info(int device, DeviceInfo** out)
{
    if (device < 0) NVFP4_CUDA_CHECK(cudaGetDevice(&device));
    if (device >= kMaxDevices) return fail(NVFP4_E_INVALID_ARGUMENT, "device %d out of range", device);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo& d = g_devices[device];
    if (!d.known) {
        NVFP4_CUDA_CHECK(cudaDeviceGetAttribute(&d.hw_sms, cudaDevAttrMultiProcessorCount, device));
        NVFP4_CUDA_CHECK(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, device));
        NVFP4_CUDA_CHECK(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, device));
        NVFP4_CUDA_CHECK(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        d.num_sms = d.hw_sms;
        d.known = true;
    }
    *out = &d;
    return NVFP4_OK;
}

int workspace_pool(int dev, cudaMemPool_t* out)
{
    static cudaMemPool_t pools[kMaxDevices] = {};
    if (dev < 0 || dev >= kMaxDevices) return fail(NVFP4_E_INVALID_ARGUMENT, "device %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (pools[dev] == nullptr) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t pool = nullptr;
        NVFP4_CUDA_CHECK(cudaMemPoolCreate(&pool, &props));
        uint64_t keep = UINT64_MAX;
        NVFP4_CUDA_CHECK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        pools[dev] = pool;
    }
    *out = pools[dev];
    return NVFP4_OK;
}

int encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                         uint64_t dim0, uint64_t dim1, uint64_t row_stride_bytes, uint32_t box0, uint32_t box1,
                         CUtensorMapSwizzle swizzle)
{
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        NVFP4_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
            return fail(NVFP4_E_CUDA, "driver has no cuTensorMapEncodeTiled");
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
        return fail(NVFP4_E_INVALID_ARGUMENT, "tensor base %p is not 16-byte aligned", base);
    if (row_stride_bytes % 16 != 0)
        return fail(NVFP4_E_INVALID_ARGUMENT, "row stride of %llu bytes is not a multiple of 16",
                    static_cast<unsigned long long>(row_stride_bytes));
    // Encoded maps are kept per (type, base, shape, stride, box, swizzle): weights keep their address from call to
    // call and the pooled workspace usually does, so an eager call costs look-ups instead of driver calls.
    // Counterpart in the reference: the per-launch encodes of src/runtime/tma_desc.hpp:56-67.
    struct Key {
        uint64_t base, dim0, dim1, stride;
        uint32_t box0, box1, dtype, swizzle;
        bool operator==(const Key& o) const
        {
            return base == o.base && dim0 == o.dim0 && dim1 == o.dim1 && stride == o.stride && box0 == o.box0 &&
                   box1 == o.box1 && dtype == o.dtype && swizzle == o.swizzle;
        }
    };
    struct Entry { Key key; CUtensorMap map; bool used; };
    constexpr uint32_t kCacheSize = 256;                       // direct-mapped: a collision just re-encodes
    static Entry cache[kCacheSize] = {};
    static std::mutex cache_mutex;
    const Key key{reinterpret_cast<uint64_t>(base), dim0, dim1, row_stride_bytes, box0, box1,
                  static_cast<uint32_t>(dtype), static_cast<uint32_t>(swizzle)};
    uint64_t h = key.base * 0x9e3779b97f4a7c15ull ^ (key.dim0 * 31 + key.dim1) * 0xbf58476d1ce4e5b9ull ^
                 (static_cast<uint64_t>(key.box0) << 40 | static_cast<uint64_t>(key.box1) << 20 | key.swizzle << 8 | key.dtype);
    h ^= h >> 29;
    Entry& slot = cache[h % kCacheSize];
    {
        std::lock_guard<std::mutex> lock(cache_mutex);
        if (slot.used && slot.key == key) { *map = slot.map; return NVFP4_OK; }
    }
    const cuuint64_t dims[2] = {dim0, dim1};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t elem_strides[2] = {1, 1};
    (void)elem_bytes;
    const CUresult r = encode(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(NVFP4_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, box %u x %u)",
                    static_cast<int>(r), static_cast<unsigned long long>(dim0),
                    static_cast<unsigned long long>(dim1), box0, box1);
    {
        std::lock_guard<std::mutex> lock(cache_mutex);
        slot.key = key;
        slot.map = *map;
        slot.used = true;
    }
    return NVFP4_OK;
}

}  // namespace nvfp4::host

using namespace nvfp4;




extern "C" {

const char* nvfp4_last_error(void) { return host::g_error; }
const char* nvfp4_version(void) { return "nvfp4_b200 0.1 sm_100a"; }

int nvfp4_get_num_sms(int device, int* out)
{
    host::clear_error();
    NVFP4_REQUIRE(out != nullptr, "out is null");
    host::DeviceInfo* d;
    if (int rc = host::device_info(device, &d)) return rc;
    *out = d->num_sms;
    return NVFP4_OK;
}

int nvfp4_set_num_sms(int device, int value)
{
    host::clear_error();
    host::DeviceInfo* d;
    if (int rc = host::device_info(device, &d)) return rc;
    NVFP4_REQUIRE(value >= 0 && value <= 2 * d->hw_sms, "num_sms %d outside [0, %d]", value, 2 * d->hw_sms);
    d->num_sms = value == 0 ? d->hw_sms : value;
    return NVFP4_OK;
}

int nvfp4_quantize_weight(const void* w, int w_dtype, int E, int N, int K, void* b, void* sfb, float* gw,
                          void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(E >= 0 && N >= 0 && K >= 0, "negative shape (E=%d, N=%d, K=%d)", E, N, K);
    NVFP4_REQUIRE(K % 64 == 0, "K=%d must be a multiple of 64", K);
    NVFP4_REQUIRE(w_dtype == NVFP4_DTYPE_BF16 || w_dtype == NVFP4_DTYPE_F32, "unknown weight dtype code %d", w_dtype);
    if (E == 0 || N == 0 || K == 0) return NVFP4_OK;
    NVFP4_REQUIRE(w && b && sfb && gw, "null pointer argument");
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(b) & 15u) == 0, "b must be 16-byte aligned");
    host::DeviceInfo* d;
    if (int rc = host::device_info(-1, &d)) return rc;
    if (d->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU, found sm_%d%d", d->cc_major, d->cc_minor);
    return launch_quantize_weight(w, w_dtype, E, N, K, b, sfb, gw, static_cast<cudaStream_t>(stream));
}

int nvfp4_quantize_weight_static(const void* w, int w_dtype, int E, int N, int K, void* b, void* sfb, float* gw,
                                 void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(E >= 0 && N >= 0 && K >= 0, "negative shape (E=%d, N=%d, K=%d)", E, N, K);
    NVFP4_REQUIRE(K % 64 == 0, "K=%d must be a multiple of 64", K);
    NVFP4_REQUIRE(w_dtype == NVFP4_DTYPE_BF16 || w_dtype == NVFP4_DTYPE_F32, "unknown weight dtype code %d", w_dtype);
    NVFP4_REQUIRE(E <= NVFP4_STATIC_MAX_EXPERTS,
                  "E=%d exceeds the %d experts the static scratch array holds; use nvfp4_quantize_weight or split the call",
                  E, NVFP4_STATIC_MAX_EXPERTS);
    if (E == 0 || N == 0 || K == 0) return NVFP4_OK;
    NVFP4_REQUIRE(w && b && sfb && gw, "null pointer argument");
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(b) & 15u) == 0, "b must be 16-byte aligned");
    host::DeviceInfo* d;
    if (int rc = host::device_info(-1, &d)) return rc;
    if (d->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU, found sm_%d%d", d->cc_major, d->cc_minor);
    return launch_quantize_weight_static(w, w_dtype, E, N, K, b, sfb, gw, static_cast<cudaStream_t>(stream));
}

// Which GEMM kernel the split path runs: tune_cluster = 2 the CTA-pair kernel (cta_group::2, 256 rows x 256 columns per
// pair), 1 the single-CTA kernel, 0 the library's choice.  A pair tile needs two row blocks of one expert, and an
// expert's odd last block costs a whole pair tile.  The pair kernel's main loop is ~5 % faster, so it is chosen when that
// waste is known to be nil (the caller states that every group is a multiple of 256 rows) or small (experts with
// 16 row blocks and more on average; with ~8 ragged row blocks per expert the two kernels measured within 3 % of each
// other either way, with ~1.5 row blocks per expert the pair kernel is 20-30 % slower).
static bool split_gemm_as_pair(const int32_t* tune, int64_t rows, int experts, bool groups_of_256)
{
    const int knob = tune ? tune[8] : 0;
    if (knob == 2) return true;
    if (knob == 1) return false;
    return groups_of_256 || (experts > 0 && rows / experts >= 2048);
}

int nvfp4_grouped_gemm_contiguous(const void* a, int64_t lda_elems, const void* b, const void* sfb, const float* gw,
                                  void* d, int64_t ldd_elems, const int32_t* m_indices, int M, int N, int K, int E,
                                  int scale_policy, int enable_residual_pass, int orientation, int m_alignment,
                                  const int32_t* tune, int32_t* device_status, void* stream)
{
    host::clear_error();
    // the reference's checks, in its order (src/api.hpp:58-79 there)
    NVFP4_REQUIRE(M >= 0 && N >= 0 && K >= 0 && E >= 0, "negative shape (M=%d, N=%d, K=%d, E=%d)", M, N, K, E);
    NVFP4_REQUIRE(K % 128 == 0 && N % 128 == 0, "N and K must be multiples of 128 (N=%d, K=%d)", N, K);
    NVFP4_REQUIRE(orientation == NVFP4_ORIENT_NORMAL || orientation == NVFP4_ORIENT_SWAP_AB, "unknown orientation %d", orientation);
    if (orientation == NVFP4_ORIENT_NORMAL) {
        if (m_alignment == 0) m_alignment = 128;
        NVFP4_REQUIRE(m_alignment == 128 || m_alignment == 256, "normal orientation needs m_alignment 128 or 256, got %d",
                      m_alignment);
    } else {
        if (m_alignment == 0) m_alignment = 32;
        NVFP4_REQUIRE(m_alignment == 16 || m_alignment == 32 || m_alignment == 64 || m_alignment == 128,
                      "swap-AB m_alignment must be 16, 32, 64 or 128, got %d", m_alignment);
    }
    NVFP4_REQUIRE(M % m_alignment == 0, "M must be a multiple of the token-tile alignment (M=%d, alignment=%d)", M, m_alignment);
    if (M == 0 || N == 0) return NVFP4_OK;
    NVFP4_REQUIRE(E > 0 && K > 0, "empty weights (E=%d, K=%d)", E, K);
    NVFP4_REQUIRE(a && b && sfb && gw && d && m_indices, "null pointer argument");
    NVFP4_REQUIRE(lda_elems >= K && ldd_elems >= N, "row strides too small (lda=%lld, ldd=%lld)",
                  static_cast<long long>(lda_elems), static_cast<long long>(ldd_elems));
    NVFP4_REQUIRE(lda_elems % 8 == 0 && ldd_elems % 8 == 0, "row strides must be multiples of 8 elements (16 bytes)");
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(d) & 15u) == 0, "d must be 16-byte aligned");
    NVFP4_REQUIRE(scale_policy >= NVFP4_POLICY_DERIVED_DIV8 && scale_policy <= NVFP4_POLICY_DIV4_RADIX8,
                  "unknown scale policy %d", scale_policy);

    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU, found sm_%d%d", dev->cc_major, dev->cc_minor);

    // tune[] follows the reference's keyword order: 0 block_n, 1 transform_warps, ..., 12 sched_group
    const int tune_block_n = tune ? tune[0] : 0;
    const int tune_xform_warps = tune ? tune[1] : 0;
    const int tune_sched_group = tune ? tune[12] : 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (orientation == NVFP4_ORIENT_SWAP_AB) {
        // token tile: the caller's choice if it divides the alignment, else the largest built tile that does
        int tile = tune_block_n > 0 ? tune_block_n : (m_alignment >= 64 ? 64 : m_alignment);
        NVFP4_REQUIRE((tile == 16 || tile == 32 || tile == 64) && m_alignment % tile == 0,
                      "token tile %d must be 16, 32 or 64 and divide m_alignment %d", tile, m_alignment);
        const int tune_block_k = tune ? tune[5] : 0;   // 0 = the largest of 512 / 256 / 128 that divides K and fits
        NVFP4_REQUIRE(tune_block_k == 0 || tune_block_k == 128 || tune_block_k == 256 || tune_block_k == 512,
                      "tune_block_k must be 0, 128, 256 or 512");
        return launch_gemm_swap(a, lda_elems, b, sfb, gw, d, ldd_elems, m_indices, M, N, K, E, enable_residual_pass != 0,
                                tile, tune_block_k, scale_policy, !(tune && tune[11]), dev->num_sms, device_status, s);
    }
    NVFP4_REQUIRE(tune_xform_warps == 0 || tune_xform_warps == 8 || tune_xform_warps == 16,
                  "tune_transform_warps must be 0, 8 or 16");
    // tune_cluster: 2 / 4 = that many CTAs share one transformed activation tile (needs N % (256 * cluster) == 0),
    // 1 = single-CTA kernel, 0 = the library's choice
    // tune_split_transform: 1 = quantise the activations once, in a kernel of their own, ahead of a GEMM without
    // transform warps (N % 256 == 0); 2 = decompose inside the GEMM main loop; 0 = the library's choice.  (In the
    // reference this keyword signals A0 readiness early inside its one kernel; here it chooses between the two paths.)
    const int tune_split = tune ? tune[13] : 0;
    const bool pdl = !(tune && tune[11]);                           // tune_no_pdl
    NVFP4_REQUIRE(tune_split >= 0 && tune_split <= 2, "tune_split_transform must be 0, 1 or 2");
    NVFP4_REQUIRE(tune_split != 1 || N % 256 == 0, "tune_split_transform=1 needs N %% 256 == 0 (N=%d)", N);
    // The library's choice: a cluster of the fused kernel spans 1024 (512) columns, so up to there an activation tile is
    // transformed once either way and the fused kernel saves the workspace round trip (measured 10 % faster at N = 1024,
    // K = 2048); on wider layers the fused kernel repeats Algorithm 1 per column span and the separate pass wins.
    // Explicit fused-kernel knobs (cluster, transform warps, direct A) keep the fused kernels.
    const bool fused_knobs = tune && (tune[8] != 0 || tune[1] != 0 || tune[9] != 0);
    if (tune_split == 1 || (tune_split == 0 && !fused_knobs && N % 256 == 0 && N > 1024)) {
        const int tune_block_k = tune ? tune[5] : 0;
        return launch_gemm_split(a, lda_elems, b, sfb, gw, d, ldd_elems, m_indices, nullptr, 0, M, N, K, E,
                                 enable_residual_pass != 0, tune_block_k, tune_sched_group, pdl, scale_policy, false,
                                 dev->num_sms, split_gemm_as_pair(tune, M, E, m_alignment == 256), device_status, s);
    }
    int cluster = tune ? tune[8] : 0;
    NVFP4_REQUIRE(cluster == 0 || cluster == 1 || cluster == 2 || cluster == 4, "tune_cluster must be 0, 1, 2 or 4");
    NVFP4_REQUIRE(cluster < 2 || N % (256 * cluster) == 0, "tune_cluster %d needs N %% %d == 0 (N=%d)", cluster, 256 * cluster, N);
    if (cluster == 0) {
        // the widest cluster N allows: every doubling halves the Algorithm-1 arithmetic per CTA
        const bool plain = tune_xform_warps == 0 && !(tune && tune[9]);
        cluster = !plain ? 1 : (N % 1024 == 0 ? 4 : (N % 512 == 0 ? 2 : 1));
    }
    if (cluster >= 2 && dev->num_sms >= cluster)
        return launch_gemm_cluster(a, lda_elems, b, sfb, gw, d, ldd_elems, m_indices, M, N, K, E,
                                   enable_residual_pass != 0, cluster, scale_policy, tune_sched_group, pdl, dev->num_sms,
                                   device_status, s);
    // tune_direct_a = 1: the transform reads activations straight from global memory instead of a TMA-fed
    // shared-memory ring (measured slower on B200: 1.89 ms against 1.06 ms on the Mixtral-like shape)
    const bool direct_a = tune && tune[9] == 1 && tune_xform_warps != 16;
    return launch_gemm_normal(a, lda_elems, b, sfb, gw, d, ldd_elems, m_indices, M, N, K, E, enable_residual_pass != 0,
                              tune_xform_warps, tune_sched_group, direct_a, scale_policy, pdl, dev->num_sms, device_status, s);
}

int nvfp4_permute_rows(const void* src, int64_t src_ld_bytes, const int64_t* src_idx, int src_div, const int64_t* dst_idx,
                       int64_t n_rows, int row_bytes, void* dst, int64_t dst_ld_bytes, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(n_rows >= 0 && row_bytes > 0 && row_bytes % 16 == 0, "row_bytes must be a positive multiple of 16 (got %d)", row_bytes);
    if (n_rows == 0) return NVFP4_OK;
    NVFP4_REQUIRE(src && dst, "null pointer argument");
    NVFP4_REQUIRE(src_div >= 1, "src_div must be at least 1");
    NVFP4_REQUIRE(src_ld_bytes % 16 == 0 && dst_ld_bytes % 16 == 0 && src_ld_bytes >= row_bytes && dst_ld_bytes >= row_bytes,
                  "row strides must be multiples of 16 bytes and at least row_bytes");
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0, "rows must be 16-byte aligned");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    return launch_permute_rows(src, src_ld_bytes, src_idx, src_div, dst_idx, n_rows, row_bytes, dst, dst_ld_bytes, dev->hw_sms,
                               static_cast<cudaStream_t>(stream));
}

int nvfp4_swiglu(const void* h, int64_t h_ld_elems, int64_t rows, int inter, void* out, int64_t out_ld_elems, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(rows >= 0 && inter > 0 && inter % 8 == 0, "inter must be a positive multiple of 8 (got %d)", inter);
    if (rows == 0) return NVFP4_OK;
    NVFP4_REQUIRE(h && out, "null pointer argument");
    NVFP4_REQUIRE(h_ld_elems % 8 == 0 && out_ld_elems % 8 == 0 && h_ld_elems >= 2 * static_cast<int64_t>(inter) && out_ld_elems >= inter,
                  "row strides must be multiples of 8 elements and cover the row");
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0, "rows must be 16-byte aligned");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    return launch_swiglu(h, h_ld_elems, rows, inter, out, out_ld_elems, dev->hw_sms, static_cast<cudaStream_t>(stream));
}

int nvfp4_combine_rows(const void* rows, int64_t rows_ld_elems, const int64_t* pos, const float* w, int64_t tokens, int k,
                       int hidden, void* y, int64_t y_ld_elems, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(tokens >= 0 && k >= 1 && hidden > 0 && hidden % 8 == 0, "k >= 1 and hidden a positive multiple of 8 (k=%d, hidden=%d)", k, hidden);
    if (tokens == 0) return NVFP4_OK;
    NVFP4_REQUIRE(rows && pos && w && y, "null pointer argument");
    NVFP4_REQUIRE(rows_ld_elems % 8 == 0 && y_ld_elems % 8 == 0 && rows_ld_elems >= hidden && y_ld_elems >= hidden,
                  "row strides must be multiples of 8 elements and cover the row");
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0, "rows must be 16-byte aligned");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    return launch_combine_rows(rows, rows_ld_elems, pos, w, tokens, k, hidden, y, y_ld_elems, dev->hw_sms,
                               static_cast<cudaStream_t>(stream));
}

int nvfp4_grouped_gemm_swiglu_contiguous(const void* h, int64_t ldh_elems, const void* b, const void* sfb, const float* gw, void* d,
                                         int64_t ldd_elems, const int32_t* m_indices, int M, int N, int K, int E,
                                         int enable_residual_pass, const int32_t* tune, int32_t* device_status, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(M >= 0 && N >= 0 && K >= 0 && E >= 0, "negative size");
    NVFP4_REQUIRE(N % 256 == 0 && K % 128 == 0, "N must be a multiple of 256 and K of 128 (N=%d, K=%d)", N, K);
    NVFP4_REQUIRE(M % 128 == 0, "M must be a multiple of 128 (M=%d)", M);
    if (M == 0 || N == 0) return NVFP4_OK;
    NVFP4_REQUIRE(E > 0 && K > 0, "empty weights (E=%d, K=%d)", E, K);
    NVFP4_REQUIRE(h && b && sfb && gw && d && m_indices, "null pointer argument");
    NVFP4_REQUIRE(ldh_elems >= 2 * static_cast<int64_t>(K) && ldd_elems >= N, "row strides too small (ldh=%lld, ldd=%lld)",
                  static_cast<long long>(ldh_elems), static_cast<long long>(ldd_elems));
    NVFP4_REQUIRE(ldh_elems % 8 == 0 && ldd_elems % 8 == 0, "row strides must be multiples of 8 elements (16 bytes)");
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(d)) & 15u) == 0, "h and d must be 16-byte aligned");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU, found sm_%d%d", dev->cc_major, dev->cc_minor);
    return launch_gemm_split(h, ldh_elems, b, sfb, gw, d, ldd_elems, m_indices, nullptr, 0, M, N, K, E,
                             enable_residual_pass != 0, tune ? tune[5] : 0, tune ? tune[12] : 0, !(tune && tune[11]),
                             NVFP4_POLICY_DERIVED_DIV8, true, dev->num_sms, split_gemm_as_pair(tune, M, E, false), device_status,
                             static_cast<cudaStream_t>(stream));
}

int nvfp4_grouped_gemm_masked(const void* a, int64_t lda_elems, const void* b, const void* sfb, const float* gw, void* d,
                              int64_t ldd_elems, const int32_t* masked_m, int E, int max_m, int N, int K, int scale_policy,
                              int enable_residual_pass, int fold_swiglu, const int32_t* tune, int32_t* device_status, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(E >= 0 && max_m >= 0 && N >= 0 && K >= 0, "negative size (E=%d, max_m=%d, N=%d, K=%d)", E, max_m, N, K);
    NVFP4_REQUIRE(N % 256 == 0 && K % 128 == 0, "N must be a multiple of 256 and K of 128 (N=%d, K=%d)", N, K);
    NVFP4_REQUIRE(max_m % 128 == 0, "max_m must be a multiple of 128 (max_m=%d)", max_m);
    NVFP4_REQUIRE(static_cast<int64_t>(E) * max_m <= INT32_MAX, "E * max_m = %lld rows exceed the 32-bit row index",
                  static_cast<long long>(E) * max_m);
    if (E == 0 || max_m == 0 || N == 0) return NVFP4_OK;
    NVFP4_REQUIRE(K > 0, "empty weights (K=%d)", K);
    NVFP4_REQUIRE(a && b && sfb && gw && d && masked_m, "null pointer argument");
    const int64_t a_cols = fold_swiglu ? 2 * static_cast<int64_t>(K) : K;
    NVFP4_REQUIRE(lda_elems >= a_cols && ldd_elems >= N, "row strides too small (lda=%lld, ldd=%lld)",
                  static_cast<long long>(lda_elems), static_cast<long long>(ldd_elems));
    NVFP4_REQUIRE(lda_elems % 8 == 0 && ldd_elems % 8 == 0, "row strides must be multiples of 8 elements (16 bytes)");
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(d)) & 15u) == 0, "a and d must be 16-byte aligned");
    NVFP4_REQUIRE(scale_policy >= NVFP4_POLICY_DERIVED_DIV8 && scale_policy <= NVFP4_POLICY_DIV4_RADIX8,
                  "unknown scale policy %d", scale_policy);
    NVFP4_REQUIRE(!fold_swiglu || scale_policy == NVFP4_POLICY_DERIVED_DIV8, "the SwiGLU-folded form is built for derived_div8 only");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU, found sm_%d%d", dev->cc_major, dev->cc_minor);
    return launch_gemm_split(a, lda_elems, b, sfb, gw, d, ldd_elems, nullptr, masked_m, max_m, E * max_m, N, K, E,
                             enable_residual_pass != 0, tune ? tune[5] : 0, tune ? tune[12] : 0, !(tune && tune[11]),
                             scale_policy, fold_swiglu != 0, dev->num_sms, split_gemm_as_pair(tune, static_cast<int64_t>(E) * (max_m / 2), E, false), device_status,
                             static_cast<cudaStream_t>(stream));
}

int nvfp4_load_checkpoint_weights(int num_parts, const void* const* weight_packed, const void* const* weight_scale,
                                  const float* const* weight_global_scale, const int32_t* part_rows,
                                  int global_scale_is_divisor, int E, int K, void* b, void* sfb, float* gw, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(num_parts >= 1 && num_parts <= NVFP4_MAX_CHECKPOINT_PARTS, "num_parts %d outside [1, %d]", num_parts,
                  NVFP4_MAX_CHECKPOINT_PARTS);
    NVFP4_REQUIRE(E >= 0 && K >= 0 && K % 64 == 0, "K=%d must be a non-negative multiple of 64 (E=%d)", K, E);
    NVFP4_REQUIRE(weight_packed && weight_scale && weight_global_scale && part_rows, "null pointer argument");
    int64_t n_total = 0;
    for (int i = 0; i < num_parts; ++i) {
        NVFP4_REQUIRE(part_rows[i] > 0, "part %d has %d rows", i, part_rows[i]);
        NVFP4_REQUIRE(weight_packed[i] && weight_scale[i] && weight_global_scale[i], "null pointer in part %d", i);
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(weight_packed[i]) & 15u) == 0 && (reinterpret_cast<uintptr_t>(weight_scale[i]) & 3u) == 0,
                      "part %d: weight_packed must be 16-byte and weight_scale 4-byte aligned", i);
        n_total += part_rows[i];
    }
    NVFP4_REQUIRE(n_total <= INT32_MAX, "too many rows");
    if (E == 0 || K == 0) return NVFP4_OK;
    NVFP4_REQUIRE(b && sfb && gw, "null pointer argument");
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(b) & 15u) == 0, "b must be 16-byte aligned");
    return launch_load_checkpoint(num_parts, weight_packed, weight_scale, weight_global_scale, part_rows,
                                  global_scale_is_divisor != 0, E, K, static_cast<int>(n_total), b, sfb, gw,
                                  static_cast<cudaStream_t>(stream));
}

int nvfp4_read_status(int32_t* device_status, int32_t* host_value, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(device_status != nullptr, "device_status is null");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int32_t v = 0;
    NVFP4_CUDA_CHECK(cudaMemcpyAsync(&v, device_status, sizeof v, cudaMemcpyDeviceToHost, s));
    NVFP4_CUDA_CHECK(cudaMemsetAsync(device_status, 0, sizeof v, s));
    NVFP4_CUDA_CHECK(cudaStreamSynchronize(s));
    if (host_value != nullptr) *host_value = v;
    if (v & 1)
        return host::fail(NVFP4_E_DEVICE_TIMEOUT, "a bounded in-kernel wait expired (device status 0x%x); the kernel unwound and "
                          "released its tensor memory, its output is undefined", v);
    if (v != 0) return host::fail(NVFP4_E_DEVICE_TIMEOUT, "device status 0x%x", v);
    return NVFP4_OK;
}

int nvfp4_debug_wait_timeout(int64_t budget_cycles, int32_t* device_status, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(budget_cycles > 0 && budget_cycles <= 2000000000ll, "budget_cycles outside (0, 2e9]");
    NVFP4_REQUIRE(device_status != nullptr, "device_status is null");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU");
    return launch_debug_wait_timeout(budget_cycles, device_status, static_cast<cudaStream_t>(stream));
}

int nvfp4_debug_split_workspace(const void* a, int64_t lda_elems, int M, int K, int scale_policy, int enable_residual_pass,
                                int fold_swiglu, void* a0, void* a1, void* sfa, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(M >= 0 && K >= 0 && M % 128 == 0 && K % 128 == 0, "M and K must be multiples of 128 (M=%d, K=%d)", M, K);
    NVFP4_REQUIRE(scale_policy >= NVFP4_POLICY_DERIVED_DIV8 && scale_policy <= NVFP4_POLICY_DIV4_RADIX8,
                  "unknown scale policy %d", scale_policy);
    NVFP4_REQUIRE(!fold_swiglu || scale_policy == NVFP4_POLICY_DERIVED_DIV8, "the SwiGLU-folded form is built for derived_div8 only");
    if (M == 0 || K == 0) return NVFP4_OK;
    NVFP4_REQUIRE(a && a0 && sfa && (a1 || !enable_residual_pass), "null pointer argument");
    NVFP4_REQUIRE(lda_elems >= (fold_swiglu ? 2 * static_cast<int64_t>(K) : K) && lda_elems % 8 == 0, "bad row stride %lld",
                  static_cast<long long>(lda_elems));
    return launch_debug_split_workspace(a, lda_elems, M, K, scale_policy, enable_residual_pass != 0, fold_swiglu != 0, a0,
                                        enable_residual_pass ? a1 : a0, sfa, static_cast<cudaStream_t>(stream));
}

int nvfp4_expert_histogram(const int64_t* ids, int64_t n, int num_experts, int64_t* counts, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(num_experts >= 1 && num_experts <= 4096 && n >= 0, "num_experts (%d) must be in [1, 4096]", num_experts);
    NVFP4_REQUIRE(counts && (n == 0 || ids), "null pointer argument");
    return launch_expert_histogram(ids, n, num_experts, counts, static_cast<cudaStream_t>(stream));
}

int nvfp4_plan_peer_masked(const int64_t* all_counts, int world, int num_experts, int rank, int cap_m, const int64_t* ids,
                           int64_t n, int64_t* base, int64_t* limit, int32_t* masked_m, int64_t* dst_row, int32_t* device_status,
                           void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(world >= 1 && num_experts >= 1 && num_experts <= 4096 && num_experts % world == 0,
                  "num_experts (%d) must be in [1, 4096] and a multiple of world (%d)", num_experts, world);
    NVFP4_REQUIRE(rank >= 0 && rank < world && cap_m >= 128 && cap_m % 128 == 0 && n >= 0, "bad rank / capacity / pair count");
    NVFP4_REQUIRE(all_counts && base && limit && masked_m && (n == 0 || (ids && dst_row)), "null pointer argument");
    return launch_plan_peer_masked(all_counts, world, num_experts, rank, cap_m, ids, n, base, limit, masked_m, dst_row, device_status,
                                   static_cast<cudaStream_t>(stream));
}

int nvfp4_peer_barrier(const int64_t* flag_peers, int rank, int world, int slot, int64_t epoch, int64_t budget_cycles,
                       int32_t* device_status, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(world >= 1 && world <= 64 && rank >= 0 && rank < world, "world (%d) must be in [1, 64] and rank (%d) inside it", world, rank);
    NVFP4_REQUIRE(slot >= 0 && slot < NVFP4_BARRIER_SLOTS && epoch > 0, "slot (%d) must be in [0, %d) and epoch positive", slot,
                  NVFP4_BARRIER_SLOTS);
    NVFP4_REQUIRE(budget_cycles > 0 && budget_cycles <= 4000000000ll, "budget_cycles outside (0, 4e9]");
    NVFP4_REQUIRE(flag_peers != nullptr, "null pointer argument");
    return launch_peer_barrier(flag_peers, rank, world, slot, epoch, budget_cycles, device_status, static_cast<cudaStream_t>(stream));
}

int nvfp4_dispatch_rows_peer(const void* src, int64_t src_ld_bytes, const int64_t* src_idx, int src_div, const int64_t* peers,
                             const int64_t* dst_rank, const int64_t* dst_row, int64_t n_rows, int row_bytes, int64_t dst_ld_bytes,
                             int world, int64_t rows_cap, int sm_budget, int32_t* device_status, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(n_rows >= 0 && row_bytes > 0 && row_bytes % 16 == 0, "row_bytes must be a positive multiple of 16 (got %d)", row_bytes);
    if (n_rows == 0) return NVFP4_OK;
    NVFP4_REQUIRE(src && peers && dst_rank && dst_row, "null pointer argument");
    NVFP4_REQUIRE(src_div >= 1 && world >= 1 && rows_cap >= 0, "src_div and world must be at least 1, rows_cap non-negative");
    NVFP4_REQUIRE(src_ld_bytes % 16 == 0 && dst_ld_bytes % 16 == 0 && src_ld_bytes >= row_bytes && dst_ld_bytes >= row_bytes,
                  "row strides must be multiples of 16 bytes and at least row_bytes");
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15u) == 0, "rows must be 16-byte aligned");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    NVFP4_REQUIRE(sm_budget >= 0, "sm_budget must not be negative");
    return launch_dispatch_rows_peer(src, src_ld_bytes, src_idx, src_div, peers, dst_rank, dst_row, n_rows, row_bytes, dst_ld_bytes,
                                     world, rows_cap, device_status, sm_budget > 0 && sm_budget < dev->hw_sms ? sm_budget : dev->hw_sms,
                                     static_cast<cudaStream_t>(stream));
}

int nvfp4_dispatch_quantized_peer(const void* x, int64_t x_ld_elems, int64_t tokens, int k, int K, const int64_t* peers,
                                  int64_t a1_offset_bytes, int64_t scale_offset_bytes, const int64_t* dst_rank,
                                  const int64_t* dst_row, int world, int64_t rows_cap, int sm_budget, int32_t* device_status,
                                  void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(tokens >= 0 && k >= 1, "tokens must not be negative and k at least 1 (tokens=%lld, k=%d)", static_cast<long long>(tokens), k);
    NVFP4_REQUIRE(K >= 1024 && K <= 8192 && K % 1024 == 0, "quantised dispatch needs K in 1024 ... 8192, a multiple of 1024 (K=%d)", K);
    if (tokens == 0) return NVFP4_OK;
    NVFP4_REQUIRE(x && peers && dst_rank && dst_row, "null pointer argument");
    NVFP4_REQUIRE(world >= 1 && rows_cap >= 0 && sm_budget >= 0, "world must be at least 1, rows_cap and sm_budget non-negative");
    NVFP4_REQUIRE(x_ld_elems >= K && x_ld_elems % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0,
                  "token rows must be 16-byte aligned with a stride of at least K elements");
    NVFP4_REQUIRE(a1_offset_bytes >= rows_cap * (K / 2) && scale_offset_bytes >= a1_offset_bytes + rows_cap * (K / 2) &&
                      a1_offset_bytes % 16 == 0 && scale_offset_bytes % 16 == 0,
                  "the three planes (a0, a1, scales) must not overlap and must start on 16-byte boundaries");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    return launch_dispatch_quantized_peer(x, x_ld_elems * 2, tokens, k, K, peers, a1_offset_bytes, scale_offset_bytes, dst_rank, dst_row,
                                          world, rows_cap, device_status,
                                          sm_budget > 0 && sm_budget < dev->hw_sms ? sm_budget : dev->hw_sms,
                                          static_cast<cudaStream_t>(stream));
}

int nvfp4_relayout_scales(const void* scale_rows, const int32_t* masked_m, int E, int max_m, int K, void* scale_atoms, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(E >= 0 && max_m >= 0 && max_m % 128 == 0 && K > 0 && K % 64 == 0,
                  "max_m must be a multiple of 128 and K of 64 (E=%d, max_m=%d, K=%d)", E, max_m, K);
    if (E == 0 || max_m == 0) return NVFP4_OK;
    NVFP4_REQUIRE(scale_rows && scale_atoms, "null pointer argument");
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(scale_rows) | reinterpret_cast<uintptr_t>(scale_atoms)) & 3u) == 0, "scale buffers must be 4-byte aligned");
    return launch_relayout_scales(scale_rows, masked_m, max_m, static_cast<int64_t>(E) * max_m, K, scale_atoms, true,
                                  static_cast<cudaStream_t>(stream));
}

int nvfp4_grouped_gemm_masked_quantized(const void* a0, const void* a1, const void* scale_atoms, const void* b, const void* sfb,
                                        const float* gw, void* d, int64_t ldd_elems, const int32_t* masked_m, int E, int max_m, int N,
                                        int K, int enable_residual_pass, const int32_t* tune, int32_t* device_status, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(E >= 0 && max_m >= 0 && N >= 0 && K >= 0, "negative size (E=%d, max_m=%d, N=%d, K=%d)", E, max_m, N, K);
    NVFP4_REQUIRE(N % 256 == 0 && K % 128 == 0, "N must be a multiple of 256 and K of 128 (N=%d, K=%d)", N, K);
    NVFP4_REQUIRE(max_m % 128 == 0, "max_m must be a multiple of 128 (max_m=%d)", max_m);
    NVFP4_REQUIRE(static_cast<int64_t>(E) * max_m <= INT32_MAX, "E * max_m = %lld rows exceed the 32-bit row index",
                  static_cast<long long>(E) * max_m);
    if (E == 0 || max_m == 0 || N == 0) return NVFP4_OK;
    NVFP4_REQUIRE(K > 0, "empty weights (K=%d)", K);
    NVFP4_REQUIRE(a0 && scale_atoms && b && sfb && gw && d && masked_m && (a1 || !enable_residual_pass), "null pointer argument");
    NVFP4_REQUIRE(ldd_elems >= N && ldd_elems % 8 == 0, "bad output row stride %lld", static_cast<long long>(ldd_elems));
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(a0) | reinterpret_cast<uintptr_t>(a1) | reinterpret_cast<uintptr_t>(scale_atoms) |
                    reinterpret_cast<uintptr_t>(d)) & 15u) == 0, "a0, a1, scale_atoms and d must be 16-byte aligned");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU, found sm_%d%d", dev->cc_major, dev->cc_minor);
    return launch_gemm_split_quantized(a0, a1, scale_atoms, b, sfb, gw, d, ldd_elems, masked_m, max_m, N, K, E, enable_residual_pass != 0,
                                       tune ? tune[5] : 0, tune ? tune[12] : 0, !(tune && tune[11]), dev->num_sms,
                                       split_gemm_as_pair(tune, static_cast<int64_t>(E) * (max_m / 2), E, false), nullptr, nullptr, nullptr,
                                       device_status, static_cast<cudaStream_t>(stream));
}

int nvfp4_grouped_gemm_masked_quantized_swiglu(const void* a0, const void* a1, const void* scale_atoms, const void* b, const void* sfb,
                                               const float* gw, void* out_a0, void* out_a1, void* out_scale_atoms,
                                               const int32_t* masked_m, int E, int max_m, int N, int K, const int32_t* tune,
                                               int32_t* device_status, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(E >= 0 && max_m >= 0 && N >= 0 && K >= 0, "negative size (E=%d, max_m=%d, N=%d, K=%d)", E, max_m, N, K);
    NVFP4_REQUIRE(N % 256 == 0 && K % 128 == 0, "N must be a multiple of 256 and K of 128 (N=%d, K=%d)", N, K);
    NVFP4_REQUIRE(max_m % 128 == 0, "max_m must be a multiple of 128 (max_m=%d)", max_m);
    NVFP4_REQUIRE(static_cast<int64_t>(E) * max_m <= INT32_MAX, "E * max_m = %lld rows exceed the 32-bit row index",
                  static_cast<long long>(E) * max_m);
    if (E == 0 || max_m == 0 || N == 0) return NVFP4_OK;
    NVFP4_REQUIRE(K > 0, "empty weights (K=%d)", K);
    NVFP4_REQUIRE(a0 && a1 && scale_atoms && b && sfb && gw && out_a0 && out_a1 && out_scale_atoms && masked_m, "null pointer argument");
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(a0) | reinterpret_cast<uintptr_t>(a1) | reinterpret_cast<uintptr_t>(scale_atoms) |
                    reinterpret_cast<uintptr_t>(out_a0) | reinterpret_cast<uintptr_t>(out_a1) | reinterpret_cast<uintptr_t>(out_scale_atoms)) & 15u) == 0,
                  "all activation buffers must be 16-byte aligned");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU, found sm_%d%d", dev->cc_major, dev->cc_minor);
    return launch_gemm_split_quantized(a0, a1, scale_atoms, b, sfb, gw, nullptr, 0, masked_m, max_m, N, K, E, true, tune ? tune[5] : 0,
                                       tune ? tune[12] : 0, !(tune && tune[11]), dev->num_sms,
                                       split_gemm_as_pair(tune, static_cast<int64_t>(E) * (max_m / 2), E, false), out_a0, out_a1,
                                       out_scale_atoms, device_status, static_cast<cudaStream_t>(stream));
}

int nvfp4_combine_rows_peer(const int64_t* peers, int64_t rows_ld_elems, const int64_t* src_rank, const int64_t* src_row,
                            const float* w, int64_t tokens, int k, int hidden, void* y, int64_t y_ld_elems, int world,
                            int64_t rows_cap, int sm_budget, int bulk_copies, int32_t* device_status, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(tokens >= 0 && k >= 1 && hidden > 0 && hidden % 8 == 0, "k >= 1 and hidden a positive multiple of 8 (k=%d, hidden=%d)", k, hidden);
    if (tokens == 0) return NVFP4_OK;
    NVFP4_REQUIRE(peers && src_rank && src_row && w && y, "null pointer argument");
    NVFP4_REQUIRE(world >= 1 && rows_cap >= 0, "world must be at least 1, rows_cap non-negative");
    NVFP4_REQUIRE(rows_ld_elems % 8 == 0 && y_ld_elems % 8 == 0 && rows_ld_elems >= hidden && y_ld_elems >= hidden,
                  "row strides must be multiples of 8 elements and cover the row");
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(y) & 15u) == 0, "rows must be 16-byte aligned");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    NVFP4_REQUIRE(sm_budget >= 0, "sm_budget must not be negative");
    return launch_combine_rows_peer(peers, rows_ld_elems, src_rank, src_row, w, tokens, k, hidden, y, y_ld_elems, world, rows_cap,
                                    sm_budget > 0 && sm_budget < dev->hw_sms ? sm_budget : dev->hw_sms, bulk_copies != 0,
                                    device_status, static_cast<cudaStream_t>(stream));
}

int nvfp4_debug_decompose(const void* a, int64_t lda_elems, int M, int K, int scale_policy, void* q0, void* q1,
                          void* s0, void* s1, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(M >= 0 && K >= 0 && M % 128 == 0 && K % 128 == 0, "M and K must be multiples of 128 (M=%d, K=%d)", M, K);
    NVFP4_REQUIRE(scale_policy >= NVFP4_POLICY_DERIVED_DIV8 && scale_policy <= NVFP4_POLICY_DIV4_RADIX8,
                  "unknown scale policy %d", scale_policy);
    if (M == 0 || K == 0) return NVFP4_OK;
    NVFP4_REQUIRE(a && q0 && q1 && s0 && s1, "null pointer argument");
    NVFP4_REQUIRE(lda_elems >= K && lda_elems % 8 == 0, "bad row stride %lld", static_cast<long long>(lda_elems));
    return launch_debug_decompose(a, lda_elems, M, K, scale_policy, q0, q1, s0, s1, static_cast<cudaStream_t>(stream));
}

int nvfp4_debug_mma_peak(int iters, double* flops_per_launch, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(iters > 0 && iters <= (1 << 20), "iters %d outside [1, 2^20]", iters);
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU");
    return launch_mma_peak(iters, dev->hw_sms, flops_per_launch, static_cast<cudaStream_t>(stream));
}

int nvfp4_debug_mma_peak_pair(int iters, double* flops_per_launch, void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(iters > 0, "iters must be positive");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU, found sm_%d%d", dev->cc_major, dev->cc_minor);
    return launch_mma_peak_pair(iters, dev->hw_sms, flops_per_launch, static_cast<cudaStream_t>(stream));
}

int nvfp4_debug_mma_pattern(int iters, int num_cp, int num_mma, int mma_n, int alt_cols, double* flops_per_launch,
                            void* stream)
{
    host::clear_error();
    NVFP4_REQUIRE(iters > 0 && iters <= (1 << 20) && num_cp >= 0 && num_cp <= 64 && num_mma >= 0 && num_mma <= 64,
                  "iters / num_cp / num_mma out of range");
    host::DeviceInfo* dev;
    if (int rc = host::device_info(-1, &dev)) return rc;
    if (dev->cc_major != 10) return host::fail(NVFP4_E_UNSUPPORTED, "needs an sm_100 GPU");
    return launch_mma_pattern(iters, num_cp, num_mma, mma_n, alt_cols, dev->hw_sms, flops_per_launch,
                              static_cast<cudaStream_t>(stream));
}

}  // extern "C"
