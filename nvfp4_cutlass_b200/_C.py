"""Binding of the C ABI (include/nvfp4_b200.h) -- the stand-in for the reference's
compiled ``_C`` extension module (src/python_api.cpp:10-14, src/api.hpp:146-204 there).

Tensors cross the boundary as raw device pointers, sizes and strides; the launch
goes onto torch's current CUDA stream, as in the reference (src/jit/launch.hpp:47).
Failures of the library surface as ``RuntimeError`` carrying its error text, where
the reference's pybind layer surfaces its C++ exception.  There is no fallback of
any kind: without the compiled library, or without a CUDA tensor, calls raise.
"""
from __future__ import annotations

import ctypes
import os

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libnvfp4_b200.so")
_lib = None

POLICY_CODES = {"derived_div8": 0, "residual_amax": 1, "derived_div4": 2, "div4_radix8": 3}

# keyword order of the reference's tune_* arguments (src/api.hpp:166-203)
TUNE_KEYS = ("tune_block_n", "tune_transform_warps", "tune_epilogue_threads", "tune_num_stages",
             "tune_swizzle_cd", "tune_block_k", "tune_epilogue_stages", "tune_swap_ab", "tune_cluster",
             "tune_direct_a", "tune_l2_pin_weights", "tune_no_pdl", "tune_sched_group",
             "tune_split_transform", "tune_timing_probe", "tune_tail_split", "tune_shallow_stages",
             "tune_produced_stages")

EXPORTS = ("nvfp4_last_error", "nvfp4_version", "nvfp4_get_num_sms", "nvfp4_set_num_sms",
           "nvfp4_quantize_weight", "nvfp4_quantize_weight_static", "nvfp4_grouped_gemm_contiguous", "nvfp4_debug_decompose",
           "nvfp4_debug_mma_peak", "nvfp4_debug_mma_peak_pair", "nvfp4_debug_mma_pattern", "nvfp4_permute_rows", "nvfp4_swiglu", "nvfp4_combine_rows",
           "nvfp4_dispatch_rows_peer", "nvfp4_dispatch_quantized_peer", "nvfp4_relayout_scales",
           "nvfp4_grouped_gemm_masked_quantized", "nvfp4_grouped_gemm_masked_quantized_swiglu", "nvfp4_combine_rows_peer", "nvfp4_expert_histogram",
           "nvfp4_grouped_gemm_swiglu_contiguous", "nvfp4_grouped_gemm_masked", "nvfp4_load_checkpoint_weights",
           "nvfp4_read_status", "nvfp4_debug_split_workspace", "nvfp4_debug_wait_timeout", "nvfp4_plan_peer_masked",
           "nvfp4_peer_barrier")


def library_path() -> str:
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python nvfp4_cutlass_b200/csrc/build.py` "
                "(there is no fallback path)")
        L = ctypes.CDLL(_LIB_PATH)
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        L.nvfp4_last_error.restype = ctypes.c_char_p
        L.nvfp4_version.restype = ctypes.c_char_p
        L.nvfp4_get_num_sms.argtypes = [i32, ctypes.POINTER(i32)]
        L.nvfp4_set_num_sms.argtypes = [i32, i32]
        L.nvfp4_quantize_weight.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
        L.nvfp4_quantize_weight_static.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
        L.nvfp4_grouped_gemm_contiguous.argtypes = [vp, i64, vp, vp, vp, vp, i64, vp, i32, i32, i32, i32,
                                                    i32, i32, i32, i32, vp, vp, vp]
        L.nvfp4_debug_decompose.argtypes = [vp, i64, i32, i32, i32, vp, vp, vp, vp, vp]
        L.nvfp4_permute_rows.argtypes = [vp, i64, vp, i32, vp, i64, i32, vp, i64, vp]
        L.nvfp4_swiglu.argtypes = [vp, i64, i64, i32, vp, i64, vp]
        L.nvfp4_dispatch_rows_peer.argtypes = [vp, i64, vp, i32, vp, vp, vp, i64, i32, i64, i32, i64, i32, vp, vp]
        L.nvfp4_plan_peer_masked.argtypes = [vp, i32, i32, i32, i32, vp, i64, vp, vp, vp, vp, vp, vp]
        L.nvfp4_peer_barrier.argtypes = [vp, i32, i32, i32, i64, i64, vp, vp]
        L.nvfp4_expert_histogram.argtypes = [vp, i64, i32, vp, vp]
        L.nvfp4_grouped_gemm_swiglu_contiguous.argtypes = [vp, i64, vp, vp, vp, vp, i64, vp, i32, i32, i32, i32, i32, vp, vp, vp]
        L.nvfp4_combine_rows_peer.argtypes = [vp, i64, vp, vp, vp, i64, i32, i32, vp, i64, i32, i64, i32, i32, vp, vp]
        L.nvfp4_combine_rows.argtypes = [vp, i64, vp, vp, i64, i32, i32, vp, i64, vp]
        L.nvfp4_dispatch_quantized_peer.argtypes = [vp, i64, i64, i32, i32, vp, i64, i64, vp, vp, i32, i64, i32, vp, vp]
        L.nvfp4_relayout_scales.argtypes = [vp, vp, i32, i32, i32, vp, vp]
        L.nvfp4_grouped_gemm_masked_quantized.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, vp, i32, i32, i32, i32, i32, vp, vp, vp]
        L.nvfp4_grouped_gemm_masked_quantized_swiglu.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, vp]
        L.nvfp4_grouped_gemm_masked.argtypes = [vp, i64, vp, vp, vp, vp, i64, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp]
        L.nvfp4_load_checkpoint_weights.argtypes = [i32, vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, vp]
        L.nvfp4_read_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
        L.nvfp4_debug_split_workspace.argtypes = [vp, i64, i32, i32, i32, i32, i32, vp, vp, vp, vp]
        L.nvfp4_debug_wait_timeout.argtypes = [i64, vp, vp]
        L.nvfp4_debug_mma_peak.argtypes = [i32, ctypes.POINTER(ctypes.c_double), vp]
        L.nvfp4_debug_mma_peak_pair.argtypes = [i32, ctypes.POINTER(ctypes.c_double), vp]
        L.nvfp4_debug_mma_pattern.argtypes = [i32, i32, i32, i32, i32, ctypes.POINTER(ctypes.c_double), vp]
        _lib = L
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"nvfp4_b200 error {rc}: {lib().nvfp4_last_error().decode()}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require(cond: bool, what: str) -> None:
    if not cond:
        raise RuntimeError(f"nvfp4_gemm: assertion failed: {what}")


def _one_device(*tensors) -> torch.device:
    """All tensors are CUDA tensors of ONE device; returns it.  The library launches on the current device and
    stream, so every wrapper below makes that device current for the call (``with torch.cuda.device(...)``): stream,
    memory pool, SM count and tensor maps then belong to the GPU that holds the operands."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        _require(isinstance(t, torch.Tensor) and t.is_cuda, "every operand is a CUDA tensor")
        dev = t.device if dev is None else dev
        _require(t.device == dev, f"all operands are on one device (found {dev} and {t.device})")
    _require(dev is not None, "at least one tensor operand")
    return dev


def init(include_root: str = "", cuda_home: str = "") -> None:
    """Kept for signature compatibility: the reference starts its JIT here; kernels
    in this build are compiled ahead of time, so this only loads the library."""
    lib()


def get_num_sms() -> int:
    out = ctypes.c_int(0)
    _check(lib().nvfp4_get_num_sms(-1, ctypes.byref(out)))
    return out.value


def set_num_sms(num_sms: int) -> None:
    _check(lib().nvfp4_set_num_sms(-1, int(num_sms)))


def set_probe_buffer(t=None) -> None:
    """The reference's in-kernel clock probe has no counterpart; accepted and ignored."""


def m_grouped_bf16_dual_nvfp4_gemm_contiguous(a, b, sfb, gw, d, m_indices, scale_policy: str = "derived_div8",
                                              enable_residual_pass: bool = True, *, device_status=None,
                                              m_alignment: int = 0, **tune) -> None:
    """d = (A0 + A1) @ W^T * gw per expert group; same contract as the reference entry
    (src/api.hpp:26-144): dtype / shape assertions first, then a silent return for
    M == 0 or N == 0, then an asynchronous launch on the current stream."""
    for key in tune:
        if key not in TUNE_KEYS:
            raise TypeError(f"m_grouped_bf16_dual_nvfp4_gemm_contiguous() got an unexpected keyword argument {key!r}")
    _require(a.dtype == torch.bfloat16, "a.dtype == bfloat16")
    _require(d.dtype == torch.bfloat16, "d.dtype == bfloat16")
    _require(b.dtype == torch.int8, "b.dtype == int8")
    _require(sfb.dtype == torch.int32, "sfb.dtype == int32")
    _require(gw.dtype == torch.float32, "gw.dtype == float32")
    _require(m_indices.dtype == torch.int32, "m_indices.dtype == int32")
    _require(a.dim() == 2 and d.dim() == 2, "a.dim() == 2 and d.dim() == 2")
    m, k = a.shape
    n = d.shape[1]
    e = gw.numel()
    _require(d.shape[0] == m, "d.size(0) == m")
    _require(m_indices.dim() == 1 and m_indices.shape[0] == m, "m_indices.size(0) == m")
    _require(b.dim() == 2 and b.shape[0] == e * n, "b.size(0) == num_groups * n")
    _require(b.shape[1] == k // 2, "b.size(1) == k / 2")
    _require(sfb.dim() == 2 and sfb.shape[0] == e * (k // 64), "sfb.size(0) == num_groups * (k / 64)")
    _require(sfb.shape[1] == n, "sfb.size(1) == n")
    for name, t in (("a", a), ("b", b), ("sfb", sfb), ("gw", gw), ("d", d), ("m_indices", m_indices)):
        _require(t.is_cuda, f"{name} is a CUDA tensor")
    dev = _one_device(a, b, sfb, gw, d, m_indices, device_status)
    _require(a.stride(1) == 1 and d.stride(1) == 1, "a and d are contiguous along their last dimension")
    _require(b.is_contiguous() and sfb.is_contiguous() and gw.is_contiguous() and m_indices.is_contiguous(),
             "b, sfb, gw, m_indices are contiguous")
    if scale_policy not in POLICY_CODES:
        raise RuntimeError("scale_policy must be 'derived_div8', 'derived_div4', 'div4_radix8' or 'residual_amax'")
    swap = int(tune.get("tune_swap_ab", 0)) != 0
    tune_arr = (ctypes.c_int32 * len(TUNE_KEYS))(*[int(tune.get(key, 0)) for key in TUNE_KEYS])
    lda = a.stride(0) if m > 1 else max(a.stride(0), k)
    ldd = d.stride(0) if m > 1 else max(d.stride(0), n)
    with torch.cuda.device(dev):
        _check(lib().nvfp4_grouped_gemm_contiguous(
            a.data_ptr(), lda, b.data_ptr(), sfb.data_ptr(), gw.data_ptr(), d.data_ptr(), ldd,
            m_indices.data_ptr(), m, n, k, e, POLICY_CODES[scale_policy], 1 if enable_residual_pass else 0,
            1 if swap else 0, int(m_alignment), ctypes.cast(tune_arr, ctypes.c_void_p),
            device_status.data_ptr() if device_status is not None else None, _stream()))


def m_grouped_bf16_dual_nvfp4_gemm_masked(a, b, sfb, gw, d, masked_m, scale_policy: str = "derived_div8",
                                          enable_residual_pass: bool = True, *, fold_swiglu: bool = False,
                                          device_status=None, **tune) -> None:
    """The same GEMM over the masked layout: ``a`` (E, max_m, K) and ``d`` (E, max_m, N) BF16 (last dimension
    contiguous, groups max_m rows apart), ``masked_m`` int32 (E,) on the device = real rows of each group.  With
    ``fold_swiglu`` ``a`` is the (E, max_m, 2 K) gate+up output and the activation is silu(gate) * up."""
    for key in tune:
        if key not in TUNE_KEYS:
            raise TypeError(f"m_grouped_bf16_dual_nvfp4_gemm_masked() got an unexpected keyword argument {key!r}")
    _require(a.dtype == torch.bfloat16 and d.dtype == torch.bfloat16, "a and d are bfloat16")
    _require(b.dtype == torch.int8 and sfb.dtype == torch.int32 and gw.dtype == torch.float32 and masked_m.dtype == torch.int32,
             "b int8, sfb int32, gw float32, masked_m int32")
    _require(a.dim() == 3 and d.dim() == 3 and a.shape[:2] == d.shape[:2], "a (E, max_m, K) and d (E, max_m, N)")
    e, max_m, ka = a.shape
    k = ka // 2 if fold_swiglu else ka
    n = d.shape[2]
    _require(gw.numel() == e and masked_m.numel() == e, "gw and masked_m have one entry per group")
    _require(b.shape == (e * n, k // 2) and sfb.shape == (e * (k // 64), n), "weight shapes do not fit")
    dev = _one_device(a, b, sfb, gw, d, masked_m, device_status)
    _require(a.stride(2) == 1 and d.stride(2) == 1 and a.stride(0) == max_m * a.stride(1) and d.stride(0) == max_m * d.stride(1),
             "a and d: last dimension contiguous, groups max_m rows apart")
    _require(b.is_contiguous() and sfb.is_contiguous() and gw.is_contiguous() and masked_m.is_contiguous(),
             "b, sfb, gw, masked_m are contiguous")
    if scale_policy not in POLICY_CODES:
        raise RuntimeError("scale_policy must be 'derived_div8', 'derived_div4', 'div4_radix8' or 'residual_amax'")
    tune_arr = (ctypes.c_int32 * len(TUNE_KEYS))(*[int(tune.get(key, 0)) for key in TUNE_KEYS])
    with torch.cuda.device(dev):
        _check(lib().nvfp4_grouped_gemm_masked(
            a.data_ptr(), a.stride(1), b.data_ptr(), sfb.data_ptr(), gw.data_ptr(), d.data_ptr(), d.stride(1),
            masked_m.data_ptr(), e, max_m, n, k, POLICY_CODES[scale_policy], 1 if enable_residual_pass else 0,
            1 if fold_swiglu else 0, ctypes.cast(tune_arr, ctypes.c_void_p),
            device_status.data_ptr() if device_status is not None else None, _stream()))


def load_checkpoint_weights(parts, global_scale_is_divisor: bool = True):
    """NVFP4 checkpoint tensors -> (b, sfb, gw).  ``parts`` lists the projections to fuse along N, in order, each as
    (weight_packed uint8 (E, rows, K/2), weight_scale float8_e4m3fn or uint8 (E, rows, K/16), weight_global_scale
    float32 (E,) or (E, 1)); gate and up of one expert MLP make a fused gate+up projection, a down projection is a
    single part.  Runs on the GPU (nvfp4_load_checkpoint_weights); see the header for the re-folding rule."""
    _require(1 <= len(parts) <= 4, "between one and four parts")
    packed, scale, glob = [], [], []
    for wp, ws, wg in parts:
        _require(wp.dim() == 3 and ws.dim() == 3 and wp.dtype in (torch.uint8, torch.int8), "weight_packed is (E, rows, K/2) bytes")
        if ws.dtype != torch.uint8:
            _require(ws.dtype == torch.float8_e4m3fn, "weight_scale is float8_e4m3fn or uint8")
            ws = ws.view(torch.uint8)
        packed.append(wp.contiguous())
        scale.append(ws.contiguous())
        glob.append(wg.reshape(-1).to(torch.float32).contiguous())
    e, _, k2 = packed[0].shape
    k = 2 * k2
    for wp, ws, wg in zip(packed, scale, glob):
        _require(wp.shape[0] == e and wp.shape[2] == k2 and ws.shape == (e, wp.shape[1], k // 16) and wg.numel() == e,
                 "parts disagree on E / K, or a scale tensor does not fit its codes")
    if k % 64 != 0:
        raise ValueError(f"K={k} must be a multiple of 64")
    dev = _one_device(*packed, *scale, *glob)
    n = sum(wp.shape[1] for wp in packed)
    b = torch.empty(e * n, k // 2, dtype=torch.int8, device=dev)
    sfb = torch.empty(e * k // 64, n, dtype=torch.int32, device=dev)
    gw = torch.empty(e, dtype=torch.float32, device=dev)
    ptrs = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    rows = (ctypes.c_int32 * len(packed))(*[wp.shape[1] for wp in packed])
    with torch.cuda.device(dev):
        _check(lib().nvfp4_load_checkpoint_weights(len(packed), ctypes.cast(ptrs(packed), ctypes.c_void_p),
                                                   ctypes.cast(ptrs(scale), ctypes.c_void_p), ctypes.cast(ptrs(glob), ctypes.c_void_p),
                                                   ctypes.cast(rows, ctypes.c_void_p), 1 if global_scale_is_divisor else 0, e, k,
                                                   b.data_ptr(), sfb.data_ptr(), gw.data_ptr(), _stream()))
    return b, sfb, gw


def read_status(device_status: torch.Tensor) -> int:
    """Reads and clears a kernel status word (synchronises the current stream); raises RuntimeError carrying
    NVFP4_E_DEVICE_TIMEOUT if a bounded in-kernel wait had expired, else returns 0."""
    _require(device_status.is_cuda and device_status.dtype == torch.int32 and device_status.numel() >= 1, "an int32 CUDA tensor")
    value = ctypes.c_int32(0)
    with torch.cuda.device(device_status.device):
        _check(lib().nvfp4_read_status(device_status.data_ptr(), ctypes.byref(value), _stream()))
    return value.value


def debug_wait_timeout(budget_cycles: int, device_status: torch.Tensor) -> None:
    """Launches the kernel whose bounded wait runs out (test hook of the unwind path)."""
    with torch.cuda.device(device_status.device):
        _check(lib().nvfp4_debug_wait_timeout(int(budget_cycles), device_status.data_ptr(), _stream()))


def debug_split_workspace(a: torch.Tensor, scale_policy: str = "derived_div8", enable_residual_pass: bool = True,
                          fold_swiglu: bool = False):
    """The split path's activation-quantisation kernel alone: returns (a0, a1, sfa) as uint8 CUDA tensors, a0 / a1
    (M, K/2) packed codes and sfa (M/128, K/64, passes, 512) scale atoms -- exactly what the GEMM kernel reads."""
    _require(a.is_cuda and a.dtype == torch.bfloat16 and a.dim() == 2 and a.stride(1) == 1, "a is a 2-D BF16 CUDA tensor")
    m, ka = a.shape
    k = ka // 2 if fold_swiglu else ka
    passes = 2 if enable_residual_pass else 1
    a0 = torch.zeros(m, k // 2, dtype=torch.uint8, device=a.device)
    a1 = torch.zeros_like(a0)
    sfa = torch.zeros(m // 128, k // 64, passes, 512, dtype=torch.uint8, device=a.device)
    with torch.cuda.device(a.device):
        _check(lib().nvfp4_debug_split_workspace(a.data_ptr(), a.stride(0), m, k, POLICY_CODES[scale_policy],
                                                 1 if enable_residual_pass else 0, 1 if fold_swiglu else 0,
                                                 a0.data_ptr(), a1.data_ptr(), sfa.data_ptr(), _stream()))
    return a0, a1, sfa


def quantize_weight(w: torch.Tensor):
    """CUDA tensor (E, N, K), BF16 or FP32 -> (b, sfb, gw) on the same device."""
    _require(w.is_cuda, "w is a CUDA tensor")
    if w.dtype not in (torch.bfloat16, torch.float32):
        w = w.to(torch.float32)
    w = w.contiguous()
    e, n, k = w.shape
    b = torch.empty(e * n, k // 2, dtype=torch.int8, device=w.device)
    sfb = torch.empty(e * k // 64, n, dtype=torch.int32, device=w.device)
    gw = torch.empty(e, dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        _check(lib().nvfp4_quantize_weight(w.data_ptr(), 0 if w.dtype == torch.bfloat16 else 1, e, n, k,
                                           b.data_ptr(), sfb.data_ptr(), gw.data_ptr(), _stream()))
    return b, sfb, gw


def _rows_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1


def permute_rows(src: torch.Tensor, n_rows: int, dst: torch.Tensor, src_idx: torch.Tensor = None, src_div: int = 1,
                 dst_idx: torch.Tensor = None) -> None:
    """dst[dst_idx[i] or i] = src[(src_idx[i] or i) // src_div] for i < n_rows (BF16 rows, int64 indices)."""
    _require(_rows_ok(src) and _rows_ok(dst) and src.shape[1] == dst.shape[1], "src and dst are 2-D BF16 CUDA tensors of one width")
    for idx in (src_idx, dst_idx):
        _require(idx is None or (idx.is_cuda and idx.dtype == torch.int64 and idx.is_contiguous() and idx.numel() >= n_rows),
                 "indices are contiguous int64 CUDA tensors with at least n_rows entries")
    with torch.cuda.device(_one_device(src, dst, src_idx, dst_idx)):
        _check(lib().nvfp4_permute_rows(src.data_ptr(), src.stride(0) * 2, src_idx.data_ptr() if src_idx is not None else None,
                                        src_div, dst_idx.data_ptr() if dst_idx is not None else None, n_rows, src.shape[1] * 2,
                                        dst.data_ptr(), dst.stride(0) * 2, _stream()))


def swiglu(h: torch.Tensor) -> torch.Tensor:
    """silu(h[:, :I]) * h[:, I:] for a (rows, 2 I) BF16 CUDA tensor."""
    _require(_rows_ok(h) and h.shape[1] % 16 == 0, "h is a 2-D BF16 CUDA tensor whose width is a multiple of 16")
    inter = h.shape[1] // 2
    out = torch.empty(h.shape[0], inter, dtype=torch.bfloat16, device=h.device)
    with torch.cuda.device(_one_device(h)):
        _check(lib().nvfp4_swiglu(h.data_ptr(), h.stride(0), h.shape[0], inter, out.data_ptr(), out.stride(0), _stream()))
    return out


def combine_rows(rows: torch.Tensor, pos: torch.Tensor, w: torch.Tensor, tokens: int) -> torch.Tensor:
    """y[t] = sum_j w[t, j] * rows[pos[t, j]] (FP32 accumulation, ascending j), BF16 out."""
    _require(_rows_ok(rows), "rows is a 2-D BF16 CUDA tensor")
    _require(pos.is_cuda and pos.dtype == torch.int64 and pos.is_contiguous() and w.is_cuda and w.dtype == torch.float32 and
             w.is_contiguous() and pos.numel() == w.numel() and pos.numel() % max(tokens, 1) == 0,
             "pos (int64) and w (float32) are contiguous CUDA tensors of tokens * k entries")
    y = torch.empty(tokens, rows.shape[1], dtype=torch.bfloat16, device=rows.device)
    k = pos.numel() // tokens if tokens else 1
    with torch.cuda.device(_one_device(rows, pos, w)):
        _check(lib().nvfp4_combine_rows(rows.data_ptr(), rows.stride(0), pos.data_ptr(), w.data_ptr(), tokens, k, rows.shape[1],
                                        y.data_ptr(), y.stride(0), _stream()))
    return y


def _i64_ok(t: torch.Tensor, n: int) -> bool:
    return t.is_cuda and t.dtype == torch.int64 and t.is_contiguous() and t.numel() >= n


def m_grouped_swiglu_dual_nvfp4_gemm_contiguous(h, b, sfb, gw, d, m_indices, enable_residual_pass: bool = True,
                                                device_status=None) -> None:
    """d = Q(silu(h[:, :K]) * h[:, K:]) @ W^T * gw[expert]: the down-projection of a SwiGLU expert MLP with the
    activation folded into the activation-quantisation kernel (normal orientation, N % 256 == 0)."""
    _require(_rows_ok(h) and _rows_ok(d) and h.shape[1] % 2 == 0, "h and d are 2-D BF16 CUDA tensors")
    m, k = h.shape[0], h.shape[1] // 2
    n, e = d.shape[1], gw.numel()
    _require(d.shape[0] == m and b.shape == (e * n, k // 2) and sfb.shape == (e * (k // 64), n) and m_indices.numel() == m,
             "operand shapes do not fit together")
    _require(b.is_contiguous() and sfb.is_contiguous() and gw.is_contiguous() and m_indices.is_contiguous(),
             "b, sfb, gw and m_indices are contiguous")
    with torch.cuda.device(_one_device(h, b, sfb, gw, d, m_indices, device_status)):
        _check(lib().nvfp4_grouped_gemm_swiglu_contiguous(
            h.data_ptr(), h.stride(0), b.data_ptr(), sfb.data_ptr(), gw.data_ptr(), d.data_ptr(), d.stride(0),
            m_indices.data_ptr(), m, n, k, e, 1 if enable_residual_pass else 0, None,
            device_status.data_ptr() if device_status is not None else None, _stream()))


def expert_histogram(ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """counts[e] = number of entries of ids equal to e (int64 CUDA tensors)."""
    _require(_i64_ok(ids, ids.numel()), "ids is a contiguous int64 CUDA tensor")
    counts = torch.empty(num_experts, dtype=torch.int64, device=ids.device)
    with torch.cuda.device(_one_device(ids)):
        _check(lib().nvfp4_expert_histogram(ids.data_ptr(), ids.numel(), num_experts, counts.data_ptr(), _stream()))
    return counts


def plan_peer_masked(all_counts: torch.Tensor, ids: torch.Tensor, world: int, rank: int, cap_m: int, status: torch.Tensor):
    """Routing plan for the masked layout; returns (masked_m int32 (E / world,), dst_row int64 (pairs,)), all on the
    device.  Overflow of an expert's capacity sets bit 2 of ``status``."""
    num_experts = all_counts.numel() // world
    _require(_i64_ok(all_counts, world * num_experts) and _i64_ok(ids, ids.numel()), "counts and ids are contiguous int64 CUDA tensors")
    dev = _one_device(all_counts, ids, status)
    base = torch.empty(num_experts, dtype=torch.int64, device=dev)
    limit = torch.empty(num_experts, dtype=torch.int64, device=dev)
    masked_m = torch.empty(num_experts // world, dtype=torch.int32, device=dev)
    dst_row = torch.empty(ids.numel(), dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        _check(lib().nvfp4_plan_peer_masked(all_counts.data_ptr(), world, num_experts, rank, cap_m, ids.data_ptr(), ids.numel(),
                                            base.data_ptr(), limit.data_ptr(), masked_m.data_ptr(), dst_row.data_ptr(),
                                            status.data_ptr(), _stream()))
    return masked_m, dst_row


def peer_barrier(flag_peers: torch.Tensor, rank: int, world: int, slot: int, epoch: int, status: torch.Tensor,
                 budget_cycles: int = 2_000_000_000) -> None:
    """Bounded barrier over the ranks whose flag arrays ``flag_peers`` lists (see the header)."""
    with torch.cuda.device(_one_device(flag_peers, status)):
        _check(lib().nvfp4_peer_barrier(flag_peers.data_ptr(), rank, world, slot, epoch, budget_cycles, status.data_ptr(), _stream()))


def dispatch_rows_peer(src: torch.Tensor, src_idx, src_div: int, peers: torch.Tensor, dst_rank: torch.Tensor,
                       dst_row: torch.Tensor, dst_ld_elems: int, rows_cap: int, status: torch.Tensor = None, sm_budget: int = 0) -> None:
    """Row src[(src_idx[i] or i) // src_div] -> row dst_row[i] of rank dst_rank[i]'s buffer (`peers`: int64 base
    addresses, `rows_cap` rows each); pairs out of range are skipped."""
    n = dst_row.numel()
    _require(_rows_ok(src), "src is a 2-D BF16 CUDA tensor")
    _require((src_idx is None or _i64_ok(src_idx, n)) and _i64_ok(dst_rank, n) and _i64_ok(dst_row, n) and _i64_ok(peers, 1),
             "indices and peer addresses are contiguous int64 CUDA tensors")
    with torch.cuda.device(_one_device(src, src_idx, peers, dst_rank, dst_row, status)):
        _check(lib().nvfp4_dispatch_rows_peer(src.data_ptr(), src.stride(0) * 2, src_idx.data_ptr() if src_idx is not None else None,
                                              src_div, peers.data_ptr(), dst_rank.data_ptr(), dst_row.data_ptr(), n, src.shape[1] * 2,
                                              dst_ld_elems * 2, peers.numel(), rows_cap, int(sm_budget),
                                              status.data_ptr() if status is not None else None, _stream()))


class QuantizedRows:
    """The three planes of a buffer of quantised activation rows, (E, max_m) rows of K elements, in one uint8 tensor
    `store` of E * max_m * (K + K // 8) bytes: packed codes of the first pass, of the residual pass, block scales
    (rows, 2, K // 16) -- the layout nvfp4_dispatch_quantized_peer writes -- plus a local tensor of scale atoms."""

    def __init__(self, store: torch.Tensor, e: int, max_m: int, k: int):
        rows = e * max_m
        _require(store.dtype == torch.uint8 and store.is_contiguous() and store.numel() == rows * (k + k // 8),
                 "store is a contiguous uint8 tensor of E * max_m * (K + K / 8) bytes")
        self.store, self.e, self.max_m, self.k = store, e, max_m, k
        self.a1_offset, self.scale_offset = rows * (k // 2), rows * k
        self.a0 = store[:self.a1_offset].view(rows, k // 2)
        self.a1 = store[self.a1_offset:self.scale_offset].view(rows, k // 2)
        self.scale_rows = store[self.scale_offset:].view(rows, 2, k // 16)
        self.scale_atoms = torch.zeros(rows // 128, k // 64, 2, 512, dtype=torch.uint8, device=store.device)


def dispatch_quantized_peer(x: torch.Tensor, k_choices: int, peers: torch.Tensor, dst_rank: torch.Tensor, dst_row: torch.Tensor,
                            rows: "QuantizedRows", status: torch.Tensor = None, sm_budget: int = 0) -> None:
    """Every token row of x, decomposed once, -> the quantised buffers (planes as in `rows`) of the ranks in `peers`."""
    n = dst_row.numel()
    _require(_rows_ok(x) and x.shape[1] == rows.k, "x is a (tokens, K) BF16 CUDA tensor")
    _require(_i64_ok(dst_rank, n) and _i64_ok(dst_row, n) and _i64_ok(peers, 1) and n == x.shape[0] * k_choices,
             "indices and peer addresses are contiguous int64 CUDA tensors, one entry per (token, choice)")
    with torch.cuda.device(_one_device(x, peers, dst_rank, dst_row, status)):
        _check(lib().nvfp4_dispatch_quantized_peer(x.data_ptr(), x.stride(0), x.shape[0], int(k_choices), rows.k, peers.data_ptr(),
                                                   rows.a1_offset, rows.scale_offset, dst_rank.data_ptr(), dst_row.data_ptr(),
                                                   peers.numel(), rows.e * rows.max_m, int(sm_budget),
                                                   status.data_ptr() if status is not None else None, _stream()))


def relayout_scales(rows: "QuantizedRows", masked_m: torch.Tensor = None) -> None:
    """rows.scale_rows -> rows.scale_atoms for the live row blocks of every group."""
    with torch.cuda.device(_one_device(rows.store, rows.scale_atoms, masked_m)):
        _check(lib().nvfp4_relayout_scales(rows.scale_rows.data_ptr(), masked_m.data_ptr() if masked_m is not None else None,
                                           rows.e, rows.max_m, rows.k, rows.scale_atoms.data_ptr(), _stream()))


def m_grouped_quantized_dual_nvfp4_gemm_masked(rows: "QuantizedRows", b, sfb, gw, d, masked_m, enable_residual_pass: bool = True,
                                               *, device_status=None, **tune) -> None:
    """The masked GEMM over activations that are already quantised (`rows` after relayout_scales)."""
    for key in tune:
        if key not in TUNE_KEYS:
            raise TypeError(f"m_grouped_quantized_dual_nvfp4_gemm_masked() got an unexpected keyword argument {key!r}")
    e, max_m, k = rows.e, rows.max_m, rows.k
    _require(d.dtype == torch.bfloat16 and d.dim() == 3 and d.shape[:2] == (e, max_m) and d.stride(2) == 1 and
             d.stride(0) == max_m * d.stride(1), "d is (E, max_m, N) BF16, last dimension contiguous, groups max_m rows apart")
    n = d.shape[2]
    _require(b.dtype == torch.int8 and sfb.dtype == torch.int32 and gw.dtype == torch.float32 and masked_m.dtype == torch.int32,
             "b int8, sfb int32, gw float32, masked_m int32")
    _require(gw.numel() == e and masked_m.numel() == e and b.shape == (e * n, k // 2) and sfb.shape == (e * (k // 64), n),
             "weight shapes do not fit")
    _require(b.is_contiguous() and sfb.is_contiguous() and gw.is_contiguous() and masked_m.is_contiguous(),
             "b, sfb, gw, masked_m are contiguous")
    tune_arr = (ctypes.c_int32 * len(TUNE_KEYS))(*[int(tune.get(key, 0)) for key in TUNE_KEYS])
    with torch.cuda.device(_one_device(rows.store, rows.scale_atoms, b, sfb, gw, d, masked_m, device_status)):
        _check(lib().nvfp4_grouped_gemm_masked_quantized(
            rows.a0.data_ptr(), rows.a1.data_ptr(), rows.scale_atoms.data_ptr(), b.data_ptr(), sfb.data_ptr(), gw.data_ptr(),
            d.data_ptr(), d.stride(1), masked_m.data_ptr(), e, max_m, n, k, 1 if enable_residual_pass else 0,
            ctypes.cast(tune_arr, ctypes.c_void_p), device_status.data_ptr() if device_status is not None else None, _stream()))


def interleave_gate_up(b: torch.Tensor, sfb: torch.Tensor, num_experts: int, inter: int):
    """Weights of a fused gate+up projection, (E * 2 I, K / 2) codes and (E * K / 64, 2 I) scale words, with their rows
    re-ordered for m_grouped_quantized_swiglu_dual_nvfp4_gemm_masked: runs of 32 gate rows followed by the 32 matching
    up rows, so that every 256-row tile holds 128 (gate, up) pairs.  inter % 128 == 0."""
    _require(inter % 128 == 0 and b.shape[0] == num_experts * 2 * inter and sfb.shape[1] == 2 * inter, "shapes do not fit I % 128 == 0")
    new = torch.arange(2 * inter, device=b.device)
    t, g, hh, i = new // 256, (new // 64) % 4, (new // 32) % 2, new % 32
    orig = hh * inter + 128 * t + 32 * g + i
    b2 = b.reshape(num_experts, 2 * inter, -1)[:, orig].reshape(b.shape).contiguous()
    return b2, sfb[:, orig].contiguous()


def m_grouped_quantized_swiglu_dual_nvfp4_gemm_masked(rows: "QuantizedRows", b, sfb, gw, out: "QuantizedRows", masked_m, *,
                                                      device_status=None, **tune) -> None:
    """Up-projection over quantised activations `rows` (E, max_m, K) with gate/up-interleaved weights (interleave_gate_up);
    writes silu(gate) * up, quantised, into `out` (E, max_m, I): its code planes and scale atoms, ready for
    m_grouped_quantized_dual_nvfp4_gemm_masked with the down-projection's weights."""
    for key in tune:
        if key not in TUNE_KEYS:
            raise TypeError(f"m_grouped_quantized_swiglu_dual_nvfp4_gemm_masked() got an unexpected keyword argument {key!r}")
    e, max_m, k = rows.e, rows.max_m, rows.k
    n = 2 * out.k
    _require(out.e == e and out.max_m == max_m and out.k % 128 == 0, "out is (E, max_m, I) with I % 128 == 0")
    _require(b.dtype == torch.int8 and sfb.dtype == torch.int32 and gw.dtype == torch.float32 and masked_m.dtype == torch.int32,
             "b int8, sfb int32, gw float32, masked_m int32")
    _require(gw.numel() == e and masked_m.numel() == e and b.shape == (e * n, k // 2) and sfb.shape == (e * (k // 64), n),
             "weight shapes do not fit")
    _require(b.is_contiguous() and sfb.is_contiguous() and gw.is_contiguous() and masked_m.is_contiguous(),
             "b, sfb, gw, masked_m are contiguous")
    tune_arr = (ctypes.c_int32 * len(TUNE_KEYS))(*[int(tune.get(key, 0)) for key in TUNE_KEYS])
    with torch.cuda.device(_one_device(rows.store, rows.scale_atoms, out.store, out.scale_atoms, b, sfb, gw, masked_m, device_status)):
        _check(lib().nvfp4_grouped_gemm_masked_quantized_swiglu(
            rows.a0.data_ptr(), rows.a1.data_ptr(), rows.scale_atoms.data_ptr(), b.data_ptr(), sfb.data_ptr(), gw.data_ptr(),
            out.a0.data_ptr(), out.a1.data_ptr(), out.scale_atoms.data_ptr(), masked_m.data_ptr(), e, max_m, n, k,
            ctypes.cast(tune_arr, ctypes.c_void_p), device_status.data_ptr() if device_status is not None else None, _stream()))


def combine_rows_peer(peers: torch.Tensor, rows_ld_elems: int, src_rank: torch.Tensor, src_row: torch.Tensor, w: torch.Tensor,
                      tokens: int, hidden: int, rows_cap: int, out: torch.Tensor = None, sm_budget: int = 0, bulk: bool = True,
                      status: torch.Tensor = None) -> torch.Tensor:
    """y[t] = sum_j w[t, j] * (row src_row[t, j] of rank src_rank[t, j]'s buffer), BF16, into `out` if given.  `bulk`:
    rows fetched by bulk copies into shared memory (a few SMs saturate NVLink) instead of per-thread loads."""
    n = src_rank.numel()
    _require(_i64_ok(src_rank, n) and _i64_ok(src_row, n) and _i64_ok(peers, 1) and w.is_cuda and w.dtype == torch.float32 and
             w.is_contiguous() and w.numel() == n and n % max(tokens, 1) == 0, "bad index / weight tensors")
    _require(out is None or (_rows_ok(out) and out.shape == (tokens, hidden)), "out is a (tokens, hidden) BF16 CUDA tensor")
    y = out if out is not None else torch.empty(tokens, hidden, dtype=torch.bfloat16, device=w.device)
    k = n // tokens if tokens else 1
    with torch.cuda.device(_one_device(peers, src_rank, src_row, w, status)):
        _check(lib().nvfp4_combine_rows_peer(peers.data_ptr(), rows_ld_elems, src_rank.data_ptr(), src_row.data_ptr(), w.data_ptr(),
                                             tokens, k, hidden, y.data_ptr(), y.stride(0), peers.numel(), rows_cap, int(sm_budget),
                                             1 if bulk else 0, status.data_ptr() if status is not None else None, _stream()))
    return y


def debug_decompose(a: torch.Tensor, scale_policy: str = "derived_div8"):
    """Algorithm 1 as the GEMM's transform warps run it; returns packed q0, q1 (M, K/2)
    and s0, s1 (M, K/16) as uint8 CUDA tensors.  Test hook."""
    _require(a.is_cuda and a.dtype == torch.bfloat16 and a.dim() == 2 and a.stride(1) == 1, "a is a 2-D BF16 CUDA tensor")
    m, k = a.shape
    q0 = torch.empty(m, k // 2, dtype=torch.uint8, device=a.device)
    q1 = torch.empty_like(q0)
    s0 = torch.empty(m, k // 16, dtype=torch.uint8, device=a.device)
    s1 = torch.empty_like(s0)
    with torch.cuda.device(_one_device(a)):
        _check(lib().nvfp4_debug_decompose(a.data_ptr(), a.stride(0), m, k, POLICY_CODES[scale_policy],
                                           q0.data_ptr(), q1.data_ptr(), s0.data_ptr(), s1.data_ptr(), _stream()))
    return q0, q1, s0, s1


def debug_mma_peak(iters: int) -> float:
    """Launches the resident-operand FP4 MMA loop once; returns the FLOPs of the launch."""
    flops = ctypes.c_double(0.0)
    _check(lib().nvfp4_debug_mma_peak(int(iters), ctypes.byref(flops), _stream()))
    return flops.value


def debug_mma_peak_pair(iters: int) -> float:
    """Launch the CTA-pair (cta_group::2) resident-operand MMA loop; returns the FLOPs of the launch."""
    flops = ctypes.c_double(0.0)
    _check(lib().nvfp4_debug_mma_peak_pair(int(iters), ctypes.byref(flops), _stream()))
    return flops.value


def debug_mma_pattern(iters: int, num_cp: int, num_mma: int, mma_n: int, alt_cols: int = 0) -> float:
    """One launch of the copy + MMA issue pattern study; returns the FLOPs of the launch."""
    flops = ctypes.c_double(0.0)
    _check(lib().nvfp4_debug_mma_pattern(int(iters), int(num_cp), int(num_mma), int(mma_n), int(alt_cols),
                                         ctypes.byref(flops), _stream()))
    return flops.value
