"""TEST INFRASTRUCTURE -- ctypes front end of the CPU oracle (not product code).

Only the tests, the smoke test and the benchmark's CPU-baseline leg import this
package.  It loads ``oracle/liboracle.so`` (the C restatement of the reference's
PyTorch emulation, see ``dual_nvfp4_oracle.c``) and, if present,
``oracle/_ref/libref_twin.so`` (the reference's own C++ host twin compiled
unmodified from its header) and ``oracle/_ref/ref_dual_nvfp4.py`` (a build-time copy
of the reference's PyTorch emulation, the CPU baseline the benchmark times).
Tensors in and out are CPU torch tensors.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_twin.so")

POLICIES = {"derived_div8": 0, "residual_amax": 1, "derived_div4": 2, "div4_radix8": 3}
E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference twin when the reference is mounted)."""
    src = os.path.join(_HERE, "dual_nvfp4_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "liboracle.so", "-B"], check=True, capture_output=True)
    subprocess.run(["make", "-C", _HERE, "ref", "ref_py"], check=True, capture_output=True)


_lib = None
_ref = None
_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_quantize_weight.restype = _i32
        _lib.orc_decompose.restype = _i32
        _lib.orc_grouped_gemm.restype = _i32
        _lib.orc_num_threads.restype = _i32
    return _lib


def ref_twin() -> ctypes.CDLL | None:
    """The reference's C++ twin, or None when it was never built."""
    global _ref
    if _ref is None and os.path.exists(_REF_PATH):
        _ref = ctypes.CDLL(_REF_PATH)
    return _ref


_emu = None


def ref_emulation():
    """The reference's own PyTorch emulation module (decompose_dual_nvfp4, dual_nvfp4_grouped_gemm, ...), loaded from
    the build-time copy in oracle/_ref/, or None when that copy was never made."""
    global _emu
    path = os.path.join(_HERE, "_ref", "ref_dual_nvfp4.py")
    if _emu is None and os.path.exists(path):
        import importlib.util
        import sys
        spec = importlib.util.spec_from_file_location("ref_dual_nvfp4", path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules["ref_dual_nvfp4"] = mod          # its dataclasses look their module up by name
        spec.loader.exec_module(mod)
        _emu = mod
    return _emu


def num_threads() -> int:
    return int(lib().orc_num_threads())


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _cpu(t: torch.Tensor, dtype=None) -> torch.Tensor:
    t = t.detach().cpu()
    if dtype is not None:
        t = t.to(dtype)
    return t.contiguous()


def e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    x = _cpu(x, torch.float32)
    out = torch.empty(x.shape, dtype=torch.uint8)
    lib().orc_e2m1_codes(_ptr(x), _ptr(out), _i64(x.numel()))
    return out


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    codes = _cpu(codes, torch.uint8)
    out = torch.empty(codes.shape, dtype=torch.float32)
    lib().orc_e2m1_decode(_ptr(codes), _ptr(out), _i64(codes.numel()))
    return out


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    x = _cpu(x, torch.float32)
    out = torch.empty(x.shape, dtype=torch.uint8)
    lib().orc_e4m3_encode(_ptr(x), _ptr(out), _i64(x.numel()))
    return out


def e4m3_decode(codes: torch.Tensor) -> torch.Tensor:
    codes = _cpu(codes, torch.uint8)
    out = torch.empty(codes.shape, dtype=torch.float32)
    lib().orc_e4m3_decode(_ptr(codes), _ptr(out), _i64(codes.numel()))
    return out


def quantize_weight(w: torch.Tensor):
    """(E, N, K) -> b int8 (E*N, K/2), sfb int32 (E*K/64, N), gw fp32 (E,)."""
    if w.dim() != 3:
        raise ValueError("expected weights shaped (E, N, K)")
    e, n, k = w.shape
    if k % 64 != 0:
        raise ValueError(f"K={k} must be a multiple of 64")
    w32 = _cpu(w, torch.float32)
    b = torch.empty(e * n, k // 2, dtype=torch.int8)
    sfb = torch.empty(e * k // 64, n, dtype=torch.int32)
    gw = torch.empty(e, dtype=torch.float32)
    rc = lib().orc_quantize_weight(_ptr(w32), e, n, k, _ptr(b), _ptr(sfb), _ptr(gw))
    assert rc == 0, rc
    return b, sfb, gw


def dequantize_weight(b, sfb, gw, num_experts: int, n: int, k: int) -> torch.Tensor:
    out = torch.empty(num_experts, n, k, dtype=torch.float32)
    lib().orc_dequantize_weight(_ptr(_cpu(b)), _ptr(_cpu(sfb)), _ptr(_cpu(gw, torch.float32)),
                                num_experts, n, k, _ptr(out))
    return out


def decompose(a: torch.Tensor, scale_policy: str = "derived_div8"):
    """Algorithm 1.  Returns (q0, q1) uint8 codes (M, K) and (s0, s1) E4M3 bytes (M, K/16)."""
    a = _cpu(a, torch.bfloat16)
    m, k = a.shape
    q0 = torch.empty(m, k, dtype=torch.uint8)
    q1 = torch.empty(m, k, dtype=torch.uint8)
    s0 = torch.empty(m, k // 16, dtype=torch.uint8)
    s1 = torch.empty(m, k // 16, dtype=torch.uint8)
    rc = lib().orc_decompose(_ptr(a.view(torch.int16)), _i64(m), _i64(k), _i64(k),
                             POLICIES[scale_policy], _ptr(q0), _ptr(q1), _ptr(s0), _ptr(s1))
    if rc != 0:
        raise ValueError(f"orc_decompose failed ({rc})")
    return q0, q1, s0, s1


def grouped_gemm(a, b, sfb, gw, m_indices, n: int, mode: str = "dual",
                 scale_policy: str = "derived_div8", n_range=None, want_f32: bool = False):
    """Algorithm 2 (mode 'dual' / 'single') or the FP32 ground truth (mode 'truth').

    Returns BF16 (M, N) for the two quantised modes, FP32 for 'truth' or when
    ``want_f32``.  ``n_range=(lo, hi)`` restricts the computed output columns.
    """
    a = _cpu(a, torch.bfloat16)
    m, k = a.shape
    e = gw.numel()
    mode_i = {"truth": 0, "single": 1, "dual": 2}[mode]
    lo, hi = n_range if n_range is not None else (0, n)
    f32 = want_f32 or mode == "truth"
    d = torch.zeros(m, n, dtype=torch.float32 if f32 else torch.bfloat16)
    rc = lib().orc_grouped_gemm(
        _ptr(a.view(torch.int16)), _i64(k), _ptr(_cpu(b)), _ptr(_cpu(sfb)),
        _ptr(_cpu(gw, torch.float32)), _ptr(_cpu(m_indices, torch.int32)), _i64(m), n, k, e,
        POLICIES[scale_policy], mode_i, lo, hi,
        None if f32 else _ptr(d.view(torch.int16)), _ptr(d) if f32 else None, _i64(n))
    if rc != 0:
        raise ValueError(f"orc_grouped_gemm failed ({rc})")
    return d


# ---- the reference's own C++ twin (present only when it was compiled) --------

def ref_twin_decompose(x: torch.Tensor):
    r = ref_twin()
    x = _cpu(x, torch.float32)
    m, k = x.shape
    q0 = torch.empty(m, k, dtype=torch.uint8)
    q1 = torch.empty(m, k, dtype=torch.uint8)
    s0 = torch.empty(m, k // 16, dtype=torch.uint8)
    s1 = torch.empty(m, k // 16, dtype=torch.uint8)
    rc = r.ref_twin_decompose(_ptr(x), _i64(m), _i64(k), _ptr(q0), _ptr(q1), _ptr(s0), _ptr(s1))
    assert rc == 0
    return q0, q1, s0, s1


def ref_twin_quantize_weight(w: torch.Tensor):
    r = ref_twin()
    w = _cpu(w, torch.float32)
    e, n, k = w.shape
    q = torch.empty(e, n, k, dtype=torch.uint8)
    sf = torch.empty(e, n, k // 16, dtype=torch.uint8)
    g = torch.empty(e, dtype=torch.float32)
    r.ref_twin_quantize_weight(_ptr(w), e, n, k, _ptr(q), _ptr(sf), _ptr(g))
    return q, sf, g


def ref_twin_dual_gemm(a, q, sf, g, expert_of_row, n: int) -> torch.Tensor:
    r = ref_twin()
    a = _cpu(a, torch.float32)
    m, k = a.shape
    out = torch.empty(m, n, dtype=torch.float32)
    r.ref_twin_dual_gemm(_ptr(a), _ptr(_cpu(q)), _ptr(_cpu(sf)), _ptr(_cpu(g, torch.float32)),
                         _ptr(_cpu(expert_of_row, torch.int32)), m, n, k, g.numel(), _ptr(out))
    return out


def ref_twin_dual_gemm_mt(a, q, sf, g, expert_of_row, n: int, threads: int) -> torch.Tensor:
    """ref::dual_gemm on every host thread (row chunks handed to independent calls)."""
    r = ref_twin()
    a = _cpu(a, torch.float32)
    m, k = a.shape
    out = torch.empty(m, n, dtype=torch.float32)
    r.ref_twin_dual_gemm_mt(_ptr(a), _ptr(_cpu(q)), _ptr(_cpu(sf)), _ptr(_cpu(g, torch.float32)),
                            _ptr(_cpu(expert_of_row, torch.int32)), m, n, k, g.numel(), _ptr(out), int(threads))
    return out
