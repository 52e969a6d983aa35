"""CPU: the host side of the drop-in surface -- layout helpers with the reference's
known answers (tests/python/test_layout.py there), argument checking, and that the
C-ABI library loads and exports every symbol include/nvfp4_b200.h declares."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT, bf16_from_bits, load_golden

import nvfp4_gemm
from nvfp4_gemm import layout


def test_public_surface():
    for name in ("m_grouped_bf16_dual_nvfp4_gemm_contiguous", "quantize_weight_nvfp4", "dequantize_weight_nvfp4",
                 "make_m_indices", "layout", "get_num_sms", "set_num_sms"):
        assert hasattr(nvfp4_gemm, name), name
    assert set(nvfp4_gemm.__all__) >= {"m_grouped_bf16_dual_nvfp4_gemm_contiguous", "quantize_weight_nvfp4"}


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    declared = set(re.findall(r"NVFP4_API\s+[\w\s\*]+?\b(nvfp4_\w+)\s*\(", header))
    assert declared and declared == set(nvfp4_gemm._C.EXPORTS)
    lib = ctypes.CDLL(nvfp4_gemm._C.library_path())          # loading needs no GPU
    for sym in declared:
        assert hasattr(lib, sym), sym
    lib.nvfp4_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.nvfp4_version()


def test_e2m1_codes_known_answers():
    # test_layout.py:33-46: codes incl. sign bit and ties
    x = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 100.0, -0.0])
    assert layout.quantize_e2m1_codes(x).tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 9, 15, 0, 2, 2, 4, 4, 6, 6, 7, 8]
    g = load_golden("e2m1.npz")
    assert torch.equal(layout.quantize_e2m1_codes(torch.from_numpy(g["x"])), torch.from_numpy(g["codes"]))


def test_nibble_order_and_scale_words():
    # test_layout.py:49-58 and :61-83
    assert (layout.pack_e2m1_pairs(torch.tensor([1, 2, 3, 4], dtype=torch.uint8)).view(torch.uint8).tolist()
            == [0x21, 0x43])
    with pytest.raises(ValueError):
        layout.pack_e2m1_pairs(torch.zeros(3, dtype=torch.uint8))
    s = torch.arange(2 * 3 * 8, dtype=torch.uint8).reshape(2, 3, 8)
    words = layout.pack_sf_atoms(s)
    assert words.shape == (2 * 2, 3) and words.dtype == torch.int32
    for e in range(2):
        for n in range(3):
            for at in range(2):
                w = int(words[e * 2 + at, n]) & 0xffffffff
                assert [(w >> (8 * j)) & 0xff for j in range(4)] == s[e, n, at * 4:at * 4 + 4].tolist()


def test_host_quantiser_matches_golden():
    g = load_golden("weights.npz")
    w = bf16_from_bits(g["w_bits"])
    b, sfb, gw = layout.quantize_weight_nvfp4(w)
    assert b.dtype == torch.int8 and sfb.dtype == torch.int32 and gw.dtype == torch.float32
    assert torch.equal(b, torch.from_numpy(g["b"]))
    assert torch.equal(sfb, torch.from_numpy(g["sfb"]))
    assert torch.equal(gw, torch.from_numpy(g["gw"]))
    assert torch.equal(layout.dequantize_weight_nvfp4(b, sfb, gw, 3, 64, 128), torch.from_numpy(g["deq"]))
    # round trip quality the reference reports (test_layout.py:86-114)
    torch.manual_seed(0)
    w = torch.randn(2, 128, 256)
    deq = layout.dequantize_weight_nvfp4(*layout.quantize_weight_nvfp4(w), 2, 128, 256)
    rel = float((deq - w).norm() / w.norm())
    cos = float(torch.dot(deq.flatten(), w.flatten()) / (deq.norm() * w.norm()))
    assert rel < 0.12 and cos > 0.995


def test_quantize_weight_errors():
    with pytest.raises(ValueError):
        layout.quantize_weight_nvfp4(torch.zeros(4, 64))
    with pytest.raises(ValueError):
        layout.quantize_weight_nvfp4(torch.zeros(1, 4, 96))


def test_make_m_indices():
    # test_layout.py:139-152
    out = layout.make_m_indices([128, 256, 0, 128])
    assert out.dtype == torch.int32 and out.shape == (512,)
    assert out[:128].eq(0).all() and out[128:384].eq(1).all() and out[384:].eq(3).all()
    with pytest.raises(ValueError):
        layout.make_m_indices([128, 100])
    assert layout.make_m_indices([32, 64], alignment=32).shape == (96,)
    assert layout.make_m_indices(torch.tensor([128])).tolist() == [0] * 128


def test_gemm_argument_checks_need_no_gpu():
    a = torch.zeros(128, 256, dtype=torch.bfloat16)
    d = torch.zeros(128, 128, dtype=torch.bfloat16)
    b = torch.zeros(128, 128, dtype=torch.int8)
    sfb = torch.zeros(4, 128, dtype=torch.int32)
    gw = torch.ones(1)
    mi = torch.zeros(128, dtype=torch.int32)
    f = nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous
    with pytest.raises(RuntimeError):                      # wrong dtype
        f(a.float(), b, sfb, gw, d, mi)
    with pytest.raises(RuntimeError):                      # wrong b shape
        f(a, b[:64], sfb, gw, d, mi)
    with pytest.raises(RuntimeError):                      # CPU tensors: no CPU path exists
        f(a, b, sfb, gw, d, mi)
    with pytest.raises(TypeError):
        f(a, b, sfb, gw, d, mi, tune_nonsense=1)
    with pytest.raises(RuntimeError):
        f(a, b, sfb, gw, d, mi, scale_policy="bogus")


def test_c_abi_validation_without_gpu():
    """Shape validation happens before any CUDA call, so the codes can be checked here."""
    lib = nvfp4_gemm._C.lib()
    rc = lib.nvfp4_grouped_gemm_contiguous(None, 0, None, None, None, None, 0, None, 128, 100, 256, 1, 0, 1, 0, 0,
                                           None, None, None)
    assert rc == 1 and b"multiples of 128" in lib.nvfp4_last_error()
    rc = lib.nvfp4_grouped_gemm_contiguous(None, 0, None, None, None, None, 0, None, 100, 128, 256, 1, 0, 1, 0, 0,
                                           None, None, None)
    assert rc == 1 and b"alignment" in lib.nvfp4_last_error()
    rc = lib.nvfp4_grouped_gemm_contiguous(None, 0, None, None, None, None, 0, None, 0, 128, 256, 1, 0, 1, 0, 0,
                                           None, None, None)
    assert rc == 0                                          # M == 0 returns silently
    assert lib.nvfp4_quantize_weight(None, 0, 1, 4, 96, None, None, None, None) == 1


def test_new_entry_points_validate_without_gpu():
    lib = nvfp4_gemm._C.lib()
    # masked layout: max_m must be a multiple of 128, N of 256
    rc = lib.nvfp4_grouped_gemm_masked(None, 0, None, None, None, None, 0, None, 4, 100, 256, 128, 0, 1, 0, None, None, None)
    assert rc == 1 and b"max_m" in lib.nvfp4_last_error()
    rc = lib.nvfp4_grouped_gemm_masked(None, 0, None, None, None, None, 0, None, 4, 128, 128, 128, 0, 1, 0, None, None, None)
    assert rc == 1 and b"256" in lib.nvfp4_last_error()
    assert lib.nvfp4_grouped_gemm_masked(None, 0, None, None, None, None, 0, None, 0, 128, 256, 128, 0, 1, 0, None, None, None) == 0
    # unknown scale policy is an argument error now that all four policies exist
    rc = lib.nvfp4_grouped_gemm_contiguous(ctypes.c_void_p(16), 256, ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16),
                                           ctypes.c_void_p(16), 128, ctypes.c_void_p(16), 128, 128, 256, 1, 7, 1, 0, 0, None, None, None)
    assert rc == 1 and b"scale policy" in lib.nvfp4_last_error()
    # checkpoint loader: part count and K
    assert lib.nvfp4_load_checkpoint_weights(0, None, None, None, None, 1, 1, 64, None, None, None, None) == 1
    assert lib.nvfp4_load_checkpoint_weights(9, None, None, None, None, 1, 1, 64, None, None, None, None) == 1
    assert lib.nvfp4_read_status(None, None, None) == 1
    assert lib.nvfp4_debug_wait_timeout(0, None, None) == 1
    # normal orientation: alignment 128, or 256 as the caller's statement of whole row pairs; nothing else
    rc = lib.nvfp4_grouped_gemm_contiguous(None, 0, None, None, None, None, 0, None, 384, 256, 128, 1, 0, 1, 0, 256, None, None, None)
    assert rc == 1 and b"multiple of the token-tile alignment" in lib.nvfp4_last_error()
    rc = lib.nvfp4_grouped_gemm_contiguous(None, 0, None, None, None, None, 0, None, 384, 256, 128, 1, 0, 1, 0, 64, None, None, None)
    assert rc == 1 and b"128 or 256" in lib.nvfp4_last_error()
    # quantised dispatch: K in steps of 1024 up to 8192; planes must not overlap
    rc = lib.nvfp4_dispatch_quantized_peer(None, 0, 4, 2, 1536, None, 0, 0, None, None, 1, 128, 0, None, None)
    assert rc == 1 and b"1024" in lib.nvfp4_last_error()
    rc = lib.nvfp4_dispatch_quantized_peer(ctypes.c_void_p(16), 1024, 4, 2, 1024, ctypes.c_void_p(16), 100, 200, ctypes.c_void_p(16),
                                           ctypes.c_void_p(16), 1, 128, 0, None, None)
    assert rc == 1 and b"planes" in lib.nvfp4_last_error()
    assert lib.nvfp4_dispatch_quantized_peer(None, 0, 0, 2, 1024, None, 0, 0, None, None, 1, 128, 0, None, None) == 0   # no tokens
    rc = lib.nvfp4_relayout_scales(None, None, 2, 100, 1024, None, None)
    assert rc == 1 and b"max_m" in lib.nvfp4_last_error()
    rc = lib.nvfp4_grouped_gemm_masked_quantized(None, None, None, None, None, None, None, 0, None, 2, 128, 128, 128, 1, None, None, None)
    assert rc == 1 and b"256" in lib.nvfp4_last_error()
    assert lib.nvfp4_grouped_gemm_masked_quantized(None, None, None, None, None, None, None, 0, None, 0, 128, 256, 128, 1, None, None, None) == 0
    assert lib.nvfp4_debug_mma_peak_pair(0, None, None) == 1


def test_operands_must_share_one_device():
    """The wrappers launch on the device that holds the operands; tensors spread over devices are refused before any
    pointer reaches the library (checked here with stand-ins that only carry what the check reads)."""
    from unittest import mock
    from nvfp4_gemm import _C

    def fake(index):
        t = mock.MagicMock(spec=torch.Tensor)
        t.is_cuda = True
        t.device = torch.device("cuda", index)
        return t

    assert _C._one_device(fake(1), None, fake(1)) == torch.device("cuda", 1)
    with pytest.raises(RuntimeError, match="one device"):
        _C._one_device(fake(0), fake(1))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _C._one_device(torch.zeros(1))


def test_oracle_radix_policies_follow_the_kernel_constants(oracle):
    """derived_div4 and div4_radix8 exist only in the reference's kernel (include/nvfp4_gemm/transform/dual_nvfp4.cuh:31-61
    there); the oracle states them in the emulation's operation order.  Known answers by hand for one block."""
    x = torch.zeros(1, 16)
    x[0, :4] = torch.tensor([6.0, 2.75, -0.3125, 1.0])
    q0, q1, s0, s1 = oracle.decompose(x.to(torch.bfloat16), "derived_div4")
    # amax 6 -> s0 = 1 (0x38), s1 = Q(1/4) = 0x28; u = x: q0 = {6, 3 (2.75 -> 3), -0.5 (0.3125 -> 0.5), 1}
    assert s0[0, 0] == 0x38 and s1[0, 0] == 0x28
    assert oracle.e2m1_decode(q0[0, :4]).tolist() == [6.0, 3.0, -0.5, 1.0]
    # residual x4: (2.75 - 3) * 4 = -1 ; (-0.3125 + 0.5) * 4 = 0.75 -> tie to 1.0
    assert oracle.e2m1_decode(q1[0, :4]).tolist() == [0.0, -1.0, 1.0, 0.0]
    q0, q1, s0, s1 = oracle.decompose(x.to(torch.bfloat16), "div4_radix8")
    # s0 = Q(6 / 4) = 1.5 (0x3c), s1 = Q(1.5 / 8) = 0.1875 (0x24); u = x / 1.5 = {4, 1.8333, -0.20833, 0.6667}
    assert s0[0, 0] == 0x3c and s1[0, 0] == 0x24
    assert oracle.e2m1_decode(q0[0, :4]).tolist() == [4.0, 2.0, -0.0, 0.5]
    # residual x8: (1.8333 - 2) * 8 = -1.333 -> -1.5 ; -0.20833 * 8 = -1.667 -> -1.5 ; (0.6667 - 0.5) * 8 = 1.333 -> 1.5
    assert oracle.e2m1_decode(q1[0, :4]).tolist() == [0.0, -1.5, -1.5, 1.5]
    # both give a usable reconstruction on Gaussian data
    g = torch.Generator().manual_seed(0)
    a = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    for policy in ("derived_div4", "div4_radix8"):
        q0, q1, s0, s1 = oracle.decompose(a, policy)
        rec = (oracle.e2m1_decode(q0) * oracle.e4m3_decode(s0).repeat_interleave(16, dim=1) +
               oracle.e2m1_decode(q1) * oracle.e4m3_decode(s1).repeat_interleave(16, dim=1))
        assert float((rec - a.float()).norm() / a.float().norm()) < 0.02


def test_checkpoint_restatement_single_part_is_identity(oracle):
    from oracle import checkpoint
    g = torch.Generator().manual_seed(1)
    e, n, k = 2, 64, 128
    w = (torch.randn(e, n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = oracle.quantize_weight(w)
    part = (b.view(torch.uint8).reshape(e, n, k // 2), layout.unpack_sf_atoms(sfb, e), gw)
    assert torch.equal(layout.pack_sf_atoms(layout.unpack_sf_atoms(sfb, e)), sfb)
    ob, osfb, ogw = checkpoint.load_checkpoint_weights([part], global_scale_is_divisor=False)
    assert torch.equal(ob, b) and torch.equal(osfb, sfb) and torch.equal(ogw, gw)
    with pytest.raises(RuntimeError):                      # the loader itself is GPU-only: no CPU path
        nvfp4_gemm.load_checkpoint_weights_nvfp4([part])


def test_gate_up_interleave_puts_every_pair_in_one_64_column_group():
    """The row order the fused up-projection epilogue relies on: in every run of 64 output columns the first 32 are gate
    rows and the next 32 the up rows of the same 32 products, 128 products per 256-column tile, products in order."""
    from nvfp4_gemm import _C
    e, inter, k = 2, 256, 128
    b = torch.arange(e * 2 * inter, dtype=torch.int64).repeat_interleave(k // 2).reshape(e * 2 * inter, k // 2)   # row id in every byte slot
    sfb = torch.arange(2 * inter, dtype=torch.int64).repeat(e * (k // 64), 1)                                      # column id in every word
    b2, sfb2 = _C.interleave_gate_up(b, sfb, e, inter)
    rows = b2[:, 0].reshape(e, 2 * inter)
    for ex in range(e):
        r = rows[ex] - ex * 2 * inter                           # original row (0 .. I: gate, I .. 2 I: up) at every new position
        groups = r.reshape(-1, 2, 32)                            # [64-column group][gate | up][32]
        assert torch.equal(groups[:, 1], groups[:, 0] + inter)   # the up row of the same product sits 32 columns further
        assert torch.equal(groups[:, 0].reshape(-1), torch.arange(inter))   # products in ascending order
    assert torch.equal(sfb2[0], rows[0]) and torch.equal(sfb2[-1], rows[0])                                        # scale columns move with the rows
    with pytest.raises(RuntimeError):
        _C.interleave_gate_up(b, sfb, e, 192)                    # I must be a multiple of 128
