"""Generate the golden vectors in this folder from the reference's own Python code.

Run once in a container where the reference project is mounted:

    python tests/golden/make_golden.py [/path/to/reference]

It imports, by file path and unmodified, the reference's CPU emulation
(tests/python/reference/dual_nvfp4.py) and its layout module
(python/nvfp4_gemm/layout.py), feeds them seeded inputs and stores inputs and
outputs as small ``.npz`` files.  The tests read only the ``.npz`` files, so they
run where the reference is absent.  Inputs are stored as bit patterns (BF16 as
uint16), never re-drawn from an RNG at test time.
"""
from __future__ import annotations

import hashlib
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)


def e4m3_bytes(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def grid_i8(t: torch.Tensor) -> np.ndarray:
    """E2M1 values are multiples of 0.5 in [-6, 6]: store 2*v as int8."""
    return (t * 2).to(torch.int8).numpy()


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def adversarial_rows(k: int, gen: torch.Generator) -> torch.Tensor:
    rows = [
        torch.zeros(k),
        torch.full((k,), 2688.0),
        torch.full((k,), -2688.0),
        torch.full((k,), 1e-8),
        torch.randn(k, generator=gen) * 1e-3,            # s0 at the 2^-6 floor
        torch.randn(k, generator=gen) * 0.05,            # s0 < 2^-3: s1 re-rounded in E4M3 subnormals
        torch.randn(k, generator=gen) * 300.0,
        # exact ties: multiples of 1/32 of a power-of-two block maximum
        (torch.randint(-192, 193, (k,), generator=gen).float() / 32.0),
        (torch.randint(-48, 49, (k,), generator=gen).float() * 0.25),
        torch.where(torch.arange(k) % 16 == 0, torch.tensor(6.0), torch.tensor(-0.0)),
    ]
    return torch.stack(rows).clamp(-2688.0, 2688.0)


def main(ref_root: str) -> None:
    emu = _load(os.path.join(ref_root, "tests/python/reference/dual_nvfp4.py"), "ref_dual_nvfp4")
    lay = _load(os.path.join(ref_root, "python/nvfp4_gemm/layout.py"), "ref_layout")

    # ---- rounding rules --------------------------------------------------
    g = torch.Generator().manual_seed(100)
    levels = torch.tensor(emu.E2M1_LEVELS)
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    special = torch.tensor([6.5, 1e4, -7.0, float("inf"), float("-inf"), -0.0, 0.0, 1e-30, -1e-30])
    near = torch.cat([torch.nextafter(mids, torch.tensor(10.0)), torch.nextafter(mids, torch.tensor(-10.0))])
    rnd = torch.randn(4096, generator=g) * 3.0
    x = torch.cat([levels, -levels, mids, -mids, near, -near, special, rnd])
    np.savez_compressed(
        os.path.join(HERE, "e2m1.npz"),
        x=x.numpy(),
        values=emu.quantize_e2m1(x).numpy(),                       # dual_nvfp4.py:51-74
        codes=lay.quantize_e2m1_codes(x).numpy(),                  # layout.py:34-48
    )
    y = torch.cat([
        torch.tensor([0.0, 2.0**-9, 2.0**-10, 1.5 * 2.0**-9, 2.0**-6, 448.0, 447.9, 463.9, 0.0146484375]),
        torch.exp(torch.rand(4096, generator=g) * 14.0 - 7.5),
        torch.rand(1024, generator=g) * 2.0**-5,
    ])
    np.savez_compressed(os.path.join(HERE, "e4m3.npz"), x=y.numpy(), codes=e4m3_bytes(y))   # layout.py:64-65

    # ---- Algorithm 1 (dual_nvfp4.py:101-158) -----------------------------
    g = torch.Generator().manual_seed(0)
    k = 256
    a = torch.cat([
        torch.randn(24, k, generator=g),
        torch.randn(8, k, generator=g) * torch.exp(0.5 * torch.randn(8, 1, generator=g)) * 4.0,
        adversarial_rows(k, g),
    ]).to(torch.bfloat16)
    out = {"a_bits": bf16_bits(a)}
    for policy in ("derived_div8", "residual_amax"):
        d = emu.decompose_dual_nvfp4(a, policy)
        out[f"{policy}_q0"] = grid_i8(d.q0)
        out[f"{policy}_q1"] = grid_i8(d.q1)
        out[f"{policy}_s0"] = e4m3_bytes(d.s0)
        out[f"{policy}_s1"] = e4m3_bytes(d.s1)
    np.savez_compressed(os.path.join(HERE, "decompose.npz"), **out)

    # ---- offline weight quantisation (layout.py:68-127, 130-152) ----------
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(3, 64, 128, generator=g) * 0.02).to(torch.bfloat16)
    w[1] *= 37.0                                    # experts with very different ranges
    w[2, :4] = 0.0                                  # all-zero blocks inside an expert
    b, sfb, gw = lay.quantize_weight_nvfp4(w)
    np.savez_compressed(
        os.path.join(HERE, "weights.npz"),
        w_bits=bf16_bits(w), b=b.numpy(), sfb=sfb.numpy(), gw=gw.numpy(),
        deq=lay.dequantize_weight_nvfp4(b, sfb, gw, 3, 64, 128).numpy(),
    )
    q, s, gg = emu.quantize_weight_nvfp4(w)         # dual_nvfp4.py:176-197 (unpacked twin)
    assert torch.equal(gg, gw)

    # ---- Algorithm 2 + ground truth (dual_nvfp4.py:200-258) ---------------
    g = torch.Generator().manual_seed(2)
    e, rows, n, k = 2, 32, 64, 256
    a = torch.randn(e * rows, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(e, n, k, generator=g) * 0.02).to(torch.bfloat16)
    q, s, gg = emu.quantize_weight_nvfp4(w)
    indptr = torch.tensor([0, rows, 2 * rows])
    b, sfb, gw = lay.quantize_weight_nvfp4(w)
    d_dual = emu.dual_nvfp4_grouped_gemm(a, q, s, gg, indptr)
    d_res = emu.dual_nvfp4_grouped_gemm(a, q, s, gg, indptr, scale_policy="residual_amax")
    d_true = emu.reference_grouped_gemm(a, q, s, gg, indptr)
    np.savez_compressed(
        os.path.join(HERE, "gemm.npz"),
        a_bits=bf16_bits(a), w_bits=bf16_bits(w), b=b.numpy(), sfb=sfb.numpy(), gw=gw.numpy(),
        m_indices=torch.arange(e).repeat_interleave(rows).to(torch.int32).numpy(),
        d_dual_bits=bf16_bits(d_dual), d_residual_amax_bits=bf16_bits(d_res), d_truth=d_true.numpy(),
    )

    # ---- scalars the reference's own tests pin, and the C1 checksums -------
    pins = {}
    torch.manual_seed(0)                            # test_dual_nvfp4_reference.py:69-85
    xs = torch.randn(512, 256).to(torch.bfloat16)
    d = emu.decompose_dual_nvfp4(xs)
    x32 = xs.float()
    s0b = d.s0.repeat_interleave(16, dim=-1)
    pins["single_rel_l2"] = float((d.q0 * s0b - x32).norm() / x32.norm())
    pins["dual_rel_l2"] = float((d.reconstruct() - x32).norm() / x32.norm())
    np.savez_compressed(os.path.join(HERE, "rel_l2_input.npz"), a_bits=bf16_bits(xs))

    # C1 of the benchmark plan: E=4 x 64 rows, N=512, K=1024, seeds act 0 / w 1.
    ga = torch.Generator().manual_seed(0)
    gw_ = torch.Generator().manual_seed(1)
    a1 = torch.randn(256, 1024, generator=ga).to(torch.bfloat16)
    w1 = (torch.randn(4, 512, 1024, generator=gw_) * 0.02).to(torch.bfloat16)
    d1 = emu.decompose_dual_nvfp4(a1)
    b1, sfb1, gw1 = lay.quantize_weight_nvfp4(w1)
    q1_, s1_, g1_ = emu.quantize_weight_nvfp4(w1)
    out1 = emu.dual_nvfp4_grouped_gemm(a1, q1_, s1_, g1_, torch.tensor([0, 64, 128, 192, 256]))
    true1 = emu.reference_grouped_gemm(a1, q1_, s1_, g1_, torch.tensor([0, 64, 128, 192, 256]))
    pins["c1"] = {
        "a_sha": sha(a1), "w_sha": sha(w1),
        "q0_sha": sha(torch.from_numpy(grid_i8(d1.q0))), "q1_sha": sha(torch.from_numpy(grid_i8(d1.q1))),
        "s0_sha": sha(torch.from_numpy(e4m3_bytes(d1.s0))), "s1_sha": sha(torch.from_numpy(e4m3_bytes(d1.s1))),
        "b_sha": sha(b1), "sfb_sha": sha(sfb1), "gw_sha": sha(gw1),
        "cosine_vs_truth": emu.cosine_similarity(out1, true1),
        "rel_l2_vs_truth": float((out1.float() - true1).norm() / true1.norm()),
    }
    np.savez_compressed(os.path.join(HERE, "c1_out.npz"), d_dual_bits=bf16_bits(out1))
    pins["torch_version"] = torch.__version__
    with open(os.path.join(HERE, "pins.json"), "w") as f:
        json.dump(pins, f, indent=1)
    print(json.dumps(pins, indent=1))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
