"""GPU parity at the real sizes of the benchmark configurations (C2, C3 up / down, C4, C5 up / down).

The CUDA call runs on the whole problem, built by the same generator as ``bench.py``; the CPU oracle then
recomputes slices of it -- for the hottest expert, an expert with a single row block and the last active expert,
on 256-column strips at the first, a middle and the last column tile -- from the very bytes the kernel read
(weights and scales copied back from the device).  Bar: relative L2 <= 2.5e-3 against the oracle's BF16 output on
every slice, rows that are all zero in A exactly zero in D, nothing written past column N, device status 0.
Shape list after the reference's acceptance test (tests/python/test_gemm.py:31-50,83-85), at the sizes its
benchmarks use.
"""
import pytest
import torch

import bench
import nvfp4_gemm
from nvfp4_gemm import _C

pytestmark = pytest.mark.gpu

REL_L2_VS_ORACLE = 2.5e-3


def rel_l2(x, y):
    x, y = x.float(), y.float()
    return float((x - y).norm() / y.norm().clamp_min(1e-30))


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a GPU"
    _C.lib()
    return torch.device("cuda:0")


def check_slices(case, d, oracle, mode="dual", policy="derived_div8", strip=256, max_rows=256):
    E, N, K = case["E"], case["N"], case["K"]
    real, padded = case["real"], case["padded"]
    starts = [sum(padded[:e]) for e in range(E)]
    active = [e for e in range(E) if real[e] > 0]
    hottest = max(active, key=lambda e: real[e])
    single = [e for e in active if padded[e] == min(padded[x] for x in active)]
    experts = sorted({hottest, single[len(single) // 2], active[-1]})
    tiles = sorted({0, (N // strip) // 2, N // strip - 1})
    worst = 0.0
    for e in experts:
        rows = min(padded[e], max_rows)
        picks = [(starts[e], rows)]
        if padded[e] > rows:                                     # the last row block of a long group as well
            picks.append((starts[e] + padded[e] - min(padded[e], 128), min(padded[e], 128)))
        for t in tiles:
            lo, hi = t * strip, (t + 1) * strip
            b_sub = case["b"][e * N + lo:e * N + hi].cpu()
            sfb_sub = case["sfb"][e * (K // 64):(e + 1) * (K // 64), lo:hi].contiguous().cpu()
            gw_sub = case["gw"][e:e + 1].cpu()
            for r0, nr in picks:
                a_sub = case["a"][r0:r0 + nr].cpu()
                want = oracle.grouped_gemm(a_sub, b_sub, sfb_sub, gw_sub, torch.zeros(nr, dtype=torch.int32), hi - lo,
                                           mode=mode, scale_policy=policy)
                got = d[r0:r0 + nr, lo:hi].cpu()
                err = rel_l2(got, want)
                worst = max(worst, err)
                assert torch.isfinite(got.float()).all()
                assert err < REL_L2_VS_ORACLE, (e, t, r0, nr, err)
    return worst


def run_case(dev, oracle, workload, extra_kw=None, **check_kw):
    case = bench.build_single_gpu_case(workload, dev, extra_kw)
    M, N = case["M"], case["N"]
    d_wide = torch.full((M, N + 128), float("nan"), dtype=torch.bfloat16, device=dev)
    d = d_wide[:, :N]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(case["a"], case["b"], case["sfb"], case["gw"], d, case["m_indices"],
                                                         device_status=status, **case["kw"])
    torch.cuda.synchronize()
    assert _C.read_status(status) == 0
    assert torch.isnan(d_wide[:, N:].float()).all(), "written past column N"
    zero_rows = (case["a"] == 0).all(dim=1)
    if bool(zero_rows.any()):
        assert float(d[zero_rows].float().abs().max()) == 0.0, "padding rows must come out as exact zeros"
    assert torch.isfinite(d[~zero_rows].float()).all()
    worst = check_slices(case, d, oracle, **check_kw)
    del case, d_wide
    torch.cuda.empty_cache()
    return worst


PATHS = {"default": None, "fused": dict(tune_split_transform=2), "single_cta_split": dict(tune_split_transform=1, tune_cluster=1),
         "pair_split": dict(tune_split_transform=1, tune_cluster=2)}


@pytest.mark.parametrize("path", ["default", "fused", "single_cta_split"])
def test_c2_mixtral_up_projection(dev, oracle, path):
    """The default is the CTA-pair GEMM here: every expert has 512 rows and the case says m_alignment=256."""
    run_case(dev, oracle, "c2", PATHS[path])


@pytest.mark.parametrize("workload", ["c3up", "c3down"])
@pytest.mark.parametrize("path", ["default", "fused"])
def test_c3_deepseek_prefill(dev, oracle, workload, path):
    run_case(dev, oracle, workload, dict(tune_split_transform=2) if path == "fused" else None)


def test_c4_decode(dev, oracle):
    run_case(dev, oracle, "c4", max_rows=16)


@pytest.mark.parametrize("workload", ["c5up", "c5down"])
@pytest.mark.parametrize("path", ["default", "pair_split"])
def test_c5_expert_parallel_gemms_at_one_rank(dev, oracle, workload, path):
    """pair_split: 128 experts with ragged row counts, so about half of them end in a left-over single row block."""
    run_case(dev, oracle, workload, PATHS[path])
