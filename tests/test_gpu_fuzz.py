"""GPU: seeded random shapes through every kernel family, against the CPU oracle.

The hand-picked cases of test_gpu_parity.py cover the corners somebody thought of; this file draws expert counts,
ragged group sizes, N, K, the scale policy, the pass count and the kernel family from a seeded generator, so that a
combination nobody thought of (an odd number of row blocks under the pair kernel, a K that only the 128-wide block
divides under the masked layout, a single expert wider than the machine) is still compared with the oracle.  Sizes
are kept small enough for the oracle to finish each case in well under a second.
"""
import random

import pytest
import torch

import nvfp4_gemm
from nvfp4_gemm import _C

pytestmark = pytest.mark.gpu

REL_L2_VS_ORACLE = 2.5e-3
POLICIES = ["derived_div8", "residual_amax", "derived_div4", "div4_radix8"]
# kernel family -> (tune knobs, constraint on N)
FAMILIES = {
    "split_single": (dict(tune_split_transform=1, tune_cluster=1), 256),
    "split_pair": (dict(tune_split_transform=1, tune_cluster=2), 256),
    "fused_quad": (dict(tune_split_transform=2, tune_cluster=4), 1024),
    "fused_pair": (dict(tune_split_transform=2, tune_cluster=2), 512),
    "fused_single": (dict(tune_split_transform=2, tune_cluster=1), 128),
    "default": (dict(), 128),
}


def rel_l2(x, y):
    x, y = x.float(), y.float()
    return float((x - y).norm() / y.norm().clamp_min(1e-30))


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a GPU"
    _C.lib()
    return torch.device("cuda:0")


def draw_case(seed: int):
    rnd = random.Random(seed)
    family = rnd.choice(list(FAMILIES))
    knobs, n_unit = FAMILIES[family]
    n = n_unit * rnd.choice([1, 1, 2, 3])
    k = 128 * rnd.choice([1, 2, 3, 4, 5, 8, 12])
    experts = rnd.choice([1, 2, 3, 5, 7])
    sizes = [128 * rnd.choice([0, 1, 1, 2, 3, 4]) for _ in range(experts)]
    if sum(sizes) == 0:
        sizes[0] = 128
    return dict(family=family, knobs=knobs, n=n, k=k, sizes=sizes, policy=rnd.choice(POLICIES), residual=rnd.random() < 0.75,
                heavy_tail=rnd.random() < 0.3)


@pytest.mark.parametrize("seed", range(48))
def test_contiguous_layout_random_case(dev, oracle, seed):
    c = draw_case(seed)
    g = torch.Generator().manual_seed(10_000 + seed)
    m = sum(c["sizes"])
    a = torch.randn(m, c["k"], generator=g)
    if c["heavy_tail"]:                                   # a few rows and a few channels much larger than the rest
        a[::7] *= 40.0
        a[:, ::53] *= 25.0
    a = a.clamp(-2688.0, 2688.0).to(torch.bfloat16)
    w = (torch.randn(len(c["sizes"]), c["n"], c["k"], generator=g) * 0.03).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(c["sizes"])
    d = torch.full((m, c["n"]), float("nan"), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(a.to(dev), b, sfb, gw, d, mi.to(dev), scale_policy=c["policy"],
                                                         enable_residual_pass=c["residual"], device_status=status, **c["knobs"])
    torch.cuda.synchronize()
    assert int(status.item()) == 0, c
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, c["n"], mode="dual" if c["residual"] else "single",
                               scale_policy=c["policy"])
    assert torch.isfinite(d.float()).all(), c
    assert rel_l2(d.cpu(), want) < REL_L2_VS_ORACLE, c


@pytest.mark.parametrize("seed", range(16))
def test_masked_layout_random_case(dev, oracle, seed):
    rnd = random.Random(500 + seed)
    groups = rnd.choice([1, 2, 4, 6])
    max_m = 128 * rnd.choice([1, 2, 3, 5])
    n = 256 * rnd.choice([1, 2, 3])
    k = 128 * rnd.choice([1, 2, 3, 4, 6])
    counts = [rnd.choice([0, 1, max_m // 2, max_m - 1, max_m, max_m + 9, rnd.randrange(0, max_m + 1)]) for _ in range(groups)]
    residual = rnd.random() < 0.75
    tune = dict(tune_cluster=rnd.choice([1, 2]))
    g = torch.Generator().manual_seed(20_000 + seed)
    a = torch.randn(groups, max_m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(groups, n, k, generator=g) * 0.03).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    d = torch.full((groups, max_m, n), float("nan"), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_masked(a.to(dev), b, sfb, gw, d, torch.tensor(counts, dtype=torch.int32, device=dev),
                                                     enable_residual_pass=residual, device_status=status, **tune)
    torch.cuda.synchronize()
    assert _C.read_status(status) == 0, (counts, tune)
    dc = d.cpu()
    for grp, cnt in enumerate(counts):
        live = min((min(cnt, max_m) + 127) // 128 * 128, max_m)
        assert torch.isnan(dc[grp, live:].float()).all(), (grp, counts, tune)
        if live == 0:
            continue
        want = oracle.grouped_gemm(a[grp, :live], b.cpu()[grp * n:(grp + 1) * n], sfb.cpu()[grp * (k // 64):(grp + 1) * (k // 64)],
                                   gw.cpu()[grp:grp + 1], torch.zeros(live, dtype=torch.int32), n, mode="dual" if residual else "single")
        assert rel_l2(dc[grp, :live], want) < REL_L2_VS_ORACLE, (grp, counts, tune)


@pytest.mark.parametrize("seed", range(12))
def test_decode_orientation_random_case(dev, oracle, seed):
    rnd = random.Random(900 + seed)
    align = rnd.choice([16, 32, 64, 128])
    experts = rnd.choice([1, 3, 6])
    n = 128 * rnd.choice([1, 2, 3, 5])
    k = 128 * rnd.choice([1, 2, 4, 5, 8])
    sizes = [align * rnd.choice([0, 1, 1, 2, 3]) for _ in range(experts)]
    if sum(sizes) == 0:
        sizes[-1] = align
    policy = rnd.choice(POLICIES)
    residual = rnd.random() < 0.75
    g = torch.Generator().manual_seed(30_000 + seed)
    a = torch.randn(sum(sizes), k, generator=g).to(torch.bfloat16)
    w = (torch.randn(experts, n, k, generator=g) * 0.03).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes, alignment=align)
    d = torch.full((sum(sizes), n), float("nan"), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(a.to(dev), b, sfb, gw, d, mi.to(dev), scale_policy=policy,
                                                         enable_residual_pass=residual, tune_swap_ab=1, m_alignment=align,
                                                         device_status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="dual" if residual else "single", scale_policy=policy)
    assert rel_l2(d.cpu(), want) < REL_L2_VS_ORACLE, (sizes, n, k, policy, residual, align)
