"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bar: weight quantisation and the activation codes/scales (q0, q1, s0, s1) bit-exact;
GEMM output within relative L2 2.5e-3 of the oracle's BF16 output (BF16 rounding of
two differently ordered FP32 sums alone gives ~1.7e-3) and cosine > 0.999 against
the FP32 ground truth (the reference's acceptance gate, tests/python/test_gemm.py:83-85).
"""
import pytest
import torch

from conftest import bf16_from_bits, grid_i8_from_codes, load_golden

import nvfp4_gemm
from nvfp4_gemm import _C

pytestmark = pytest.mark.gpu

REL_L2_VS_ORACLE = 2.5e-3


def unpack_codes(packed: torch.Tensor) -> torch.Tensor:
    u = packed.cpu().view(torch.uint8)
    return torch.stack([u & 0xF, u >> 4], dim=-1).reshape(u.shape[0], -1)


def rel_l2(x, y):
    x, y = x.float(), y.float()
    return float((x - y).norm() / y.norm().clamp_min(1e-30))


def cosine(x, y):
    x, y = x.float().flatten(), y.float().flatten()
    return float(torch.dot(x, y) / (x.norm() * y.norm()).clamp_min(1e-30))


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a GPU"
    _C.lib()                                   # fail loudly if the library is missing
    return torch.device("cuda:0")


# ---------------------------------------------------------------- weights
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_weight_quantiser_bit_exact_golden(dev, oracle, dtype):
    g = load_golden("weights.npz")
    w = bf16_from_bits(g["w_bits"]).to(dtype)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    assert torch.equal(b.cpu(), torch.from_numpy(g["b"]))
    assert torch.equal(sfb.cpu(), torch.from_numpy(g["sfb"]))
    assert torch.equal(gw.cpu(), torch.from_numpy(g["gw"]))


@pytest.mark.parametrize("shape", [(1, 128, 64), (4, 512, 1024), (2, 384, 4096), (3, 100, 192)])
def test_weight_quantiser_bit_exact_random(dev, oracle, shape):
    g = torch.Generator().manual_seed(sum(shape))
    w = (torch.randn(*shape, generator=g) * 0.02).to(torch.bfloat16)
    w[0, 0, :16] = 0.0
    if shape[0] > 1:
        w[1] *= 123.0
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    ob, osfb, ogw = oracle.quantize_weight(w)
    assert torch.equal(gw.cpu(), ogw)
    assert torch.equal(sfb.cpu(), osfb)
    assert torch.equal(b.cpu(), ob)


def test_weight_quantiser_fp32_input_and_zero_expert(dev, oracle):
    g = torch.Generator().manual_seed(9)
    w = torch.randn(2, 64, 128, generator=g) * 0.3
    w[1] = 0.0                                   # G clamps to the smallest normal float
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    ob, osfb, ogw = oracle.quantize_weight(w)
    assert torch.equal(gw.cpu(), ogw) and torch.equal(sfb.cpu(), osfb) and torch.equal(b.cpu(), ob)


# ---------------------------------------------------------------- Algorithm 1
POLICIES = ["derived_div8", "residual_amax", "derived_div4", "div4_radix8"]


def check_decompose(dev, oracle, a, policy="derived_div8"):
    q0, q1, s0, s1 = _C.debug_decompose(a.to(dev), scale_policy=policy)
    o0, o1, os0, os1 = oracle.decompose(a, scale_policy=policy)
    assert torch.equal(s0.cpu(), os0), "s0 bytes differ"
    assert torch.equal(s1.cpu(), os1), "s1 bytes differ"
    assert torch.equal(grid_i8_from_codes(unpack_codes(q0)), grid_i8_from_codes(o0)), "q0 differs"
    assert torch.equal(grid_i8_from_codes(unpack_codes(q1)), grid_i8_from_codes(o1)), "q1 differs"


@pytest.mark.parametrize("policy", POLICIES[:2])       # the two policies the reference's emulation has
def test_decompose_bit_exact_golden(dev, oracle, policy):
    g = load_golden("decompose.npz")
    a = bf16_from_bits(g["a_bits"])                          # 42 x 256, incl. adversarial rows
    a = torch.cat([a, torch.zeros(128 - a.shape[0], a.shape[1], dtype=torch.bfloat16)])
    q0, q1, s0, s1 = _C.debug_decompose(a.to(dev), scale_policy=policy)
    n = g["a_bits"].shape[0]
    assert torch.equal(s0.cpu()[:n], torch.from_numpy(g[policy + "_s0"]))
    assert torch.equal(s1.cpu()[:n], torch.from_numpy(g[policy + "_s1"]))
    assert torch.equal(grid_i8_from_codes(unpack_codes(q0))[:n], torch.from_numpy(g[policy + "_q0"]))
    assert torch.equal(grid_i8_from_codes(unpack_codes(q1))[:n], torch.from_numpy(g[policy + "_q1"]))


@pytest.mark.parametrize("policy", POLICIES)
def test_decompose_bit_exact_c1_and_distributions(dev, oracle, policy):
    g = torch.Generator().manual_seed(0)
    a = torch.randn(256, 1024, generator=g).to(torch.bfloat16)                       # config C1 activations
    check_decompose(dev, oracle, a, policy)
    a = (torch.randn(256, 512, generator=g) * torch.exp(0.5 * torch.randn(256, 1, generator=g))).to(torch.bfloat16)
    check_decompose(dev, oracle, a, policy)
    t = torch.randn(128, 512, generator=g) / torch.sqrt(torch.randn(128, 512, 4, generator=g).pow(2).mean(-1))
    check_decompose(dev, oracle, t.clamp(-2688, 2688).to(torch.bfloat16), policy)    # Student-t(4)
    a = torch.randn(128, 1024, generator=g)
    a[:, torch.randperm(1024, generator=g)[:2]] *= 50.0                               # outlier channels
    check_decompose(dev, oracle, a.to(torch.bfloat16), policy)
    a = torch.randn(128, 256, generator=g) * 1e-3                                     # tiny blocks: the scale floors
    check_decompose(dev, oracle, a.to(torch.bfloat16), policy)


@pytest.mark.parametrize("policy", POLICIES)
def test_decompose_bit_exact_every_scale_and_value(dev, oracle, policy):
    """Every E4M3 scale the floor allows x every BF16 magnitude up to the block maximum:
    each 16-block carries one element that pins s0 and fifteen probe values."""
    blocks = []
    for code in range(0x01 if policy == "residual_amax" else 0x08, 0x7F):
        s0 = torch.tensor([code], dtype=torch.uint8).view(torch.float8_e4m3fn).float().item()
        top = torch.tensor((4.0 if policy == "div4_radix8" else 6.0) * s0).to(torch.bfloat16)
        bits = torch.arange(0, int(top.view(torch.int16).item()) + 1, 7, dtype=torch.int32)
        ties = (torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.28125, 1.53125, 3.25, 5.5, 0.3125, 1.0625, 2.15625]) * s0)
        vals = torch.cat([bits.to(torch.int16).view(torch.bfloat16).float(), ties])
        vals = torch.cat([vals, -vals])
        pad = (-vals.numel()) % 15
        vals = torch.cat([vals, torch.zeros(pad)]).reshape(-1, 15)
        blocks.append(torch.cat([torch.full((vals.shape[0], 1), float(top)), vals], dim=1))
    flat = torch.cat(blocks).reshape(-1)
    k = 1024
    pad = (-flat.numel()) % (128 * k)
    a = torch.cat([flat, torch.zeros(pad)]).reshape(-1, k).to(torch.bfloat16)
    check_decompose(dev, oracle, a, policy)


# ---------------------------------------------------------------- GEMM
def make_case(e, rows, n, k, seed, act_scale=1.0, w_scale=0.02):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(e * rows, k, generator=g) * act_scale).to(torch.bfloat16)
    w = (torch.randn(e, n, k, generator=g) * w_scale).to(torch.bfloat16)
    return a, w


def run_gemm(dev, a, b, sfb, gw, m_indices, n, **kw):
    d = torch.full((a.shape[0], n), float("nan"), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(a.to(dev), b, sfb, gw, d, m_indices.to(dev),
                                                         device_status=status, **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device status {int(status.item())}"
    return d.cpu()


# the reference's acceptance shapes (tests/python/test_gemm.py:31-36) plus edge shapes
SHAPES = [(1, 128, 128, 256), (2, 128, 256, 512), (4, 256, 1024, 2048), (4, 512, 2048, 512),
          (1, 128, 256, 128), (3, 128, 384, 256), (2, 384, 512, 1024)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("residual", [True, False])
def test_gemm_matches_oracle(dev, oracle, shape, residual):
    e, rows, n, k = shape
    a, w = make_case(e, rows, n, k, seed=1000 + n + k)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual)
    assert torch.isfinite(d.float()).all()
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="dual" if residual else "single")
    truth = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="truth")
    assert rel_l2(d, want) < REL_L2_VS_ORACLE, (rel_l2(d, want), cosine(d, truth))
    if residual:
        assert cosine(d, truth) > 0.999
        assert rel_l2(d, truth) <= rel_l2(want, truth) * 1.02 + 1e-4     # no worse than the reference chain


@pytest.mark.parametrize("tune", [dict(tune_direct_a=1), dict(tune_transform_warps=16), dict(tune_sched_group=4),
                                  dict(tune_split_transform=2, tune_sched_group=4)])
@pytest.mark.parametrize("residual", [True, False])
def test_gemm_kernel_variants_agree(dev, oracle, tune, residual):
    """The direct-global-read transform, the 16-warp transform and another tile order against the
    oracle; K blocks odd in number and more tiles than SMs so that every ring wraps."""
    e, rows, n, k = 3, 256, 2048, 640
    a, w = make_case(e, rows, n, k, seed=31)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual, **tune)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="dual" if residual else "single")
    assert rel_l2(d, want) < REL_L2_VS_ORACLE


@pytest.mark.parametrize("shape", [(1, 128, 512, 128), (1, 128, 512, 1024), (4, 256, 1024, 2048), (3, 256, 2048, 640)])
@pytest.mark.parametrize("residual", [True, False])
@pytest.mark.parametrize("cluster", [2, 4])
def test_gemm_cluster_matches_oracle(dev, oracle, shape, residual, cluster):
    """tune_cluster=2 / 4: the CTAs of a cluster transform a share of the tile each and exchange the
    shares; short and long K (every ring wraps), one and many tiles per cluster."""
    if shape[2] % (256 * cluster):
        pytest.skip("N is not a multiple of the cluster's column span")
    e, rows, n, k = shape
    a, w = make_case(e, rows, n, k, seed=500 + n + k)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual, tune_cluster=cluster)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="dual" if residual else "single")
    assert rel_l2(d, want) < REL_L2_VS_ORACLE


@pytest.mark.parametrize("shape", [(1, 128, 256, 128), (1, 128, 512, 1024), (4, 256, 1024, 2048), (3, 256, 2048, 640),
                                   (2, 384, 768, 256)])
@pytest.mark.parametrize("residual", [True, False])
@pytest.mark.parametrize("block_k", [0, 128, 130])
def test_gemm_split_matches_oracle(dev, oracle, shape, residual, block_k):
    """tune_split_transform=1: the activations are quantised once by a kernel of their own and the GEMM reads
    codes and scale atoms from the workspace; short and long K, K that only the 128-wide block divides,
    both K-block widths."""
    e, rows, n, k = shape
    a, w = make_case(e, rows, n, k, seed=700 + n + k)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual, tune_split_transform=1, tune_block_k=block_k)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="dual" if residual else "single")
    assert torch.isfinite(d.float()).all()
    assert rel_l2(d, want) < REL_L2_VS_ORACLE
    fused = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual, tune_split_transform=2)
    assert rel_l2(d, fused) < 1e-3        # same codes and scales; only the summation order may differ


PAIR = dict(tune_split_transform=1, tune_cluster=2)     # split path with the CTA-pair (cta_group::2) GEMM kernel


@pytest.mark.parametrize("sizes", [[256], [128], [128, 128], [384, 128, 256, 640, 128], [256, 256, 256], [128] * 5, [1152]],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("nk", [(256, 128), (1024, 2048), (2048, 640)])
@pytest.mark.parametrize("residual", [True, False])
def test_gemm_split_pair_kernel_matches_oracle(dev, oracle, sizes, nk, residual):
    """tune_split_transform=1 + tune_cluster=2: two CTAs share one MMA over 256 rows x 256 columns.  Experts with one,
    an even and an odd number of row blocks (a left-over block is a unit of its own: the odd CTA stores nothing),
    expert boundaries on odd row blocks, short and long K, K that only the 128-wide block divides.  Same K order as
    the single-CTA kernel, so the two must agree bit for bit."""
    n, k = nk
    g = torch.Generator().manual_seed(900 + n + k + len(sizes))
    a = torch.randn(sum(sizes), k, generator=g).to(torch.bfloat16)
    w = (torch.randn(len(sizes), n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual, **PAIR)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="dual" if residual else "single")
    assert torch.isfinite(d.float()).all()
    assert rel_l2(d, want) < REL_L2_VS_ORACLE
    single = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual, tune_split_transform=1, tune_cluster=1)
    assert torch.equal(d, single)


def test_groups_of_256_rows_take_the_pair_kernel_by_default(dev, oracle):
    """m_alignment=256 is the caller's statement that every expert's rows are whole 256-row pairs; the split path then
    runs the CTA-pair kernel by itself.  Same bits as the explicitly chosen kernels; M % 256 is enforced."""
    sizes, n, k = [512, 256, 768], 2048, 1024
    g = torch.Generator().manual_seed(4242)
    a = torch.randn(sum(sizes), k, generator=g).to(torch.bfloat16)
    w = (torch.randn(len(sizes), n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes, alignment=256)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, m_alignment=256)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n)
    assert rel_l2(d, want) < REL_L2_VS_ORACLE
    assert torch.equal(d, run_gemm(dev, a, b, sfb, gw, mi, n, **PAIR))
    assert torch.equal(d, run_gemm(dev, a, b, sfb, gw, mi, n, tune_split_transform=1, tune_cluster=1))
    with pytest.raises(RuntimeError, match="multiple of the token-tile alignment"):
        run_gemm(dev, a[:384], b, sfb, gw, mi[:384], n, m_alignment=256)


@pytest.mark.parametrize("tune", [dict(tune_split_transform=1), PAIR], ids=["single", "pair"])
def test_gemm_split_many_tiles_strided(dev, oracle, tune):
    """Split path with more tiles than SMs, ragged experts, a strided activation matrix and a strided output."""
    sizes = [128, 384, 256, 128, 512, 128, 256, 640]
    n, k = 4096, 512
    g = torch.Generator().manual_seed(123)
    a_wide = torch.randn(sum(sizes), k + 64, generator=g).to(torch.bfloat16).to(dev)
    a = a_wide[:, :k]
    w = (torch.randn(len(sizes), n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes)
    d_wide = torch.full((sum(sizes), n + 128), float("nan"), dtype=torch.bfloat16, device=dev)
    d = d_wide[:, :n]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for _ in range(3):                    # repeated calls reuse the pooled workspace
        nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(a, b, sfb, gw, d, mi.to(dev), device_status=status, **tune)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = oracle.grouped_gemm(a.cpu().contiguous(), b.cpu(), sfb.cpu(), gw.cpu(), mi, n)
    assert rel_l2(d.cpu(), want) < REL_L2_VS_ORACLE
    assert torch.isnan(d_wide[:, n:].float()).all()          # nothing written past the N columns


@pytest.mark.parametrize("kw", [dict(tune_split_transform=1), dict(tune_split_transform=2), dict(tune_swap_ab=1, m_alignment=128)],
                         ids=["split", "fused", "swap_ab"])
def test_cuda_graph_replay_matches_eager(dev, kw):
    """One warm-up call, then the call is captured into a CUDA graph (the reference's contract: capturable after a
    warm-up) and replayed on fresh inputs written into the same buffers."""
    e, rows, n, k = 2, 256, 1024, 1024
    a0, w = make_case(e, rows, n, k, seed=31)
    a1, _ = make_case(e, rows, n, k, seed=32)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e).to(dev)
    a = a0.to(dev).clone()
    d = torch.empty(e * rows, n, dtype=torch.bfloat16, device=dev)

    def call():
        nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(a, b, sfb, gw, d, mi, **kw)

    call()
    torch.cuda.synchronize()
    eager0 = d.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    d.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(d, eager0)
    a.copy_(a1.to(dev))
    graph.replay()
    torch.cuda.synchronize()
    replayed = d.clone()
    call()
    torch.cuda.synchronize()
    assert torch.equal(replayed, d) and not torch.equal(replayed, eager0)


def test_split_path_on_two_streams_at_once(dev, oracle):
    """The split path's workspace is allocated stream-ordered from a pool: calls in flight on two streams must not
    share it."""
    e, rows, n, k = 2, 256, 2048, 512
    cases = [make_case(e, rows, n, k, seed=41 + i) for i in range(2)]
    quant = [nvfp4_gemm.quantize_weight_nvfp4(w.to(dev)) for _, w in cases]
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [torch.empty(e * rows, n, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    acts = [a.to(dev) for a, _ in cases]
    mid = mi.to(dev)
    torch.cuda.synchronize()
    for _ in range(8):
        for i in range(2):
            with torch.cuda.stream(streams[i]):
                nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(acts[i], *quant[i], outs[i], mid, tune_split_transform=1)
    torch.cuda.synchronize()
    for i in range(2):
        want = oracle.grouped_gemm(cases[i][0], quant[i][0].cpu(), quant[i][1].cpu(), quant[i][2].cpu(), mi, n)
        assert rel_l2(outs[i].cpu(), want) < REL_L2_VS_ORACLE


@pytest.mark.parametrize("shape", [(1, 128, 128, 256), (2, 128, 256, 512), (4, 256, 1024, 2048), (4, 512, 2048, 512), (3, 128, 384, 256)])
@pytest.mark.parametrize("residual", [True, False])
@pytest.mark.parametrize("policy", POLICIES[1:])
def test_gemm_other_scale_policies_match_oracle(dev, oracle, shape, residual, policy):
    """residual_amax, derived_div4 and div4_radix8 on the reference's acceptance shapes (tests/python/test_gemm.py:31-36
    there) through the default dispatch: the split path for N % 256 == 0 and N > 1024, a fused kernel otherwise."""
    e, rows, n, k = shape
    a, w = make_case(e, rows, n, k, seed=900 + n + k)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual, scale_policy=policy)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="dual" if residual else "single",
                               scale_policy=policy)
    truth = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="truth")
    assert rel_l2(d, want) < REL_L2_VS_ORACLE
    if residual:
        assert cosine(d, truth) > 0.999
        if policy == "residual_amax":
            div8 = run_gemm(dev, a, b, sfb, gw, mi, n)
            assert rel_l2(d, truth) <= rel_l2(div8, truth) * 1.05       # the second amax pass buys accuracy


@pytest.mark.parametrize("policy", POLICIES)
@pytest.mark.parametrize("kw", [dict(tune_split_transform=2, tune_cluster=4), dict(tune_split_transform=2, tune_cluster=2),
                                dict(tune_split_transform=2, tune_cluster=1), dict(tune_split_transform=1)],
                         ids=["cluster4", "cluster2", "single_cta", "split"])
def test_every_kernel_family_runs_every_policy(dev, oracle, policy, kw):
    e, rows, n, k = 2, 256, 1024, 640
    a, w = make_case(e, rows, n, k, seed=1234)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, scale_policy=policy, **kw)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, scale_policy=policy)
    assert rel_l2(d, want) < REL_L2_VS_ORACLE


@pytest.mark.parametrize("case", [([16, 48, 16, 32], 16, 384, 1024), ([64, 128], 64, 256, 384), ([32] * 4, 32, 512, 2048)])
@pytest.mark.parametrize("policy", POLICIES[1:])
def test_gemm_swap_ab_other_policies_match_oracle(dev, oracle, case, policy):
    sizes, align, n, k = case
    g = torch.Generator().manual_seed(6000 + n + k)
    a = torch.randn(sum(sizes), k, generator=g).to(torch.bfloat16)
    w = (torch.randn(len(sizes), n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes, alignment=align)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, tune_swap_ab=1, m_alignment=align, scale_policy=policy)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, scale_policy=policy)
    assert rel_l2(d, want) < REL_L2_VS_ORACLE


def test_gemm_many_tiles_ragged_experts(dev, oracle):
    """More tiles than SMs, ragged expert sizes: every CTA loops over several tiles."""
    sizes = [128, 384, 256, 128, 512, 128, 256, 640]
    n, k = 4096, 256
    g = torch.Generator().manual_seed(99)
    a = torch.randn(sum(sizes), k, generator=g).to(torch.bfloat16)
    w = (torch.randn(len(sizes), n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes)
    d = run_gemm(dev, a, b, sfb, gw, mi, n)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n)
    assert rel_l2(d, want) < REL_L2_VS_ORACLE


def test_gemm_rejects_n_below_contract(dev):
    g = load_golden("gemm.npz")                       # E=2 x 32 rows: pad each expert to 128 rows
    a = bf16_from_bits(g["a_bits"])
    k = a.shape[1]
    ap = torch.zeros(256, k, dtype=torch.bfloat16)
    ap[0:32] = a[0:32]
    ap[128:160] = a[32:64]
    b, sfb, gw = (torch.from_numpy(g[x]).to(dev) for x in ("b", "sfb", "gw"))
    # N = 64 is below the kernel's N % 128 contract: check the contract instead
    with pytest.raises(RuntimeError):
        run_gemm(dev, ap, b, sfb, gw, nvfp4_gemm.make_m_indices([128, 128]), 64)


def test_gemm_c1_padded(dev, oracle):
    """Config C1 (E=4 x 64 rows, N=512, K=1024, seeds 0 / 1), each expert padded to 128 rows."""
    a = torch.randn(256, 1024, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    w = (torch.randn(4, 512, 1024, generator=torch.Generator().manual_seed(1)) * 0.02).to(torch.bfloat16)
    ap = torch.zeros(512, 1024, dtype=torch.bfloat16)
    for e in range(4):
        ap[e * 128:e * 128 + 64] = a[e * 64:(e + 1) * 64]
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    d = run_gemm(dev, ap, b, sfb, gw, nvfp4_gemm.make_m_indices([128] * 4), 512)
    real = torch.cat([d[e * 128:e * 128 + 64] for e in range(4)])
    ref = bf16_from_bits(load_golden("c1_out.npz")["d_dual_bits"])        # the reference emulation's output
    assert rel_l2(real, ref) < REL_L2_VS_ORACLE
    pad = torch.cat([d[e * 128 + 64:(e + 1) * 128] for e in range(4)])
    assert float(pad.float().abs().max()) == 0.0                          # zero rows give exact zeros


def test_gemm_one_hot_rows_localise_layout(dev, oracle):
    """A with a single 6.0 per row (s0 = 1, q0 = 6, q1 = 0: a_hat is exactly 6): row r of
    D must be 6 x column k(r) of dequant(W), which pins every layout rotation at once."""
    e, n, k = 1, 256, 256
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(e, n, k, generator=g) * 0.02).to(torch.bfloat16)
    a = torch.zeros(128, k, dtype=torch.bfloat16)
    cols = (torch.arange(128) * 37 + 5) % k
    a[torch.arange(128), cols] = 6.0
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    d = run_gemm(dev, a, b, sfb, gw, nvfp4_gemm.make_m_indices([128]), n)
    wdq = oracle.dequantize_weight(b.cpu(), sfb.cpu(), gw.cpu(), e, n, k)[0]          # (n, k)
    want = (6.0 * wdq[:, cols].T)
    # one product per output: only the order of the two FP32 roundings can differ
    assert float((d.float() - want).abs().max()) <= float(want.abs().max()) * 2 ** -8
    assert float((d.view(torch.int16) == want.to(torch.bfloat16).view(torch.int16)).float().mean()) > 0.9


def test_gemm_strided_rows_and_negative_index(dev, oracle):
    e, rows, n, k = 2, 128, 256, 256
    a, w = make_case(e, rows, n, k, seed=77)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    mi[:128] = -1                                             # negative ids read as expert 0
    a_wide = torch.zeros(a.shape[0], k + 64, dtype=torch.bfloat16, device=dev)
    a_wide[:, :k] = a.to(dev)
    d_wide = torch.zeros(a.shape[0], n + 128, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(a_wide[:, :k], b, sfb, gw, d_wide[:, :n], mi.to(dev),
                                                         device_status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n)
    assert rel_l2(d_wide[:, :n].cpu(), want) < REL_L2_VS_ORACLE
    assert float(d_wide[:, n:].float().abs().max()) == 0.0     # nothing written past N


def test_gemm_empty_and_errors(dev):
    b = torch.zeros(128, 128, dtype=torch.int8, device=dev)
    sfb = torch.zeros(4, 128, dtype=torch.int32, device=dev)
    gw = torch.ones(1, device=dev)
    f = nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous
    f(torch.zeros(0, 256, dtype=torch.bfloat16, device=dev), b, sfb, gw,
      torch.zeros(0, 128, dtype=torch.bfloat16, device=dev), torch.zeros(0, dtype=torch.int32, device=dev))
    with pytest.raises(RuntimeError):                          # M not a multiple of 128
        f(torch.zeros(64, 256, dtype=torch.bfloat16, device=dev), b, sfb, gw,
          torch.zeros(64, 128, dtype=torch.bfloat16, device=dev), torch.zeros(64, dtype=torch.int32, device=dev))


def test_num_sms_roundtrip(dev):
    hw = nvfp4_gemm.get_num_sms()
    assert hw == torch.cuda.get_device_properties(0).multi_processor_count
    nvfp4_gemm.set_num_sms(hw - 16)
    assert nvfp4_gemm.get_num_sms() == hw - 16
    nvfp4_gemm.set_num_sms(0)
    assert nvfp4_gemm.get_num_sms() == hw
    with pytest.raises(RuntimeError):
        nvfp4_gemm.set_num_sms(10 * hw)


# ---------------------------------------------------------------- decode orientation (swap-AB)
SWAP_CASES = [
    # (group sizes, alignment, N, K)
    ([16, 16], 16, 128, 256),
    ([32, 64, 32], 32, 256, 512),
    ([16, 48, 16, 32], 16, 384, 1024),
    ([64, 128], 64, 256, 384),           # K not a multiple of 256: the 128-wide K block variant
    ([128, 128], 128, 512, 256),
    ([32] * 8, 32, 1024, 2048),
]


@pytest.mark.parametrize("case", SWAP_CASES)
@pytest.mark.parametrize("residual", [True, False])
def test_gemm_swap_ab_matches_oracle(dev, oracle, case, residual):
    sizes, align, n, k = case
    e = len(sizes)
    g = torch.Generator().manual_seed(4000 + n + k + align)
    a = torch.randn(sum(sizes), k, generator=g).to(torch.bfloat16)
    w = (torch.randn(e, n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes, alignment=align)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, enable_residual_pass=residual, tune_swap_ab=1, m_alignment=align)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="dual" if residual else "single")
    truth = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n, mode="truth")
    assert torch.isfinite(d.float()).all()
    assert rel_l2(d, want) < REL_L2_VS_ORACLE, (rel_l2(d, want), cosine(d, truth))
    if residual:
        assert cosine(d, truth) > 0.999


def test_gemm_swap_ab_decode_routing(dev, oracle):
    """Decode-style routing: many experts, 1-16 real rows each padded to 16, the rest of
    every tile zero; padded rows must come out as exact zeros."""
    e, n, k = 24, 256, 512
    g = torch.Generator().manual_seed(11)
    real = torch.randint(1, 17, (e,), generator=g).tolist()
    real[3] = 0                                       # an expert without tokens gets no rows at all
    sizes = [((r + 15) // 16) * 16 for r in real]
    a = torch.zeros(sum(sizes), k, dtype=torch.bfloat16)
    off = 0
    for r, s_ in zip(real, sizes):
        a[off:off + r] = torch.randn(r, k, generator=g).to(torch.bfloat16)
        off += s_
    w = (torch.randn(e, n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes, alignment=16)
    d = run_gemm(dev, a, b, sfb, gw, mi, n, tune_swap_ab=1, m_alignment=16)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n)
    assert rel_l2(d, want) < REL_L2_VS_ORACLE
    zero_rows = a.float().abs().sum(dim=1) == 0
    assert float(d[zero_rows].float().abs().max()) == 0.0


@pytest.mark.parametrize("tile", [16, 32])
def test_gemm_swap_ab_k_block_variants_agree(dev, oracle, tile):
    """The decode kernel has 128-, 256- and 512-wide K blocks; on a K all three divide they must agree with
    the oracle and with each other (same codes and products, same summation order per accumulator)."""
    sizes, n, k = [tile, 3 * tile, tile], 384, 1536
    g = torch.Generator().manual_seed(77 + tile)
    a = torch.randn(sum(sizes), k, generator=g).to(torch.bfloat16)
    w = (torch.randn(len(sizes), n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices(sizes, alignment=tile)
    want = oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n)
    outs = [run_gemm(dev, a, b, sfb, gw, mi, n, tune_swap_ab=1, m_alignment=tile, tune_block_k=bk)
            for bk in (128, 256, 512)]
    for d in outs:
        assert rel_l2(d, want) < REL_L2_VS_ORACLE
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


def test_both_orientations_agree(dev):
    e, rows, n, k = 2, 128, 256, 512
    a, w = make_case(e, rows, n, k, seed=5)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    d0 = run_gemm(dev, a, b, sfb, gw, mi, n)
    d1 = run_gemm(dev, a, b, sfb, gw, mi, n, tune_swap_ab=1, m_alignment=128)
    assert rel_l2(d1, d0) < 1e-3          # same codes, same products; only the summation order differs


# ---------------------------------------------------------------- the split path's own bytes
def workspace_from_oracle(oracle, a, policy, residual):
    """oracle.decompose re-laid into the workspace layout of the split path."""
    o0, o1, s0, s1 = oracle.decompose(a, scale_policy=policy)
    m, k = a.shape
    atoms = torch.zeros(m // 128, k // 64, 2 if residual else 1, 512, dtype=torch.uint8)
    r = torch.arange(m)
    off = (r % 128 % 32) * 16 + (r % 128 // 32) * 4
    for p, sc in enumerate((s0, s1) if residual else (s0,)):
        sc4 = sc.reshape(m, k // 64, 4)
        for j in range(4):
            atoms[r // 128, :, p, off + j] = sc4[:, :, j]
    return o0, o1, atoms


@pytest.mark.parametrize("policy", POLICIES)
@pytest.mark.parametrize("residual", [True, False])
def test_split_workspace_byte_for_byte(dev, oracle, policy, residual):
    """The quantised activations the split GEMM consumes -- packed codes and the scale atoms in their tensor-memory
    image -- against the oracle, on config C1's activations and on the lognormal / Student-t / outlier inputs."""
    g = torch.Generator().manual_seed(0)
    inputs = [torch.randn(256, 1024, generator=g)]
    inputs.append(torch.randn(256, 512, generator=g) * torch.exp(0.5 * torch.randn(256, 1, generator=g)))
    inputs.append((torch.randn(128, 512, generator=g) / torch.sqrt(torch.randn(128, 512, 4, generator=g).pow(2).mean(-1))).clamp(-2688, 2688))
    x = torch.randn(128, 1024, generator=g)
    x[:, torch.randperm(1024, generator=g)[:2]] *= 50.0
    inputs.append(x)
    inputs.append(torch.randn(128, 256, generator=g) * 1e-3)
    for x in inputs:
        a = x.to(torch.bfloat16)
        a0, a1, sfa = _C.debug_split_workspace(a.to(dev), scale_policy=policy, enable_residual_pass=residual)
        o0, o1, atoms = workspace_from_oracle(oracle, a, policy, residual)
        assert torch.equal(sfa.cpu(), atoms), "scale atoms differ"
        assert torch.equal(grid_i8_from_codes(unpack_codes(a0)), grid_i8_from_codes(o0)), "A0 codes differ"
        if residual:
            assert torch.equal(grid_i8_from_codes(unpack_codes(a1)), grid_i8_from_codes(o1)), "A1 codes differ"


@pytest.mark.parametrize("residual", [True, False])
def test_split_workspace_swiglu_fold_byte_for_byte(dev, oracle, residual):
    """The SwiGLU-folded form: the workspace must hold Algorithm 1 of the BF16-rounded product silu(gate) * up as the
    stand-alone SwiGLU kernel computes it."""
    g = torch.Generator().manual_seed(5)
    h = (torch.randn(256, 2 * 384 + 16, generator=g) * 2).to(torch.bfloat16).to(dev)[:, :2 * 384]      # strided rows
    act = _C.swiglu(h.contiguous()).cpu()
    a0, a1, sfa = _C.debug_split_workspace(h, enable_residual_pass=residual, fold_swiglu=True)
    o0, o1, atoms = workspace_from_oracle(oracle, act, "derived_div8", residual)
    assert torch.equal(sfa.cpu(), atoms)
    assert torch.equal(grid_i8_from_codes(unpack_codes(a0)), grid_i8_from_codes(o0))
    if residual:
        assert torch.equal(grid_i8_from_codes(unpack_codes(a1)), grid_i8_from_codes(o1))


# ---------------------------------------------------------------- masked layout
@pytest.mark.parametrize("residual", [True, False])
@pytest.mark.parametrize("k", [512, 640])
@pytest.mark.parametrize("tune", [{}, dict(tune_cluster=2)], ids=["single", "pair"])
def test_gemm_masked_layout_matches_oracle(dev, oracle, residual, k, tune):
    """Groups with device-side row counts: empty groups, a full group, counts that are not multiples of 128, a count
    above max_m (clamped); rows past a group's last row block must stay untouched."""
    e, max_m, n = 6, 512, 1024
    counts = [300, 0, 512, 1, 129, 900]
    g = torch.Generator().manual_seed(77 + k)
    a = torch.randn(e, max_m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(e, n, k, generator=g) * 0.02).to(torch.bfloat16)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    d = torch.full((e, max_m, n), float("nan"), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    masked_m = torch.tensor(counts, dtype=torch.int32, device=dev)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_masked(a.to(dev), b, sfb, gw, d, masked_m, enable_residual_pass=residual,
                                                     device_status=status, **tune)
    torch.cuda.synchronize()
    assert _C.read_status(status) == 0
    dc = d.cpu()
    for grp, c in enumerate(counts):
        live = min((min(c, max_m) + 127) // 128 * 128, max_m)
        assert torch.isnan(dc[grp, live:].float()).all(), "rows past the last row block were written"
        if live == 0:
            continue
        want = oracle.grouped_gemm(a[grp, :live], b.cpu()[grp * n:(grp + 1) * n], sfb.cpu()[grp * (k // 64):(grp + 1) * (k // 64)],
                                   gw.cpu()[grp:grp + 1], torch.zeros(live, dtype=torch.int32), n,
                                   mode="dual" if residual else "single")
        assert rel_l2(dc[grp, :live], want) < REL_L2_VS_ORACLE, grp


def test_gemm_masked_layout_with_swiglu_fold_equals_contiguous(dev):
    """The masked call on full groups against the contiguous call on the same rows: same kernels, same bits."""
    e, max_m, inter, hidden = 3, 256, 384, 512
    g = torch.Generator().manual_seed(21)
    h = (torch.randn(e, max_m, 2 * inter, generator=g) * 2).to(torch.bfloat16).to(dev)
    w = (torch.randn(e, hidden, inter, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w)
    d_masked = torch.zeros(e, max_m, hidden, dtype=torch.bfloat16, device=dev)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_masked(h, b, sfb, gw, d_masked, torch.full((e,), max_m, dtype=torch.int32, device=dev),
                                                     fold_swiglu=True)
    d_contig = torch.zeros(e * max_m, hidden, dtype=torch.bfloat16, device=dev)
    _C.m_grouped_swiglu_dual_nvfp4_gemm_contiguous(h.reshape(e * max_m, -1), b, sfb, gw, d_contig,
                                                   nvfp4_gemm.make_m_indices([max_m] * e).to(dev))
    torch.cuda.synchronize()
    assert torch.equal(d_masked.reshape(e * max_m, hidden), d_contig)


@pytest.mark.parametrize("inter,k", [(128, 256), (384, 640), (512, 1024)])
@pytest.mark.parametrize("cluster", [1, 2], ids=["single", "pair"])
def test_up_projection_with_swiglu_and_quantisation_in_its_epilogue(dev, inter, k, cluster):
    """The masked up-projection that writes the down-projection's quantised workspace straight from its epilogue
    (gate/up-interleaved weights) against the unfused sequence -- BF16 gate+up output, then the SwiGLU-folded activation
    quantisation: codes and scale atoms of every live row block byte for byte; then the down-projection on both."""
    e, max_m, hidden_out = 3, 384, 256
    counts = [384, 130, 0]
    g = torch.Generator().manual_seed(60 + inter + k)
    a = torch.randn(e * max_m, k, generator=g).to(torch.bfloat16).to(dev)
    w_up = (torch.randn(e, 2 * inter, k, generator=g) * 0.08).to(torch.bfloat16).to(dev)
    w_down = (torch.randn(e, hidden_out, inter, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    up, down = nvfp4_gemm.quantize_weight_nvfp4(w_up), nvfp4_gemm.quantize_weight_nvfp4(w_down)
    masked_m = torch.tensor(counts, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rows = _C.QuantizedRows(torch.zeros(e * max_m * (k + k // 8), dtype=torch.uint8, device=dev), e, max_m, k)
    a0, a1, sfa = _C.debug_split_workspace(a)
    rows.a0.copy_(a0); rows.a1.copy_(a1); rows.scale_atoms.copy_(sfa)
    tune = dict(tune_cluster=cluster)
    # unfused: BF16 h, then quantise silu(gate) * up
    h = torch.zeros(e, max_m, 2 * inter, dtype=torch.bfloat16, device=dev)
    _C.m_grouped_quantized_dual_nvfp4_gemm_masked(rows, *up, h, masked_m, device_status=status, **tune)
    want0, want1, want_sf = _C.debug_split_workspace(h.reshape(e * max_m, 2 * inter), fold_swiglu=True)
    # fused
    hq = _C.QuantizedRows(torch.zeros(e * max_m * (inter + inter // 8), dtype=torch.uint8, device=dev), e, max_m, inter)
    bi, sfbi = _C.interleave_gate_up(up[0], up[1], e, inter)
    _C.m_grouped_quantized_swiglu_dual_nvfp4_gemm_masked(rows, bi, sfbi, up[2], hq, masked_m, device_status=status, **tune)
    torch.cuda.synchronize()
    assert _C.read_status(status) == 0
    for grp, c in enumerate(counts):
        live = (c + 127) // 128 * 128
        lo = grp * max_m
        assert torch.equal(hq.a0[lo:lo + live], want0[lo:lo + live]) and torch.equal(hq.a1[lo:lo + live], want1[lo:lo + live]), grp
        assert torch.equal(hq.scale_atoms[lo // 128:(lo + live) // 128], want_sf[lo // 128:(lo + live) // 128]), grp
        assert int(hq.a0[lo + live:lo + max_m].max() if live < max_m else 0) == 0          # dead row blocks untouched
    d_fused = torch.zeros(e, max_m, hidden_out, dtype=torch.bfloat16, device=dev)
    d_plain = torch.zeros_like(d_fused)
    _C.m_grouped_quantized_dual_nvfp4_gemm_masked(hq, *down, d_fused, masked_m, device_status=status)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_masked(h, *down, d_plain, masked_m, fold_swiglu=True, device_status=status)
    torch.cuda.synchronize()
    assert _C.read_status(status) == 0 and torch.equal(d_fused, d_plain)


# ---------------------------------------------------------------- checkpoint loader
def to_checkpoint(b, sfb, gw, e, n, k, divisor):
    from nvfp4_cutlass_b200.layout import unpack_sf_atoms
    return (b.view(torch.uint8).reshape(e, n, k // 2), unpack_sf_atoms(sfb, e), (1.0 / gw) if divisor else gw.clone())


@pytest.mark.parametrize("divisor", [False, True])
def test_checkpoint_loader_fuses_gate_and_up_byte_exact(dev, oracle, divisor):
    """Gate and up projections quantised separately (own global scales) -> one fused (b, sfb, gw): byte for byte
    against the CPU restatement of the re-folding rule, and close to the two parts dequantised on their own."""
    from oracle import checkpoint
    e, n_half, k = 4, 192, 256
    g = torch.Generator().manual_seed(8)
    wg = (torch.randn(e, n_half, k, generator=g) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(e, n_half, k, generator=g) * 0.07).to(torch.bfloat16)
    wu[2] *= 0.1                                                       # an expert whose gate scale is the larger one
    qg, qu = oracle.quantize_weight(wg), oracle.quantize_weight(wu)
    parts = [to_checkpoint(*qg, e, n_half, k, divisor), to_checkpoint(*qu, e, n_half, k, divisor)]
    b, sfb, gw = nvfp4_gemm.load_checkpoint_weights_nvfp4([tuple(t.to(dev) for t in p) for p in parts], global_scale_is_divisor=divisor)
    ob, osfb, ogw = checkpoint.load_checkpoint_weights(parts, global_scale_is_divisor=divisor)
    assert torch.equal(gw.cpu(), ogw) and torch.equal(sfb.cpu(), osfb) and torch.equal(b.cpu(), ob)
    fused = oracle.dequantize_weight(b.cpu(), sfb.cpu(), gw.cpu(), e, 2 * n_half, k)
    apart = torch.cat([oracle.dequantize_weight(*qg, e, n_half, k), oracle.dequantize_weight(*qu, e, n_half, k)], dim=1)
    assert rel_l2(fused, apart) < 0.03                                 # one more E4M3 rounding of the block scales
    # and the fused weights run: GEMM on them against the oracle on the same bytes
    a = torch.randn(e * 128, k, generator=g).to(torch.bfloat16)
    mi = nvfp4_gemm.make_m_indices([128] * e)
    d = run_gemm(dev, a, b, sfb, gw, mi, 2 * n_half)
    assert rel_l2(d, oracle.grouped_gemm(a, ob, osfb, ogw, mi, 2 * n_half)) < REL_L2_VS_ORACLE


def test_checkpoint_loader_single_part_round_trip(dev, oracle):
    """A down projection (one part): the loader returns the checkpoint's own codes and scales bit for bit."""
    e, n, k = 3, 256, 384 + 128
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(e, n, k, generator=g) * 0.03).to(torch.bfloat16)
    ob, osfb, ogw = oracle.quantize_weight(w)
    part = to_checkpoint(ob, osfb, ogw, e, n, k, divisor=False)
    b, sfb, gw = nvfp4_gemm.load_checkpoint_weights_nvfp4([tuple(t.to(dev) for t in part)], global_scale_is_divisor=False)
    assert torch.equal(b.cpu(), ob) and torch.equal(sfb.cpu(), osfb) and torch.equal(gw.cpu(), ogw)


# ---------------------------------------------------------------- bounded waits and status
def test_bounded_wait_runs_out_cleanly(dev, oracle):
    """A wait nobody satisfies expires after its budget: status bit 0 is set, the kernel returns, tensor memory is
    free again (a GEMM that needs all 512 columns runs right after it) and read_status reports the timeout once."""
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _C.debug_wait_timeout(1_000_000, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    with pytest.raises(RuntimeError, match="error 4"):
        _C.read_status(status)
    assert _C.read_status(status) == 0                         # cleared by the read
    e, rows, n, k = 1, 128, 256, 256
    a, w = make_case(e, rows, n, k, seed=3)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    d = run_gemm(dev, a, b, sfb, gw, mi, n)
    assert rel_l2(d, oracle.grouped_gemm(a, b.cpu(), sfb.cpu(), gw.cpu(), mi, n)) < REL_L2_VS_ORACLE


@pytest.mark.parametrize("no_pdl", [0, 1])
def test_back_to_back_calls_chained_by_dependent_launch(dev, oracle, no_pdl):
    """up -> down -> up ... on one stream without host synchronisation, every kernel launched with programmatic
    stream serialisation (or without: tune_no_pdl): each call must see the previous call's output."""
    e, rows, hidden, inter = 2, 256, 512, 1024
    g = torch.Generator().manual_seed(15)
    x = torch.randn(e * rows, hidden, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(e, inter, hidden, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(e, hidden, inter, generator=g) * 0.05).to(torch.bfloat16)
    q1, q2 = nvfp4_gemm.quantize_weight_nvfp4(w1.to(dev)), nvfp4_gemm.quantize_weight_nvfp4(w2.to(dev))
    mi = nvfp4_gemm.make_m_indices([rows] * e)
    mid, xd = mi.to(dev), x.to(dev)
    h = torch.empty(e * rows, inter, dtype=torch.bfloat16, device=dev)
    y = torch.empty(e * rows, hidden, dtype=torch.bfloat16, device=dev)
    for kw in (dict(), dict(tune_split_transform=2), dict(tune_swap_ab=1, m_alignment=128)):
        h.zero_(); y.zero_()
        for _ in range(3):
            nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(xd, *q1, h, mid, tune_no_pdl=no_pdl, **kw)
            nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(h, *q2, y, mid, tune_no_pdl=no_pdl, **kw)
        torch.cuda.synchronize()
        h_want = oracle.grouped_gemm(x, q1[0].cpu(), q1[1].cpu(), q1[2].cpu(), mi, inter)
        assert rel_l2(h.cpu(), h_want) < REL_L2_VS_ORACLE
        y_want = oracle.grouped_gemm(h.cpu(), q2[0].cpu(), q2[1].cpu(), q2[2].cpu(), mi, hidden)
        assert rel_l2(y.cpu(), y_want) < REL_L2_VS_ORACLE
