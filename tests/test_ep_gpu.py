"""GPU tests of the expert-parallel layer's own kernels (row movers, SwiGLU, weighted combine) and of one
layer step on one rank, against the same computation written with tensor operations."""
import pytest
import torch

import nvfp4_gemm
from nvfp4_cutlass_b200 import _C
from nvfp4_cutlass_b200.ep import ExpertParallelMoE, route_topk

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def test_permute_rows_gather_scatter_and_fused(dev):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(37, 264, generator=g).to(torch.bfloat16).to(dev)[:, :256]       # strided rows
    k, n = 3, 37 * 3
    order = torch.randperm(n, generator=g).to(dev)
    place = torch.randperm(200, generator=g)[:n].to(dev)
    gathered = torch.empty(n, 256, dtype=torch.bfloat16, device=dev)
    _C.permute_rows(x, n, gathered, src_idx=order, src_div=k)
    assert torch.equal(gathered, x[order // k])
    scattered = torch.zeros(200, 256, dtype=torch.bfloat16, device=dev)
    _C.permute_rows(gathered, n, scattered, dst_idx=place)
    want = torch.zeros_like(scattered)
    want[place] = x[order // k]
    assert torch.equal(scattered, want)
    fused = torch.zeros_like(scattered)
    _C.permute_rows(x, n, fused, src_idx=order, src_div=k, dst_idx=place)
    assert torch.equal(fused, want)
    _C.permute_rows(x, 0, fused)                                                     # empty: no launch, no error


def test_swiglu_matches_tensor_ops(dev):
    g = torch.Generator().manual_seed(2)
    h = (torch.randn(300, 512, generator=g) * 3).to(torch.bfloat16).to(dev)
    got = _C.swiglu(h)
    gate, up = h.float().chunk(2, dim=-1)
    want = (torch.nn.functional.silu(gate) * up).to(torch.bfloat16)
    assert got.shape == want.shape
    assert rel_l2(got, want) < 2e-3          # same FP32 formula; exp differs in the last bits


@pytest.mark.parametrize("residual", [True, False])
def test_swiglu_folded_into_the_down_projection_is_bit_identical(dev, residual):
    """nvfp4_grouped_gemm_swiglu_contiguous against nvfp4_swiglu followed by the split-path GEMM."""
    e, rows, inter, hidden = 3, 256, 384, 512
    g = torch.Generator().manual_seed(12)
    h = (torch.randn(e * rows, 2 * inter + 16, generator=g) * 2).to(torch.bfloat16).to(dev)[:, :2 * inter]   # strided rows
    w = (torch.randn(e, hidden, inter, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    b, sfb, gw = nvfp4_gemm.quantize_weight_nvfp4(w)
    mi = nvfp4_gemm.make_m_indices([rows] * e).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    fused = torch.empty(e * rows, hidden, dtype=torch.bfloat16, device=dev)
    _C.m_grouped_swiglu_dual_nvfp4_gemm_contiguous(h, b, sfb, gw, fused, mi, enable_residual_pass=residual, device_status=status)
    plain = torch.empty_like(fused)
    nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(_C.swiglu(h.contiguous()), b, sfb, gw, plain, mi,
                                                         enable_residual_pass=residual, tune_split_transform=1, device_status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.isfinite(fused.float()).all() and torch.equal(fused, plain)


def test_combine_rows_matches_tensor_ops(dev):
    g = torch.Generator().manual_seed(3)
    tokens, k, hidden = 50, 4, 384
    rows = torch.randn(tokens * k + 9, hidden, generator=g).to(torch.bfloat16).to(dev)
    pos = torch.randperm(tokens * k + 9, generator=g)[:tokens * k].to(dev)
    w = torch.rand(tokens * k, generator=g).to(dev)
    got = _C.combine_rows(rows, pos, w, tokens)
    want = (rows[pos].float() * w.unsqueeze(1)).reshape(tokens, k, hidden).sum(dim=1).to(torch.bfloat16)
    assert rel_l2(got, want) < 2e-3


@pytest.mark.parametrize("hidden,k", [(1024, 8), (4096, 8), (2048, 3), (512, 16)])
def test_combine_over_peer_memory_bulk_copies_equal_thread_loads(dev, hidden, k):
    """The combine that fetches rows by bulk copies into shared memory against the one that loads them per thread and
    against tensor operations: same ascending-j FP32 sum, same bits; pairs out of range contribute nothing; more tokens
    than the ring has slots per CTA."""
    tokens, rows_cap = 700, 3000
    g = torch.Generator().manual_seed(31 + hidden)
    rows = torch.randn(rows_cap, hidden, generator=g).to(torch.bfloat16).to(dev)
    src_row = torch.randint(0, rows_cap, (tokens * k,), generator=g).to(dev)
    src_row[3] = -1
    src_row[11] = rows_cap + 5
    src_rank = torch.zeros(tokens * k, dtype=torch.int64, device=dev)
    src_rank[20] = 7                                                       # no such rank
    w = torch.rand(tokens * k, generator=g).to(dev)
    peers = torch.tensor([rows.data_ptr()], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    bulk = _C.combine_rows_peer(peers, hidden, src_rank, src_row, w, tokens, hidden, rows_cap, bulk=True, status=status)
    few = _C.combine_rows_peer(peers, hidden, src_rank, src_row, w, tokens, hidden, rows_cap, bulk=True, status=status, sm_budget=3)
    plain = _C.combine_rows_peer(peers, hidden, src_rank, src_row, w, tokens, hidden, rows_cap, bulk=False)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(bulk, plain) and torch.equal(few, plain)
    ok = (src_row >= 0) & (src_row < rows_cap) & (src_rank == 0)
    want = (rows[src_row.clamp(0, rows_cap - 1)].float() * (w * ok).unsqueeze(1)).reshape(tokens, k, hidden).sum(dim=1)
    assert rel_l2(bulk, want.to(torch.bfloat16)) < 4e-3


def test_layer_step_native_glue_matches_tensor_glue(dev):
    """One rank, 8 experts: the layer with the library's kernels against the layer with tensor operations
    around the same GEMM calls."""
    e, hidden, inter, tokens, k = 8, 512, 256, 640, 2
    g = torch.Generator().manual_seed(4)
    up_w = (torch.randn(e, 2 * inter, hidden, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    down_w = (torch.randn(e, hidden, inter, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    up, down = nvfp4_gemm.quantize_weight_nvfp4(up_w), nvfp4_gemm.quantize_weight_nvfp4(down_w)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(dev)
    ids, wts = route_topk(torch.randn(tokens, e, generator=g).to(dev), k)
    native = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128)(x, ids, wts)
    plain = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, native_glue=False)(x, ids, wts)
    planned = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=512)   # masked layout, local buffers
    assert planned.peer is not None
    fast = [planned(x, ids, wts) for _ in range(2)]
    halves = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=512, micro_batches=2)(x, ids, wts)
    tiny = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=128)      # some expert overflows
    repeated = tiny(x, ids, wts)
    torch.cuda.synchronize()
    assert native.shape == (tokens, hidden) and torch.isfinite(native.float()).all()
    assert rel_l2(native, plain) < 5e-3
    # same rows in the same order per expert, same kernels, same summation order: the same bits
    assert torch.equal(fast[0], native) and torch.equal(fast[1], native) and torch.equal(halves, native)
    assert planned.steps_repeated == 0 and tiny.steps_repeated == 1 and torch.equal(repeated, native)


@pytest.mark.parametrize("hidden", [1024, 3072])
def test_quantized_dispatch_writes_the_gemm_workspace_byte_for_byte(dev, hidden):
    """The sender-side quantisation against the GEMM's own: rows scattered as NVFP4 codes + scale rows (and re-laid into
    atoms) must equal, byte for byte, what the split path's quantisation kernel makes of the same BF16 rows after the
    BF16 dispatch.  Out-of-range pairs are skipped and reported."""
    tokens, k, e, cap_m = 200, 3, 2, 384
    g = torch.Generator().manual_seed(77)
    x = (torch.randn(tokens, hidden, generator=g) * torch.exp(torch.randn(tokens, 1, generator=g))).to(torch.bfloat16).to(dev)
    perm = torch.randperm(e * cap_m, generator=g)[:tokens * k]
    dst_row = perm.to(dev)
    dst_row[5] = -1                                                        # a pair that did not fit: skipped silently
    dst_rank = torch.zeros(tokens * k, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rows = _C.QuantizedRows(torch.zeros(e * cap_m * (hidden + hidden // 8), dtype=torch.uint8, device=dev), e, cap_m, hidden)
    peers = torch.tensor([rows.store.data_ptr()], dtype=torch.int64, device=dev)
    _C.dispatch_quantized_peer(x, k, peers, dst_rank, dst_row, rows, status)
    _C.relayout_scales(rows)
    bf16 = torch.zeros(e * cap_m, hidden, dtype=torch.bfloat16, device=dev)
    _C.dispatch_rows_peer(x, None, k, torch.tensor([bf16.data_ptr()], dtype=torch.int64, device=dev), dst_rank, dst_row, hidden,
                          e * cap_m, status)
    a0, a1, sfa = _C.debug_split_workspace(bf16)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    live = torch.zeros(e * cap_m, dtype=torch.bool, device=dev)
    live[dst_row[dst_row >= 0]] = True
    assert torch.equal(rows.a0[live], a0[live]) and torch.equal(rows.a1[live], a1[live])
    # scale atoms: compare the words of the live rows (rows nobody wrote hold zeros on one side, the scale floor on the other)
    r = torch.arange(e * cap_m, device=dev)
    def words(atoms):
        at = atoms.reshape(e * cap_m // 128, hidden // 64, 2, 32, 4, 4)    # [row block][atom][pass][r % 32][r / 32][byte]
        return at[r // 128, :, :, r % 32, (r % 128) // 32]                 # (rows, atoms, passes, 4 bytes)
    assert torch.equal(words(rows.scale_atoms)[live], words(sfa)[live])
    dst_row[7] = e * cap_m + 3                                             # out of range: skipped, bit 3
    _C.dispatch_quantized_peer(x, k, peers, dst_rank, dst_row, rows, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 8


def test_layer_with_quantized_dispatch_equals_bf16_dispatch(dev):
    """One rank: the layer whose dispatch sends NVFP4 codes against the layer whose dispatch sends BF16 rows -- the same
    codes reach the same GEMM kernels, so the outputs are identical; both against the all-to-all path."""
    e, hidden, inter, tokens, k = 4, 1024, 128, 300, 2
    g = torch.Generator().manual_seed(15)
    up_w = (torch.randn(e, 2 * inter, hidden, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    down_w = (torch.randn(e, hidden, inter, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    up, down = nvfp4_gemm.quantize_weight_nvfp4(up_w), nvfp4_gemm.quantize_weight_nvfp4(down_w)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(dev)
    ids, wts = route_topk(torch.randn(tokens, e, generator=g).to(dev), k)
    quant = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=256)
    plain = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=256, quantized_dispatch=False)
    unfused = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=256, fused_swiglu=False)
    assert quant.peer[0].q is not None and plain.peer[0].q is None
    # SwiGLU + the down-projection's quantisation in the up-projection's epilogue is on by default with quantised rows
    assert quant.peer[0].hq is not None and unfused.peer[0].hq is None and unfused.peer[0].q is not None
    yq = [quant(x, ids, wts) for _ in range(2)]
    yp = plain(x, ids, wts)
    assert torch.equal(unfused(x, ids, wts), yp)
    ya = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128)(x, ids, wts)
    torch.cuda.synchronize()
    assert quant.steps_repeated == 0 and plain.steps_repeated == 0
    assert torch.equal(yq[0], yp) and torch.equal(yq[1], yp) and torch.equal(yp, ya)


def test_layer_step_against_the_oracle_dense_reference(dev):
    """One rank, the layer with the CUDA kernels against the single-process oracle statement of the same layer (per
    expert, oracle GEMMs on its rows): the layer is compared with the CPU oracle, not only with itself."""
    import oracle
    from test_ep_cpu import _dense_reference
    e, hidden, inter, tokens, k = 4, 256, 128, 96, 2
    g = torch.Generator().manual_seed(14)
    up_w = (torch.randn(e, 2 * inter, hidden, generator=g) * 0.05).to(torch.bfloat16)
    down_w = (torch.randn(e, hidden, inter, generator=g) * 0.05).to(torch.bfloat16)
    up, down = nvfp4_gemm.quantize_weight_nvfp4(up_w.to(dev)), nvfp4_gemm.quantize_weight_nvfp4(down_w.to(dev))
    oup = oracle.quantize_weight(up_w)
    assert all(torch.equal(a.cpu(), b) for a, b in zip(up, oup))
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    ids, wts = route_topk(torch.randn(tokens, e, generator=g), k)
    ref = _dense_reference(x, ids, wts, up_w, down_w, 128)
    for kw in (dict(), dict(peer_rows_cap=128)):
        y = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, **kw)(x.to(dev), ids.to(dev), wts.to(dev))
        torch.cuda.synchronize()
        # the SwiGLU in between uses the device exponential; one BF16 ulp of the intermediate moves a few codes
        assert rel_l2(y.cpu(), ref) < 2e-2, kw


def test_bounded_barrier_times_out_without_hanging(dev):
    """A barrier whose peer never arrives: two 'ranks' whose flag arrays both live on this GPU, only rank 0 ever calls.
    The wait runs out after its budget, bit 1 of the status word is set, the stream carries on and the context stays
    usable; a later call with the peer's flag set passes at once."""
    flags = torch.zeros(2, 8 * 2, dtype=torch.int64, device=dev)          # [rank][slot * world + src]
    peers = torch.tensor([flags[0].data_ptr(), flags[1].data_ptr()], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _C.peer_barrier(peers, 0, 2, 3, 1, status, budget_cycles=2_000_000)
    torch.cuda.synchronize()
    assert int(status.item()) == 2
    assert int(flags[1, 3 * 2 + 0].item()) == 1                           # rank 0 did announce itself to rank 1
    status.zero_()
    flags[0, 3 * 2 + 1] = 2                                               # "rank 1 has reached epoch 2"
    _C.peer_barrier(peers, 0, 2, 3, 2, status, budget_cycles=2_000_000)
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def _two_rank_worker(rank, world, port, results, hidden):
    import os
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        e, hidden, inter, tokens, k = 8, hidden, 256, 384 + 128 * rank, 2
        e_local = e // world
        g = torch.Generator().manual_seed(4)
        up_w = (torch.randn(e, 2 * inter, hidden, generator=g) * 0.05).to(torch.bfloat16)
        down_w = (torch.randn(e, hidden, inter, generator=g) * 0.05).to(torch.bfloat16)
        lo = rank * e_local
        up = nvfp4_gemm.quantize_weight_nvfp4(up_w[lo:lo + e_local].to(dev))
        down = nvfp4_gemm.quantize_weight_nvfp4(down_w[lo:lo + e_local].to(dev))
        g = torch.Generator().manual_seed(40 + rank)
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(dev)
        ids, wts = route_topk(torch.randn(tokens, e, generator=g).to(dev), k)
        a2a = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128)
        peer = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=512)
        y_a2a = a2a(x, ids, wts)
        ys = [peer(x, ids, wts) for _ in range(3)]            # repeated steps reuse the buffers
        # other tokens through the same buffers: nothing of the earlier steps may survive in any cache on the way
        x2 = (x.float() * -0.5 + 0.25).to(torch.bfloat16)
        fresh = rel_l2(peer(x2, ids, wts), a2a(x2, ids, wts))
        halves = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=512, micro_batches=2)
        y_halves = [halves(x, ids, wts) for _ in range(2)][1]
        tiny = ExpertParallelMoE(e, hidden, inter, up, down, alignment=128, peer_rows_cap=128)
        y_fallback = tiny(x, ids, wts)                        # does not fit: every rank takes the all-to-all path
        torch.cuda.synchronize()
        results[rank] = (peer.peer is not None and (peer.peer[0].q is not None) == (hidden % 1024 == 0), peer.peer_error,
                         rel_l2(ys[0], y_a2a), rel_l2(ys[2], y_a2a),
                         max(rel_l2(y_fallback, y_a2a), rel_l2(y_halves, y_a2a), fresh), bool(torch.isfinite(ys[2].float()).all()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("hidden", [512, 1024], ids=["bf16_rows", "quantised_rows"])
def test_two_ranks_peer_memory_path_matches_all_to_all_path(hidden):
    """Two GPUs: dispatch/combine over peer memory against the NCCL all-to-all path, same routing; hidden = 1024 sends
    the rows quantised."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_two_rank_worker, args=(2, port, results, hidden), nprocs=2, join=True)
    for rank in range(2):
        has_peer, err, first, third, fallback, finite = results[rank]
        assert has_peer, err
        assert finite
        assert first < 1e-6 and third < 1e-6, (first, third)     # same rows, same kernels, same summation order
        assert fallback < 1e-6


@pytest.mark.parametrize("rank", [0, 2, 3])
@pytest.mark.parametrize("cap_m", [2048, 128])
def test_masked_plan_kernels_match_tensor_ops(dev, rank, cap_m):
    """The plan kernels of the masked layout against the same plan written with tensor operations (the CPU form of
    plan_dispatch_masked): rows, per-expert counts and the overflow bit; the small capacity overflows."""
    from nvfp4_cutlass_b200.ep import plan_dispatch_masked
    world, num_experts, n = 4, 16, 3000
    g = torch.Generator().manual_seed(9)
    ids_all = [torch.randint(0, num_experts, (n + 37 * s,), generator=g) for s in range(world)]
    for t in ids_all:
        t[t == 5] = 6                                            # an expert nobody routes to
    all_counts = torch.stack([torch.bincount(t, minlength=num_experts) for t in ids_all])
    flat = ids_all[rank]
    assert torch.equal(_C.expert_histogram(flat.to(dev), num_experts).cpu(), all_counts[rank])
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    masked_m, dst_row = _C.plan_peer_masked(all_counts.reshape(-1).to(dev), flat.to(dev), world, rank, cap_m, status)
    torch.cuda.synchronize()
    # the tensor-operation form, fed the same gathered counts through a stand-in for the all-gather
    import torch.distributed as dist
    from unittest import mock
    with mock.patch.object(dist, "all_gather_into_tensor", lambda out, inp, group=None: out.copy_(all_counts.reshape(-1))):
        want = plan_dispatch_masked(flat.reshape(-1, 1), num_experts, world, rank, cap_m)
    assert torch.equal(dst_row.cpu(), want.dst_row)
    assert torch.equal(masked_m.cpu(), want.masked_m)
    assert bool(int(status.item()) & 4) == bool(want.overflow) == (cap_m == 128)
