"""CPU: the expert-parallel layer's routing, dispatch, padding and combine logic on gloo
ranks (world size 1 and 2), with the CPU oracle standing in for the CUDA GEMM."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _oracle_gemm(a, b, sfb, gw, d, m_indices, **_):
    import oracle
    d.copy_(oracle.grouped_gemm(a, b, sfb, gw, m_indices, d.shape[1]))


def _make_layer_inputs(num_experts, hidden, inter, tokens, top_k, seed):
    g = torch.Generator().manual_seed(seed)
    w_up = (torch.randn(num_experts, 2 * inter, hidden, generator=g) * 0.05).to(torch.bfloat16)
    w_down = (torch.randn(num_experts, hidden, inter, generator=g) * 0.05).to(torch.bfloat16)
    return w_up, w_down


def _dense_reference(x, ids, wts, w_up, w_down, alignment):
    """Single-process statement of the same layer: per expert, oracle GEMMs on its rows."""
    import oracle
    from nvfp4_cutlass_b200.ep import swiglu
    y = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32)
    for e in range(w_up.shape[0]):
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        up = oracle.quantize_weight(w_up[e:e + 1])
        down = oracle.quantize_weight(w_down[e:e + 1])
        mi = torch.zeros(tok.numel(), dtype=torch.int32)
        h = oracle.grouped_gemm(x[tok], *up, mi, w_up.shape[1])
        o = oracle.grouped_gemm(swiglu(h), *down, mi, w_down.shape[1])
        y.index_add_(0, tok, o.float() * wts[tok, slot].unsqueeze(1))
    return y.to(torch.bfloat16)


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from nvfp4_cutlass_b200.ep import ExpertParallelMoE, route_topk
        num_experts, hidden, inter, tokens, top_k, alignment = 8, 128, 64, 40, 2, 16
        w_up, w_down = _make_layer_inputs(num_experts, hidden, inter, tokens, top_k, seed=5)
        e_local = num_experts // world
        lo = rank * e_local
        up = oracle.quantize_weight(w_up[lo:lo + e_local])
        down = oracle.quantize_weight(w_down[lo:lo + e_local])
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
        logits = torch.randn(tokens, num_experts, generator=g)
        logits[:, 5] = -1e9                                   # an expert nobody routes to
        ids, wts = route_topk(logits, top_k)
        layer = ExpertParallelMoE(num_experts, hidden, inter, up, down, alignment=alignment, gemm=_oracle_gemm)
        y = layer(x, ids, wts)
        ref = _dense_reference(x, ids, wts, w_up, w_down, alignment)
        err = float((y.float() - ref.float()).norm() / ref.float().norm())
        plan = layer.last
        ok_pad = all(s % alignment == 0 for s in plan.group_sizes) and plan.rows_padded == sum(plan.group_sizes)
        results[rank] = (err, ok_pad, sum(plan.real_sizes))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [1, 2])
def test_expert_parallel_layer_matches_dense(world):
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world
    total_rows = 0
    for rank in range(world):
        err, ok_pad, rows = results[rank]
        assert ok_pad
        assert err < 2e-2, err          # same rows, same codes; only BF16 rounding of the weighted sum differs
        total_rows += rows
    assert total_rows == world * 40 * 2  # every (token, expert) pair arrived somewhere exactly once


def test_plan_dispatch_places_rows_by_expert():
    from nvfp4_cutlass_b200.ep import plan_dispatch
    ids = torch.tensor([[0, 3], [3, 1], [2, 3], [0, 1]])
    plan = plan_dispatch(ids, num_experts=4, world=1, alignment=4)
    assert plan.real_sizes == [2, 2, 1, 3] and plan.group_sizes == [4, 4, 4, 4]
    flat = ids.reshape(-1)
    experts_in_order = flat[plan.order]
    assert experts_in_order.tolist() == sorted(flat.tolist())
    # rows of expert e land in [4e, 4e + real)
    for pos, e in zip(plan.place.tolist(), experts_in_order.tolist()):
        assert 4 * e <= pos < 4 * e + plan.real_sizes[e]
    assert len(set(plan.place.tolist())) == flat.numel()


def _peer_plan_worker(rank, world, port, results):
    """The peer-memory (masked layout) plan against the all-to-all plan: storing every rank's rows at (dst_rank,
    dst_row) must give every local expert, in the first masked_m rows of its cap_m-row group, exactly the rows -- in
    the same order -- that the all-to-all dispatch puts into that expert's padded group."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvfp4_cutlass_b200.ep import ExpertParallelMoE, plan_dispatch_masked, route_topk
        num_experts, hidden, tokens, top_k, alignment, cap_m = 8, 32, 24 + 5 * rank, 3, 16, 48
        e_local = num_experts // world
        g = torch.Generator().manual_seed(7 + rank)
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
        logits = torch.randn(tokens, num_experts, generator=g)
        logits[:, 2] = -1e9
        ids, _ = route_topk(logits, top_k)
        layer = ExpertParallelMoE(num_experts, hidden, 16, None, None, alignment=alignment, gemm=_oracle_gemm)
        plan_a2a, a_want = layer.dispatch(x, ids)
        plan = plan_dispatch_masked(ids, num_experts, world, rank, cap_m)
        tight = plan_dispatch_masked(ids, num_experts, world, rank, 2)          # a capacity nobody fits
        rows = x[torch.arange(tokens * top_k) // top_k]
        mine = [None] * world
        dist.all_gather_object(mine, (plan.dst_rank.tolist(), plan.dst_row.tolist(), rows.float().tolist()))
        a_got = torch.zeros(e_local, cap_m, hidden, dtype=torch.bfloat16)
        written = set()
        for dst_rank, dst_row, r in mine:
            for dr, row, vals in zip(dst_rank, dst_row, r):
                if dr == rank:
                    assert row not in written and 0 <= row < e_local * cap_m
                    written.add(row)
                    a_got.reshape(-1, hidden)[row] = torch.tensor(vals).to(torch.bfloat16)
        same = True
        start = 0
        for j in range(e_local):
            real, padded = plan_a2a.real_sizes[j], plan_a2a.group_sizes[j]
            same &= int(plan.masked_m[j]) == real
            same &= torch.equal(a_got[j, :real], a_want[start:start + real])
            same &= bool((a_got[j, real:] == 0).all())
            start += padded
        results[rank] = (same, len(written) == sum(plan_a2a.real_sizes), not bool(plan.overflow), bool(tight.overflow),
                         int((tight.dst_row == -1).sum()) > 0 and int(tight.masked_m.max()) <= 2)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_masked_peer_plan_gives_every_expert_the_rows_of_the_all_to_all_plan(world):
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_peer_plan_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        assert all(results[rank]), results[rank]
