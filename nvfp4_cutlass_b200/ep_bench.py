"""Benchmark leg of the expert-parallel MoE layer (called by bench.py for workload c5).

Qwen3-235B-A22B-like layer: E = 128 experts split evenly over the ranks, 16384 tokens per
rank (weak scaling), top-8 softmax routing of Gaussian logits, hidden 4096, expert
intermediate 1536 (up N = 3072 = 2 x 1536, K = 4096; down N = 4096, K = 1536), Student-t(4)
activations clamped to +-2688.  A step is dispatch all-to-all -> up GEMM -> SwiGLU -> down
GEMM -> combine all-to-all + weighted sum.  ``value`` is the logical GEMM TFLOP/s of the
whole job: sum over ranks of 2 * real rows * (N_up * K_up + N_down * K_down), divided by
the slowest rank's device time.
"""
from __future__ import annotations

import json
import os
import statistics
import time

import torch
import torch.distributed as dist

E_TOTAL, HIDDEN, INTER, TOKENS, TOP_K = 128, 4096, 1536, 16384, 8


def expert_rows_cap(world: int, micro: int) -> int:
    """Rows every local expert owns per micro-batch: 1.5 x the average it receives, plus a tile."""
    avg = TOKENS * TOP_K * world // E_TOTAL // micro
    return (avg * 3 // 2 + 128 + 127) // 128 * 128


def one_gpu_record(dev, local: int, fp4_peak: float, steps: int = 5) -> dict:
    """The layer at one rank (all 128 experts local, the dispatch and combine kernels on local buffers), as a
    sub-record of the one-GPU benchmark line: ms per step and its phases."""
    import bench
    import nvfp4_gemm  # noqa: F401
    from .ep import ExpertParallelMoE, route_topk
    up = bench.build_weights(E_TOTAL, 2 * INTER, HIDDEN, dev, seed=20)
    down = bench.build_weights(E_TOTAL, HIDDEN, INTER, dev, seed=40)
    g = torch.Generator(device=dev).manual_seed(10)
    z = torch.randn(TOKENS, HIDDEN, generator=g, device=dev)
    chi = torch.randn(TOKENS, HIDDEN, 4, generator=g, device=dev).pow(2).mean(-1).sqrt()
    x = (z / chi).clamp(-2688.0, 2688.0).to(torch.bfloat16)
    del z, chi
    logits = torch.randn(TOKENS, E_TOTAL, generator=torch.Generator(device=dev).manual_seed(30), device=dev)
    ids, wts = route_topk(logits, TOP_K)
    layer = ExpertParallelMoE(E_TOTAL, HIDDEN, INTER, up, down, alignment=128, peer_rows_cap=expert_rows_cap(1, 1),
                              check_each_step=False)
    sampler = bench.ClockSampler(local)
    sampler.start()
    ms, t0, t1 = bench.timed(lambda: layer(x, ids, wts), steps, 3, lambda: None)
    clocks = sampler.stop(t0, t1)
    assert layer.read_status() == 0, "an expert overflowed its rows"
    marks = []
    layer.forward_peer(x, ids, wts, marks)
    torch.cuda.synchronize()
    phases = [marks[i].elapsed_time(marks[i + 1]) for i in range(4)]
    real_rows = float(TOKENS * TOP_K)
    flops = 2.0 * real_rows * (2 * INTER * HIDDEN + HIDDEN * INTER)
    return {"workload": f"expert-parallel MoE layer at one rank: E={E_TOTAL}, {TOKENS} tokens, top-{TOP_K}", "ms_per_step": ms,
            "steps": steps, "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "phases_ms": {"plan": phases[0], "dispatch": phases[1], "experts": phases[2], "combine": phases[3]},
            "experts_frac": 2.0 * flops / (phases[2] * 1e-3) / 1e12 / fp4_peak, "bound": "tensor", "clocks": clocks}


def run(args, workload: str, world: int, rank: int, local: int) -> None:
    import bench
    import nvfp4_gemm
    from .ep import ExpertParallelMoE, route_topk

    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    steps = args.steps or 20
    warmup = max(args.warmup if args.warmup is not None else 3, 3)
    e_local = E_TOTAL // world
    tokens = TOKENS

    # this rank's experts, random-init BF16 ~ N(0, 0.02), quantised on the device
    up = bench.build_weights(e_local, 2 * INTER, HIDDEN, dev, seed=20 + rank)
    down = bench.build_weights(e_local, HIDDEN, INTER, dev, seed=40 + rank)
    g = torch.Generator(device=dev).manual_seed(10 + rank)
    z = torch.randn(tokens, HIDDEN, generator=g, device=dev)
    chi = torch.randn(tokens, HIDDEN, 4, generator=g, device=dev).pow(2).mean(-1).sqrt()
    x = (z / chi).clamp(-2688.0, 2688.0).to(torch.bfloat16)
    del z, chi
    logits = torch.randn(tokens, E_TOTAL, generator=torch.Generator(device=dev).manual_seed(30 + rank), device=dev)
    ids, wts = route_topk(logits, TOP_K)
    extra = {kv.split('=')[0]: int(kv.split('=')[1]) for kv in getattr(args, "tune", [])}
    # several GPUs: dispatch and combine over peer memory unless ep_peer=0 asks for the NCCL all-to-all path;
    # room for 1.5 x the average rows a rank receives (a step that does not fit falls back by itself)
    use_peer = extra.get("ep_peer", 1) != 0
    # Micro-batches on streams of their own (the NVLink traffic of one part under the GEMMs of another, the parts' GEMM
    # phases chained one after the other).  Measured, ms per step as one batch / two / four parts: 2 GPUs 4.04 / 4.19 / 4.10,
    # 4 GPUs 4.12 / 4.76 / 3.83, 8 GPUs 4.37 / 4.73 / 4.77 (with 16 local experts a quarter of the rows makes GEMMs too small
    # to pay for what they hide).  So four parts on 4 GPUs, one batch otherwise.
    micro = extra.get("ep_micro", 4 if world == 4 else 1)
    layer = ExpertParallelMoE(E_TOTAL, HIDDEN, INTER, up, down, alignment=128,
                              peer_rows_cap=expert_rows_cap(world, micro) if use_peer else 0, micro_batches=micro,
                              check_each_step=False, comm_sms=extra.get("ep_comm_sms", 24),
                              quantized_dispatch=extra.get("ep_quant", 1) != 0, bulk_combine=extra.get("ep_bulk", 1) != 0,
                              fused_swiglu=extra.get("ep_fuse", 1) != 0)
    exchange = "nccl all_to_all"
    if layer.peer is not None:
        rows_as = ("rows quantised by the sender, NVFP4 codes + scales over NVLink (1.125 B/element)" if layer.peer[0].q is not None
                   else "BF16 rows over NVLink")
        exchange = ((f"peer memory, masked layout, {micro} micro-batch(es) on streams of their own (dispatch: {rows_as}, NVLink stores; "
                     "combine: NVLink loads, bounded flag barriers)") if world > 1 else
                    f"one rank: the dispatch and combine kernels on local buffers, masked layout ({rows_as})")
    elif use_peer:
        exchange = "nccl all_to_all (symmetric memory unavailable: %s)" % (layer.peer_error or "?")[:200]

    def barrier():
        if world > 1:
            dist.barrier()

    def step():
        return layer(x, ids, wts)

    sampler = bench.ClockSampler(local)
    sampler.start()
    ms, t0, t1 = bench.timed(step, steps, warmup, barrier)
    clocks = sampler.stop(t0, t1)
    # the timed steps checked nothing on the host: did every step fit its buffers, did every wait end in time?
    status_bits = layer.read_status() if layer.peer is not None else 0
    assert status_bits == 0, f"peer-memory steps reported status {status_bits:#x}"

    # per-phase device times on this rank (one extra, untimed pass over the all-to-all path, whose phases are
    # separate calls)
    plan, a = layer.dispatch(x, ids)                     # first use of the all-to-all path may set up NCCL channels
    layer.combine(layer.experts(a, plan), plan, wts, tokens)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    plan, a = layer.dispatch(x, ids)
    ev[1].record()
    out = layer.experts(a, plan)
    ev[2].record()
    y = layer.combine(out, plan, wts, tokens)
    ev[3].record()
    torch.cuda.synchronize()
    phases = [ev[i].elapsed_time(ev[i + 1]) for i in range(3)]
    real_rows = float(sum(plan.real_sizes))
    # agreement of the two exchange paths on this rank's tokens
    peer_vs_a2a, peer_phases = None, None
    if layer.peer is not None:
        marks = []
        y_peer = layer.forward_peer(x, ids, wts, marks)
        torch.cuda.synchronize()
        assert layer.read_status() == 0
        peer_vs_a2a = float((y_peer.float() - y.float()).norm() / y.float().norm().clamp_min(1e-30))
        peer_phases = [marks[i].elapsed_time(marks[i + 1]) for i in range(4)]
    del plan, a, out

    # end to end: activations and routing come from pinned host memory, the layer output goes back
    x_host, ids_host, w_host = x.cpu().pin_memory(), ids.cpu().pin_memory(), wts.cpu().pin_memory()
    y_host = torch.empty(tokens, HIDDEN, dtype=torch.bfloat16).pin_memory()
    xd, idd, wd = torch.empty_like(x), torch.empty_like(ids), torch.empty_like(wts)

    def e2e_step():
        xd.copy_(x_host, non_blocking=True)
        idd.copy_(ids_host, non_blocking=True)
        wd.copy_(w_host, non_blocking=True)
        y_host.copy_(layer(xd, idd, wd), non_blocking=True)

    e2e_steps = max(4, min(steps, 10)) // 2 * 2
    e2e_seq_ms, _, _ = bench.timed(e2e_step, e2e_steps, 3, barrier)

    # The same steps as a three-stage pipeline: inputs of step i + 1 go up and the result of step i - 1 comes back (both over
    # PCIe, on streams of their own) while step i computes.  Every step still copies its own inputs and its own result.
    up, down, cur = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev), torch.cuda.current_stream()
    bufs = [dict(x=torch.empty_like(x), ids=torch.empty_like(ids), w=torch.empty_like(wts),
                 out=torch.empty(tokens, HIDDEN, dtype=torch.bfloat16).pin_memory(), loaded=None, computed=None, stored=None)
            for _ in range(2)]

    def piped_step(i):
        b = bufs[i % 2]
        with torch.cuda.stream(up):
            if b["computed"] is not None:
                up.wait_event(b["computed"])              # step i - 2 has read these inputs
            b["x"].copy_(x_host, non_blocking=True)
            b["ids"].copy_(ids_host, non_blocking=True)
            b["w"].copy_(w_host, non_blocking=True)
            b["loaded"] = torch.cuda.Event()
            b["loaded"].record()
        cur.wait_event(b["loaded"])
        y_dev = layer(b["x"], b["ids"], b["w"])
        b["computed"] = torch.cuda.Event()
        b["computed"].record()
        with torch.cuda.stream(down):
            down.wait_event(b["computed"])
            y_dev.record_stream(down)
            b["out"].copy_(y_dev, non_blocking=True)

    for i in range(4):
        piped_step(i)
    torch.cuda.synchronize()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    up.wait_event(ev0)
    down.wait_event(ev0)
    for i in range(e2e_steps):
        piped_step(i)
    cur.wait_stream(up)
    cur.wait_stream(down)
    ev1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = ev0.elapsed_time(ev1) / e2e_steps
    e2e_same = bool(torch.equal(bufs[0]["out"], y_host))
    del bufs

    flops_rank = 2.0 * real_rows * (2 * INTER * HIDDEN + HIDDEN * INTER)
    stats = torch.tensor([ms, e2e_ms, flops_rank, phases[0], phases[1], phases[2]] + (peer_phases or [0.0] * 4) + [e2e_seq_ms],
                         dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    else:
        mx, sm = stats, stats
    ms_max, e2e_max, flops_all = float(mx[0]), float(mx[1]), float(sm[2])
    # kernels of this library per step: 2 GEMMs x (activation quantisation + GEMM), SwiGLU, and the row movers
    # (+ histogram and the two plan kernels on the peer-memory path)
    # peer path, per micro-batch: histogram, 3 plan kernels, dispatch, scale relayout, up GEMM, down quantise + GEMM, combine
    # (+ 3 barriers); with BF16 dispatch the relayout is an activation-quantisation kernel instead
    fused = layer.peer is not None and layer.peer[0].hq is not None     # no activation-quantisation kernel between the GEMMs
    kernels_per_step = (micro * ((9 if fused else 10) + (3 if world > 1 else 0)) if layer.peer is not None else
                        4 + (0 if layer.gemm_swiglu is not None else 1) + (2 if world == 1 else 4))
    if rank == 0:
        fp4_peak = bench.measure_fp4_peak()
        value = flops_all / (ms_max * 1e-3) / 1e12
        gemm_ms = float(mx[4])
        achieved = 2.0 * flops_rank / (gemm_ms * 1e-3) / 1e12
        dispatch_bytes_per_elem = 1.125 if (layer.peer is not None and layer.peer[0].q is not None) else 2.0
        off_rank_elems = tokens * TOP_K * HIDDEN * (world - 1) / world
        off_rank_bytes = off_rank_elems * 2.0
        line = {"metric": "grouped_gemm_logical_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "nvfp4 (e2m1 x ue4m3 block 16), fp32 accumulate, bf16 in/out", "data": "synthetic",
                "config": {"workload": f"expert-parallel MoE layer: E={E_TOTAL} over {world} ranks, {TOKENS} tokens/rank, top-{TOP_K}, "
                                       f"up N={2 * INTER} K={HIDDEN}, down N={HIDDEN} K={INTER}", "name": "c5",
                           "parallelism": f"ep{world}", "l2": "operands larger than L2, no flush", "exchange": exchange,
                           "step": ("dispatch, up GEMM with SwiGLU and the down-projection's activation quantisation in its epilogue, "
                                    "down GEMM, combine") if fused else
                                   "dispatch, up GEMM, down GEMM with SwiGLU folded into its activation quantisation, combine"},
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s",
                             "frac": achieved / fp4_peak, "traffic": None,
                             "note": "the two grouped GEMMs + SwiGLU glue of rank 0, both NVFP4 passes counted",
                             "peak_source": "resident-operand tcgen05 kind::mxf4nvf4 loop measured in this run"},
                "phases_ms_max_over_ranks_all_to_all_path": {"dispatch": float(mx[3]), "experts": gemm_ms, "combine": float(mx[5])},
                "phases_ms_max_over_ranks_peer_path": ({"plan": float(mx[6]), "dispatch": float(mx[7]), "experts": float(mx[8]),
                                                        "combine": float(mx[9]),
                                                        "note": "first micro-batch of one extra step, its stream sharing the GPU with the others'"}
                                                       if peer_phases else None),
                "micro_batches": micro,
                "peer_vs_all_to_all_rel_l2": peer_vs_a2a,
                "all_to_all_bytes_per_rank_per_direction": off_rank_bytes,
                "nvlink_bytes_per_rank_peer_path": {"dispatch": off_rank_elems * dispatch_bytes_per_elem, "combine": off_rank_bytes},
                "e2e": {"value": flops_all / (e2e_max * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_max,
                        "h2d_bytes_per_step": x_host.numel() * 2 + ids_host.numel() * 8 + w_host.numel() * 4,
                        "d2h_bytes_per_step": y_host.numel() * 2, "one_step_at_a_time_ms": float(mx[10]),
                        "result_equals_sequential": e2e_same,
                        "note": "three-stage pipeline: the next step's inputs go up and the previous step's result comes back "
                                "(PCIe, streams of their own) while a step computes; each step copies its own inputs and result"},
                "gpu_launches": kernels_per_step * steps, "kernels_per_step": kernels_per_step, "clocks": clocks}
        if world == 1:
            # the one-GPU point of a scaling series: the headline configuration C2 rides along as a sub-record, and the
            # CPU baseline is timed here as on every one-GPU line
            del layer, up, down, x, logits
            torch.cuda.empty_cache()
            c2 = bench.single_gpu_line("c2", dev, local, 20, 5, {}, cpu_baseline=False, also=False, e2e=False, sustained=False)
            line["also"] = {"c2": {k: c2[k] for k in ("ms_per_step", "value", "unit", "north_star_path", "rel_l2_vs_fp32")}
                            | {"frac": c2["roofline"]["frac"], "workload": c2["config"]["workload"]}}
            if not getattr(args, "no_cpu_baseline", False):
                base = bench.cpu_reference_sample("c5")
                line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
