#!/usr/bin/env python
"""Benchmark of the grouped dual-NVFP4 GEMM hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3up|c3down|c4|c5] [--impl reference]

A step is one call of ``m_grouped_bf16_dual_nvfp4_gemm_contiguous`` over one batch of
seeded synthetic input.  At N = 1 the default workload is the Mixtral-8x7B-like expert
up-projection (E=8, 512 rows per expert, N=28672, K=4096).  ``value`` is logical
TFLOP/s (2*M*N*K / t, the figure the reference prints) with every operand resident in
HBM; ``e2e`` is the same figure through the public call with the activations coming
from pinned host memory and the output going back to the host inside the timed region.
``roofline`` relates the kernel to the tensor-pipe ceiling (both NVFP4 passes count) or,
for the decode workload, to HBM bandwidth.  ``--impl reference`` times the reference's
CPU implementation of the same chain on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: experts, N, K, description
    "c2": dict(E=8, N=28672, K=4096, desc="Mixtral-8x7B-like up-projection: E=8 x 512 rows, N=28672, K=4096"),
    "c3up": dict(E=256, N=4096, K=7168, desc="DeepSeek-V3-style prefill up: E=256, 32768 rows Zipf(1.1) padded to 128, N=4096, K=7168"),
    "c3down": dict(E=256, N=7168, K=2048, desc="DeepSeek-V3-style prefill down: E=256, 32768 rows Zipf(1.1) padded to 128, N=7168, K=2048"),
    "c4": dict(E=256, N=4096, K=7168, desc="decode: E=256, 64 tokens x top-8 (1-16 rows per active expert, padded to 16), N=4096, K=7168"),
    # reduced copies of c2 / c4 (operands still larger than L2) for profiler captures
    # the reference's own sweep (benchmarks/bench_moe_forward.py:37-52, bench_decode.py there): Qwen3.5-35B-A3B expert
    # shapes, 32 local experts, balanced rows per expert; q*4k..32k = 128..1024 rows per expert, qdec* = decode
    **{f"qup{t}k": dict(E=32, N=1024, K=2048, rows=t * 32, desc=f"reference sweep gate_up: E=32 x {t * 32} rows, N=1024, K=2048")
       for t in (4, 8, 16, 32)},
    **{f"qdown{t}k": dict(E=32, N=2048, K=512, rows=t * 32, desc=f"reference sweep down: E=32 x {t * 32} rows, N=2048, K=512")
       for t in (4, 8, 16, 32)},
    **{f"qdec{t}": dict(E=32, N=1024, K=2048, decode_tokens=t,
                        desc=f"reference decode sweep gate_up: {t} tokens x top-8 of 256 experts, 32 local experts, N=1024, K=2048")
       for t in (16, 32, 128)},
    # the up-projection of the expert-parallel layer (the dominant GEMM of config C5); the layer itself is built in
    # nvfp4_cutlass_b200/ep_bench.py, this entry gives the CPU reference arm its shape
    "c5": dict(E=128, N=3072, K=4096, desc="expert-parallel MoE layer (C5): up-projection E=128, N=3072, K=4096"),
    # the two GEMMs of that layer at one rank, as plain grouped-GEMM workloads (same routing rule: top-8 softmax of
    # Gaussian logits over 16384 tokens, groups padded to 128 rows, Student-t(4) activations)
    "c5up": dict(E=128, N=3072, K=4096, ep_tokens=16384, desc="C5 up-projection at one rank: E=128, 131072 rows top-8 routed, N=3072, K=4096"),
    "c5down": dict(E=128, N=4096, K=1536, ep_tokens=16384, desc="C5 down-projection at one rank: E=128, 131072 rows top-8 routed, N=4096, K=1536"),
    "c2s": dict(E=8, N=8192, K=4096, desc="reduced c2 for profiling: E=8 x 512 rows, N=8192, K=4096"),
    "c4s": dict(E=64, N=4096, K=7168, desc="reduced c4 for profiling: E=64, 16 tokens x top-8, N=4096, K=7168"),
}


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch from the ncu captures summarised
# under profiles/, on the reduced workloads c2s / c4s (the full ones exceed what a multi-pass capture should
# hold), as (bytes measured, algorithmic bytes of that captured launch).  Both kernels stream every operand
# once, so traffic grows in proportion to the algorithmic bytes; a full launch is scaled by that ratio.
NCU_TRAFFIC = {"normal": (246.45e6, 251.66e6, "split-path kernels (CTA-pair GEMM) on c2s, captured at commit 253fbe0"),
               "swap_ab": (925.44e6, 911.22e6, "decode kernel on c4s, captured at commit 70bfc9c")}


def scaled_traffic(orientation: str, algo_bytes: float) -> dict:
    measured, algo_small, src = NCU_TRAFFIC[orientation]
    return {"traffic": measured / algo_small * algo_bytes,
            "traffic_source": f"one ncu capture of a launch on a reduced workload ({src}), scaled by algorithmic bytes"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 + 0.06] or [r for _, r in self.rows[-3:]]
        mhz, reasons, mx = [], set(), None
        for r in rows:
            try:
                mhz.append(float(r[0])); mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ----------------------------------------------------------------------------- workloads
def routing_rows(workload: str, E: int, gen: torch.Generator):
    """Real rows per expert and the padded group sizes the kernel sees."""
    if workload in ("c2", "c2s"):
        real = [512] * E
        return real, real, 128, False
    if workload in ("c3up", "c3down"):
        p = torch.arange(1, E + 1, dtype=torch.float64).pow(-1.1)
        real = torch.multinomial(p / p.sum(), 32768, replacement=True, generator=gen).bincount(minlength=E).tolist()
        return real, [((r + 127) // 128) * 128 for r in real], 128, False
    if workload in ("c4", "c4s"):
        counts = torch.zeros(E, dtype=torch.int64)
        for _ in range(64 if workload == "c4" else 16):     # 64 tokens, 8 distinct experts each
            counts[torch.randperm(E, generator=gen)[:8]] += 1
        real = counts.clamp(max=16).tolist()
        return real, [((r + 15) // 16) * 16 for r in real], 16, True
    cfg = WORKLOADS[workload]
    if "ep_tokens" in cfg:                                  # top-8 softmax routing of Gaussian logits
        logits = torch.randn(cfg["ep_tokens"], E, generator=gen)
        ids = torch.topk(torch.softmax(logits, dim=-1), 8, dim=-1).indices
        real = torch.bincount(ids.reshape(-1), minlength=E).tolist()
        return real, [((r + 127) // 128) * 128 for r in real], 128, False
    if "rows" in cfg:
        real = [cfg["rows"]] * E
        return real, real, 128, False
    if "decode_tokens" in cfg:                              # each token picks 8 of 256 experts; 32 of them live here
        counts = torch.zeros(256, dtype=torch.int64)
        for _ in range(cfg["decode_tokens"]):
            counts[torch.randperm(256, generator=gen)[:8]] += 1
        real = counts[:E].tolist()
        return real, [((r + 15) // 16) * 16 for r in real], 16, True
    raise ValueError(workload)


def build_weights(E: int, N: int, K: int, dev, seed: int):
    """Random-init BF16 weights ~N(0, 0.02), quantised expert by expert (bounds device memory)."""
    import nvfp4_gemm
    b = torch.empty(E * N, K // 2, dtype=torch.int8, device=dev)
    sfb = torch.empty(E * K // 64, N, dtype=torch.int32, device=dev)
    gw = torch.empty(E, dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(seed)
    for e in range(E):
        w = (torch.randn(1, N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        be, se, ge = nvfp4_gemm.quantize_weight_nvfp4(w)
        b[e * N:(e + 1) * N] = be
        sfb[e * (K // 64):(e + 1) * (K // 64)] = se
        gw[e] = ge[0]
    return b, sfb, gw


def build_single_gpu_case(workload: str, dev, extra_kw=None, weights=None):
    """Seeded synthetic operands of a workload, on the device.  `weights` = (b, sfb, gw) of an earlier case with the
    same E, N, K (c4 shares c3up's)."""
    import nvfp4_gemm
    cfg = WORKLOADS[workload]
    E, N, K = cfg["E"], cfg["N"], cfg["K"]
    gen = torch.Generator().manual_seed(3)
    real, padded, align, swap = routing_rows(workload, E, gen)
    M = sum(padded)
    ga = torch.Generator(device=dev).manual_seed(0)
    a = torch.zeros(M, K, dtype=torch.bfloat16, device=dev)
    x = torch.randn(sum(real), K, generator=ga, device=dev)
    if workload in ("c2", "c2s"):                           # per-row lognormal(0, 0.5) scale
        x = x * torch.exp(0.5 * torch.randn(sum(real), 1, generator=ga, device=dev))
    if "ep_tokens" in cfg:                                  # Student-t(4), in row chunks to bound memory
        for r0 in range(0, x.shape[0], 16384):
            chi = torch.randn(min(16384, x.shape[0] - r0), K, 4, generator=ga, device=dev).pow(2).mean(-1).sqrt()
            x[r0:r0 + 16384] /= chi
            del chi
    if workload.startswith("c3"):                           # 0.1 % outlier channels x50
        cols = torch.randperm(K, generator=torch.Generator().manual_seed(1))[:max(1, K // 1000)]
        x[:, cols.to(dev)] *= 50.0
    x = x.clamp(-2688.0, 2688.0).to(torch.bfloat16)
    off_r = off_p = 0
    for r, pz in zip(real, padded):
        a[off_p:off_p + r] = x[off_r:off_r + r]
        off_r += r
        off_p += pz
    m_indices = nvfp4_gemm.make_m_indices(padded, alignment=align).to(dev)
    b, sfb, gw = weights if weights is not None else build_weights(E, N, K, dev, seed=2)
    kw = dict(tune_swap_ab=1, m_alignment=align) if swap else {}
    if not swap and all(pz % 256 == 0 for pz in padded):
        kw["m_alignment"] = 256                             # every group is whole 256-row pairs: the caller may say so
    kw.update(extra_kw or {})
    active = sum(1 for r in real if r > 0)
    return dict(a=a, b=b, sfb=sfb, gw=gw, m_indices=m_indices, M=M, N=N, K=K, E=E, real_rows=sum(real),
                active_experts=active, kw=kw, swap=swap, padded=padded, real=real)


def accuracy_sample(case, d, dev):
    """rel-L2 / cosine of the kernel output against FP32 A_bf16 @ dequant(W)^T on the rows of one expert
    and a 1024-column slice (torch ops are the checker here, never the product)."""
    import nvfp4_gemm
    E, N, K = case["E"], case["N"], case["K"]
    e = max(range(E), key=lambda i: case["real"][i])
    start = sum(case["padded"][:e])
    rows = min(case["real"][e], 256)
    ncols = min(N, 1024)
    be = case["b"][e * N:e * N + ncols]
    se = case["sfb"][e * (K // 64):(e + 1) * (K // 64), :ncols].contiguous()
    wdq = nvfp4_gemm.dequantize_weight_nvfp4(be, se, case["gw"][e:e + 1], 1, ncols, K)[0]
    ref = case["a"][start:start + rows].float() @ wdq.T
    got = d[start:start + rows, :ncols].float()
    rel = float((got - ref).norm() / ref.norm())
    cos = float(torch.dot(got.flatten(), ref.flatten()) / (got.norm() * ref.norm()))
    return rel, cos


# ----------------------------------------------------------------------------- CPU baseline
class CpuReference:
    """The reference's CPU chain on a bounded sample of the workload (the rows of one expert x a slice of its output
    columns x full K), on all host threads.  Preferred: the reference's own PyTorch emulation
    (tests/python/reference/dual_nvfp4.py there: decompose -> dequantise -> FP32 matmul -> G_W -> BF16), copied at
    build time into the git-ignored oracle/_ref/ by oracle/Makefile.  Without it: the reference's C++ host twin
    (oracle/_ref/libref_twin.so), else the C restatement (oracle/).  The sample is prepared once (weights quantised,
    untimed, as on the GPU arm); run() times one pass of the chain over it."""

    def __init__(self, workload: str, seconds_target: float = 10.0):
        import oracle
        self.oracle = oracle
        cfg = WORKLOADS.get(workload, WORKLOADS["c2"])
        self.K, N = cfg["K"], cfg["N"]
        self.threads = os.cpu_count() or 1
        self.emu = oracle.ref_emulation()
        self.twin = oracle.ref_twin() is not None and hasattr(oracle.ref_twin(), "ref_twin_dual_gemm_mt")
        self.kind = "reference" if self.emu is not None else ("reference-cpp" if self.twin else "port")
        # one expert's rows as the workload has them (512 at C2), columns sized for the time target
        rows = min(512, cfg.get("rows", 512))
        ncols = min(N, 1024)
        # one cheap probe, then the final sample prepared once: columns grow up to N, then the rows (large FP32 matmuls
        # run ~2x more efficiently than the probe, hence the factor)
        self._prepare(rows, ncols)
        t_probe = min(self.run() for _ in range(2))
        scale = 2.0 * seconds_target / max(t_probe, 1e-3)
        if scale >= 1.5:
            new_cols = min(N, max(ncols, int(ncols * scale) // 64 * 64))
            scale /= new_cols / ncols
            ncols = new_cols
            if scale >= 1.5:
                rows = min(4096, max(rows, int(rows * scale) // 128 * 128))
            self._prepare(rows, ncols)

    def _prepare(self, rows, ncols):
        g = torch.Generator().manual_seed(0)
        self.rows, self.ncols = rows, ncols
        self.a = torch.randn(rows, self.K, generator=g).to(torch.bfloat16)
        w = (torch.randn(1, ncols, self.K, generator=g) * 0.02).to(torch.bfloat16)
        self.mi = torch.zeros(rows, dtype=torch.int32)
        if self.emu is not None:
            torch.set_num_threads(self.threads)
            self.w = self.emu.quantize_weight_nvfp4(w.float())
        elif self.twin:
            self.w = self.oracle.ref_twin_quantize_weight(w.float())
        else:
            self.w = self.oracle.quantize_weight(w)

    def run(self) -> float:
        t = time.perf_counter()
        if self.emu is not None:
            self.emu.dual_nvfp4_grouped_gemm(self.a, *self.w, torch.tensor([0, self.rows]))
        elif self.twin:
            self.oracle.ref_twin_dual_gemm_mt(self.a.float(), *self.w, self.mi, self.ncols, self.threads)
        else:
            self.oracle.grouped_gemm(self.a, *self.w, self.mi, self.ncols, mode="dual")
        return time.perf_counter() - t

    def record(self, seconds: float) -> dict:
        flops = 2.0 * self.rows * self.ncols * self.K
        what = {"reference": "the reference's PyTorch emulation (dual_nvfp4_grouped_gemm, FP32 matmul)",
                "reference-cpp": "the reference's C++ host twin", "port": "the C restatement of the reference's emulation"}[self.kind]
        return dict(value=flops / seconds / 1e12, unit="TFLOP/s", cores=self.threads if self.kind != "port" else self.oracle.num_threads(),
                    kind=self.kind, seconds=seconds,
                    sample=f"{what}: {self.rows} rows of one expert x {self.ncols} output columns x K={self.K} "
                           f"({flops / 1e9:.1f} GFLOP, {seconds:.1f} s)")


def cpu_reference_sample(workload: str, seconds_target: float = 10.0):
    ref = CpuReference(workload, seconds_target)
    return ref.record(ref.run())


def default_workload(args, world: int) -> str:
    """C2 (the configuration the headline metric is quoted on) for a one-GPU run on a one-GPU box.  The expert-parallel
    layer C5 for several ranks, and also for a one-rank run under a torchrun-style launcher or on a box with several
    GPUs: that is the N = 1 point of a 1 -> 8 scaling series, which must be the same workload as its N > 1 points."""
    if args.workload:
        return args.workload
    if world > 1 or args.gpus > 1:
        return "c5"
    scaling_series = "WORLD_SIZE" in os.environ or (torch.cuda.is_available() and torch.cuda.device_count() > 1)
    return "c5" if scaling_series else "c2"


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    base = None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    workload = default_workload(args, max(world, args.gpus))      # the same default as the main arm
    # each step is one pass over the same bounded sample, sized so that warm-up + steps end within a few minutes
    ref = CpuReference(workload, seconds_target=max(1.0, min(6.0, 150.0 / max(1, args.warmup + args.steps))))
    for i in range(args.warmup + args.steps):
        base = ref.record(ref.run())
        if i >= args.warmup:
            times.append(base["value"])
    value = statistics.mean(times)
    line = {"impl": "reference", "metric": "grouped_gemm_logical_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["seconds"] * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 codes, fp32 accumulate",
            "data": "synthetic", "config": {"workload": WORKLOADS.get(workload, {}).get("desc", workload),
                                            "note": "bounded sample of the workload on the host cores"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    line["cpu_baseline"]["value"] = value
    print(json.dumps(line))


# ----------------------------------------------------------------------------- main arm
def timed_graph(fn, steps, warmup):
    """The reference's timing method (benchmarks/bench_moe_forward.py:87-124 there): one call captured into a CUDA
    graph, replayed back to back; host launch cost is out of the picture and the operands are the same (L2-warm
    when they fit) on every replay."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        fn()
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    s.record()
    for _ in range(steps):
        graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps, t0, time.time()


def timed(fn, steps, warmup, barrier):
    for _ in range(warmup):
        fn()
    barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    s.record()
    for _ in range(steps):
        fn()
    e.record()
    torch.cuda.synchronize()
    barrier()
    return s.elapsed_time(e) / steps, t0, time.time()


def measure_fp4_peak():
    from nvfp4_gemm import _C
    _C.debug_mma_peak(256)
    torch.cuda.synchronize()
    best = 0.0
    for _ in range(3):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fl = _C.debug_mma_peak(4096)
        e.record()
        torch.cuda.synchronize()
        best = max(best, fl / (s.elapsed_time(e) * 1e-3) / 1e12)
    return best


def measure_fp4_peak_sustained(seconds: float = 0.25):
    """The same resident-operand MMA loop launched back to back for about `seconds`: the rate the tensor
    pipe holds once the power cap has pulled the SM clock down (what a long timed region can reach)."""
    from nvfp4_gemm import _C
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fl = _C.debug_mma_peak(4096)
    e.record()
    torch.cuda.synchronize()
    n = max(4, int(seconds * 1e3 / max(s.elapsed_time(e), 1e-3)))
    s.record()
    for _ in range(n):
        fl = _C.debug_mma_peak(4096)
    e.record()
    torch.cuda.synchronize()
    return n * fl / (s.elapsed_time(e) * 1e-3) / 1e12


def split_default(case, extra) -> bool:
    """Whether the dispatcher (csrc/abi.cu) sends this call to the two-kernel split path."""
    fused_knobs = any(extra.get(k, 0) for k in ("tune_cluster", "tune_transform_warps", "tune_direct_a"))
    mode = extra.get("tune_split_transform", 0)
    return (not case["swap"]) and case["N"] % 256 == 0 and (mode == 1 or (mode == 0 and not fused_knobs and case["N"] > 1024))


def gemm_record(case, dev, steps, warmup, fp4_peak, graph=False, extra=None, sample_clocks=True, local=0):
    """One timed run of the grouped GEMM on `case`: ms, logical TFLOP/s, roofline record, accuracy sample."""
    import nvfp4_gemm
    from nvfp4_gemm import _C
    extra = dict(extra or {})
    kw = dict(case["kw"], **extra)
    M, N, K = case["M"], case["N"], case["K"]
    d = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def step():
        nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(case["a"], case["b"], case["sfb"], case["gw"], d,
                                                             case["m_indices"], device_status=status, **kw)

    sampler = ClockSampler(local) if sample_clocks else None
    if sampler:
        sampler.start()
    ms, t0, t1 = (timed_graph(step, steps, warmup) if graph else timed(step, steps, warmup, lambda: None))
    clocks = sampler.stop(t0, t1) if sampler else None
    assert _C.read_status(status) == 0, "kernel reported a device-side timeout"
    rel, cos = accuracy_sample(case, d, dev)
    logical = 2.0 * case["real_rows"] * N * K
    pk = peaks()
    if case["swap"]:
        algo_bytes = (case["active_experts"] * (N * K // 2 + N * K // 16) + 2 * case["real_rows"] * K +
                      2 * case["real_rows"] * N + 4 * case["E"] + 4 * M)
        achieved = algo_bytes / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], **scaled_traffic("swap_ab", algo_bytes), "peak_source": pk["source"],
                    "algorithmic_bytes_per_launch": algo_bytes}
    else:
        achieved = 2.0 * logical / (ms * 1e-3) / 1e12       # both NVFP4 passes run on the tensor pipe
        algo_bytes = case["b"].numel() + case["sfb"].numel() * 4 + case["a"].numel() * 2 + d.numel() * 2
        roofline = {"bound": "tensor", "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s",
                    "frac": achieved / fp4_peak, **scaled_traffic("normal", algo_bytes),
                    "algorithmic_bytes_per_launch": algo_bytes, "tensor_flops_per_launch": 2.0 * logical,
                    "hbm_gbs_min": algo_bytes / (ms * 1e-3) / 1e9, "hbm_frac_min": algo_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
    rec = {"ms_per_step": ms, "steps": steps, "value": logical / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "roofline": roofline,
           "frac": roofline["frac"], "rel_l2_vs_fp32": rel, "cosine_vs_fp32": cos,
           "timing": "CUDA-graph replay of one call" if graph else "back-to-back launches",
           "kernels_per_step": 2 if split_default(case, extra) else 1}
    if clocks is not None:
        rec["clocks"] = clocks
    return rec, d, step


def north_star_record(case, dev, steps, fp4_peak, graph=False):
    """The path the project is named for -- Algorithm 1 inside the GEMM main loop, nothing quantised written to
    global memory -- on this workload: the fused cluster kernel for the normal orientation (the decode kernel
    always decomposes in its main loop)."""
    rec, _, _ = gemm_record(case, dev, steps, 3, fp4_peak, graph=graph, extra=dict(tune_split_transform=2), sample_clocks=False)
    return {"ms_per_step": rec["ms_per_step"], "steps": rec["steps"], "value": rec["value"], "unit": "TFLOP/s", "frac": rec["frac"],
            "rel_l2_vs_fp32": rec["rel_l2_vs_fp32"], "cosine_vs_fp32": rec["cosine_vs_fp32"], "kernels_per_step": 1,
            "note": "tune_split_transform=2: Algorithm 1 inside the GEMM main loop (cluster kernel, transform shared over distributed shared memory)"}


def slim(rec):
    """A sub-record of the JSON line: the figures, without the long provenance strings."""
    out = {k: rec[k] for k in ("ms_per_step", "steps", "value", "unit", "frac", "rel_l2_vs_fp32", "cosine_vs_fp32", "timing",
                               "kernels_per_step") if k in rec}
    out["bound"] = rec["roofline"]["bound"]
    if "hbm_frac_min" in rec["roofline"]:
        out["hbm_frac_min"] = rec["roofline"]["hbm_frac_min"]
    if "clocks" in rec:
        out["clocks"] = rec["clocks"]
    if "north_star_path" in rec:
        out["north_star_path"] = rec["north_star_path"]
    return out


def also_records(dev, fp4_peak, local, budget_s=120.0):
    """The other configurations and the reference's own sweep, bounded, in the same run: C3 up / down, C4, and the
    Qwen-shaped gate_up / down / decode shapes the reference publishes (graph-timed like there, split and fused)."""
    t_start = time.time()
    out = {}
    shared = {}
    for name, steps in (("c3up", 10), ("c4", 20), ("c3down", 10)):
        if time.time() - t_start > budget_s:
            out[name] = {"skipped": "time budget of the default run"}
            continue
        case = build_single_gpu_case(name, dev, weights=shared.get((WORKLOADS[name]["E"], WORKLOADS[name]["N"], WORKLOADS[name]["K"])))
        shared[(case["E"], case["N"], case["K"])] = (case["b"], case["sfb"], case["gw"])
        rec, _, _ = gemm_record(case, dev, steps, 3, fp4_peak, local=local)
        if not case["swap"]:
            rec["north_star_path"] = north_star_record(case, dev, max(3, steps // 2), fp4_peak)
        out[name] = slim(rec)
        out[name]["workload"] = WORKLOADS[name]["desc"]
        del case
        if name == "c4":
            shared.clear()
        torch.cuda.empty_cache()
    sweep = {}
    for name in ("qup8k", "qup16k", "qup32k", "qdown8k", "qdown16k", "qdown32k", "qdec16", "qdec32", "qdec128"):
        if time.time() - t_start > budget_s:
            sweep[name] = {"skipped": "time budget of the default run"}
            continue
        case = build_single_gpu_case(name, dev)
        rec, _, _ = gemm_record(case, dev, 100, 3, fp4_peak, graph=True, sample_clocks=False)
        entry = {"us": rec["ms_per_step"] * 1e3, "value": rec["value"], "frac": rec["frac"], "bound": rec["roofline"]["bound"],
                 "cosine_vs_fp32": rec["cosine_vs_fp32"]}
        if not case["swap"]:
            other = 1 if rec["kernels_per_step"] == 1 else 2         # the path the dispatcher did not take
            ns, _, _ = gemm_record(case, dev, 100, 3, fp4_peak, graph=True, extra=dict(tune_split_transform=other), sample_clocks=False)
            entry["path"] = "fused" if rec["kernels_per_step"] == 1 else "split"
            entry["fused_us" if other == 2 else "split_us"] = ns["ms_per_step"] * 1e3
        sweep[name] = entry
        del case
    out["ref_sweep"] = {"timing": "CUDA-graph replay of one call, 100 replays (the reference's method)", "unit": "us per call",
                        "shapes": sweep}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default=None, help="c2 (default at 1 GPU), c3up, c3down, c4, c5up, c5down, c5 (default at >1 GPU)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the sub-records of the other configurations")
    ap.add_argument("--quick", action="store_true", help="the timed region only: no sustained / end-to-end / north-star / "
                    "other-configuration / CPU legs (what a profiler capture wants)")
    ap.add_argument("--graph", action="store_true", help="time CUDA-graph replays of one call (the reference's method)")
    ap.add_argument("--tune", action="append", default=[], help="tune_xxx=int passed to the GEMM call (experiments)")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = args.steps or 2
        args.warmup = args.warmup if args.warmup is not None else 1
        return run_reference_arm(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    workload = default_workload(args, world)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 or workload == "c5":
        from nvfp4_cutlass_b200 import ep_bench
        return ep_bench.run(args, workload, world, rank, local)

    steps = args.steps or 20
    warmup = max(args.warmup if args.warmup is not None else 5, 3)
    extra = {kv.split('=')[0]: int(kv.split('=')[1]) for kv in args.tune}
    if args.quick:
        line = single_gpu_line(workload, dev, local, steps, warmup, extra, args.graph, cpu_baseline=False, also=False, e2e=False,
                               sustained=False, north_star=False)
    else:
        line = single_gpu_line(workload, dev, local, steps, warmup, extra, args.graph, cpu_baseline=not args.no_cpu_baseline,
                               also=not args.no_also and workload == "c2" and not extra)
    print(json.dumps(line))


def single_gpu_line(workload, dev, local, steps, warmup, extra, graph=False, cpu_baseline=True, also=False, e2e=True, sustained=True,
                    north_star=True):
    """The JSON line of a one-GPU grouped-GEMM workload."""
    import nvfp4_gemm
    case = build_single_gpu_case(workload, dev, extra)
    M, N, K = case["M"], case["N"], case["K"]
    fp4_peak = measure_fp4_peak()
    rec, d, step = gemm_record(case, dev, steps, warmup, fp4_peak, graph=graph, extra=extra, local=local)
    roofline = rec["roofline"]
    is_split = split_default(case, extra)
    pair = case["kw"].get("m_alignment") == 256 or extra.get("tune_cluster") == 2 or case["M"] // case["E"] >= 2048
    if extra.get("tune_cluster") == 1:
        pair = False
    path = ("split: quantize_activation_kernel (Algorithm 1 once per element, into an L2-resident workspace) + " +
            ("gemm_split_pair_kernel (block-scaled FP4 GEMM, CTA pairs: tcgen05.mma.cta_group::2 over 256 rows x 256 columns; "
             "the call states m_alignment=256)" if pair else "gemm_split_kernel (block-scaled FP4 GEMM)")) if is_split else (
            "decode: gemm_swap_kernel, Algorithm 1 in the main loop" if case["swap"] else
            "fused: Algorithm 1 in the main loop of the GEMM kernel")
    logical = 2.0 * case["real_rows"] * N * K
    pk = peaks()
    if not case["swap"]:
        fp4_sustained = measure_fp4_peak_sustained()
        roofline.update({"peak_source": "resident-operand tcgen05 kind::mxf4nvf4 loop measured in this run (burst)",
                         "peak_sustained": fp4_sustained, "frac_of_sustained": roofline["achieved"] / fp4_sustained,
                         "peak_sustained_source": "the same loop launched back to back for 0.25 s (power-capped clock)",
                         "peak_4x_measured_bf16": 4.0 * pk["bf16_tflops"],
                         "frac_of_4x_measured_bf16": roofline["achieved"] / (4.0 * pk["bf16_tflops"]), "peak_bf16_source": pk["source"]})

    line = {"metric": "grouped_gemm_logical_tflops", "value": rec["value"], "unit": "TFLOP/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 (e2m1 x ue4m3 block 16), fp32 accumulate, bf16 in/out", "data": "synthetic",
            "config": {"workload": WORKLOADS[workload]["desc"], "name": workload, "M_padded": M, "M_real": case["real_rows"],
                       "N": N, "K": K, "E": case["E"], "passes": 2, "orientation": "swap_ab" if case["swap"] else "normal",
                       "tune": extra, "path": path, "kernels_per_step": rec["kernels_per_step"], "timing": rec["timing"],
                       "l2": ("operands larger than L2 (weights %.0f MB), no flush" if case["b"].numel() > 126e6 else
                              "weights %.0f MB fit in L2 and are not flushed (the reference's sweep is timed the same way)")
                             % (case["b"].numel() / 1e6)},
            "roofline": roofline, "gpu_launches": steps * rec["kernels_per_step"], "clocks": rec["clocks"],
            "rel_l2_vs_fp32": rec["rel_l2_vs_fp32"], "cosine_vs_fp32": rec["cosine_vs_fp32"]}

    # the same call for >= 0.25 s back to back: what the kernel holds once the power cap has settled the clock
    if sustained and not graph:
        n_sus = max(steps, int(0.3 / max(rec["ms_per_step"] * 1e-3, 1e-6)))
        sampler = ClockSampler(local)
        sampler.start()
        sus_ms, t0, t1 = timed(step, n_sus, 3, lambda: None)
        sus_clocks = sampler.stop(t0, t1)
        ach = (2.0 * logical / (sus_ms * 1e-3) / 1e12) if not case["swap"] else roofline["algorithmic_bytes_per_launch"] / (sus_ms * 1e-3) / 1e9
        line["sustained"] = {"ms_per_step": sus_ms, "steps": n_sus, "value": logical / (sus_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                             "frac": ach / roofline["peak"], "clocks": sus_clocks}
        if not case["swap"]:
            line["sustained"]["frac_of_sustained_peak"] = ach / roofline["peak_sustained"]

    # the north-star path (Algorithm 1 inside the GEMM main loop) on the same inputs, whatever the default is
    if not north_star:
        pass
    elif case["swap"]:
        line["north_star_path"] = {"ms_per_step": rec["ms_per_step"], "value": rec["value"], "unit": "TFLOP/s", "frac": rec["frac"],
                                   "note": "the decode kernel decomposes the activations inside its main loop: this is the default path"}
    elif not is_split:
        line["north_star_path"] = {"ms_per_step": rec["ms_per_step"], "value": rec["value"], "unit": "TFLOP/s", "frac": rec["frac"],
                                   "note": "the timed path is the fused kernel"}
    else:
        line["north_star_path"] = north_star_record(case, dev, max(5, min(steps, 50)), fp4_peak, graph=graph)
        line["fused_in_mainloop"] = dict(line["north_star_path"], roofline_frac=line["north_star_path"]["frac"])
        step()                                    # leave the default path's output in d

    if e2e:
        # end to end through the public call: activations and routing index come from pinned host memory every step and
        # the output goes back to pinned host memory (weights are model state, resident on the device)
        a_host = case["a"].cpu().pin_memory()
        mi_host = case["m_indices"].cpu().pin_memory()
        d_host = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
        a_dev = torch.empty_like(case["a"])
        mi_dev = torch.empty_like(case["m_indices"])
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        kw = dict(case["kw"])

        def e2e_step():
            a_dev.copy_(a_host, non_blocking=True)
            mi_dev.copy_(mi_host, non_blocking=True)
            nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(a_dev, case["b"], case["sfb"], case["gw"], d, mi_dev,
                                                                 device_status=status, **kw)
            d_host.copy_(d, non_blocking=True)

        e2e_steps = max(6, min(steps, 30)) // 2 * 2
        seq_ms, _, _ = timed(e2e_step, e2e_steps, 3, lambda: None)
        # The same steps with two in flight: each on a stream and a set of buffers of its own, so that one step's copy back
        # (PCIe, the longest leg) runs while the next step's inputs go up and its kernels run.  Every step still copies its
        # own inputs in and its own result out inside the timed region.
        lanes = []
        for _ in range(2):
            lanes.append(dict(stream=torch.cuda.Stream(device=dev), a=torch.empty_like(case["a"]), mi=torch.empty_like(case["m_indices"]),
                              d=torch.empty_like(d), out=torch.empty(M, N, dtype=torch.bfloat16).pin_memory()))

        def piped_step(i):
            ln = lanes[i % 2]
            with torch.cuda.stream(ln["stream"]):
                ln["a"].copy_(a_host, non_blocking=True)
                ln["mi"].copy_(mi_host, non_blocking=True)
                nvfp4_gemm.m_grouped_bf16_dual_nvfp4_gemm_contiguous(ln["a"], case["b"], case["sfb"], case["gw"], ln["d"], ln["mi"],
                                                                     device_status=status, **kw)
                ln["out"].copy_(ln["d"], non_blocking=True)

        cur = torch.cuda.current_stream()
        for i in range(4):
            piped_step(i)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for ln in lanes:
            ln["stream"].wait_event(ev0)
        for i in range(e2e_steps):
            piped_step(i)
        for ln in lanes:
            cur.wait_stream(ln["stream"])
        ev1.record()
        torch.cuda.synchronize()
        e2e_ms = ev0.elapsed_time(ev1) / e2e_steps
        same = bool(torch.equal(lanes[0]["out"], d_host)) and int(status.item()) == 0
        line["e2e"] = {"value": logical / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                       "h2d_bytes_per_step": a_host.numel() * 2 + mi_host.numel() * 4, "d2h_bytes_per_step": d_host.numel() * 2,
                       "in_flight": 2, "one_step_at_a_time_ms": seq_ms, "one_step_at_a_time_value": logical / (seq_ms * 1e-3) / 1e12,
                       "result_equals_sequential": same,
                       "note": "two steps in flight on streams of their own (copy back of one under the next); "
                               "each step copies its inputs from pinned host memory and its result back"}
        del lanes
        del a_host, d_host, a_dev
    del case, d
    torch.cuda.empty_cache()
    if also:
        line["also"] = also_records(dev, fp4_peak, local)
        try:
            from nvfp4_cutlass_b200 import ep_bench
            line["also"]["c5_one_gpu"] = ep_bench.one_gpu_record(dev, local, fp4_peak)
        except Exception as exc:                                  # the headline must survive a failure of a side record
            line["also"]["c5_one_gpu"] = {"error": repr(exc)[:300]}
    if cpu_baseline:
        base = cpu_reference_sample(workload)
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    return line


if __name__ == "__main__":
    main()
