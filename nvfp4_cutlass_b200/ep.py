"""Expert-parallel MoE layer around the grouped dual-NVFP4 GEMM.

The GEMM shards by expert: tiles of different experts never meet, so rank r of R owns
experts [r*E/R, (r+1)*E/R) with their quantised weights resident, tokens stay data
parallel, and there is one exchange before and one after the two GEMMs:

  dispatch   every (token, chosen expert) pair is one BF16 row that goes to the rank that
             owns the expert, into that rank's expert-major buffer with every group padded
             to the kernel's row alignment
  compute    up-GEMM -> SwiGLU -> down-GEMM on the local buffer
  combine    every token sums the outputs of its k experts with the routing weights

Two ways to move the rows.  Peer memory (``peer_rows_cap > 0``; GPUs of one NVLink domain, or
one rank): every local expert owns a fixed number of rows of its rank's symmetric buffer (the
GEMM's masked layout), the ranks all-gather the (rank, expert) histograms, two plan kernels
give every pair its row in the owner's buffer and the owner its per-expert row counts -- all
on the device, nothing about the routing comes back to the host -- one kernel stores the
token rows straight into the owners' buffers, the two masked GEMMs run on them, and one
kernel loads the k output rows of every token back; three bounded barriers separate the
phases, and with ``micro_batches`` > 1 the tokens are split and the parts run on streams of
their own so that one part's NVLink traffic overlaps another's GEMMs.  All-to-all (the
fallback when an expert overflows its rows, and the form the CPU tests run on gloo): counts
all-to-all, gather, ``all_to_all_single`` with split sizes, scatter; the reverse for the
combine.  Both give every expert the same rows in the same order.

The reference project has no multi-GPU mode; this one follows the contiguous-layout
contract of its GEMM (python/nvfp4_gemm/layout.py:155-169 there: rows grouped by expert,
group starts aligned).  Collectives go through ``torch.distributed`` (NCCL over NVLink on
GPUs, gloo in the CPU tests).  Row movement, SwiGLU, the weighted sum and the peer-path plan
run as CUDA kernels of the library for CUDA tensors and as tensor operations for the CPU
tests of the host logic.  The GEMM is injectable so that
the CPU tests can stand in a checker.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


def route_topk(logits: torch.Tensor, k: int):
    """Softmax routing: top-k expert ids (T, k) and their weights renormalised to sum to 1."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(probs, k, dim=-1)
    return ids, w / w.sum(dim=-1, keepdim=True)


@dataclass
class Dispatch:
    """Everything the combine step needs to undo the dispatch."""
    order: torch.Tensor          # (T*k,) pair index sorted by global expert id
    send_counts: list            # rows sent to each rank
    recv_counts: list            # rows received from each rank
    place: torch.Tensor          # (rows received,) row of the padded expert-major buffer
    group_sizes: list            # padded rows per local expert
    real_sizes: list             # real rows per local expert
    rows_padded: int


def _pad(n: torch.Tensor, alignment: int) -> torch.Tensor:
    return (n + alignment - 1) // alignment * alignment


def plan_dispatch(topk_ids: torch.Tensor, num_experts: int, world: int, alignment: int,
                  group: Optional[dist.ProcessGroup] = None) -> Dispatch:
    """Sort the (token, expert) pairs by destination, exchange the count matrix and work out
    where each received row lands in the padded expert-major buffer."""
    e_local = num_experts // world
    flat = topk_ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts).reshape(world, e_local)   # [dest rank, local expert]
    if world > 1:
        recv = torch.empty_like(counts)
        dist.all_to_all_single(recv, counts.contiguous(), group=group)             # recv[src, e] rows src sends for my expert e
    else:
        recv = counts
    send_counts = counts.sum(dim=1).tolist()
    recv_counts = recv.sum(dim=1).tolist()
    per_expert = recv.sum(dim=0)                                                   # real rows per local expert
    padded = _pad(per_expert, alignment)
    starts = torch.cumsum(padded, 0) - padded                                      # padded start of each expert
    # rows arrive source-major, expert-minor; inside expert e the rows of source s follow those of sources < s
    before = torch.cumsum(recv, dim=0) - recv                                      # [src, e] rows of e from earlier sources
    seg_start = (starts.unsqueeze(0) + before).reshape(-1)                         # start of segment (src, e)
    seg_len = recv.reshape(-1)
    seg_id = torch.repeat_interleave(torch.arange(seg_len.numel(), device=flat.device), seg_len)
    first = torch.cumsum(seg_len, 0) - seg_len
    place = seg_start[seg_id] + (torch.arange(seg_id.numel(), device=flat.device) - first[seg_id])
    return Dispatch(order=order, send_counts=send_counts, recv_counts=recv_counts, place=place,
                    group_sizes=padded.tolist(), real_sizes=per_expert.tolist(), rows_padded=int(padded.sum()))


@dataclass
class MaskedDispatch:
    """Routing plan of the peer-memory path: where every (token, choice) pair lives in its owner's buffer, in which
    every local expert owns `cap_m` rows (the masked layout).  Everything is a device tensor."""
    dst_rank: torch.Tensor       # (T*k,) owner rank of pair p = token * k + choice
    dst_row: torch.Tensor        # (T*k,) row in the owner's buffer (local expert * cap_m + position), -1 = does not fit
    masked_m: torch.Tensor       # (E_local,) int32 real rows of this rank's experts (clamped to cap_m)
    overflow: Optional[torch.Tensor] = None    # CPU form only: whether some expert anywhere exceeds cap_m


def plan_dispatch_masked(topk_ids: torch.Tensor, num_experts: int, world: int, rank: int, cap_m: int,
                         group: Optional[dist.ProcessGroup] = None, status: Optional[torch.Tensor] = None) -> MaskedDispatch:
    """Every rank gathers the whole (source rank, expert) count matrix and from it works out, without a second
    exchange and without a host read-back, the row of each of its pairs in the owner's buffer: expert-major with
    cap_m rows per expert, inside an expert the rows of lower source ranks first and a rank's own pairs in their
    order -- the same order the all-to-all plan produces."""
    e_local = num_experts // world
    flat = topk_ids.reshape(-1).contiguous()
    if flat.is_cuda:
        from . import _C
        counts = _C.expert_histogram(flat, num_experts)
    else:
        counts = torch.zeros(num_experts, dtype=torch.int64).scatter_add_(0, flat, torch.ones_like(flat))
    if world > 1:
        gathered = counts.new_empty(world * num_experts)
        dist.all_gather_into_tensor(gathered, counts, group=group)
    else:
        gathered = counts
    dst_rank = torch.div(flat, e_local, rounding_mode="floor")
    if flat.is_cuda:
        masked_m, dst_row = _C.plan_peer_masked(gathered, flat, world, rank, cap_m, status)
        return MaskedDispatch(dst_rank=dst_rank, dst_row=dst_row, masked_m=masked_m)
    # the same plan as tensor operations (CPU tests of the host logic)
    all_counts = gathered.reshape(world, num_experts)
    total = all_counts.sum(dim=0)
    before = (torch.cumsum(all_counts, dim=0) - all_counts)[rank]             # rows of each expert from lower ranks
    order = torch.argsort(flat, stable=True)
    first = torch.cumsum(counts, 0) - counts                                  # first sorted index of each expert
    expert_sorted = flat[order]
    within = before[expert_sorted] + torch.arange(order.numel()) - first[expert_sorted]
    row_sorted = torch.where(within < cap_m, (expert_sorted % e_local) * cap_m + within, torch.full_like(within, -1))
    dst_row = torch.empty_like(row_sorted)
    dst_row[order] = row_sorted
    masked_m = total.reshape(world, e_local)[rank].clamp(max=cap_m).to(torch.int32)
    return MaskedDispatch(dst_rank=dst_rank, dst_row=dst_row, masked_m=masked_m, overflow=(total > cap_m).any())


class PeerBuffers:
    """What one in-flight step of the peer-memory path owns: the symmetric input and output buffers of this rank's
    experts in the masked layout (E_local, cap_m, hidden), mapped into every rank of the group, the local gate+up
    buffer, the address tables, the flag array of the bounded barrier and the step's status word."""

    NUM_SLOTS = 8

    def __init__(self, e_local: int, cap_m: int, hidden: int, inter: int, device: torch.device, group=None, world: int = 1,
                 rank: int = 0, quantized: bool = False, fused_swiglu: bool = False):
        self.e_local, self.cap_m, self.hidden, self.world, self.rank = e_local, cap_m, hidden, world, rank
        self.rows_cap = e_local * cap_m
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        # between the two GEMMs: the (rows, 2 I) BF16 gate+up output, or -- SwiGLU and the down-projection's activation
        # quantisation folded into the up-projection's epilogue -- the quantised (rows, I) activation itself
        self.h, self.hq = None, None
        if fused_swiglu:
            from . import _C
            self.hq = _C.QuantizedRows(torch.zeros(self.rows_cap * (inter + inter // 8), dtype=torch.uint8, device=device), e_local, cap_m, inter)
        else:
            self.h = torch.zeros(e_local, cap_m, 2 * inter, dtype=torch.bfloat16, device=device)
        self.epoch = [0] * self.NUM_SLOTS
        # the input buffer holds BF16 rows, or -- quantised dispatch -- the senders' NVFP4 codes and block scales
        # (1.125 bytes per element: three planes in one allocation, see _C.QuantizedRows)
        in_shape = (self.rows_cap * (hidden + hidden // 8),) if quantized else (e_local, cap_m, hidden)
        in_dtype = torch.uint8 if quantized else torch.bfloat16
        self.q = None
        if world == 1:                      # one rank: the same kernels on ordinary buffers, nobody to wait for
            self.a = torch.zeros(in_shape, dtype=in_dtype, device=device)
            self.out = torch.zeros(e_local, cap_m, hidden, dtype=torch.bfloat16, device=device)
            self.a_peers = torch.tensor([self.a.data_ptr()], dtype=torch.int64, device=device)
            self.out_peers = torch.tensor([self.out.data_ptr()], dtype=torch.int64, device=device)
            self.flag_peers = None
            if quantized:
                from . import _C
                self.q = _C.QuantizedRows(self.a, e_local, cap_m, hidden)
            return
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.a = symm.empty(*in_shape, dtype=in_dtype, device=device)
        self.out = symm.empty(e_local, cap_m, hidden, dtype=torch.bfloat16, device=device)
        self.flags = symm.empty(self.NUM_SLOTS * world, dtype=torch.int64, device=device)
        handles = [symm.rendezvous(t, group) for t in (self.a, self.out, self.flags)]
        self.a.zero_()                      # rows past an expert's count are computed like real rows: keep them finite
        self.out.zero_()
        self.flags.zero_()
        if quantized:
            from . import _C
            self.q = _C.QuantizedRows(self.a, e_local, cap_m, hidden)
        self.a_peers, self.out_peers, self.flag_peers = (
            torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=device) for h in handles)
        torch.cuda.synchronize(device)
        handles[0].barrier(channel=0)       # set-up only: every rank's buffers and flags are zero before the first step
        torch.cuda.synchronize(device)

    def barrier(self, slot: int, budget_cycles: int = 2_000_000_000) -> None:
        """All ranks of the group, ordered on the current stream.  The wait is bounded: a peer that never arrives costs
        `budget_cycles` clock cycles and bit 1 of the status word, not a hung GPU."""
        if self.world == 1:
            return
        from . import _C
        self.epoch[slot] += 1
        _C.peer_barrier(self.flag_peers, self.rank, self.world, slot, self.epoch[slot], self.status, budget_cycles)


def _exchange(rows: torch.Tensor, send_counts, recv_counts, group) -> torch.Tensor:
    out = rows.new_empty(sum(recv_counts), rows.shape[1])
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts,
                           group=group)
    return out


def swiglu(gate_up: torch.Tensor, native: bool = True) -> torch.Tensor:
    """silu(gate) * up on the fused (rows, 2*I) up-projection output, BF16 in and out."""
    if gate_up.is_cuda and native:
        from . import _C
        return _C.swiglu(gate_up)
    gate, up = gate_up.float().chunk(2, dim=-1)
    return (torch.nn.functional.silu(gate) * up).to(torch.bfloat16)


class ExpertParallelMoE:
    """One MoE layer with its experts split evenly over the ranks of ``group``.

    ``up`` / ``down`` are (b, sfb, gw) triples of this rank's experts as produced by
    ``quantize_weight_nvfp4``: up (E_local, 2*I, H), down (E_local, H, I).
    ``gemm(a, b, sfb, gw, d, m_indices)`` defaults to the CUDA kernel.
    """

    def __init__(self, num_experts: int, hidden: int, inter: int, up, down, group=None, alignment: int = 128,
                 gemm: Optional[Callable] = None, native_glue: bool = True, peer_rows_cap: int = 0, micro_batches: int = 1,
                 check_each_step: bool = True, comm_sms: int = 24, quantized_dispatch: bool = True, bulk_combine: bool = True,
                 fused_swiglu: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts do not split evenly over {self.world} ranks")
        self.num_experts, self.hidden, self.inter, self.alignment = num_experts, hidden, inter, alignment
        self.e_local = num_experts // self.world
        self.up, self.down = up, down
        self.gemm_swiglu = None                # SwiGLU folded into the down-projection (CUDA library only)
        self.gemm_masked = None
        if gemm is None:
            from . import _C
            gemm = _C.m_grouped_bf16_dual_nvfp4_gemm_contiguous
            self.gemm_masked = _C.m_grouped_bf16_dual_nvfp4_gemm_masked
            if hidden % 256 == 0:
                self.gemm_swiglu = _C.m_grouped_swiglu_dual_nvfp4_gemm_contiguous
        self.gemm = gemm
        self.native_glue = native_glue         # False: tensor operations even for CUDA tensors (a test's comparison arm)
        # peer_rows_cap > 0: dispatch and combine go through peer memory.  It is the number of rows every local expert
        # owns in this rank's buffers, per micro-batch (rounded up to the GEMM's 128-row tile); a step in which some
        # expert receives more takes the all-to-all path instead -- on every rank, since all see the same histograms.
        self.micro = max(1, int(micro_batches))
        self.check_each_step = check_each_step
        # With several micro-batches the dispatch and combine kernels get `comm_sms` SMs to themselves and the GEMMs are
        # sized to the others, so that one micro-batch's NVLink traffic runs beside another's GEMMs whichever is
        # launched first; with one micro-batch nothing overlaps and every kernel uses the whole GPU.
        self.comm_sms = int(comm_sms) if self.micro > 1 else 0
        self.peer = None                       # list of PeerBuffers, one per micro-batch in flight
        self.peer_error = None
        self.steps_repeated = 0                # steps that overflowed the buffers and were repeated over the all-to-all path
        masked_ok = self.gemm_masked is not None and (2 * inter) % 256 == 0 and hidden % 256 == 0
        # Quantised dispatch: the sender runs Algorithm 1 once per token and the rows cross NVLink as NVFP4 codes and
        # scales (1.125 instead of 2 bytes per element); the owners' up-projection then starts from the codes.  Same
        # codes as quantising the BF16 rows on arrival, so the layer's output does not change by a bit.
        self.quantized_dispatch = bool(quantized_dispatch) and hidden % 1024 == 0 and hidden <= 8192
        self.bulk_combine = bool(bulk_combine)   # combine fetches rows by bulk copies into shared memory (see combine_rows_bulk_kernel)
        # SwiGLU and the down-projection's activation quantisation in the up-projection's epilogue (needs the quantised
        # dispatch's GEMM entry and gate/up-interleaved weights; same bits as the separate kernels)
        self.fused_swiglu = bool(fused_swiglu) and self.quantized_dispatch and inter % 128 == 0 and self.gemm_masked is not None
        self.up_interleaved = None
        if peer_rows_cap > 0 and torch.cuda.is_available() and masked_ok:
            dev = torch.device("cuda", torch.cuda.current_device())
            cap_m = (int(peer_rows_cap) + 127) // 128 * 128
            try:
                self.peer = [PeerBuffers(self.e_local, cap_m, hidden, inter, dev, group, self.world, self.rank,
                                         quantized=self.quantized_dispatch, fused_swiglu=self.fused_swiglu)
                             for _ in range(self.micro)]
                if self.fused_swiglu:
                    from . import _C
                    self.up_interleaved = (*_C.interleave_gate_up(up[0], up[1], self.e_local, inter), up[2])
                self.streams = [torch.cuda.Stream(device=dev) for _ in range(self.micro)] if self.micro > 1 else []
            except Exception as exc:                                   # symmetric memory unavailable: keep the NCCL path
                self.peer = None
                self.peer_error = repr(exc)
            if self.world > 1:
                # every rank must take the same path: one rank without buffers sends all of them to the all-to-all
                ok = torch.tensor([1 if self.peer is not None else 0], dtype=torch.int32, device=dev)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) == 0 and self.peer is not None:
                    self.peer = None
                    self.peer_error = "symmetric memory unavailable on another rank"
        self.last = None                       # Dispatch of the most recent call (for accounting)

    def dispatch(self, x: torch.Tensor, topk_ids: torch.Tensor):
        k = topk_ids.shape[1]
        plan = plan_dispatch(topk_ids, self.num_experts, self.world, self.alignment, self.group)
        a = x.new_zeros(plan.rows_padded, x.shape[1])
        if x.is_cuda and self.native_glue:
            from . import _C
            n = plan.order.numel()
            if self.world > 1:
                rows = x.new_empty(n, x.shape[1])
                _C.permute_rows(x, n, rows, src_idx=plan.order, src_div=k)                  # token rows in send order
                recv = _exchange(rows, plan.send_counts, plan.recv_counts, self.group)
                _C.permute_rows(recv, recv.shape[0], a, dst_idx=plan.place)                 # into the padded groups
            else:
                _C.permute_rows(x, n, a, src_idx=plan.order, src_div=k, dst_idx=plan.place)  # both in one pass
            return plan, a
        rows = x[plan.order // k]
        recv = _exchange(rows, plan.send_counts, plan.recv_counts, self.group) if self.world > 1 else rows
        a[plan.place] = recv
        return plan, a

    def experts(self, a: torch.Tensor, plan: Dispatch) -> torch.Tensor:
        from .layout import make_m_indices
        m_indices = make_m_indices(plan.group_sizes, device=a.device, alignment=self.alignment)
        h = torch.empty(a.shape[0], 2 * self.inter, dtype=torch.bfloat16, device=a.device)
        self.gemm(a, *self.up, h, m_indices)
        out = torch.empty(a.shape[0], self.hidden, dtype=torch.bfloat16, device=a.device)
        self._down(h, out, m_indices)
        return out

    def _down(self, h: torch.Tensor, out: torch.Tensor, m_indices: torch.Tensor) -> None:
        """SwiGLU and the down-projection; one fused call where the library offers it."""
        if self.gemm_swiglu is not None and self.native_glue and h.is_cuda:
            self.gemm_swiglu(h, *self.down, out, m_indices)
        else:
            self.gemm(swiglu(h, native=self.native_glue), *self.down, out, m_indices)

    def combine(self, out: torch.Tensor, plan: Dispatch, topk_w: torch.Tensor, tokens: int) -> torch.Tensor:
        k = topk_w.shape[1]
        if out.is_cuda and self.native_glue:
            from . import _C
            n = plan.place.numel()
            inverse = torch.empty_like(plan.order)
            inverse[plan.order] = torch.arange(plan.order.numel(), device=out.device)      # pair (t, j) -> its row in send order
            if self.world > 1:
                rows = out.new_empty(n, out.shape[1])
                _C.permute_rows(out, n, rows, src_idx=plan.place)
                back = _exchange(rows, plan.recv_counts, plan.send_counts, self.group)
                return _C.combine_rows(back, inverse, topk_w.float().contiguous().reshape(-1), tokens)
            # one rank: row i of the send order sits at place[i] of the expert-major buffer
            return _C.combine_rows(out, plan.place[inverse], topk_w.float().contiguous().reshape(-1), tokens)
        rows = out[plan.place]
        back = _exchange(rows, plan.recv_counts, plan.send_counts, self.group) if self.world > 1 else rows
        y = torch.zeros(tokens, self.hidden, dtype=torch.float32, device=out.device)
        y.index_add_(0, plan.order // k, back.float() * topk_w.reshape(-1)[plan.order].unsqueeze(1))
        return y.to(torch.bfloat16)

    def _peer_step(self, buf: "PeerBuffers", x, topk_ids, topk_w, y, marks: Optional[list] = None, gemm_gate=None) -> None:
        """One (micro-)step over peer memory on the current stream, into `y`.  Nothing here reads anything back to the
        host.  Everything that can fail on this rank alone -- argument checks, allocations -- happens before the first
        barrier; if a call between the barriers raises all the same, the remaining barriers are still enqueued before
        the exception travels on, so that the other ranks' waits are not left to run into their time limit."""
        from . import _C

        def mark():
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append(ev)

        k = topk_ids.shape[1]
        _C._require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == self.hidden and x.stride(1) == 1,
                    "x is a (tokens, hidden) BF16 CUDA tensor")
        _C._require(topk_ids.shape == topk_w.shape and topk_ids.shape[0] == x.shape[0] and topk_ids.dtype == torch.int64,
                    "topk_ids (int64) and topk_w have one row per token")
        w_flat = topk_w.float().contiguous().reshape(-1)
        mark()
        plan = plan_dispatch_masked(topk_ids, self.num_experts, self.world, self.rank, buf.cap_m, self.group, buf.status)
        self.last = plan
        mark()
        pending = [0, 1, 2]                         # barrier slots of this step still to be enqueued
        try:
            buf.barrier(pending.pop(0))             # every rank has finished with these buffers (its previous step on them)
            if buf.q is not None:
                _C.dispatch_quantized_peer(x, k, buf.a_peers, plan.dst_rank, plan.dst_row, buf.q, buf.status, sm_budget=self.comm_sms)
            else:
                _C.dispatch_rows_peer(x, None, k, buf.a_peers, plan.dst_rank, plan.dst_row, self.hidden, buf.rows_cap, buf.status,
                                      sm_budget=self.comm_sms)
            buf.barrier(pending.pop(0))             # all rows have landed everywhere
            mark()
            # Micro-batches: the GEMMs of the parts run one part after the other (each fills the SMs it is given), so
            # that a part's combine has the whole GEMM phase of the next part to hide under.  Left to the hardware's
            # choice the parts' GEMM kernels alternate, every part finishes late and the combines pile up at the end.
            if gemm_gate is not None and gemm_gate[0] is not None:
                torch.cuda.current_stream().wait_event(gemm_gate[0])
            if buf.hq is not None:
                _C.relayout_scales(buf.q, plan.masked_m)
                _C.m_grouped_quantized_swiglu_dual_nvfp4_gemm_masked(buf.q, *self.up_interleaved, buf.hq, plan.masked_m,
                                                                     device_status=buf.status)
                _C.m_grouped_quantized_dual_nvfp4_gemm_masked(buf.hq, *self.down, buf.out, plan.masked_m, device_status=buf.status)
            else:
                if buf.q is not None:
                    _C.relayout_scales(buf.q, plan.masked_m)
                    _C.m_grouped_quantized_dual_nvfp4_gemm_masked(buf.q, *self.up, buf.h, plan.masked_m, device_status=buf.status)
                else:
                    self.gemm_masked(buf.a, *self.up, buf.h, plan.masked_m, device_status=buf.status)
                self.gemm_masked(buf.h, *self.down, buf.out, plan.masked_m, fold_swiglu=True, device_status=buf.status)
            if gemm_gate is not None:
                gemm_gate[0] = torch.cuda.Event()
                gemm_gate[0].record()
            mark()
            buf.barrier(pending.pop(0))             # every rank's expert outputs are complete
            _C.combine_rows_peer(buf.out_peers, self.hidden, plan.dst_rank, plan.dst_row, w_flat, x.shape[0], self.hidden,
                                 buf.rows_cap, out=y, sm_budget=self.comm_sms, bulk=self.bulk_combine, status=buf.status)
            mark()
        except BaseException:
            for slot in pending:
                buf.barrier(slot)
            raise

    def forward_peer(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, marks: Optional[list] = None):
        """One step over peer memory.  With micro_batches > 1 the tokens are cut into that many parts, each with buffers
        and a stream of its own, so that the NVLink traffic of one part runs under the GEMMs of another; every token's
        result is the same whichever part it is in.  `marks`, if given, receives a CUDA event after each phase of the
        (first) part: start, plan, dispatch, experts, combine."""
        tokens = x.shape[0]
        y = torch.empty(tokens, self.hidden, dtype=torch.bfloat16, device=x.device)
        if self.micro == 1 or tokens < self.micro:
            self._peer_step(self.peer[0], x, topk_ids, topk_w, y, marks)
            return y
        from . import _C
        cur = torch.cuda.current_stream()
        bounds = [tokens * i // self.micro for i in range(self.micro + 1)]
        all_sms = _C.get_num_sms()
        _C.set_num_sms(max(all_sms - self.comm_sms, 1))      # the GEMMs leave the communication kernels their SMs
        gate = [None]                                        # event after the previous part's GEMMs
        try:
            for i, stream in enumerate(self.streams):
                lo, hi = bounds[i], bounds[i + 1]
                stream.wait_stream(cur)
                with torch.cuda.stream(stream):
                    self._peer_step(self.peer[i], x[lo:hi], topk_ids[lo:hi], topk_w[lo:hi], y[lo:hi], marks if i == 0 else None, gate)
            for stream in self.streams:
                cur.wait_stream(stream)
        finally:
            _C.set_num_sms(all_sms)
        return y

    def read_status(self) -> int:
        """Reads and clears the status words of the peer-memory buffers (synchronises): bit 0 a GEMM's wait expired,
        bit 1 a barrier's wait expired (a peer never arrived), bit 2 an expert received more rows than it owns, bit 3 a
        routing entry out of range.  Bits 0, 1 and 3 raise; the overflow bit is returned for the caller to act on."""
        bits = 0
        for buf in self.peer or []:
            bits |= int(buf.status.item())
            buf.status.zero_()
        if bits & 0b1011:
            raise RuntimeError(f"expert-parallel step failed on the device (status {bits:#x}: "
                               f"{'GEMM wait expired; ' if bits & 1 else ''}{'a peer never reached a barrier; ' if bits & 2 else ''}"
                               f"{'routing entry out of range' if bits & 8 else ''})")
        return bits

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
        if self.peer is not None and x.is_cuda:
            y = self.forward_peer(x, topk_ids, topk_w)
            # the one host read of a step, after everything has been enqueued: did every expert fit its rows?
            if not self.check_each_step or not (self.read_status() & 4):
                return y
            self.steps_repeated += 1
        plan, a = self.dispatch(x, topk_ids)
        self.last = plan
        out = self.experts(a, plan)
        return self.combine(out, plan, topk_w, x.shape[0])

    __call__ = forward
