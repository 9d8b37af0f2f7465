"""Expert-parallel MoE layer: experts sharded over the ranks of one NVSwitch box, tokens stay with their rank.

Not in the reference (it has no collective anywhere); built on the reference's seam
`_compute_experts(hidden_states, router_weights, selected_experts)`
(cute_kernels/kernels/scattermoe/torch_implementation.py:135-137).

Per forward pass on rank r (R ranks, E experts, E/R experts per rank, T local tokens, k slots):
  1. route locally: stable sort of the flat expert ids -> rows ordered by (owning rank, expert), counts (E)
  2. counts all-to-all (int32 (R, E/R), equal splits) -> how many rows every source sends to each local expert
  3. dispatch gather: send[n, :] = x[token(n), :] in sorted order (one HBM pass)
  4. rows all-to-all with variable splits (NCCL over NVLink); received rows land in local HBM
  5. local experts on the received rows: the fused SwiGLU expert path with k = 1 and unit gates
  6. rows all-to-all back (same splits reversed)
  7. un-sort to (token, slot) order and gate-weighted sum over the k slots at the source rank
Backward mirrors it: autograd replays steps 7..1 with the all-to-alls swapped, so a pass moves four row
payloads in total.  The gate gradient d<gate> = <unweighted expert output, upstream gradient> is formed at
the source rank in step 7's backward, so no extra payload travels for it.

The one host synchronisation per pass is the read of the split sizes (NCCL wants them as host integers).

Row operations (gather, combine, routing sort) are injected: the default runs this package's CUDA kernels;
the CPU test-suite passes torch-indexing doubles to exercise the exchange logic over gloo.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class CudaRowOps:
    """Row operations on this package's kernels."""

    @staticmethod
    def route(flat_ids: torch.Tensor, num_experts: int, k: int):
        from .scattermoe import route

        se, ss, _, counts, _, _ = route(flat_ids, num_experts, k, True, False)
        return ss, counts

    @staticmethod
    def plan_tables(counts_all: torch.Tensor, ss: torch.Tensor, world: int, rank: int, num_experts: int):
        """The tables of the direct exchange in one launch (`b200moe_ep_plan`): start, base, dest_pos, local_offsets,
        summary, inverse permutation.  None when the sizes are outside the kernel's limits."""
        from . import _lib

        if world * num_experts > 4096 or num_experts > 256 or counts_all.dtype != torch.int32 or ss.dtype != torch.int64:
            return None
        dev, M = ss.device, ss.numel()
        start = torch.empty(world + 1, dtype=torch.int32, device=dev)
        base = torch.empty(world, dtype=torch.int32, device=dev)
        dest_pos = torch.empty(M, dtype=torch.int32, device=dev)
        local_offsets = torch.empty(num_experts // world, dtype=torch.int64, device=dev)
        summary = torch.empty(2, dtype=torch.int64, device=dev)
        inv = torch.empty(M, dtype=torch.int64, device=dev)
        _lib.check(_lib.lib().b200moe_ep_plan(_lib.ptr(counts_all), _lib.ptr(ss), world, rank, num_experts, M, _lib.ptr(start), _lib.ptr(base),
                                              _lib.ptr(dest_pos), _lib.ptr(local_offsets), _lib.ptr(summary), _lib.ptr(inv), _lib.stream_ptr(dev)), "ep_plan")
        return start, base, dest_pos, local_offsets, summary, inv

    @staticmethod
    def gather(x: torch.Tensor, idx: torch.Tensor, fan_out: int, coeff: torch.Tensor | None = None) -> torch.Tensor:
        """out[n, :] = x[idx[n] // fan_out, :] * coeff[idx[n]] (coeff optional), one pass."""
        from .ops import group

        out = torch.empty(idx.numel(), x.size(1), dtype=x.dtype, device=x.device)
        group(x, idx, out, coeff, fan_out)
        return out

    @staticmethod
    def combine(expanded: torch.Tensor, gates: torch.Tensor | None, k: int) -> torch.Tensor:
        from .ops import combine

        out = torch.empty(expanded.size(0) // k, expanded.size(1), dtype=expanded.dtype, device=expanded.device)
        combine(expanded, gates, out, k)
        return out

    @staticmethod
    def gate_grad(expanded: torch.Tensor, grad: torch.Tensor, k: int) -> torch.Tensor:
        """d_gates[t, j] = <expanded[t*k + j, :], grad[t, :]>."""
        from .ops import gate_grad

        return gate_grad(expanded, grad, k)


class _AllToAllRows(torch.autograd.Function):
    """Variable-split row exchange; the backward is the same exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, rows, send_splits, recv_splits, group):
        ctx.splits = (send_splits, recv_splits)
        ctx.group = group
        out = torch.empty(sum(recv_splits), rows.size(1), dtype=rows.dtype, device=rows.device)
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        send_splits, recv_splits = ctx.splits
        out = torch.empty(sum(send_splits), grad.size(1), dtype=grad.dtype, device=grad.device)
        dist.all_to_all_single(out, grad.contiguous(), output_split_sizes=send_splits, input_split_sizes=recv_splits, group=ctx.group)
        return out, None, None, None


class _DispatchGather(torch.autograd.Function):
    """send[n, :] = x[ss[n] // k, :].  Backward: un-sort the row gradients and sum the k slots of a token."""

    @staticmethod
    def forward(ctx, x, ss, inv, k, ops):
        ctx.save_for_backward(inv)
        ctx.k, ctx.ops = k, ops
        return ops.gather(x, ss, k)

    @staticmethod
    def backward(ctx, grad):
        (inv,) = ctx.saved_tensors
        expanded = ctx.ops.gather(grad.contiguous(), inv, 1)
        return ctx.ops.combine(expanded, None, ctx.k), None, None, None, None


class _UnsortCombine(torch.autograd.Function):
    """y[t, :] = sum_j gates[t, j] * rows[inv[t*k + j], :] with gradients for the rows and the gates."""

    @staticmethod
    def forward(ctx, rows, gates, ss, inv, ops):
        k = gates.size(1)
        expanded = ops.gather(rows, inv, 1)  # (token, slot) order
        ctx.save_for_backward(expanded, gates, ss)
        ctx.ops = ops
        return ops.combine(expanded, gates.contiguous(), k)

    @staticmethod
    def backward(ctx, grad):
        expanded, gates, ss = ctx.saved_tensors
        T, k = gates.shape
        grad = grad.contiguous()
        d_gates = _gate_grad_via(ctx.ops, expanded, grad, k).to(gates.dtype)
        # gradient of row n (sorted order) = gates[ss[n]] * grad[ss[n] // k]
        d_rows = ctx.ops.gather(grad, ss, k, gates.reshape(-1).contiguous())
        return d_rows, d_gates, None, None, None


def exchange_counts(counts: torch.Tensor, world: int, group) -> torch.Tensor:
    """counts: int32 (E) rows this rank sends to every expert.  Returns int32 (R, E/R): rows every source
    rank sends to each of this rank's experts."""
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts.contiguous(), group=group)
    return recv.view(world, -1)


last_received_rows = None  # rows this rank's experts received in the most recent exchange pass (load report)
_last_plan = None          # plan of the most recent peer-memory pass (its received-row count may not have been read yet)


def received_rows_of_last_pass() -> int:
    """Rows this rank's experts received in the most recent pass; reads the count from the plan where the pass itself
    ran without a host read."""
    if last_received_rows is not None:
        return int(last_received_rows)
    return _last_plan.received_rows() if _last_plan is not None else 0


def ep_experts(x, router_weights, selected_experts, num_experts: int, local_experts_fn: Callable, group, ops=CudaRowOps):
    """Routed experts over an expert-parallel group.  `local_experts_fn(rows, local_expert_ids)` evaluates
    this rank's experts on the received rows (unit gates, one expert per row) and must be differentiable."""
    world = dist.get_world_size(group)
    T, k = selected_experts.shape
    e_local = num_experts // world
    with torch.no_grad():
        flat = selected_experts.reshape(-1)
        ss, counts = ops.route(flat, num_experts, k)
        inv = torch.empty_like(ss)
        inv[ss] = torch.arange(ss.numel(), device=ss.device)
        recv_counts = exchange_counts(counts, world, group)
        # one host read per pass: NCCL takes the split sizes as host integers
        host = torch.cat([counts.view(world, e_local).sum(1), recv_counts.sum(1), ]).tolist()
        send_splits, recv_splits = [int(v) for v in host[:world]], [int(v) for v in host[world:]]
        global last_received_rows
        last_received_rows = sum(recv_splits)
        local_ids = torch.repeat_interleave(
            torch.arange(e_local, device=x.device).repeat(world), recv_counts.flatten().long(), output_size=sum(recv_splits)
        )
    send = _DispatchGather.apply(x, ss, inv, k, ops)
    recv = _AllToAllRows.apply(send, send_splits, recv_splits, group)
    out_rows = local_experts_fn(recv, local_ids)
    back = _AllToAllRows.apply(out_rows, recv_splits, send_splits, group)
    return _UnsortCombine.apply(back, router_weights.to(x.dtype), ss, inv, ops)


# --------------------------------------------------------------------------------------------------
# exchange over peer memory: this package's kernels store to / load from the peers' buffers directly
# --------------------------------------------------------------------------------------------------

BARRIER_LIMIT_CYCLES = 4_000_000_000  # about two seconds of SM clock: a peer that never arrives ends the wait with status 302


def _phase(name: str):
    from .scattermoe import phase

    return phase(name)


class PeerExchange:
    """Four symmetric (cap_rows, H) buffers per rank, mapped into every rank of the group:
    "x" (dispatched tokens), "y" (expert outputs), "dy" (dispatched output gradients), "dx" (input gradients of the
    received rows), plus a symmetric flag array for `barrier()`, which orders the ranks on the current stream with
    this package's bounded barrier kernel (a missing peer gives status 302 after about two seconds instead of a hang).

    The three methods `push`, `pull` and `barrier` are the whole interface the exchange logic uses; the CPU tests
    substitute an object with the same methods that moves rows between per-rank host tensors."""

    def __init__(self, group, cap_rows: int, width: int, dtype: torch.dtype, device: torch.device):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        self.group, self.cap_rows, self.width = group, cap_rows, width
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device(device)
        self.bufs, self.peer_ptrs, self._handles = {}, {}, {}
        for name in ("x", "y", "dy", "dx"):
            t = symm.empty(cap_rows, width, dtype=dtype, device=device)
            hdl = symm.rendezvous(t, group)
            self.bufs[name], self._handles[name] = t, hdl
            self.peer_ptrs[name] = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        flags = symm.empty(64, dtype=torch.int32, device=device)
        flags.zero_()
        fh = symm.rendezvous(flags, group)
        self._flags, self._flags_handle = flags, fh
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in fh.buffer_ptrs])
        self._epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flags are zero before anyone publishes an epoch
        self.backward_reads_pending = False
        self.sync_free = False  # True: no host read per pass (see _PeerDispatch.forward)
        self.direct = False     # True: rows are exchanged in the receiver's padded grouped order (see ep_experts_p2p)
        self.max_blocks = 0     # > 0: cap on the grid of the transfer kernels (one block per SM when they run beside GEMMs)
        self.host_rows = torch.empty(2, dtype=torch.int64).pin_memory()  # landing place of the per-pass host read

    def barrier(self) -> None:
        from ._lib import check, lib, ptr, status_word, stream_ptr

        self._epoch += 1
        with _phase("ep_barrier"):
            check(lib().b200moe_ep_barrier(self._flag_ptrs, self.rank, self.world, self._epoch, BARRIER_LIMIT_CYCLES, ptr(status_word(self.device)), stream_ptr(self.device)), "ep_barrier")

    def push(self, name: str, src, idx, fan_out: int, coeff, plan: "_Plan") -> None:
        from ._lib import check, dtype_code, lib, ptr, status_word, stream_ptr

        with _phase("ep_push_" + name):
            check(
                lib().b200moe_ep_push_rows_at(ptr(src), src.stride(0), ptr(idx), fan_out, ptr(coeff), self.peer_ptrs[name], ptr(plan.start), ptr(plan.base),
                                              ptr(plan.dest_pos), self.world, plan.ss.numel(), src.size(1), self.cap_rows, self.max_blocks, dtype_code(src),
                                              ptr(status_word(src.device)), stream_ptr(src.device)),
                "ep_push_rows",
            )

    def zero_fillers(self, name: str, plan: "_Plan") -> None:
        """Clears the filler rows of this rank's own buffer (peers only store real rows)."""
        from ._lib import check, dtype_code, lib, ptr, stream_ptr

        buf = self.bufs[name]
        check(lib().b200moe_zero_filler_rows(ptr(buf), buf.stride(0), ptr(plan.local_offsets), plan.local_offsets.numel(), buf.size(1), buf.size(0), dtype_code(buf),
                                             stream_ptr(buf.device)), "zero_filler_rows")

    def pull(self, name: str, gates, out, expanded, plan: "_Plan") -> None:
        from ._lib import check, dtype_code, lib, ptr, stream_ptr

        with _phase("ep_pull_" + name):
            check(
                lib().b200moe_ep_pull_combine_at(self.peer_ptrs[name], ptr(plan.inv), ptr(plan.start), ptr(plan.base), ptr(plan.dest_pos), self.world, self.cap_rows, self.max_blocks, ptr(gates),
                                                 ptr(out), out.stride(0), ptr(expanded), out.size(0), plan.k, out.size(1), dtype_code(out), stream_ptr(out.device)),
                "ep_pull_combine",
            )


class _Chain:
    """Orders the dispatches of the slices of one pipelined pass: a slice starts sending only when the slice before it has
    finished its own dispatch (and so has begun its expert GEMMs), so that every transfer but the first runs beside GEMMs
    instead of beside the other slices' transfers."""

    def __init__(self):
        self.fwd_event = None
        self.bwd_event = None

    def wait(self, which: str) -> None:
        ev = getattr(self, which)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def mark(self, which: str) -> None:
        ev = torch.cuda.Event()
        ev.record()
        setattr(self, which, ev)


class _Plan:
    """Where this rank's sorted rows go: computed once per pass from the all-gathered expert counts."""

    __slots__ = ("ss", "inv", "start", "base", "m_recv", "max_recv", "local_ids", "k", "_recv_counts", "_host", "_event", "_e_local", "_world", "chain", "dest_pos", "local_offsets")

    def local_ids_for_capacity(self, cap_rows: int) -> torch.Tensor:
        """Local expert of every row of a receive buffer of `cap_rows` rows, -1 for the rows past the received ones,
        computed on the device without knowing the received count on the host."""
        dev = self._recv_counts.device
        cum = self._recv_counts.reshape(-1).long().cumsum(0)
        seg = torch.searchsorted(cum, torch.arange(cap_rows, device=dev), right=True)
        ids = torch.cat([torch.arange(self._e_local, device=dev).repeat(self._world), torch.full((1,), -1, device=dev, dtype=torch.long)])
        return ids[seg.clamp(max=self._world * self._e_local)]

    def received_rows(self) -> int:
        """Rows this rank received in the pass of this plan (waits for the small host copy queued with the plan)."""
        if self._event is not None:
            self._event.synchronize()
        return int(self._host[0].item())

    def resolve(self) -> None:
        """Finish the plan with the one host read of the pass: the number of rows this rank receives (it sizes the local
        tensors) and the largest number any rank receives (every rank sees the same value, so a buffer overflow is
        refused by all ranks together).  The copy was queued when the plan was made, before the dispatch kernel; called
        after that kernel and its barrier are queued, the read returns while the GPU is still busy with them, so the
        device never waits for the host to catch up."""
        if self.m_recv is not None:
            return
        if self._event is not None:
            self._event.synchronize()
        self.m_recv, self.max_recv = int(self._host[0].item()), int(self._host[1].item())
        global last_received_rows
        last_received_rows = self.m_recv
        dev = self._recv_counts.device
        self.local_ids = torch.repeat_interleave(
            torch.arange(self._e_local, device=dev).repeat(self._world), self._recv_counts.reshape(-1).long(), output_size=self.m_recv
        )


def _make_plan(selected_experts, num_experts: int, world: int, rank: int, group, ops, host_rows=None, direct: bool = False) -> "_Plan":
    """`direct`: also compute, for every sorted row, its row in the RECEIVER's padded grouped order (`dest_pos`) and this
    rank's own inclusive expert offsets over everything it receives (`local_offsets`), so that rows can be stored where
    the receiver's expert GEMMs read them."""
    T, k = selected_experts.shape
    e_local = num_experts // world
    plan = _Plan()
    plan.chain = None
    plan.dest_pos = plan.local_offsets = None
    plan.k = k
    ss, counts = ops.route(selected_experts.reshape(-1), num_experts, k)
    plan.ss = ss
    counts_all = torch.empty(world * num_experts, dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(counts_all, counts.contiguous(), group=group)
    fused = ops.plan_tables(counts_all, ss, world, rank, num_experts) if direct and ss.is_cuda and hasattr(ops, "plan_tables") else None
    counts_all = counts_all.view(world, num_experts)
    if fused is not None:
        plan.start, plan.base, plan.dest_pos, plan.local_offsets, summary, plan.inv = fused
        plan._recv_counts, plan._e_local, plan._world = counts_all[:, rank * e_local : (rank + 1) * e_local], e_local, world
        plan.m_recv, plan.max_recv, plan.local_ids = None, None, None
        plan._host = host_rows if host_rows is not None else torch.empty(2, dtype=torch.int64).pin_memory()
        plan._host.copy_(summary, non_blocking=True)
        plan._event = torch.cuda.Event()
        plan._event.record()
        return plan
    plan.inv = torch.empty_like(ss)
    plan.inv[ss] = torch.arange(ss.numel(), device=ss.device)
    to_rank = counts_all.view(world, world, e_local).sum(-1)  # [source, destination]
    zero = torch.zeros(1, dtype=torch.int64, device=ss.device)
    plan.start = torch.cat([zero, to_rank[rank].cumsum(0)]).to(torch.int32)
    plan.base = (to_rank.cumsum(0) - to_rank)[rank].to(torch.int32)  # rows of lower-ranked sources in each destination
    recv_counts = counts_all[:, rank * e_local : (rank + 1) * e_local]
    plan._recv_counts, plan._e_local, plan._world = recv_counts, e_local, world
    plan.m_recv, plan.max_recv, plan.local_ids = None, None, None
    received = to_rank.sum(0).to(torch.int64)  # rows every rank receives: identical on all ranks
    if direct:
        ca = counts_all.long()
        total = ca.sum(0)                                              # rows of every expert over all sources
        padded = (total + 127) // 128 * 128                            # its segment in the owner's padded grouped order
        pv = padded.view(world, e_local)
        pad_start = (pv.cumsum(1) - pv).reshape(-1)                    # first row of the segment in the owner's buffers
        before = (ca.cumsum(0) - ca)[rank]                             # rows of lower-ranked sources inside the segment
        own = counts.long()
        excl = own.cumsum(0) - own                                     # first sorted row of every expert on this rank
        se = torch.repeat_interleave(torch.arange(num_experts, device=ss.device), own, output_size=ss.numel())
        plan.dest_pos = (pad_start[se] + before[se] + (torch.arange(ss.numel(), device=ss.device) - excl[se])).to(torch.int32)
        plan.local_offsets = total[rank * e_local : (rank + 1) * e_local].cumsum(0)
        summary = torch.stack([received[rank], pv.sum(1).max()])       # real rows here; most padded rows any rank's buffers must hold
    else:
        summary = torch.stack([received[rank], received.max()])
    if ss.is_cuda:
        plan._host = host_rows if host_rows is not None else torch.empty(2, dtype=torch.int64).pin_memory()
        plan._host.copy_(summary, non_blocking=True)
        plan._event = torch.cuda.Event()
        plan._event.record()
    else:
        plan._host, plan._event = summary.clone(), None
    return plan


def _gate_grad_via(ops, expanded: torch.Tensor, grad: torch.Tensor, k: int) -> torch.Tensor:
    """d_gates (T, k) through the row operations' `gate_grad` when they have one (the CUDA kernels do), else as the
    batched product of the reference (injected torch doubles on CPU)."""
    fn = getattr(ops, "gate_grad", None)
    if fn is not None:
        return fn(expanded, grad, k)
    return torch.bmm(expanded.view(grad.size(0), k, -1), grad.unsqueeze(2)).squeeze(-1)


class _PeerDispatch(torch.autograd.Function):
    """Forward: every rank stores its routed rows into the owners' "x" buffers.  Backward: the owners publish the
    input gradients of the rows they received in "dx"; the source pulls them and sums the k slots of a token.

    The backward's barrier is part of the protocol on every rank: the layer's input must require a gradient on all
    ranks or on none (`ep_experts_p2p` checks this across the group when `check_uniform` is set)."""

    @staticmethod
    def forward(ctx, x, xc, plan):
        ctx.xc, ctx.plan, ctx.shape = xc, plan, x.shape
        # Normally no barrier before the push: every rank finished reading its "x" rows of the previous pass before
        # it reached that pass's "y written" barrier (forward reads) and "dx written" barrier (the backward reads them
        # again for the weight gradient), and this rank has passed both.  If the previous pass may still run a backward
        # that never reached the "dx written" barrier (its input needed no gradient), order the ranks explicitly.
        if xc.backward_reads_pending:
            xc.barrier()
        xc.backward_reads_pending = torch.is_grad_enabled()
        if plan.chain is not None:
            plan.chain.wait("fwd_event")
        xc.push("x", x.contiguous(), plan.ss, plan.k, None, plan)
        xc.barrier()  # all rows have landed
        if plan.chain is not None:
            plan.chain.mark("fwd_event")
        if plan.dest_pos is not None:
            # rows sit in this rank's padded grouped order already; only the filler rows need clearing
            xc.zero_fillers("x", plan)
            plan.m_recv = xc.cap_rows
            return xc.bufs["x"]
        if getattr(xc, "sync_free", False):
            # No host read: the local tensors are sized by the buffer capacity and the rows past the received ones carry
            # no expert.  A buffer that is too small shows up as status word 301 (rows skipped), not as an exception.
            plan.m_recv = xc.cap_rows
            plan.local_ids = plan.local_ids_for_capacity(xc.cap_rows)
            return xc.bufs["x"]
        plan.resolve()
        # The decision is the same on every rank (the largest receive count of the group), so either all ranks go on to
        # the next barrier or none does.  Rows that did not fit were skipped by the push kernel (status 301).
        if plan.max_recv > xc.cap_rows:
            raise RuntimeError(f"expert-parallel exchange buffer too small: a rank receives {plan.max_recv} rows (this one {plan.m_recv}), capacity {xc.cap_rows}")
        return xc.bufs["x"][: plan.m_recv]

    @staticmethod
    def backward(ctx, grad_recv):
        xc, plan = ctx.xc, ctx.plan
        buf = xc.bufs["dx"][: plan.m_recv]
        if grad_recv.data_ptr() != buf.data_ptr():  # the fused kernels normally wrote it in place already
            buf.copy_(grad_recv)
        xc.barrier()  # every rank's "dx" rows are written
        xc.backward_reads_pending = False
        dx = torch.empty(ctx.shape, dtype=grad_recv.dtype, device=grad_recv.device)
        xc.pull("dx", None, dx, None, plan)
        # the next write into "dx" comes after the next pass's barriers, which no rank passes before it finished this pull
        return dx, None, None


class _PeerCombine(torch.autograd.Function):
    """Forward: the owners publish their output rows in "y"; the source pulls the k rows of each token and forms the
    gate-weighted sum.  Backward: gate gradients locally, gate-scaled output gradients stored into the owners' "dy"."""

    @staticmethod
    def forward(ctx, out_rows, gates, xc, plan, ops):
        T, k = gates.shape
        buf = xc.bufs["y"][: plan.m_recv]
        if out_rows.data_ptr() != buf.data_ptr():
            buf.copy_(out_rows)
        xc.barrier()  # every rank's "y" rows are written
        y = torch.empty(T, out_rows.size(1), dtype=out_rows.dtype, device=out_rows.device)
        expanded = torch.empty(T * k, out_rows.size(1), dtype=out_rows.dtype, device=out_rows.device)
        gates = gates.contiguous()
        xc.pull("y", gates, y, expanded, plan)
        ctx.save_for_backward(expanded, gates)
        ctx.xc, ctx.plan, ctx.ops = xc, plan, ops
        return y

    @staticmethod
    def backward(ctx, grad_y):
        expanded, gates = ctx.saved_tensors
        xc, plan = ctx.xc, ctx.plan
        T, k = gates.shape
        grad_y = grad_y.contiguous()
        with _phase("ep_gate_grad"):
            d_gates = _gate_grad_via(ctx.ops, expanded, grad_y, k).to(gates.dtype)
        if plan.chain is not None:
            plan.chain.wait("bwd_event")
        xc.push("dy", grad_y, plan.ss, k, gates.reshape(-1), plan)
        xc.barrier()  # all gradient rows have landed
        if plan.chain is not None:
            plan.chain.mark("bwd_event")
        if plan.dest_pos is not None:
            xc.zero_fillers("dy", plan)
        return xc.bufs["dy"][: plan.m_recv], d_gates, None, None, None


def ep_experts_p2p(x, router_weights, selected_experts, num_experts: int, local_experts_fn: Callable, xc, ops=CudaRowOps, plan=None):
    """Routed experts over an expert-parallel group with the row exchange done by this package's kernels on peer
    memory (see PeerExchange).  Same contract as `ep_experts`.  `x.requires_grad` must agree across the ranks.
    `plan`: a placement plan made beforehand with `_make_plan` for exactly these `selected_experts`."""
    world, rank = xc.world, dist.get_rank(xc.group)
    direct = getattr(xc, "direct", False)
    if plan is None:
        with torch.no_grad(), _phase("ep_plan"):
            plan = _make_plan(selected_experts, num_experts, world, rank, xc.group, ops, getattr(xc, "host_rows", None), direct)
    global _last_plan, last_received_rows
    _last_plan = plan
    if getattr(xc, "sync_free", False) or direct:
        last_received_rows = None
    recv = _PeerDispatch.apply(x, xc, plan)
    if direct:
        # Rows were stored straight into this rank's padded grouped order: the local layer needs only the expert offsets.
        # The one host read of the pass (largest padded row count of the group, for the collective overflow refusal) comes
        # after everything is queued: its copy was queued with the plan, so it has long finished.
        out_rows = local_experts_fn(recv, plan.local_offsets)
        y = _PeerCombine.apply(out_rows, router_weights.to(x.dtype), xc, plan, ops)
        if plan._event is not None:
            plan._event.synchronize()
        plan.max_recv = int(plan._host[1].item())
        if plan.max_recv > xc.cap_rows:
            raise RuntimeError(f"expert-parallel exchange buffer too small: a rank needs {plan.max_recv} padded rows, capacity {xc.cap_rows}")
        return y
    out_rows = local_experts_fn(recv, plan.local_ids)
    return _PeerCombine.apply(out_rows, router_weights.to(x.dtype), xc, plan, ops)


# --------------------------------------------------------------------------------------------------
# expert -> rank placement
# --------------------------------------------------------------------------------------------------


def make_placement(kind, num_experts: int, world: int, expected_load=None) -> torch.Tensor | None:
    """slot_of_expert (int64, E): the position of every expert in the rank-major order (rank = slot // (E / R)).

    "contiguous" (None): expert e at slot e, i.e. rank r owns experts [r*E/R, (r+1)*E/R).
    "strided": expert e on rank e % R.
    "balanced": greedy longest-first assignment of `expected_load` (one non-negative number per expert, e.g. running
        token counts) to the rank with the smallest load that still has a free slot, so that a skewed routing does not
        pile the popular experts onto one rank.
    A tensor / sequence of E distinct slots is taken as given.
    """
    e_local = num_experts // world
    if kind is None or (isinstance(kind, str) and kind == "contiguous"):
        return None
    if isinstance(kind, str) and kind == "strided":
        e = torch.arange(num_experts)
        return (e % world) * e_local + e // world
    if isinstance(kind, str) and kind == "balanced":
        assert expected_load is not None and len(expected_load) == num_experts
        load = torch.as_tensor(expected_load, dtype=torch.float64)
        order = torch.argsort(load, descending=True, stable=True).tolist()
        rank_load, rank_used = [0.0] * world, [0] * world
        slot = torch.empty(num_experts, dtype=torch.int64)
        for e in order:
            r = min((r_ for r_ in range(world) if rank_used[r_] < e_local), key=lambda r_: (rank_load[r_], r_))
            slot[e] = r * e_local + rank_used[r]
            rank_used[r] += 1
            rank_load[r] += float(load[e])
        return slot
    slot = torch.as_tensor(kind, dtype=torch.int64).clone()
    assert slot.numel() == num_experts and torch.equal(slot.sort().values, torch.arange(num_experts)), "placement must be a permutation of the expert slots"
    return slot


class MoE_B200_EP(nn.Module):
    """Expert-parallel MoE layer.  The gate is replicated; rank r holds the E/R experts whose slots
    (`make_placement`; default: expert e at slot e) fall into [r*E/R, (r+1)*E/R).

    Weights are drawn expert by expert from a seed shared by all ranks, so the union of the shards equals
    the single-GPU layer built from the same seed with `full_state_dict`-style gathering, whatever the placement.
    """

    def __init__(self, num_experts, num_experts_per_tok, hidden_size, intermediate_size, activation_function, is_glu, add_bias, std,
                 group=None, device=None, dtype=torch.float32, seed: int = 0, ops=CudaRowOps, local_experts_fn=None,
                 num_shared_experts: int = 0, shared_intermediate_size: int | None = None, router_scoring: str = "softmax",
                 exchange: str = "nccl", exchange_rows: int | None = None, placement=None, expected_load=None, micro_batches: int = 1, sync_free: bool = False, direct: bool = True):
        super().__init__()
        assert is_glu, "the expert-parallel layer implements GLU experts"
        assert router_scoring in ("softmax", "sigmoid")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        assert num_experts % self.world == 0, "experts must divide evenly over the ranks"
        self.num_experts, self.top_k = num_experts, num_experts_per_tok
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.e_local = num_experts // self.world
        # expert -> slot in the rank-major order; the routing sees slots, so everything after it is placement-agnostic
        slot_of_expert = make_placement(placement, num_experts, self.world, expected_load)
        self.register_buffer("slot_of_expert", None if slot_of_expert is None else slot_of_expert.to(device), persistent=False)
        expert_of_slot = torch.arange(num_experts) if slot_of_expert is None else torch.argsort(slot_of_expert)
        self.expert_of_slot = expert_of_slot.tolist()
        self.ops = ops
        self._local_experts_fn = local_experts_fn
        self.act = activation_function
        self.router_scoring = router_scoring
        self.num_shared_experts = num_shared_experts
        assert exchange in ("nccl", "p2p")
        # "p2p": rows move by this package's kernels over peer memory; exchange_rows = capacity of each buffer in rows
        def buffer_rows(rows: int) -> int:
            # the padded grouped order needs up to 127 filler rows per local expert on top of the rows themselves
            return (rows + (128 * self.e_local if direct else 0) + 127) // 128 * 128

        self.exchange = PeerExchange(self.group, buffer_rows(exchange_rows), hidden_size, dtype, torch.device(device)) if exchange == "p2p" else None
        # Pipelining (peer-memory exchange only): the rank's tokens are split into `micro_batches` parts, each with its own
        # exchange buffers and stream, so that the row transfers of one part run while the expert GEMMs of another do.
        # `direct` (peer-memory exchange): dispatched rows are stored in the receiver's padded grouped order and results are
        # fetched from there, so the receiving rank runs no sort, no gather pass and needs no host read
        if self.exchange is not None:
            self.exchange.sync_free = sync_free
            self.exchange.direct = direct
        self.micro_batches = micro_batches if exchange == "p2p" else 1
        self._pipe = None
        if self.micro_batches > 1:
            rows = buffer_rows((exchange_rows + self.micro_batches - 1) // self.micro_batches)
            self._pipe = [(PeerExchange(self.group, rows, hidden_size, dtype, torch.device(device)), torch.cuda.Stream(device)) for _ in range(self.micro_batches)]
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            for xc_, _ in self._pipe:
                xc_.sync_free = sync_free
                xc_.direct = direct
                xc_.max_blocks = sms  # the transfers of a slice run beside the other slices' GEMM CTAs: one block per SM
        # every rank draws with the same per-expert seeds on the same kind of device, so shards agree across ranks
        gen_dev = torch.device(device) if device is not None and torch.device(device).type == "cuda" else torch.device("cpu")

        def draw(shape, seed_, scale):
            g = torch.Generator(device=gen_dev).manual_seed(seed_)
            return (torch.randn(*shape, generator=g, device=gen_dev) * scale).to(dtype)

        self.gate = nn.Linear(hidden_size, num_experts, bias=False, device=device, dtype=dtype)
        with torch.no_grad():
            self.gate.weight.copy_(draw((num_experts, hidden_size), seed * 100003 + 1, hidden_size**-0.5))
        lo = self.rank * self.e_local
        mine = self.expert_of_slot[lo : lo + self.e_local]  # global ids of this rank's experts, in slot order
        fc = [draw((2 * intermediate_size, hidden_size), seed * 100003 + 17 + 2 * e, std) for e in mine]
        proj = [draw((hidden_size, intermediate_size), seed * 100003 + 18 + 2 * e, std) for e in mine]
        self.c_fc_weight = nn.Parameter(torch.stack(fc).to(device))
        self.c_proj_weight = nn.Parameter(torch.stack(proj).to(device))
        del fc, proj
        if num_shared_experts > 0:  # replicated; they see this rank's tokens only
            i_s = shared_intermediate_size or intermediate_size
            self.shared_c_fc_weight = nn.Parameter(torch.stack([draw((2 * i_s, hidden_size), seed * 100003 + 7 + 2 * s_, std) for s_ in range(num_shared_experts)]).to(device))
            self.shared_c_proj_weight = nn.Parameter(torch.stack([draw((hidden_size, i_s), seed * 100003 + 8 + 2 * s_, std) for s_ in range(num_shared_experts)]).to(device))

    def local_experts(self, rows: torch.Tensor, local_ids: torch.Tensor, exchange=None) -> torch.Tensor:
        """This rank's experts on the rows it received.  `local_ids`: the local expert of every row; with an exchange that
        places rows directly in the padded grouped order (`exchange.direct`) it is the inclusive expert offsets instead."""
        if self._local_experts_fn is not None:
            return self._local_experts_fn(rows, local_ids, self.c_fc_weight, self.c_proj_weight)
        from .scattermoe import fused_swiglu_experts, grouped_experts

        exchange = exchange if exchange is not None else self.exchange
        if exchange is not None and getattr(exchange, "direct", False):
            return grouped_experts(rows, self.c_fc_weight, self.c_proj_weight, local_ids, exchange.bufs["y"], exchange.bufs["dx"])
        ones = torch.ones(rows.size(0), 1, dtype=rows.dtype, device=rows.device)
        y_out = dx_out = None
        if exchange is not None and hasattr(exchange, "peer_ptrs"):  # the kernels write straight into the buffers the other ranks read
            y_out, dx_out = exchange.bufs["y"], exchange.bufs["dx"]
        return fused_swiglu_experts(rows, self.c_fc_weight, self.c_proj_weight, ones, local_ids.view(-1, 1), y_out, dx_out)

    def forward(self, hidden_states: torch.Tensor):
        shape = hidden_states.shape
        flat = hidden_states.view(-1, self.hidden_size)
        router_logits = self.gate(flat)
        vals, selected = router_logits.max(-1, keepdim=True) if self.top_k == 1 else router_logits.topk(self.top_k, dim=-1)
        if self.router_scoring == "sigmoid":
            scores = torch.sigmoid(vals.float())
            router_weights = (scores / scores.sum(-1, keepdim=True)).type_as(flat)
        else:
            router_weights = F.softmax(vals.float(), dim=-1).type_as(flat)
        out = self._compute_experts(flat, router_weights, selected)
        if self.num_shared_experts > 0:
            out = out + self._compute_shared_experts(flat)
        return out.view(shape), router_logits

    def _compute_shared_experts(self, hidden_states):
        from .scattermoe import fused_swiglu_experts

        T, S = hidden_states.shape[0], self.num_shared_experts
        ones = torch.ones(T, S, dtype=hidden_states.dtype, device=hidden_states.device)
        ids = torch.arange(S, device=hidden_states.device).expand(T, S)
        return fused_swiglu_experts(hidden_states, self.shared_c_fc_weight, self.shared_c_proj_weight, ones, ids)

    def allreduce_shared_grads(self) -> None:
        """Sums the gradients of the replicated shared experts over the ranks."""
        for p in (getattr(self, "shared_c_fc_weight", None), getattr(self, "shared_c_proj_weight", None)):
            if p is not None and p.grad is not None:
                dist.all_reduce(p.grad, group=self.group)

    def _compute_experts(self, hidden_states, router_weights, selected_experts):
        if self.slot_of_expert is not None:
            selected_experts = self.slot_of_expert[selected_experts]
        if self._pipe is not None and hidden_states.size(0) >= self.micro_batches:
            return self._compute_experts_pipelined(hidden_states, router_weights, selected_experts)
        if self.exchange is not None:
            return ep_experts_p2p(hidden_states, router_weights, selected_experts, self.num_experts, self.local_experts, self.exchange, self.ops)
        return ep_experts(hidden_states, router_weights, selected_experts, self.num_experts, self.local_experts, self.group, self.ops)

    def _compute_experts_pipelined(self, hidden_states, router_weights, selected_experts):
        """The same pass over `micro_batches` slices of the tokens, one stream and one set of exchange buffers per slice.
        The host queues slice after slice; on the GPU the dispatch of slice i+1 and the return of slice i-1 overlap the
        expert GEMMs of slice i (the GEMM kernels fill the SMs, the copy kernels run beside them).  Autograd runs every
        slice's backward on the stream of its forward, so the backward pass pipelines the same way.  Every rank must use
        the same number of slices."""
        main = torch.cuda.current_stream(hidden_states.device)
        T = hidden_states.size(0)
        bounds = [T * i // self.micro_batches for i in range(self.micro_batches + 1)]
        outs, received = [], 0
        sync_free_mode = self._pipe[0][0].sync_free
        global last_received_rows
        # The placement plans of all slices come first, on the calling stream: their small kernels (sort, count all-gather)
        # do not fit on an SM beside a GEMM CTA and would otherwise wait behind the previous slice's expert kernels.
        plans, chain = [], _Chain()
        with torch.no_grad(), _phase("ep_plan"):
            for i, (xc, _) in enumerate(self._pipe):
                plans.append(_make_plan(selected_experts[bounds[i] : bounds[i + 1]], self.num_experts, self.world, self.rank, xc.group, self.ops, xc.host_rows, xc.direct))
                plans[-1].chain = chain
        for i, (xc, stream) in enumerate(self._pipe):
            lo, hi = bounds[i], bounds[i + 1]
            stream.wait_stream(main)
            with torch.cuda.stream(stream):
                y_i = ep_experts_p2p(hidden_states[lo:hi], router_weights[lo:hi], selected_experts[lo:hi], self.num_experts,
                                     lambda rows, ids, xc=xc: self.local_experts(rows, ids, xc), xc, self.ops, plan=plans[i])
            y_i.record_stream(main)
            outs.append(y_i)
            received += received_rows_of_last_pass() if not sync_free_mode else 0
        for _, stream in self._pipe:
            main.wait_stream(stream)
        last_received_rows = received if not sync_free_mode else None
        self._plans_of_last_pass = plans
        return torch.cat(outs)

    def received_rows(self) -> int:
        """Rows this rank's experts received in the most recent pass (load report; may wait for a small host copy)."""
        plans = getattr(self, "_plans_of_last_pass", None)
        if self._pipe is not None and plans:
            return sum(p.received_rows() for p in plans)
        return received_rows_of_last_pass()

    def allreduce_replicated_grads(self) -> None:
        """Sums the gradient of the replicated gate over the ranks (tokens are data-parallel)."""
        if self.gate.weight.grad is not None:
            dist.all_reduce(self.gate.weight.grad, group=self.group)

    def full_state_dict(self) -> dict:
        """Gathers the expert shards into the single-GPU layer's `state_dict` layout (on every rank)."""
        fc = [torch.empty_like(self.c_fc_weight) for _ in range(self.world)]
        proj = [torch.empty_like(self.c_proj_weight) for _ in range(self.world)]
        dist.all_gather(fc, self.c_fc_weight.detach().contiguous(), group=self.group)
        dist.all_gather(proj, self.c_proj_weight.detach().contiguous(), group=self.group)
        fc, proj = torch.cat(fc), torch.cat(proj)  # slot order
        if self.slot_of_expert is not None:
            fc, proj = fc[self.slot_of_expert], proj[self.slot_of_expert]  # expert order
        return {"gate.weight": self.gate.weight.detach().clone(), "c_fc.weight": fc, "c_proj.weight": proj}

    def load_full_state_dict(self, sd: dict) -> None:
        lo, hi = self.rank * self.e_local, (self.rank + 1) * self.e_local
        mine = torch.as_tensor(self.expert_of_slot[lo:hi], device=sd["c_fc.weight"].device)
        with torch.no_grad():
            self.gate.weight.copy_(sd["gate.weight"])
            self.c_fc_weight.copy_(sd["c_fc.weight"][mine])
            self.c_proj_weight.copy_(sd["c_proj.weight"][mine])

    def expert_grads_in_expert_order(self):
        """(d_c_fc, d_c_proj) of this rank's experts together with their global expert ids (int64, e_local)."""
        lo = self.rank * self.e_local
        return self.c_fc_weight.grad, self.c_proj_weight.grad, torch.as_tensor(self.expert_of_slot[lo : lo + self.e_local])


# --------------------------------------------------------------------------------------------------
# multi-rank self check: the expert-parallel layer against the single-GPU layer on the union of the tokens
# --------------------------------------------------------------------------------------------------


def _rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def parity_selfcheck(group, device, cases=None) -> dict:
    """Runs small layers through `MoE_B200_EP` with both exchanges (and a strided placement) on every rank of `group` and
    compares outputs and gradients with the single-GPU layer `MoE_B200` holding the gathered weights, evaluated on the
    all-gathered tokens.  Token counts differ per rank.  Returns {"cases": {...: {y, dx, d_w_fc, d_w_proj, d_gate}},
    "worst": ..., "ok": bool}, identical on all ranks (the errors are max-reduced over the group).  Tolerances: relative L2
    1e-5 for fp32 and 1e-2 for bf16 (20x that for the gate-weight gradient, which sums over every token of the job)."""
    from . import _lib
    from .ops import swiglu_unchunked_torch
    from .scattermoe import MoE_B200

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if cases is None:
        bf = ("bf16_E64_k6_H512_I768", torch.bfloat16, 64, 6, 512, 768, 800)
        cases = [("fp32_E16_k4_H256_I384", torch.float32, 16, 4, 256, 384, 800, {}), bf + ({},),
                 (bf[0] + "_strided",) + bf[1:] + ({"placement": "strided"},),
                 (bf[0] + "_pipelined3",) + bf[1:] + ({"micro_batches": 3},),
                 (bf[0] + "_received_order",) + bf[1:] + ({"direct": False},),
                 (bf[0] + "_received_order_no_host_read",) + bf[1:] + ({"direct": False, "sync_free": True},)]
    report, ok = {}, True
    for name, dtype, E, k, H, I, T, extra in cases:
        if E % world:
            continue
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        counts = [T + 37 * r for r in range(world)]  # uneven shards
        gen = torch.Generator().manual_seed(4242)
        xs = [torch.randn(c, H, generator=gen) for c in counts]
        gs = [torch.randn(c, H, generator=gen) for c in counts]
        x_all, g_all = torch.cat(xs).to(device, dtype), torch.cat(gs).to(device, dtype)
        lo = sum(counts[:rank])
        p2p_only = any(key in extra for key in ("micro_batches", "direct", "sync_free"))
        for exchange in ("p2p",) if p2p_only else ("p2p", "nccl"):
            cap = (sum(counts) * k + 127) // 128 * 128
            layer = MoE_B200_EP(E, k, H, I, swiglu_unchunked_torch, True, False, 0.05, group=group, device=device, dtype=dtype, seed=5,
                                exchange=exchange, exchange_rows=cap, **extra)
            ref = MoE_B200(E, k, H, I, swiglu_unchunked_torch, True, False, 0.05).to(device).to(dtype)
            ref.load_state_dict(layer.full_state_dict())
            x = x_all[lo : lo + counts[rank]].clone().requires_grad_(True)
            y, _ = layer(x)
            y.backward(g_all[lo : lo + counts[rank]])
            layer.allreduce_replicated_grads()
            # The reference layer sees the shards one after the other, each with the shape the owning rank's router saw,
            # so that both sides select the same experts (a differently shaped gate GEMM may round a logit differently);
            # its parameter gradients accumulate over the shards.
            y_ref = dx_ref = None
            off = 0
            for r, c in enumerate(counts):
                xr = x_all[off : off + c].clone().requires_grad_(True)
                yr, _ = ref(xr)
                yr.backward(g_all[off : off + c])
                if r == rank:
                    y_ref, dx_ref = yr.detach(), xr.grad
                off += c
            _lib.check_status(torch.device(device))
            d_fc, d_proj, mine = layer.expert_grads_in_expert_order()
            mine = mine.to(device)
            errs = torch.tensor([
                _rel_l2(y.detach(), y_ref),
                _rel_l2(x.grad, dx_ref),
                _rel_l2(d_fc, ref.c_fc.weight.grad[mine]),
                _rel_l2(d_proj, ref.c_proj.weight.grad[mine]),
                _rel_l2(layer.gate.weight.grad, ref.gate.weight.grad),
            ], device=device, dtype=torch.float64)
            dist.all_reduce(errs, op=dist.ReduceOp.MAX, group=group)
            e = dict(zip(("y", "dx", "d_w_fc", "d_w_proj", "d_gate"), [float(v) for v in errs.cpu()]))
            report[f"{name}_{exchange}"] = e
            ok = ok and all(v < (20 * tol if n == "d_gate" else tol) for n, v in e.items()) and all(v == v for v in e.values())
            del layer, ref
    worst = max((v for e in report.values() for n, v in e.items() if n != "d_gate"), default=0.0)
    return {"cases": report, "worst": worst, "ok": bool(ok), "ranks": world}
