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
        return _gate_grad(expanded, grad, k)


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
        gate_grad = getattr(ctx.ops, "gate_grad", None)  # optional in injected row operations
        if gate_grad is not None:
            d_gates = gate_grad(expanded, grad, k).to(gates.dtype)
        else:
            d_gates = torch.bmm(expanded.view(T, k, -1), grad.unsqueeze(2)).squeeze(-1).to(gates.dtype)
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


class PeerExchange:
    """Four symmetric (cap_rows, H) buffers per rank, mapped into every rank of the group:
    "x" (dispatched tokens), "y" (expert outputs), "dy" (dispatched output gradients), "dx" (input gradients of the
    received rows).  `barrier()` orders the ranks on the current stream through the symmetric-memory signal pads."""

    def __init__(self, group, cap_rows: int, width: int, dtype: torch.dtype, device: torch.device):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        self.group, self.cap_rows, self.width = group, cap_rows, width
        self.world = dist.get_world_size(group)
        self.bufs, self.peer_ptrs, self._handles = {}, {}, {}
        for name in ("x", "y", "dy", "dx"):
            t = symm.empty(cap_rows, width, dtype=dtype, device=device)
            hdl = symm.rendezvous(t, group)
            self.bufs[name], self._handles[name] = t, hdl
            self.peer_ptrs[name] = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        self._barrier_handle = self._handles["x"]
        self.backward_reads_pending = False
        self.host_rows = torch.empty(1, dtype=torch.int64).pin_memory()  # landing place of the per-pass host read

    def barrier(self) -> None:
        self._barrier_handle.barrier(channel=0)


class _Plan:
    """Where this rank's sorted rows go: computed once per pass from the all-gathered expert counts."""

    __slots__ = ("ss", "inv", "start", "base", "m_recv", "local_ids", "k", "_recv_counts", "_host", "_event", "_e_local", "_world")

    def resolve(self) -> None:
        """Finish the plan with the one host read of the pass (the number of rows this rank receives sizes its local
        tensors).  The copy was queued when the plan was made, before the dispatch kernel; called after that kernel and
        its barrier are queued, the read returns while the GPU is still busy with them, so the device never waits for
        the host to catch up."""
        if self.m_recv is not None:
            return
        self._event.synchronize()
        self.m_recv = int(self._host.item())
        global last_received_rows
        last_received_rows = self.m_recv
        dev = self._recv_counts.device
        self.local_ids = torch.repeat_interleave(
            torch.arange(self._e_local, device=dev).repeat(self._world), self._recv_counts.reshape(-1).long(), output_size=self.m_recv
        )


def _make_plan(selected_experts, num_experts: int, world: int, rank: int, group, ops, host_rows=None) -> "_Plan":
    T, k = selected_experts.shape
    e_local = num_experts // world
    plan = _Plan()
    plan.k = k
    ss, counts = ops.route(selected_experts.reshape(-1), num_experts, k)
    plan.ss = ss
    plan.inv = torch.empty_like(ss)
    plan.inv[ss] = torch.arange(ss.numel(), device=ss.device)
    counts_all = torch.empty(world, num_experts, dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(counts_all, counts.contiguous(), group=group)
    to_rank = counts_all.view(world, world, e_local).sum(-1)  # [source, destination]
    zero = torch.zeros(1, dtype=torch.int64, device=ss.device)
    plan.start = torch.cat([zero, to_rank[rank].cumsum(0)]).to(torch.int32)
    plan.base = (to_rank.cumsum(0) - to_rank)[rank].to(torch.int32)  # rows of lower-ranked sources in each destination
    recv_counts = counts_all[:, rank * e_local : (rank + 1) * e_local]
    plan._recv_counts, plan._e_local, plan._world = recv_counts, e_local, world
    plan.m_recv, plan.local_ids = None, None
    plan._host = host_rows if host_rows is not None else torch.empty(1, dtype=torch.int64).pin_memory()
    plan._host.copy_(recv_counts.sum().to(torch.int64).reshape(1), non_blocking=True)
    plan._event = torch.cuda.Event()
    plan._event.record()
    return plan


def _push(xc: PeerExchange, name: str, src, idx, fan_out: int, coeff, plan: "_Plan") -> None:
    from .scattermoe import _launch

    _launch("ep_push_" + name, _push_impl, xc, name, src, idx, fan_out, coeff, plan)


def _pull(xc: PeerExchange, name: str, gates, out, expanded, plan: "_Plan") -> None:
    from .scattermoe import _launch

    _launch("ep_pull_" + name, _pull_impl, xc, name, gates, out, expanded, plan)


def _push_impl(xc: PeerExchange, name: str, src, idx, fan_out: int, coeff, plan: "_Plan") -> None:
    from ._lib import check, dtype_code, lib, ptr, status_word, stream_ptr

    M = plan.ss.numel()
    check(
        lib().b200moe_ep_push_rows(ptr(src), src.stride(0), ptr(idx), fan_out, ptr(coeff), xc.peer_ptrs[name], ptr(plan.start), ptr(plan.base),
                                   xc.world, M, src.size(1), xc.cap_rows, dtype_code(src), ptr(status_word(src.device)), stream_ptr(src.device)),
        "ep_push_rows",
    )


def _pull_impl(xc: PeerExchange, name: str, gates, out, expanded, plan: "_Plan") -> None:
    from ._lib import check, dtype_code, lib, ptr, stream_ptr

    check(
        lib().b200moe_ep_pull_combine(xc.peer_ptrs[name], ptr(plan.inv), ptr(plan.start), ptr(plan.base), xc.world, ptr(gates), ptr(out), out.stride(0),
                                      ptr(expanded), out.size(0), plan.k, out.size(1), dtype_code(out), stream_ptr(out.device)),
        "ep_pull_combine",
    )


def _gate_grad(expanded: torch.Tensor, grad_y: torch.Tensor, k: int) -> torch.Tensor:
    """d_gates (T, k): dot products of the kept expert rows with the output gradient of their token."""
    from ._lib import check, dtype_code, lib, ptr, stream_ptr

    T = grad_y.size(0)
    d_gates = torch.empty(T, k, dtype=grad_y.dtype, device=grad_y.device)
    check(
        lib().b200moe_ep_gate_grad(ptr(expanded), expanded.stride(0), ptr(grad_y), grad_y.stride(0), ptr(d_gates), T, k, grad_y.size(1), dtype_code(grad_y), stream_ptr(grad_y.device)),
        "ep_gate_grad",
    )
    return d_gates


class _PeerDispatch(torch.autograd.Function):
    """Forward: every rank stores its routed rows into the owners' "x" buffers.  Backward: the owners publish the
    input gradients of the rows they received in "dx"; the source pulls them and sums the k slots of a token."""

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
        _push(xc, "x", x.contiguous(), plan.ss, plan.k, None, plan)
        xc.barrier()  # all rows have landed
        plan.resolve()
        if plan.m_recv > xc.cap_rows:  # the push kernel skipped the rows that did not fit and raised status 301
            raise RuntimeError(f"expert-parallel exchange buffer too small: {plan.m_recv} rows arrive, capacity {xc.cap_rows}")
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
        _pull(xc, "dx", None, dx, None, plan)
        # the next write into "dx" comes after the next pass's barriers, which no rank passes before it finished this pull
        return dx, None, None


class _PeerCombine(torch.autograd.Function):
    """Forward: the owners publish their output rows in "y"; the source pulls the k rows of each token and forms the
    gate-weighted sum.  Backward: gate gradients locally, gate-scaled output gradients stored into the owners' "dy"."""

    @staticmethod
    def forward(ctx, out_rows, gates, xc, plan):
        T, k = gates.shape
        buf = xc.bufs["y"][: plan.m_recv]
        if out_rows.data_ptr() != buf.data_ptr():
            buf.copy_(out_rows)
        xc.barrier()  # every rank's "y" rows are written
        y = torch.empty(T, out_rows.size(1), dtype=out_rows.dtype, device=out_rows.device)
        expanded = torch.empty(T * k, out_rows.size(1), dtype=out_rows.dtype, device=out_rows.device)
        gates = gates.contiguous()
        _pull(xc, "y", gates, y, expanded, plan)
        ctx.save_for_backward(expanded, gates)
        ctx.xc, ctx.plan = xc, plan
        return y

    @staticmethod
    def backward(ctx, grad_y):
        expanded, gates = ctx.saved_tensors
        xc, plan = ctx.xc, ctx.plan
        T, k = gates.shape
        grad_y = grad_y.contiguous()
        d_gates = _gate_grad(expanded, grad_y, k)
        _push(xc, "dy", grad_y, plan.ss, k, gates.reshape(-1), plan)
        xc.barrier()  # all gradient rows have landed
        return xc.bufs["dy"][: plan.m_recv], d_gates, None, None


def ep_experts_p2p(x, router_weights, selected_experts, num_experts: int, local_experts_fn: Callable, xc: PeerExchange, ops=CudaRowOps):
    """Routed experts over an expert-parallel group with the row exchange done by this package's kernels on peer
    memory (see PeerExchange).  Same contract as `ep_experts`."""
    world, rank = xc.world, dist.get_rank(xc.group)
    with torch.no_grad():
        plan = _make_plan(selected_experts, num_experts, world, rank, xc.group, ops, xc.host_rows)
    recv = _PeerDispatch.apply(x, xc, plan)
    out_rows = local_experts_fn(recv, plan.local_ids)
    return _PeerCombine.apply(out_rows, router_weights.to(x.dtype), xc, plan)


class MoE_B200_EP(nn.Module):
    """Expert-parallel MoE layer.  The gate is replicated; rank r holds experts [r*E/R, (r+1)*E/R).

    Weights are drawn expert by expert from a seed shared by all ranks, so the union of the shards equals
    the single-GPU layer built from the same seed with `full_state_dict`-style gathering.
    """

    def __init__(self, num_experts, num_experts_per_tok, hidden_size, intermediate_size, activation_function, is_glu, add_bias, std,
                 group=None, device=None, dtype=torch.float32, seed: int = 0, ops=CudaRowOps, local_experts_fn=None,
                 num_shared_experts: int = 0, shared_intermediate_size: int | None = None, router_scoring: str = "softmax",
                 exchange: str = "nccl", exchange_rows: int | None = None):
        super().__init__()
        assert is_glu, "the expert-parallel layer implements GLU experts"
        assert router_scoring in ("softmax", "sigmoid")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        assert num_experts % self.world == 0, "experts must divide evenly over the ranks"
        self.num_experts, self.top_k = num_experts, num_experts_per_tok
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.e_local = num_experts // self.world
        self.ops = ops
        self._local_experts_fn = local_experts_fn
        self.act = activation_function
        self.router_scoring = router_scoring
        self.num_shared_experts = num_shared_experts
        assert exchange in ("nccl", "p2p")
        # "p2p": rows move by this package's kernels over peer memory; exchange_rows = capacity of each buffer in rows
        self.exchange = PeerExchange(self.group, exchange_rows, hidden_size, dtype, torch.device(device)) if exchange == "p2p" else None
        # every rank draws with the same per-expert seeds on the same kind of device, so shards agree across ranks
        gen_dev = torch.device(device) if device is not None and torch.device(device).type == "cuda" else torch.device("cpu")

        def draw(shape, seed_, scale):
            g = torch.Generator(device=gen_dev).manual_seed(seed_)
            return (torch.randn(*shape, generator=g, device=gen_dev) * scale).to(dtype)

        self.gate = nn.Linear(hidden_size, num_experts, bias=False, device=device, dtype=dtype)
        with torch.no_grad():
            self.gate.weight.copy_(draw((num_experts, hidden_size), seed * 100003 + 1, hidden_size**-0.5))
        lo = self.rank * self.e_local
        fc = [draw((2 * intermediate_size, hidden_size), seed * 100003 + 17 + 2 * e, std) for e in range(lo, lo + self.e_local)]
        proj = [draw((hidden_size, intermediate_size), seed * 100003 + 18 + 2 * e, std) for e in range(lo, lo + self.e_local)]
        self.c_fc_weight = nn.Parameter(torch.stack(fc).to(device))
        self.c_proj_weight = nn.Parameter(torch.stack(proj).to(device))
        del fc, proj
        if num_shared_experts > 0:  # replicated; they see this rank's tokens only
            i_s = shared_intermediate_size or intermediate_size
            self.shared_c_fc_weight = nn.Parameter(torch.stack([draw((2 * i_s, hidden_size), seed * 100003 + 7 + 2 * s_, std) for s_ in range(num_shared_experts)]).to(device))
            self.shared_c_proj_weight = nn.Parameter(torch.stack([draw((hidden_size, i_s), seed * 100003 + 8 + 2 * s_, std) for s_ in range(num_shared_experts)]).to(device))

    def local_experts(self, rows: torch.Tensor, local_ids: torch.Tensor) -> torch.Tensor:
        if self._local_experts_fn is not None:
            return self._local_experts_fn(rows, local_ids, self.c_fc_weight, self.c_proj_weight)
        from .scattermoe import fused_swiglu_experts

        ones = torch.ones(rows.size(0), 1, dtype=rows.dtype, device=rows.device)
        y_out = dx_out = None
        if self.exchange is not None:  # the kernels write straight into the buffers the other ranks read
            y_out, dx_out = self.exchange.bufs["y"], self.exchange.bufs["dx"]
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
        if self.exchange is not None:
            return ep_experts_p2p(hidden_states, router_weights, selected_experts, self.num_experts, self.local_experts, self.exchange, self.ops)
        return ep_experts(hidden_states, router_weights, selected_experts, self.num_experts, self.local_experts, self.group, self.ops)

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
        return {"gate.weight": self.gate.weight.detach().clone(), "c_fc.weight": torch.cat(fc), "c_proj.weight": torch.cat(proj)}

    def load_full_state_dict(self, sd: dict) -> None:
        lo, hi = self.rank * self.e_local, (self.rank + 1) * self.e_local
        with torch.no_grad():
            self.gate.weight.copy_(sd["gate.weight"])
            self.c_fc_weight.copy_(sd["c_fc.weight"][lo:hi])
            self.c_proj_weight.copy_(sd["c_proj.weight"][lo:hi])
