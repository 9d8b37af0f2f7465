"""MoE layer modules and the autograd functions behind them.

Public names follow the reference so that a user can switch packages without touching call sites:
`MoE_Torch` (eager torch module, the on-device reference), `MoE_Triton` / `MoE_B200` (this package's
kernels; the former name is kept as an alias), `Experts_Torch`, `Experts_Triton` / `Experts_B200`,
`scattered_experts` (cute_kernels/kernels/scattermoe/torch_implementation.py:10-199,
cute_kernels/kernels/scattermoe/triton_implementation/__init__.py:11-101, ops.py:133-301).

Two execution paths exist in `MoE_B200._compute_experts`:
  * fused: taken when the layer is a GLU layer whose activation is SwiGLU on the fused tensor or `nn.GLU()`, or a plain
    layer whose activation is `nn.GELU(approximate="tanh")` (the two activations of the reference's layer test).  One
    routing call, then up-projection + SwiGLU, down-projection + gate scaling, slot sum; the backward
    runs five kernels.  Intermediates live in the padded grouped order.
  * generic: any other activation callable.  The same sequence of operators as the reference
    (`scattered_experts` twice around `self.act`), each operator running on this package's kernels.
"""

from __future__ import annotations

import os
from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from ._lib import check, dtype_code, lib, ptr, status_word, stream_ptr
from .custom_op import b200_op
from .router import fused_router, fused_router_supported
from .ops import _workspace, combine, contiguous_count_cute, gate_grad, group, group_bwd_W, scatter2scatter, swiglu_unchunked_cute, swiglu_unchunked_torch

# --------------------------------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------------------------------


def padded_rows_cap(M: int, E: int) -> int:
    return (M // 128 + E) * 128


def _route_fake(expert_ids: torch.Tensor, num_experts: int, k: int, want_sorted: bool, want_row_maps: bool):
    M, dev = expert_ids.numel(), expert_ids.device
    cap = padded_rows_cap(M, num_experts) if want_row_maps else 0
    return (
        torch.empty(M if want_sorted else 0, dtype=torch.int64, device=dev),
        torch.empty(M if want_sorted else 0, dtype=torch.int64, device=dev),
        torch.empty(num_experts, dtype=torch.int64, device=dev),
        torch.empty(num_experts, dtype=torch.int32, device=dev),
        torch.empty(cap, dtype=torch.int32, device=dev),
        torch.empty(cap, dtype=torch.int32, device=dev),
    )


@b200_op("route", mutates_args=(), fake_func=_route_fake)
def route(expert_ids: torch.Tensor, num_experts: int, k: int, want_sorted: bool, want_row_maps: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Stable sort of flat expert ids by expert with histogram and inclusive offsets.

    Returns (sorted_expert_idxs int64 (M), sorted_scattered_idxs int64 (M), expert_offsets int64 (E),
    counts int32 (E), row_token int32 (cap), row_slot int32 (cap)); the first two are empty unless
    `want_sorted`, the last two unless `want_row_maps`.  Equals `ids.sort(stable=True)`,
    `bincount(minlength=E)` and its `cumsum` bit for bit.
    """
    assert expert_ids.dim() == 1 and expert_ids.dtype == torch.int64 and expert_ids.is_cuda
    expert_ids = expert_ids.contiguous()
    M, dev = expert_ids.numel(), expert_ids.device
    outs = _route_fake(expert_ids, num_experts, k, want_sorted, want_row_maps)
    se, ss, offsets, counts, row_token, row_slot = outs
    if want_sorted:
        # an id outside [0, E) is skipped by the sort (status 101): the tail of the two lists then stays unwritten
        se.zero_()
        ss.zero_()
    nbytes = lib().b200moe_route_workspace_bytes(M, num_experts)
    ws = _workspace(dev, nbytes)
    check(
        lib().b200moe_route(
            ptr(expert_ids), M, num_experts, k,
            ptr(se) if want_sorted else None, ptr(ss) if want_sorted else None, ptr(offsets), ptr(counts),
            ptr(row_token) if want_row_maps else None, ptr(row_slot) if want_row_maps else None, row_token.numel(),
            ptr(ws), ws.numel(), ptr(status_word(dev)), stream_ptr(dev),
        ),
        "route",
    )
    return outs


# --------------------------------------------------------------------------------------------------
# generic path: the reference's autograd function on this package's operators
# --------------------------------------------------------------------------------------------------


class _ScatteredExperts(torch.autograd.Function):
    """One expert projection with fused gather / scatter; same contract as the reference's function of
    the same name (cute_kernels/kernels/scattermoe/triton_implementation/ops.py:133-277)."""

    @staticmethod
    def forward(ctx, x, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates=None, grouped_in=False, grouped_out=False):
        M = sorted_expert_idxs.size(0)
        expanded = torch.empty(M, expert_weights.size(-1), device=x.device, dtype=x.dtype)
        scatter2scatter(X=x, W=expert_weights, sorted_expert_idxs=sorted_expert_idxs, sorted_scattered_idxs=sorted_scattered_idxs, out=expanded, FAN_OUT=k, x_grouped=grouped_in, y_grouped=grouped_out)
        if gates is None:
            output, kept = expanded, None
        else:
            output = torch.empty(gates.size(0), expanded.size(1), device=x.device, dtype=x.dtype)
            combine(expanded, gates, output, gates.size(1))
            kept = expanded
        ctx.save_for_backward(x, expert_weights, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates, kept)
        ctx.flags = (k, grouped_in, grouped_out)
        return output

    @staticmethod
    def backward(ctx, grad_out):
        x, expert_weights, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates, expanded = ctx.saved_tensors
        k, grouped_in, grouped_out = ctx.flags
        M, E = sorted_expert_idxs.size(0), expert_weights.size(0)
        grad_out = grad_out.contiguous()

        d_gates = None
        if gates is not None:
            # d_gates[t, j] = <expanded[t, j, :], grad_out[t, :]>
            d_gates = gate_grad(expanded, grad_out, gates.size(1))

        if grouped_out:
            grouped_grad_out = grad_out
        else:
            # the expanded buffer is dead after d_gates: reuse it for the grouped upstream gradient
            grouped_grad_out = expanded if expanded is not None else torch.empty(M, grad_out.size(1), device=x.device, dtype=x.dtype)
            group(A=grad_out, sorted_expert_idxs=sorted_scattered_idxs, out=grouped_grad_out, coeff=None if gates is None else gates.flatten(), fan_out=1 if gates is None else gates.size(1))

        if grouped_in:
            grouped_x = x
            d_expanded_input = torch.empty(M, expert_weights.size(1), device=x.device, dtype=x.dtype)
        else:
            grouped_x = torch.empty(M, x.size(1), dtype=x.dtype, device=x.device)
            group(A=x, sorted_expert_idxs=sorted_scattered_idxs, out=grouped_x, fan_out=k)
            d_expanded_input = grouped_x  # overwritten only after the weight gradient has consumed it

        # same strides as the (possibly permuted) weight view; every element is written by the kernel
        d_weights = torch.empty_like(expert_weights)
        group_bwd_W(DY=grouped_grad_out, X=grouped_x, expert_offsets=expert_offsets, DW=d_weights, E=E)

        scatter2scatter(X=grouped_grad_out, W=expert_weights.permute(0, 2, 1), sorted_expert_idxs=sorted_expert_idxs, sorted_scattered_idxs=sorted_scattered_idxs, out=d_expanded_input, FAN_OUT=1, x_grouped=True, y_grouped=grouped_in)

        if k == 1:
            d_input = d_expanded_input
        else:
            d_input = torch.empty(x.size(0), d_expanded_input.size(1), device=x.device, dtype=x.dtype)
            combine(d_expanded_input, None, d_input, k)
        return d_input, d_weights, None, None, None, None, d_gates, None, None


def scattered_experts(inputs, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates=None, grouped_in=False, grouped_out=False):
    return _ScatteredExperts.apply(inputs, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates, grouped_in, grouped_out)


# --------------------------------------------------------------------------------------------------
# fused path
# --------------------------------------------------------------------------------------------------

# Device-side failures (a bounded wait that expired, an expert id outside [0, E), an exchange buffer overrun) are
# written to a per-device status word that the host reads with `_lib.check_status(device)`.  Reading it synchronises the
# stream, so the layers do not do it on their own; with this switch on (or B200MOE_CHECK_STATUS=1 in the environment)
# the fused path checks at the end of every forward and backward pass and raises on a recorded failure.
CHECK_STATUS = os.environ.get("B200MOE_CHECK_STATUS", "0") == "1"


def _maybe_check_status(device: torch.device) -> None:
    if CHECK_STATUS and not torch.compiler.is_compiling():
        _lib.check_status(device)


# When a list is installed here, every grouped-GEMM launch of the fused path is bracketed by two CUDA
# events on the current stream and (name, start, end) is appended; the benchmark reads kernel durations
# from it without synchronising inside the step.
_timing_sink: list | None = None

# The backward pass needs the token rows in the padded grouped order again (weight gradient of the up projection).
# True: the forward's gathered copy (k rows per token) is kept for it; False: only the tokens are kept and the rows
# are gathered a second time, which trades one HBM pass for k-1 token copies of memory.
KEEP_GATHERED_INPUT = True


def set_timing_sink(sink: list | None) -> None:
    global _timing_sink
    _timing_sink = sink


class phase:
    """Context manager: with a timing sink installed, brackets the kernels queued inside it with two CUDA events on the
    current stream and records them under `name` (no synchronisation); otherwise does nothing."""

    def __init__(self, name: str):
        self.name, self.start = name, None

    def __enter__(self):
        if _timing_sink is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        sink = _timing_sink
        if self.start is not None and sink is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            sink.append((self.name, self.start, end))
        return False


def _launch(name: str, fn, *args) -> None:
    sink = _timing_sink
    if sink is None:
        fn(*args)
        return
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn(*args)
    end.record()
    sink.append((name, start, end))



@b200_op("gather_rows", mutates_args={"out"})
def _gather_rows(src: torch.Tensor, row_map: torch.Tensor, out: torch.Tensor) -> None:
    """out[p, :] = src[row_map[p], :], zeros where row_map[p] < 0 (rows of the padded grouped order)."""
    check(
        lib().b200moe_gather_rows(ptr(src), src.stride(0), ptr(row_map), ptr(out), out.stride(0), out.size(0), src.size(1), dtype_code(src), stream_ptr(src.device)),
        "gather_rows",
    )


@b200_op("up_forward", mutates_args={"h", "a"})
def _up_forward(x: torch.Tensor, w_fc: torch.Tensor, expert_offsets: torch.Tensor, row_token: torch.Tensor | None, h: torch.Tensor, a: torch.Tensor, activation: int = 0) -> None:
    E, F_, H = w_fc.shape
    I = F_ if activation == ACTIVATIONS["gelu_tanh"] else F_ // 2
    check(
        lib().b200moe_up_forward(ptr(x), x.stride(0), ptr(w_fc), ptr(expert_offsets), ptr(row_token), ptr(h), ptr(a), x.size(0), H, I, E, h.size(0), activation, dtype_code(x), ptr(status_word(x.device)), stream_ptr(x.device)),
        "up_forward",
    )


@b200_op("down_forward", mutates_args={"y_expanded"})
def _down_forward(a: torch.Tensor, w_proj: torch.Tensor, expert_offsets: torch.Tensor, row_slot: torch.Tensor | None, gates: torch.Tensor | None, y_expanded: torch.Tensor) -> None:
    E, H, I = w_proj.shape
    check(
        lib().b200moe_down_forward(ptr(a), ptr(w_proj), ptr(expert_offsets), ptr(row_slot), ptr(gates), ptr(y_expanded), y_expanded.stride(0), y_expanded.size(0), H, I, E, a.size(0), dtype_code(a), ptr(status_word(a.device)), stream_ptr(a.device)),
        "down_forward",
    )


@b200_op("gather_grad_rows", mutates_args={"out", "d_gates"})
def _gather_grad_rows(grad: torch.Tensor, row_token: torch.Tensor, row_slot: torch.Tensor, gates: torch.Tensor | None, y_expanded: torch.Tensor | None, out: torch.Tensor, d_gates: torch.Tensor | None, y_grouped: bool = False) -> None:
    """out[p, :] = gates[row_slot[p]] * grad[row_token[p], :] (zeros on filler rows) and, when the unweighted expert
    outputs are given, d_gates[s] = <y_expanded[s, :], grad[t, :]> in the same pass (`y_grouped`: the outputs are in
    the padded grouped order, row p instead of row s)."""
    check(
        lib().b200moe_gather_grad_rows(ptr(grad), grad.stride(0), ptr(row_token), ptr(row_slot), ptr(gates), ptr(y_expanded), y_expanded.stride(0) if y_expanded is not None else 0,
                                       int(y_grouped), ptr(out), out.stride(0), ptr(d_gates), out.size(0), grad.size(1), dtype_code(grad), stream_ptr(grad.device)),
        "gather_grad_rows",
    )


@b200_op("combine_rows", mutates_args={"out"})
def _combine_rows(rows: torch.Tensor, pos: torch.Tensor, gates: torch.Tensor | None, out: torch.Tensor, k: int) -> None:
    """out[t, :] = sum_j gates[t, j] * rows[pos[t*k + j], :] (gates None: plain sum)."""
    check(
        lib().b200moe_combine_rows(ptr(rows), rows.stride(0), ptr(pos), ptr(gates), ptr(out), out.stride(0), out.size(0), k, out.size(1), dtype_code(rows), stream_ptr(rows.device)),
        "combine_rows",
    )


@b200_op("invert_row_map", mutates_args={"slot_row"})
def _invert_row_map(row_slot: torch.Tensor, slot_row: torch.Tensor) -> None:
    """slot_row[row_slot[p]] = p for the real rows of the padded grouped order."""
    check(lib().b200moe_invert_row_map(ptr(row_slot), row_slot.numel(), ptr(slot_row), slot_row.numel(), stream_ptr(row_slot.device)), "invert_row_map")


@b200_op("down_dgrad", mutates_args={"dh"})
def _down_dgrad(grad_rows: torch.Tensor, w_proj: torch.Tensor, expert_offsets: torch.Tensor, row_token: torch.Tensor | None, h: torch.Tensor, dh: torch.Tensor, activation: int = 0) -> None:
    E, H, I = w_proj.shape
    check(
        lib().b200moe_down_dgrad(ptr(grad_rows), grad_rows.stride(0), ptr(w_proj), ptr(expert_offsets), ptr(row_token), ptr(h), ptr(dh),
                                 grad_rows.size(0), H, I, E, h.size(0), activation, dtype_code(h), ptr(status_word(h.device)), stream_ptr(h.device)),
        "down_dgrad",
    )


@b200_op("wgrad", mutates_args={"DW"})
def _wgrad(P: torch.Tensor, p_map: torch.Tensor | None, Q: torch.Tensor, q_map: torch.Tensor | None, expert_offsets: torch.Tensor, DW: torch.Tensor, m_cap: int) -> None:
    E, n_out, n_in = DW.shape
    check(
        lib().b200moe_wgrad(ptr(P), P.stride(0), ptr(p_map), ptr(Q), Q.stride(0), ptr(q_map), ptr(expert_offsets), ptr(DW), n_out, n_in, E, m_cap, dtype_code(P), ptr(status_word(P.device)), stream_ptr(P.device)),
        "wgrad",
    )


@b200_op("up_dgrad", mutates_args={"dx_expanded"})
def _up_dgrad(dh: torch.Tensor, w_fc: torch.Tensor, expert_offsets: torch.Tensor, row_slot: torch.Tensor | None, dx_expanded: torch.Tensor) -> None:
    E, I2, H = w_fc.shape
    check(
        lib().b200moe_up_dgrad(ptr(dh), ptr(w_fc), ptr(expert_offsets), ptr(row_slot), ptr(dx_expanded), dx_expanded.stride(0), dx_expanded.size(0), H, I2 // 2, E, dh.size(0), dtype_code(dh), ptr(status_word(dh.device)), stream_ptr(dh.device)),
        "up_dgrad",
    )


class _FusedSwiGLUExperts(torch.autograd.Function):
    """Routed SwiGLU experts with externally supplied routing, forward and backward, on the fused kernels.

    Same mathematical contract as `MoE_Triton._compute_experts` with the SwiGLU activation
    (cute_kernels/kernels/scattermoe/triton_implementation/__init__.py:76-101): gradients flow to the
    input, both weight tensors (in their stored (E, out, in) layout) and the router weights.
    """

    @staticmethod
    def forward(ctx, x, w_fc, w_proj, router_weights, selected_experts, out_bufs=None, activation=0):
        # out_bufs = (y_out, dx_out), k == 1 only: caller-owned (rows >= T, H) buffers that receive the output / the
        # input gradient directly, e.g. exchange buffers other ranks read from.  Passed as a tuple so that autograd
        # does not see them as inputs.
        y_out, dx_out = out_bufs if out_bufs is not None else (None, None)
        T, H = x.shape
        E, I2, _ = w_fc.shape  # I2: output features of the up projection (2I for a gated layer, I otherwise)
        I = I2 if activation == ACTIVATIONS["gelu_tanh"] else I2 // 2
        k = selected_experts.size(1)
        M = T * k
        assert w_fc.is_contiguous() and w_proj.is_contiguous(), "expert weights must be stored contiguously as (E, out, in)"
        assert w_proj.shape == (E, H, I) and router_weights.shape == (T, k)
        if x.stride(1) != 1:
            x = x.contiguous()
        gates = router_weights.to(x.dtype).contiguous()
        with torch.no_grad(), phase("route"):
            _, _, offsets, _, row_token, row_slot = route(selected_experts.reshape(-1), E, k, False, True)
        cap = row_token.numel()
        h = torch.empty(cap, I2, device=x.device, dtype=x.dtype)
        a = torch.empty(cap, I, device=x.device, dtype=x.dtype)
        # rows of x in the padded grouped order: one HBM pass, after which every operand is a plain TMA tile
        x_rows = torch.empty(cap, H, device=x.device, dtype=x.dtype)
        _launch("gather_x", _gather_rows, x, row_token, x_rows)
        _launch("up_forward", _up_forward, x_rows, w_fc, offsets, None, h, a, activation)
        if not KEEP_GATHERED_INPUT:
            x_rows = None
        need_gate_grad = ctx.needs_input_grad[3]
        if k == 1 and y_out is not None and not need_gate_grad:
            # the rows must land in a caller's buffer in their original order (expert-parallel exchange): the epilogue
            # scatters them there and applies the gate
            y = y_out[:M]
            _launch("down_forward", _down_forward, a, w_proj, offsets, row_slot, gates, y)
            slot_row = y_rows = None
        else:
            # The rows leave the down projection unweighted and in the padded grouped order (whole tiles stored by TMA);
            # the combine pass un-sorts them while it forms the gate-weighted sum over the slots, which is the
            # reference's bmm over its `output_expanded`.  The backward forms the gate gradient from the kept rows.
            y_rows = torch.empty(cap, H, device=x.device, dtype=x.dtype)
            _launch("down_forward", _down_forward, a, w_proj, offsets, None, None, y_rows)
            slot_row = torch.full((M,), -1, device=x.device, dtype=torch.int32)  # -1: a slot without an expert contributes nothing
            _invert_row_map(row_slot, slot_row)
            y = y_out[:T] if (k == 1 and y_out is not None) else torch.empty(T, H, device=x.device, dtype=x.dtype)
            _launch("combine_y", _combine_rows, y_rows, slot_row, gates, y, k)
            if not need_gate_grad:
                y_rows = None
        ctx.save_for_backward(x, w_fc, w_proj, gates, offsets, row_token, row_slot, h, a, x_rows, y_rows, slot_row)
        ctx.k = k
        ctx.activation = activation
        ctx.rw_dtype = router_weights.dtype
        ctx.dx_out = dx_out if k == 1 else None
        _maybe_check_status(x.device)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, w_fc, w_proj, gates, offsets, row_token, row_slot, h, a, x_rows, y_rows, slot_row = ctx.saved_tensors
        k = ctx.k
        T, H = x.shape
        E, I2, _ = w_fc.shape
        M, cap = T * k, h.size(0)
        grad_y = grad_y.contiguous()
        need_x, need_w1, need_w2, need_g = ctx.needs_input_grad[:4]

        # upstream gradient rows in the padded grouped order, scaled by their gates (the reference's
        # `group(grad_out, coeff=gates)`), and the gate gradient <unweighted expert output, upstream gradient>
        g_rows = torch.empty(cap, H, device=x.device, dtype=x.dtype)
        d_gates = torch.zeros(M, device=x.device, dtype=torch.float32) if (need_g and y_rows is not None) else None  # slots without an expert keep 0
        _launch("gather_grad", _gather_grad_rows, grad_y, row_token, row_slot, gates, y_rows if d_gates is not None else None, g_rows, d_gates, True)
        del y_rows

        d_w_proj = d_w_fc = d_x = d_rw = None
        dh = None
        if need_w1 or need_x:
            dh = torch.empty(cap, I2, device=x.device, dtype=x.dtype)
            _launch("down_dgrad", _down_dgrad, g_rows, w_proj, offsets, None, h, dh, ctx.activation)
        if need_w2:
            d_w_proj = torch.empty_like(w_proj)
            _launch("down_wgrad", _wgrad, g_rows, None, a, None, offsets, d_w_proj, cap)
        del a
        if need_w1:
            d_w_fc = torch.empty_like(w_fc)
            if x_rows is None:
                x_rows = g_rows  # the gathered gradient rows are dead now: reuse the buffer
                _gather_rows(x, row_token, x_rows)
            _launch("up_wgrad", _wgrad, dh, None, x_rows, None, offsets, d_w_fc, cap)
        del g_rows
        if need_x:
            if ctx.dx_out is not None:  # k == 1: the rows go straight into the caller's buffer, in their original order
                d_x = ctx.dx_out[:M]
                _launch("up_dgrad", _up_dgrad, dh, w_fc, offsets, row_slot, d_x)
            else:
                dx_rows = torch.empty(cap, H, device=x.device, dtype=x.dtype)
                _launch("up_dgrad", _up_dgrad, dh, w_fc, offsets, None, dx_rows)
                if slot_row is None:
                    slot_row = torch.full((M,), -1, device=x.device, dtype=torch.int32)
                    _invert_row_map(row_slot, slot_row)
                d_x = torch.empty(T, H, device=x.device, dtype=x.dtype)
                _launch("combine_dx", _combine_rows, dx_rows, slot_row, None, d_x, k)
        if d_gates is not None:
            d_rw = d_gates.view(T, k).to(ctx.rw_dtype)
        _maybe_check_status(x.device)
        return d_x, d_w_fc, d_w_proj, d_rw, None, None, None


class _GroupedExperts(torch.autograd.Function):
    """Experts on rows that already sit in the padded grouped order (every expert's segment starts at a multiple of 128
    rows, filler rows are zero): no sort, no gather, no un-sort.  `x_rows (cap, H)` and `expert_offsets` (inclusive row
    counts) describe the input; the output rows `y_rows (cap, H)` have the same order.  `bufs = (y_buf, dx_buf)` may name
    caller-owned buffers that receive the output and the input gradient (exchange buffers other ranks read from).  This is
    the local layer of the expert-parallel pass whose dispatch kernel places rows directly in this order."""

    @staticmethod
    def forward(ctx, x_rows, w_fc, w_proj, expert_offsets, bufs=None, activation=0):
        y_buf, dx_buf = bufs if bufs is not None else (None, None)
        cap, H = x_rows.shape
        E, I2, _ = w_fc.shape
        I = I2 if activation == ACTIVATIONS["gelu_tanh"] else I2 // 2
        assert cap % 128 == 0 and w_fc.is_contiguous() and w_proj.is_contiguous() and w_proj.shape == (E, H, I)
        h = torch.empty(cap, I2, device=x_rows.device, dtype=x_rows.dtype)
        a = torch.empty(cap, I, device=x_rows.device, dtype=x_rows.dtype)
        _launch("up_forward", _up_forward, x_rows, w_fc, expert_offsets, None, h, a, activation)
        y_rows = y_buf if y_buf is not None else torch.empty(cap, H, device=x_rows.device, dtype=x_rows.dtype)
        _launch("down_forward", _down_forward, a, w_proj, expert_offsets, None, None, y_rows)
        ctx.save_for_backward(x_rows, w_fc, w_proj, expert_offsets, h, a)
        ctx.activation, ctx.dx_buf = activation, dx_buf
        _maybe_check_status(x_rows.device)
        return y_rows

    @staticmethod
    def backward(ctx, g_rows):
        x_rows, w_fc, w_proj, offsets, h, a = ctx.saved_tensors
        cap, H = x_rows.shape
        need_x, need_w1, need_w2 = ctx.needs_input_grad[:3]
        if g_rows.stride(1) != 1 or g_rows.stride(0) != H:
            g_rows = g_rows.contiguous()
        d_w_proj = d_w_fc = d_x = dh = None
        if need_w1 or need_x:
            dh = torch.empty_like(h)
            _launch("down_dgrad", _down_dgrad, g_rows, w_proj, offsets, None, h, dh, ctx.activation)
        if need_w2:
            d_w_proj = torch.empty_like(w_proj)
            _launch("down_wgrad", _wgrad, g_rows, None, a, None, offsets, d_w_proj, cap)
        if need_w1:
            d_w_fc = torch.empty_like(w_fc)
            _launch("up_wgrad", _wgrad, dh, None, x_rows, None, offsets, d_w_fc, cap)
        if need_x:
            d_x = ctx.dx_buf if ctx.dx_buf is not None else torch.empty(cap, H, device=x_rows.device, dtype=x_rows.dtype)
            _launch("up_dgrad", _up_dgrad, dh, w_fc, offsets, None, d_x)
        _maybe_check_status(x_rows.device)
        return d_x, d_w_fc, d_w_proj, None, None, None


def grouped_experts(x_rows, w_fc, w_proj, expert_offsets, y_buf=None, dx_buf=None, activation: str = "swiglu"):
    """Experts on rows already in the padded grouped order; see `_GroupedExperts`."""
    bufs = (y_buf, dx_buf) if (y_buf is not None or dx_buf is not None) else None
    return _GroupedExperts.apply(x_rows, w_fc, w_proj, expert_offsets, bufs, ACTIVATIONS[activation])


# a = h[:, :I] * silu(h[:, I:]) / h[:, :I] * sigmoid(h[:, I:]) for gated layers (w_fc (E, 2I, H)); a = gelu_tanh(h) for a plain
# layer (w_fc (E, I, H))
ACTIVATIONS = {"swiglu": 0, "glu": 1, "gelu_tanh": 2}


def fused_swiglu_experts(x, w_fc, w_proj, router_weights, selected_experts, y_out=None, dx_out=None, activation: str = "swiglu"):
    """Routed experts on the fused kernels; `activation` (`ACTIVATIONS`) selects the gate function of a GLU layer or the
    un-gated tanh-GELU of a plain one.  A negative entry of `selected_experts` is a slot without an expert (padding, a
    dropped token): it contributes nothing to the output and receives a zero router-weight gradient."""
    if x.size(0) == 0:
        # no tokens: nothing to launch; the zero-weighted sums keep every input in the graph with a zero gradient
        return x.new_zeros(0, x.size(1)) + 0 * (x.sum() + w_fc.sum() + w_proj.sum() + router_weights.sum())
    out_bufs = (y_out, dx_out) if (y_out is not None or dx_out is not None) else None
    return _FusedSwiGLUExperts.apply(x, w_fc, w_proj, router_weights, selected_experts, out_bufs, ACTIVATIONS[activation])


# --------------------------------------------------------------------------------------------------
# modules
# --------------------------------------------------------------------------------------------------


class Experts_Torch(nn.Module):
    """Per-expert linear layers held as one (E, out, in) parameter; eager evaluation expert by expert."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool = True, std: float | None = None) -> None:
        super().__init__()
        self.num_experts, self.in_features, self.out_features, self.std = num_experts, in_features, out_features, std
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(num_experts, out_features)) if add_bias else None
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if self.bias is not None:
            self.bias.zero_()

    def forward(self, input, expert_frequency: torch.Tensor, return_list: bool):
        chunks = input.split(expert_frequency.tolist(), dim=0) if isinstance(input, torch.Tensor) else input
        outs = [F.linear(chunks[e], self.weight[e], None if self.bias is None else self.bias[e]) for e in range(self.num_experts)]
        return outs if return_list else torch.cat(outs)

    def extra_repr(self) -> str:
        return f"num_experts={self.num_experts}, in_features={self.in_features}, out_features={self.out_features}"


class MoE_Torch(nn.Module):
    """Eager torch MoE layer: linear router, top-k with softmax over the selected logits, per-expert MLPs,
    gate-weighted sum.  Used as the on-device reference of the kernels.

    The first eight arguments are the reference's.  Two optional extensions follow (the reference has neither):
    `num_shared_experts` always-on SwiGLU experts whose output is added for every token (parameters
    `shared_c_fc.weight (S, 2*I_s, H)`, `shared_c_proj.weight (S, H, I_s)`, created only when S > 0), and
    `router_scoring="sigmoid"`: sigmoid of the top-k logits, normalised to sum one, instead of their softmax.
    """

    experts_cls = Experts_Torch

    def __init__(self, num_experts: int, num_experts_per_tok: int, hidden_size: int, intermediate_size: int, activation_function: Callable, is_glu: bool, add_bias: bool, std: float,
                 num_shared_experts: int = 0, shared_intermediate_size: int | None = None, router_scoring: str = "softmax") -> None:
        super().__init__()
        assert router_scoring in ("softmax", "sigmoid")
        self.num_experts, self.top_k = num_experts, num_experts_per_tok
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.is_glu = is_glu
        self.router_scoring = router_scoring
        self.num_shared_experts = num_shared_experts
        self.gate = nn.Linear(in_features=hidden_size, out_features=num_experts, bias=False)
        self.c_fc = self.experts_cls(num_experts, hidden_size, 2 * intermediate_size if is_glu else intermediate_size, add_bias=add_bias, std=std)
        self.act = activation_function
        self.c_proj = self.experts_cls(num_experts, intermediate_size, hidden_size, add_bias=add_bias, std=std)
        if num_shared_experts > 0:
            i_s = shared_intermediate_size or intermediate_size
            self.shared_c_fc = Experts_Torch(num_shared_experts, hidden_size, 2 * i_s, add_bias=False, std=std)
            self.shared_c_proj = Experts_Torch(num_shared_experts, i_s, hidden_size, add_bias=False, std=std)

    def forward(self, hidden_states: torch.Tensor):
        shape = hidden_states.shape
        flat = hidden_states.view(-1, self.hidden_size)
        router_logits, router_weights, selected_experts = self._compute_routing_weights(flat)
        out = self._compute_experts(flat, router_weights, selected_experts)
        if self.num_shared_experts > 0:
            out = out + self._compute_shared_experts(flat)
        return out.view(shape), router_logits

    def _get_topk(self, x: torch.Tensor):
        return x.max(dim=-1, keepdim=True) if self.top_k == 1 else x.topk(self.top_k, dim=-1)

    def _compute_routing_weights(self, hidden_states: torch.Tensor):
        router_logits = self.gate(hidden_states)
        top_vals, selected_experts = self._get_topk(router_logits)
        if self.router_scoring == "sigmoid":
            scores = torch.sigmoid(top_vals.float())
            router_weights = (scores / scores.sum(-1, keepdim=True)).type_as(hidden_states)
        else:
            router_weights = F.softmax(top_vals.float(), dim=-1).type_as(hidden_states)
        return router_logits, router_weights, selected_experts

    def _compute_experts(self, hidden_states: torch.Tensor, router_weights: torch.Tensor, selected_experts: torch.Tensor) -> torch.Tensor:
        T = hidden_states.shape[0]
        flat_experts = selected_experts.flatten()
        frequency = flat_experts.bincount(minlength=self.num_experts)
        order = flat_experts.argsort(stable=True)
        token_of_row = order // self.top_k
        rows = self.c_fc(hidden_states[token_of_row], frequency, return_list=True)
        rows = [self.act(r) for r in rows]
        rows = self.c_proj(rows, frequency, return_list=False)
        rows = rows * router_weights.flatten()[order].unsqueeze(-1)
        return torch.zeros(T, self.hidden_size, dtype=rows.dtype, device=rows.device).index_add(0, token_of_row, rows)

    def _compute_shared_experts(self, hidden_states: torch.Tensor) -> torch.Tensor:
        out = torch.zeros_like(hidden_states)
        for s_ in range(self.num_shared_experts):
            out = out + F.linear(swiglu_unchunked_torch(F.linear(hidden_states, self.shared_c_fc.weight[s_])), self.shared_c_proj.weight[s_])
        return out


class Experts_B200(Experts_Torch):
    """Expert projection evaluated by the grouped-GEMM operator; the bias, if any, is not applied (the
    reference's scatter module ignores it as well)."""

    def forward(self, inputs, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates=None, grouped_in=False, grouped_out=False):
        return scattered_experts(inputs, self.weight.permute(0, 2, 1), k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, gates, grouped_in, grouped_out)


_SWIGLU_CALLABLES = (swiglu_unchunked_torch, swiglu_unchunked_cute)


def is_swiglu_callable(fn) -> bool:
    if fn in _SWIGLU_CALLABLES:
        return True
    return getattr(fn, "__name__", "") in ("swiglu_unchunked_torch", "swiglu_unchunked_cute")


def fused_activation(fn, is_glu: bool = True) -> str | None:
    """Name of the fused activation an activation callable maps to, or None (the layer then runs it un-fused).  GLU
    layers: SwiGLU on the fused tensor, `nn.GLU()`.  Plain layers: `nn.GELU(approximate="tanh")`."""
    if not is_glu:
        return "gelu_tanh" if isinstance(fn, nn.GELU) and fn.approximate == "tanh" else None
    if is_swiglu_callable(fn):
        return "swiglu"
    if isinstance(fn, nn.GLU) and fn.dim in (-1, 1):  # the layer applies it to 2-D (rows, 2I) tensors
        return "glu"
    return None


class MoE_B200(MoE_Torch):
    """MoE layer on the sm_100a kernels.  Same constructor, parameters and `state_dict` keys as `MoE_Torch`.

    `fused_router` (attribute, default False): route 16-bit tensors with the one-launch router kernel instead of the
    eager gate / top-k / softmax sequence.  Off by default so that the selected experts are those of the eager router
    bit for bit (see `router.py` for where the two can differ).
    """

    experts_cls = Experts_B200
    fused_router = False

    def _compute_routing_weights(self, hidden_states: torch.Tensor):
        if self.fused_router and fused_router_supported(hidden_states, self.num_experts, self.top_k, self.gate.weight):
            logits, weights, selected_experts, _ = fused_router(hidden_states, self.gate.weight, self.top_k, self.router_scoring)
            return logits, weights, selected_experts
        return super()._compute_routing_weights(hidden_states)

    def _compute_experts(self, hidden_states: torch.Tensor, router_weights: torch.Tensor, selected_experts: torch.Tensor) -> torch.Tensor:
        fused = fused_activation(self.act, self.is_glu)
        if fused == "gelu_tanh" and self.intermediate_size % 2:
            fused = None
        if fused is not None:
            return fused_swiglu_experts(hidden_states, self.c_fc.weight, self.c_proj.weight, router_weights, selected_experts, activation=fused)
        with torch.no_grad():
            sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, _, _, _ = route(selected_experts.flatten(), self.num_experts, self.top_k, True, False)
        h = self.c_fc(hidden_states, self.top_k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, grouped_out=True)
        h = self.act(h)
        return self.c_proj(h, 1, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, grouped_in=True, gates=router_weights)

    def _compute_shared_experts(self, hidden_states: torch.Tensor) -> torch.Tensor:
        # every token visits every shared expert with weight one: the routed-expert kernels with a trivial routing
        T, S = hidden_states.shape[0], self.num_shared_experts
        ones = torch.ones(T, S, dtype=hidden_states.dtype, device=hidden_states.device)
        ids = torch.arange(S, device=hidden_states.device).expand(T, S)
        return fused_swiglu_experts(hidden_states, self.shared_c_fc.weight, self.shared_c_proj.weight, ones, ids)


# drop-in names of the reference
Experts_Triton = Experts_B200
MoE_Triton = MoE_B200
