"""Fused router: gate projection, top-k, scores and expert histogram in one launch.

Replaces `_compute_routing_weights` + `_get_topk` of the reference module
(cute_kernels/kernels/scattermoe/torch_implementation.py:120-133,193-199) for 16-bit tensors.  The eager router runs a
GEMM, a top-k, a cast, a softmax and a cast back (and the layer then counts the selected experts); here the logits
never leave the accumulator before the top-k is taken.

Selection differs from the eager router only where two logits of a row are equal after rounding to the tensor type
(the fused kernel picks the lower expert; `torch.topk` leaves the order of equal values unspecified) or where the
two GEMMs round a logit differently (different summation order, at most one unit in the last place), which can
exchange two experts whose logits are that close.  The layer keeps the eager router by default for that reason
(`MoE_B200.fused_router = False`) and switches with `fused_router=True`.
"""

from __future__ import annotations

import torch

from ._lib import check, dtype_code, lib, ptr, status_word, stream_ptr
from .custom_op import b200_op

SCORING = {"softmax": 0, "sigmoid": 1}
MAX_EXPERTS, MAX_TOP_K = 256, 8


def _router_fake(x: torch.Tensor, gate_weight: torch.Tensor, top_k: int, scoring: int, row_scale: torch.Tensor | None = None):
    T, E = x.size(0), gate_weight.size(0)
    return (
        torch.empty(T, E, dtype=x.dtype, device=x.device),
        torch.empty(T, top_k, dtype=x.dtype, device=x.device),
        torch.empty(T, top_k, dtype=torch.int64, device=x.device),
        torch.empty(E, dtype=torch.int32, device=x.device),
    )


@b200_op("router_forward", mutates_args=(), fake_func=_router_fake)
def router_forward(x: torch.Tensor, gate_weight: torch.Tensor, top_k: int, scoring: int, row_scale: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(logits (T, E), weights (T, k), selected_experts int64 (T, k), counts int32 (E)) of x (T, H), gate_weight (E, H).
    `row_scale` (fp32, T): optional factor per token applied to the logits before they are rounded."""
    if not (x.is_cuda and gate_weight.is_cuda):
        raise RuntimeError("router_forward: CUDA tensors required (there is no CPU path)")
    assert x.dim() == 2 and gate_weight.dim() == 2 and x.size(1) == gate_weight.size(1) and x.dtype == gate_weight.dtype
    assert x.stride(1) == 1 and gate_weight.stride(1) == 1
    outs = _router_fake(x, gate_weight, top_k, scoring)
    logits, weights, indices, counts = outs
    assert row_scale is None or (row_scale.dtype == torch.float32 and row_scale.numel() == x.size(0) and row_scale.is_contiguous())
    check(
        lib().b200moe_router_forward_scaled(
            ptr(x), x.stride(0), ptr(gate_weight), gate_weight.stride(0), ptr(row_scale), x.size(0), x.size(1), gate_weight.size(0), top_k, scoring,
            ptr(logits), logits.stride(0), ptr(weights), ptr(indices), ptr(counts), dtype_code(x), ptr(status_word(x.device)), stream_ptr(x.device),
        ),
        "router_forward",
    )
    return outs


def fused_router_supported(x: torch.Tensor, num_experts: int, top_k: int, gate_weight: torch.Tensor | None = None) -> bool:
    """True when the one-launch router can take these tensors as they are: 16-bit CUDA tensors, rows that start on
    16-byte boundaries and are multiples of 16 bytes long, unit inner stride (for x and, when given, the gate weight)."""

    def rows_ok(t: torch.Tensor) -> bool:
        return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0

    return (
        x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and num_experts <= MAX_EXPERTS and top_k <= MAX_TOP_K
        and x.size(-1) % 8 == 0 and rows_ok(x) and (gate_weight is None or (gate_weight.dtype == x.dtype and rows_ok(gate_weight)))
    )


def _scores(top_vals: torch.Tensor, scoring: int, dtype: torch.dtype) -> torch.Tensor:
    if scoring == SCORING["sigmoid"]:
        s = torch.sigmoid(top_vals.float())
        return (s / s.sum(-1, keepdim=True)).to(dtype)
    return torch.softmax(top_vals.float(), dim=-1).to(dtype)


class _FusedRouter(torch.autograd.Function):
    """Differentiable wrapper: gradients of the logits and of the routing weights flow to x and to the gate weight."""

    @staticmethod
    def forward(ctx, x, gate_weight, top_k, scoring):
        logits, weights, indices, counts = router_forward(x.detach(), gate_weight.detach(), top_k, scoring)
        ctx.save_for_backward(x, gate_weight, logits, indices)
        ctx.scoring = scoring
        ctx.mark_non_differentiable(indices, counts)
        return logits, weights, indices, counts

    @staticmethod
    def backward(ctx, d_logits, d_weights, _d_indices, _d_counts):
        x, gate_weight, logits, indices = ctx.saved_tensors
        total = None if d_logits is None else d_logits.clone()
        if d_weights is not None:
            # scores as a function of the selected logits: the eager formula, differentiated by autograd on (T, k) values
            with torch.enable_grad():
                vals = logits.gather(1, indices).detach().requires_grad_(True)
                w = _scores(vals, ctx.scoring, logits.dtype)
                (d_vals,) = torch.autograd.grad(w, vals, d_weights)
            total = torch.zeros_like(logits) if total is None else total
            total.scatter_add_(1, indices, d_vals.to(total.dtype))
        if total is None:
            return None, None, None, None
        dx = _logit_grad_to_input(total, gate_weight) if ctx.needs_input_grad[0] else None
        dw = _logit_grad_to_weight(total, x) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def _one_group_indices(rows: int, device):
    """Index tensors that describe `rows` rows of one single expert, already in grouped order."""
    return torch.zeros(rows, dtype=torch.int64, device=device), torch.arange(rows, dtype=torch.int64, device=device), torch.full((1,), rows, dtype=torch.int64, device=device)


def _logit_grad_to_input(d_logits: torch.Tensor, gate_weight: torch.Tensor) -> torch.Tensor:
    """d_logits (T, E) @ gate_weight (E, H) on this package's grouped-GEMM operator (one group holding every row);
    falls back to the library product only for expert counts the operator's tensor-core path cannot take."""
    from .ops import scatter2scatter

    T, E = d_logits.shape
    if E % 8 or gate_weight.size(1) % 8 or T == 0:
        return d_logits @ gate_weight
    se, ss, _ = _one_group_indices(T, d_logits.device)
    out = torch.empty(T, gate_weight.size(1), dtype=d_logits.dtype, device=d_logits.device)
    scatter2scatter(X=d_logits.contiguous(), W=gate_weight.detach().unsqueeze(0), sorted_expert_idxs=se, sorted_scattered_idxs=ss, out=out, FAN_OUT=1, x_grouped=True, y_grouped=True)
    return out


def _logit_grad_to_weight(d_logits: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """d_logits (T, E)^T @ x (T, H) on this package's weight-gradient operator (one group holding every row)."""
    from .ops import group_bwd_W

    T, E = d_logits.shape
    if E % 8 or x.size(1) % 8 or T == 0:
        return d_logits.t() @ x
    _, _, off = _one_group_indices(T, d_logits.device)
    dw = torch.empty(1, E, x.size(1), dtype=x.dtype, device=x.device)
    group_bwd_W(DY=x.contiguous(), X=d_logits.contiguous(), expert_offsets=off, DW=dw, E=1)
    return dw[0]


def fused_router(x: torch.Tensor, gate_weight: torch.Tensor, top_k: int, scoring: str = "softmax"):
    """Router of the MoE layer in one launch; returns (logits, weights, selected_experts, counts).

    `counts` (int32, one entry per expert) is the histogram the layer's sort needs, produced on the way.
    """
    if top_k > MAX_TOP_K or gate_weight.size(0) > MAX_EXPERTS:
        raise RuntimeError(f"fused_router: at most {MAX_EXPERTS} experts and {MAX_TOP_K} experts per token")
    return _FusedRouter.apply(x, gate_weight, top_k, SCORING[scoring])


class _FusedNormRouter(torch.autograd.Function):
    """RMSNorm of the hidden states and the router of the layer that follows it.  The normalised rows are written once
    (the experts read them); the logits come from the UN-normalised rows: with r[t] = 1 / rms(x[t]),
    logits[t] = r[t] * (x[t] @ (gate_weight * norm_weight)^T), so the gate projection reads x while the norm kernel's only
    contribution to it is the per-row factor, applied in the router's epilogue."""

    @staticmethod
    def forward(ctx, x, norm_weight, gate_weight, eps, top_k, scoring):
        from .ops import _rmsnorm_forward

        T, H = x.shape
        y = torch.empty_like(x)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        _rmsnorm_forward(x, norm_weight, y, rstd, eps)
        folded = gate_weight if norm_weight is None else (gate_weight.float() * norm_weight.float()).to(gate_weight.dtype)
        logits, weights, indices, counts = router_forward(x.detach(), folded.detach().contiguous(), top_k, scoring, rstd)
        ctx.save_for_backward(x, norm_weight, gate_weight, rstd, y, logits, indices)
        ctx.eps, ctx.scoring = eps, scoring
        ctx.mark_non_differentiable(indices, counts)
        return y, logits, weights, indices, counts

    @staticmethod
    def backward(ctx, d_y, d_logits, d_weights, _d_indices, _d_counts):
        from .ops import _rmsnorm_backward

        x, norm_weight, gate_weight, rstd, y, logits, indices = ctx.saved_tensors
        total = None if d_logits is None else d_logits.clone()
        if d_weights is not None:
            with torch.enable_grad():
                vals = logits.gather(1, indices).detach().requires_grad_(True)
                w = _scores(vals, ctx.scoring, logits.dtype)
                (d_vals,) = torch.autograd.grad(w, vals, d_weights)
            total = torch.zeros_like(logits) if total is None else total
            total.scatter_add_(1, indices, d_vals.to(total.dtype))
        # the logits are a linear function of the normalised rows y: their gradient joins the upstream gradient of y
        d_gate = None
        dy_total = d_y
        if total is not None:
            if ctx.needs_input_grad[2]:
                d_gate = _logit_grad_to_weight(total, y)
            contrib = _logit_grad_to_input(total, gate_weight)
            dy_total = contrib if d_y is None else d_y + contrib
        if dy_total is None:
            return None, None, d_gate, None, None, None
        dx = torch.empty_like(x)
        d_norm = torch.empty_like(norm_weight) if (norm_weight is not None and ctx.needs_input_grad[1]) else None
        _rmsnorm_backward(x, norm_weight, dy_total.contiguous(), rstd, dx, d_norm, ctx.eps)
        return dx, d_norm, d_gate, None, None, None


def fused_rmsnorm_router(x: torch.Tensor, norm_weight: torch.Tensor | None, gate_weight: torch.Tensor, eps: float, top_k: int, scoring: str = "softmax"):
    """RMSNorm feeding an MoE layer, fused with that layer's gate projection
    (cute_kernels/kernels/rmsnorm/triton_implementation/kernels_forward.py:19-60 followed by
    cute_kernels/kernels/scattermoe/torch_implementation.py:120-133).  x: (T, H) 16-bit CUDA tensor.
    Returns (normalised x, logits, routing weights, selected_experts, counts); differentiable in x, both weights.
    Like the fused router, it can pick a different expert where two logits differ by one unit in the last place."""
    if top_k > MAX_TOP_K or gate_weight.size(0) > MAX_EXPERTS:
        raise RuntimeError(f"fused_rmsnorm_router: at most {MAX_EXPERTS} experts and {MAX_TOP_K} experts per token")
    assert x.dim() == 2 and x.stride(1) == 1
    return _FusedNormRouter.apply(x, norm_weight, gate_weight, eps, top_k, SCORING[scoring])
