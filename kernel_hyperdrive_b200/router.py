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


def _router_fake(x: torch.Tensor, gate_weight: torch.Tensor, top_k: int, scoring: int):
    T, E = x.size(0), gate_weight.size(0)
    return (
        torch.empty(T, E, dtype=x.dtype, device=x.device),
        torch.empty(T, top_k, dtype=x.dtype, device=x.device),
        torch.empty(T, top_k, dtype=torch.int64, device=x.device),
        torch.empty(E, dtype=torch.int32, device=x.device),
    )


@b200_op("router_forward", mutates_args=(), fake_func=_router_fake)
def router_forward(x: torch.Tensor, gate_weight: torch.Tensor, top_k: int, scoring: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(logits (T, E), weights (T, k), selected_experts int64 (T, k), counts int32 (E)) of x (T, H), gate_weight (E, H)."""
    if not (x.is_cuda and gate_weight.is_cuda):
        raise RuntimeError("router_forward: CUDA tensors required (there is no CPU path)")
    assert x.dim() == 2 and gate_weight.dim() == 2 and x.size(1) == gate_weight.size(1) and x.dtype == gate_weight.dtype
    assert x.stride(1) == 1 and gate_weight.stride(1) == 1
    outs = _router_fake(x, gate_weight, top_k, scoring)
    logits, weights, indices, counts = outs
    check(
        lib().b200moe_router_forward(
            ptr(x), x.stride(0), ptr(gate_weight), gate_weight.stride(0), x.size(0), x.size(1), gate_weight.size(0), top_k, scoring,
            ptr(logits), logits.stride(0), ptr(weights), ptr(indices), ptr(counts), dtype_code(x), ptr(status_word(x.device)), stream_ptr(x.device),
        ),
        "router_forward",
    )
    return outs


def fused_router_supported(x: torch.Tensor, num_experts: int, top_k: int) -> bool:
    return (
        x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and num_experts <= MAX_EXPERTS and top_k <= MAX_TOP_K
        and x.size(-1) % 8 == 0
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
        dx = total @ gate_weight if ctx.needs_input_grad[0] else None
        dw = total.t() @ x if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def fused_router(x: torch.Tensor, gate_weight: torch.Tensor, top_k: int, scoring: str = "softmax"):
    """Router of the MoE layer in one launch; returns (logits, weights, selected_experts, counts).

    `counts` (int32, one entry per expert) is the histogram the layer's sort needs, produced on the way.
    """
    if top_k > MAX_TOP_K or gate_weight.size(0) > MAX_EXPERTS:
        raise RuntimeError(f"fused_router: at most {MAX_EXPERTS} experts and {MAX_TOP_K} experts per token")
    return _FusedRouter.apply(x, gate_weight, top_k, SCORING[scoring])
