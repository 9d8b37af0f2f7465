"""CPU oracle for the scattermoe MoE path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-on-CPU (fp32 / fp64) and numpy integer code, the algorithm of
the reference's MoE layer so that the CUDA path can be checked against it.  Nothing in the product
package imports it: only the test-suite, the smoke check and the CPU-baseline leg of the benchmark do.

Parity status: pinned.  `tests/golden/*.npz` hold outputs of the reference's own `MoE_Torch`
(cute_kernels/kernels/scattermoe/torch_implementation.py:61-199) produced by
`tests/golden/make_golden.py`; `tests/test_oracle.py` checks every function here against them.

Each function cites the reference lines it follows (paths relative to the reference project root).
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------------
# integer routing
# --------------------------------------------------------------------------------------------------


def contiguous_count(x: np.ndarray, size: int) -> np.ndarray:
    """Histogram of ids in [0, size) as int32.

    Follows cute_kernels/kernels/contiguous_count/__init__.py:8-24 (the op) whose defining
    equivalence is `bincount(minlength=size)` (tests/kernels/contiguous_count_test.py:34-37).
    """
    x = np.asarray(x).reshape(-1)
    out = np.zeros(size, dtype=np.int32)
    for v in x:  # plain loop on purpose: this is the definition, not a fast path
        out[int(v)] += 1
    return out


def contiguous_count_fast(x: np.ndarray, size: int) -> np.ndarray:
    """Vectorised form of `contiguous_count` for the larger parity cases."""
    return np.bincount(np.asarray(x).reshape(-1), minlength=size).astype(np.int32)


def route(selected_experts: np.ndarray, num_experts: int):
    """Expert sort + histogram + inclusive offsets.

    Follows cute_kernels/kernels/scattermoe/triton_implementation/__init__.py:79-81:
    `sorted_expert_idxs, sorted_scattered_idxs = selected_experts.flatten().sort()` and
    `expert_offsets = contiguous_count(sorted_expert_idxs, E).cumsum(-1)`.
    The reference's sort is not stable, so `sorted_scattered_idxs` is defined only up to the
    order inside one expert's segment; the oracle fixes the stable order (ascending flat index
    inside each segment), which is what the CUDA path produces.
    Returns int64 (M), int64 (M), int64 (E) inclusive offsets, int32 (E) counts.
    """
    flat = np.asarray(selected_experts).reshape(-1).astype(np.int64)
    order = np.argsort(flat, kind="stable").astype(np.int64)
    sorted_expert_idxs = flat[order]
    counts = contiguous_count_fast(sorted_expert_idxs, num_experts)
    expert_offsets = np.cumsum(counts.astype(np.int64))
    return sorted_expert_idxs, order, expert_offsets, counts


def padded_layout(counts: np.ndarray, tile: int = 128):
    """Start row of each expert's segment when every segment is padded to a multiple of `tile`.

    Not in the reference: this is the internal layout of the CUDA path's grouped buffers.
    Returns int64 (E+1) padded starts; entry E is the padded total.
    """
    counts = np.asarray(counts).astype(np.int64)
    padded = (counts + tile - 1) // tile * tile
    out = np.zeros(len(counts) + 1, dtype=np.int64)
    out[1:] = np.cumsum(padded)
    return out


# --------------------------------------------------------------------------------------------------
# the four reference ops, restated on dense torch tensors
# --------------------------------------------------------------------------------------------------


def scatter2scatter(X, W, sorted_expert_idxs, sorted_scattered_idxs, FAN_OUT, x_grouped=False, y_grouped=False):
    """Grouped GEMM with row gather / scatter.

    Follows cute_kernels/kernels/scattermoe/triton_implementation/kernels.py:61-102,129-130:
    for m in [0, M): e = sorted_expert_idxs[m], s = sorted_scattered_idxs[m],
    src = m if x_grouped else s // FAN_OUT, dst = m if y_grouped else s,
    Y[dst, :] = X[src, :] @ W[e]   with W viewed (E, K, N).
    """
    se = torch.as_tensor(sorted_expert_idxs, dtype=torch.long)
    ss = torch.as_tensor(sorted_scattered_idxs, dtype=torch.long)
    M = se.numel()
    rows = torch.arange(M)
    src = rows if x_grouped else ss // FAN_OUT
    dst = rows if y_grouped else ss
    out = torch.zeros(M, W.shape[-1], dtype=X.dtype)
    for e in range(W.shape[0]):
        sel = (se == e).nonzero().flatten()
        if sel.numel():
            out[dst[sel]] = X[src[sel]] @ W[e]
    return out


def group(A, sorted_scattered_idxs, coeff=None, fan_out=1):
    """Row gather into grouped order with an optional per-row coefficient.

    Follows cute_kernels/kernels/scattermoe/triton_implementation/kernels.py:245-298:
    out[n, :] = A[idx[n] // fan_out, :] * coeff[idx[n]].
    """
    idx = torch.as_tensor(sorted_scattered_idxs, dtype=torch.long)
    out = A[idx // fan_out]
    if coeff is not None:
        out = out * coeff[idx].unsqueeze(-1)
    return out


def group_bwd_W(DY, X, expert_offsets, E):
    """Per-expert weight gradient on grouped tensors.

    Follows cute_kernels/kernels/scattermoe/triton_implementation/kernels.py:152-240:
    DW[e] (K, N) = X[off[e-1]:off[e]]^T @ DY[off[e-1]:off[e]], off[-1] := 0; empty experts stay zero.
    """
    off = [0] + [int(v) for v in expert_offsets]
    DW = torch.zeros(E, X.shape[1], DY.shape[1], dtype=X.dtype)
    for e in range(E):
        if off[e + 1] > off[e]:
            DW[e] = X[off[e] : off[e + 1]].t() @ DY[off[e] : off[e + 1]]
    return DW


def swiglu_unchunked(x):
    """y = x[..., :h] * silu(x[..., h:]).

    Follows cute_kernels/kernels/swiglu_unchunked/torch_implementation.py:5-7.
    """
    up, gate = x.chunk(2, dim=-1)
    return up * F.silu(gate)


def swiglu_unchunked_backward(x, dy):
    """Gradient of `swiglu_unchunked`.

    Follows cute_kernels/kernels/swiglu_unchunked/triton_implementation/kernels_backward.py:13-48:
    dgate = dy * up * (sig + gate * sig * (1 - sig)),  dup = dy * gate * sig, written into the two halves.
    """
    up, gate = x.chunk(2, dim=-1)
    sig = torch.sigmoid(gate)
    dup = dy * gate * sig
    dgate = dy * up * (sig + gate * sig * (1 - sig))
    return torch.cat([dup, dgate], dim=-1)


# --------------------------------------------------------------------------------------------------
# whole layer
# --------------------------------------------------------------------------------------------------


def routing_weights(x, gate_weight, top_k):
    """Router of the reference module.

    Follows cute_kernels/kernels/scattermoe/torch_implementation.py:120-133,193-199:
    logits = x @ gate_weight^T, top-k (max when k == 1), softmax over the selected logits in fp32,
    cast back to x.dtype.  Returns (logits, weights, selected_experts int64).
    """
    logits = F.linear(x, gate_weight)
    if top_k == 1:
        vals, idx = logits.max(dim=-1, keepdim=True)
    else:
        vals, idx = logits.topk(top_k, dim=-1)
    weights = F.softmax(vals.float(), dim=-1).type_as(x)
    return logits, weights, idx


def experts_torch_style(x, w_fc, w_proj, router_weights, selected_experts, act=swiglu_unchunked):
    """Expert computation in the formulation of the reference's torch module.

    Follows cute_kernels/kernels/scattermoe/torch_implementation.py:135-191,30-47:
    argsort the flat expert ids, fan_in_index = order // k, gather rows, per-expert linear over the
    split by expert frequency, activation per expert, per-expert down projection, scale by the
    gathered gates, `zeros.index_add(0, fan_in_index, .)`.
    Differentiable through torch autograd (x, w_fc, w_proj, router_weights).
    """
    T, k = selected_experts.shape
    E = w_fc.shape[0]
    flat = selected_experts.flatten()
    freq = flat.bincount(minlength=E)
    order = flat.argsort(stable=True)
    fan_in_index = order // k
    batch_gates = router_weights.flatten()[order]
    xs = x[fan_in_index].split(freq.tolist(), dim=0)
    hs = [F.linear(xs[e], w_fc[e]) for e in range(E)]
    hs = [act(h) for h in hs]
    ys = torch.cat([F.linear(hs[e], w_proj[e]) for e in range(E)])
    ys = ys * batch_gates.unsqueeze(-1)
    zeros = torch.zeros(T, x.shape[1], dtype=ys.dtype)
    return zeros.index_add(0, fan_in_index, ys)


def experts_scatter_style(x, w_fc, w_proj, router_weights, selected_experts):
    """Expert computation in the formulation of the reference's scatter module, forward and backward
    written out (no autograd), SwiGLU activation.

    Forward follows cute_kernels/kernels/scattermoe/triton_implementation/__init__.py:76-101 and
    ops.py:133-180; backward follows ops.py:182-277 for both projections with the SwiGLU backward
    in between.  Returns a dict of every intermediate the CUDA path also produces, so that tests can
    pin them one by one.  `w_fc` is (E, 2I, H), `w_proj` is (E, H, I) as stored by the module.
    """
    T, k = selected_experts.shape
    E = w_fc.shape[0]
    se, ss, off, counts = route(selected_experts.numpy(), E)
    W1 = w_fc.permute(0, 2, 1)  # (E, H, 2I) view, as Experts_Triton.forward passes it
    W2 = w_proj.permute(0, 2, 1)  # (E, I, H)
    h = scatter2scatter(x, W1, se, ss, k, x_grouped=False, y_grouped=True)
    a = swiglu_unchunked(h)
    y_exp = scatter2scatter(a, W2, se, ss, 1, x_grouped=True, y_grouped=False)
    y_exp3 = y_exp.view(T, k, -1)
    y = torch.bmm(router_weights.unsqueeze(1), y_exp3).squeeze(1)
    out = dict(sorted_expert_idxs=se, sorted_scattered_idxs=ss, expert_offsets=off, counts=counts, h=h, a=a, y_expanded=y_exp, y=y)

    def backward(grad_out):
        d_gates = torch.bmm(y_exp3, grad_out.unsqueeze(2)).squeeze(-1)
        ggo = group(grad_out, ss, coeff=router_weights.flatten(), fan_out=k)
        dW2 = group_bwd_W(ggo, a, off, E)  # (E, I, H): gradient of the permuted view
        da = scatter2scatter(ggo, W2.permute(0, 2, 1), se, ss, 1, x_grouped=True, y_grouped=True)
        dh = swiglu_unchunked_backward(h, da)
        gx = group(x, ss, fan_out=k)
        dW1 = group_bwd_W(dh, gx, off, E)  # (E, H, 2I)
        dx_exp = scatter2scatter(dh, W1.permute(0, 2, 1), se, ss, 1, x_grouped=True, y_grouped=False)
        dx = dx_exp.view(T, k, -1).sum(-2) if k > 1 else dx_exp
        return dict(
            d_gates=d_gates,
            grouped_grad_out=ggo,
            da=da,
            dh=dh,
            dx_expanded=dx_exp,
            dx=dx,
            d_w_fc=dW1.permute(0, 2, 1),  # back to the stored (E, 2I, H) orientation
            d_w_proj=dW2.permute(0, 2, 1),  # (E, H, I)
        )

    out["backward"] = backward
    return out


def moe_layer(x, gate_weight, w_fc, w_proj, top_k, grad_out=None, act=swiglu_unchunked):
    """Whole layer, forward (+ backward through autograd when `grad_out` is given).

    Follows cute_kernels/kernels/scattermoe/torch_implementation.py:101-118.
    Returns dict(y, logits, weights, selected_experts[, dx, d_gate_weight, d_w_fc, d_w_proj]).
    """
    x = x.detach().clone().requires_grad_(grad_out is not None)
    gw = gate_weight.detach().clone().requires_grad_(grad_out is not None)
    w1 = w_fc.detach().clone().requires_grad_(grad_out is not None)
    w2 = w_proj.detach().clone().requires_grad_(grad_out is not None)
    logits, weights, sel = routing_weights(x, gw, top_k)
    y = experts_torch_style(x, w1, w2, weights, sel, act=act)
    res = dict(y=y.detach(), logits=logits.detach(), weights=weights.detach(), selected_experts=sel)
    if grad_out is not None:
        y.backward(grad_out)
        res.update(dx=x.grad, d_gate_weight=gw.grad, d_w_fc=w1.grad, d_w_proj=w2.grad)
    return res


def experts_with_grads(x, w_fc, w_proj, router_weights, selected_experts, grad_out, act=swiglu_unchunked):
    """Externally supplied routing (the seam `_compute_experts(hidden_states, router_weights,
    selected_experts)`, cute_kernels/kernels/scattermoe/torch_implementation.py:135-137), forward and
    autograd backward.  Returns dict(y, dx, d_router_weights, d_w_fc, d_w_proj).
    """
    x = x.detach().clone().requires_grad_(True)
    rw = router_weights.detach().clone().requires_grad_(True)
    w1 = w_fc.detach().requires_grad_(True)  # detach() shares storage: no copy of the (large) weights
    w2 = w_proj.detach().requires_grad_(True)
    y = experts_torch_style(x, w1, w2, rw, selected_experts, act=act)
    y.backward(grad_out)
    return dict(y=y.detach(), dx=x.grad, d_router_weights=rw.grad, d_w_fc=w1.grad, d_w_proj=w2.grad)


def shared_experts(x, w_fc_shared, w_proj_shared):
    """Always-on shared experts: dense SwiGLU MLPs added to the routed output.

    Not in the reference (its module has routed experts only,
    cute_kernels/kernels/scattermoe/torch_implementation.py:81-99); restated from the same expert
    math: sum_s linear(swiglu(linear(x, Wfc_s)), Wproj_s).
    """
    y = torch.zeros_like(x)
    for s in range(w_fc_shared.shape[0]):
        y = y + F.linear(swiglu_unchunked(F.linear(x, w_fc_shared[s])), w_proj_shared[s])
    return y


def sigmoid_routing(logits, top_k, normalise=True):
    """Sigmoid scoring of the top-k logits (not in the reference, which only has the softmax of
    cute_kernels/kernels/scattermoe/torch_implementation.py:130): scores = sigmoid(logits) at the
    top-k positions, optionally normalised to sum to one.
    """
    vals, idx = logits.topk(top_k, dim=-1)
    w = torch.sigmoid(vals.float())
    if normalise:
        w = w / w.sum(-1, keepdim=True)
    return w.type_as(logits), idx


def rmsnorm(x, weight, eps):
    """y = x / sqrt(mean(x^2, last dim) + eps) * weight (weight may be None), in the arithmetic type of x.

    Follows cute_kernels/kernels/rmsnorm/torch_implementation.py:5-6 (F.rms_norm) and the kernel
    cute_kernels/kernels/rmsnorm/triton_implementation/kernels_forward.py:44-60.
    """
    inverse_rms = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    y = x * inverse_rms
    return y if weight is None else y * weight


def rmsnorm_backward(x, weight, dy, eps):
    """(dx, dweight) of `rmsnorm`; dweight is None without a weight.

    Follows cute_kernels/kernels/rmsnorm/triton_implementation/kernels_backward.py:64-96:
    g = dy * weight; dx = r * g - (1/H) * r^3 * x * sum(g * x); dweight = sum over rows of dy * x * r.
    """
    H = x.shape[-1]
    r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    g = dy if weight is None else dy * weight
    dx = r * g - (1.0 / H) * r * r * r * x * (g * x).sum(dim=-1, keepdim=True)
    dw = None if weight is None else (dy * x * r).reshape(-1, H).sum(dim=0)
    return dx, dw


def rel_l2(a, b) -> float:
    a = torch.as_tensor(a).double().flatten()
    b = torch.as_tensor(b).double().flatten()
    denom = b.norm().item()
    return (a - b).norm().item() / (denom if denom > 0 else 1.0)
