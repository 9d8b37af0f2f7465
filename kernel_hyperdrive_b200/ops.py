"""The reference's operators with their signatures, running on the b200moe C-ABI library.

`scatter2scatter`, `group_bwd_W`, `group` (cute_kernels/kernels/scattermoe/triton_implementation/ops.py:16-130),
`contiguous_count_cute` (cute_kernels/kernels/contiguous_count/__init__.py:8-24) and the SwiGLU on a fused
tensor (cute_kernels/kernels/swiglu_unchunked/__init__.py:11-69).  Same argument names and meaning, same
assertions; tensors must live on a CUDA device.
"""

from __future__ import annotations

import torch

from . import _lib
from ._lib import check, dtype_code, lib, ptr, status_word, stream_ptr
from .custom_op import b200_op

torch._dynamo.config.capture_scalar_outputs = True


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("b200moe operators run on CUDA tensors only (there is no CPU path)")


def _row_major(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or (t.size(1) > 1 and t.stride(1) != 1):
        raise ValueError(f"{name}: expected a 2-D tensor with unit inner stride, got shape {tuple(t.shape)} strides {t.stride()}")


# ---- histogram -----------------------------------------------------------------------------------


def _contiguous_count_fake(x: torch.Tensor, size: int) -> torch.Tensor:
    return torch.empty(size, dtype=torch.int32, device=x.device)


@b200_op("contiguous_count", mutates_args=(), fake_func=_contiguous_count_fake)
def _contiguous_count(x: torch.Tensor, size: int) -> torch.Tensor:
    _require_cuda(x)
    out = torch.empty(size, dtype=torch.int32, device=x.device)
    check(lib().b200moe_contiguous_count(ptr(x), int(x.dtype == torch.int64), x.numel(), ptr(out), size, stream_ptr(x.device)), "contiguous_count")
    return out


@torch.no_grad()
def contiguous_count_cute(x: torch.Tensor, size: int, kernel_backend=None, BLOCK_SIZE_B: int = 64) -> torch.Tensor:
    """int32 histogram of the values of a 1-D int32/int64 tensor in [0, size).

    `kernel_backend` and `BLOCK_SIZE_B` are accepted for signature compatibility and ignored: there is one
    backend and its launch shape is fixed.
    """
    assert x.dim() == 1, "x should be 1-dimensional"
    assert x.dtype in [torch.int32, torch.long]
    return _contiguous_count(x.contiguous(), size)


# ---- grouped GEMMs -------------------------------------------------------------------------------

_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Grow-only scratch buffer per (device, stream); kernels on one stream run in order, so sharing is safe."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


@b200_op("scatter2scatter", mutates_args={"out"})
def scatter2scatter(
    X: torch.Tensor,
    W: torch.Tensor,
    sorted_expert_idxs: torch.Tensor,
    sorted_scattered_idxs: torch.Tensor,
    out: torch.Tensor,
    FAN_OUT: int,
    x_grouped: bool = False,
    y_grouped: bool = False,
) -> None:
    assert sorted_scattered_idxs.size(0) == sorted_expert_idxs.size(0)
    assert sorted_scattered_idxs.size(0) == X.size(0) * FAN_OUT
    assert out.size(0) == sorted_expert_idxs.size(0)
    assert out.size(1) == W.size(-1)
    _require_cuda(X, W, out, sorted_expert_idxs, sorted_scattered_idxs)
    _row_major(X, "X")
    _row_major(out, "out")
    assert W.dim() == 3 and W.size(1) == X.size(1) and W.dtype == X.dtype == out.dtype
    assert sorted_expert_idxs.dtype == torch.int64 and sorted_scattered_idxs.dtype == torch.int64
    M, E = sorted_expert_idxs.size(0), W.size(0)
    nbytes = lib().b200moe_scatter2scatter_workspace_bytes(M, E)
    ws = _workspace(X.device, nbytes)
    check(
        lib().b200moe_scatter2scatter(
            ptr(X), X.stride(0), ptr(W), W.stride(0), W.stride(1), W.stride(2),
            ptr(sorted_expert_idxs.contiguous()), ptr(sorted_scattered_idxs.contiguous()),
            ptr(out), out.stride(0), M, X.size(1), out.size(1), E, FAN_OUT, int(x_grouped), int(y_grouped),
            dtype_code(X), ptr(ws), ws.numel(), ptr(status_word(X.device)), stream_ptr(X.device),
        ),
        "scatter2scatter",
    )


@b200_op("group_bwd_W", mutates_args={"DW"})
def group_bwd_W(DY: torch.Tensor, X: torch.Tensor, expert_offsets: torch.Tensor, DW: torch.Tensor, E: int) -> None:
    _require_cuda(DY, X, expert_offsets, DW)
    _row_major(DY, "DY")
    _row_major(X, "X")
    assert DW.dim() == 3 and DW.size(0) == E and DW.size(1) == X.size(1) and DW.size(2) == DY.size(1)
    assert DY.size(0) == X.size(0) and DY.dtype == X.dtype == DW.dtype
    offsets = expert_offsets.to(torch.int64).contiguous()
    check(
        lib().b200moe_group_bwd_W(
            ptr(DY), DY.stride(0), ptr(X), X.stride(0), ptr(offsets), ptr(DW), DW.stride(0), DW.stride(1), DW.stride(2),
            X.size(0), X.size(1), DY.size(1), E, dtype_code(X), ptr(status_word(X.device)), stream_ptr(X.device),
        ),
        "group_bwd_W",
    )


@b200_op("group", mutates_args={"out"})
def group(
    A: torch.Tensor,
    sorted_expert_idxs: torch.Tensor,
    out: torch.Tensor,
    coeff: torch.Tensor | None = None,
    fan_out: int = 1,
) -> None:
    N = sorted_expert_idxs.size(0)
    K = A.size(1)
    assert A.size(0) * fan_out == N
    _require_cuda(A, sorted_expert_idxs, out, coeff)
    _row_major(A, "A")
    _row_major(out, "out")
    assert out.size(0) == N and out.size(1) == K and out.dtype == A.dtype
    assert sorted_expert_idxs.dtype == torch.int64
    if coeff is not None:
        assert coeff.dtype == A.dtype and coeff.numel() == N
        coeff = coeff.contiguous()
    check(
        lib().b200moe_group(ptr(A), A.stride(0), ptr(sorted_expert_idxs.contiguous()), ptr(out), out.stride(0), ptr(coeff), fan_out, N, K, dtype_code(A), stream_ptr(A.device)),
        "group",
    )


@b200_op("combine", mutates_args={"out"})
def combine(expanded: torch.Tensor, gates: torch.Tensor | None, out: torch.Tensor, k: int) -> None:
    """out[t, :] = sum_j gates[t, j] * expanded[t*k + j, :] (plain sum without gates), fp32 accumulation."""
    _require_cuda(expanded, gates, out)
    _row_major(expanded, "expanded")
    _row_major(out, "out")
    T = out.size(0)
    assert expanded.size(0) == T * k and expanded.size(1) == out.size(1) and expanded.dtype == out.dtype
    if gates is not None:
        assert gates.numel() == T * k and gates.dtype == out.dtype
        gates = gates.contiguous()
    check(
        lib().b200moe_combine(ptr(expanded), expanded.stride(0), ptr(gates), ptr(out), out.stride(0), T, k, out.size(1), dtype_code(out), stream_ptr(out.device)),
        "combine",
    )


# ---- SwiGLU on a fused tensor ---------------------------------------------------------------------


@b200_op("gate_grad", mutates_args={"d_gates"})
def _gate_grad_op(expanded: torch.Tensor, grad: torch.Tensor, d_gates: torch.Tensor, k: int) -> None:
    check(
        lib().b200moe_ep_gate_grad(ptr(expanded), expanded.stride(0), ptr(grad), grad.stride(0), ptr(d_gates), grad.size(0), k, grad.size(1), dtype_code(grad), stream_ptr(grad.device)),
        "gate_grad",
    )


def gate_grad(expanded: torch.Tensor, grad: torch.Tensor, k: int) -> torch.Tensor:
    """d_gates[t, j] = <expanded[t*k + j, :], grad[t, :]> (fp32 sums in a fixed order, stored in the tensor type): the
    gate gradient the reference forms with a batched product
    (cute_kernels/kernels/scattermoe/triton_implementation/ops.py:204)."""
    _require_cuda(expanded, grad)
    _row_major(expanded, "expanded")
    _row_major(grad, "grad")
    d_gates = torch.empty(grad.size(0), k, dtype=grad.dtype, device=grad.device)
    _gate_grad_op(expanded, grad, d_gates, k)
    return d_gates


def swiglu_unchunked_torch(x: torch.Tensor) -> torch.Tensor:
    """Eager definition: first half of the last dimension times silu of the second half."""
    up, gate = x.chunk(2, dim=-1)
    return up * torch.nn.functional.silu(gate)


@b200_op("swiglu_unchunked_forward", mutates_args={"output"})
def _swiglu_forward(x: torch.Tensor, output: torch.Tensor) -> None:
    _require_cuda(x, output)
    h = output.size(1)
    check(lib().b200moe_swiglu_unchunked_forward(ptr(x), x.stride(0), ptr(output), output.stride(0), x.size(0), h, dtype_code(x), stream_ptr(x.device)), "swiglu_unchunked_forward")


@b200_op("swiglu_unchunked_backward", mutates_args={"x_grad"})
def _swiglu_backward(x: torch.Tensor, output_grad: torch.Tensor, x_grad: torch.Tensor) -> None:
    _require_cuda(x, output_grad, x_grad)
    h = output_grad.size(1)
    check(
        lib().b200moe_swiglu_unchunked_backward(ptr(x), x.stride(0), ptr(output_grad), output_grad.stride(0), ptr(x_grad), x_grad.stride(0), x.size(0), h, dtype_code(x), stream_ptr(x.device)),
        "swiglu_unchunked_backward",
    )


class _SwigluUnchunked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        assert shape[-1] % 2 == 0
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        out = torch.empty(x2.size(0), shape[-1] // 2, dtype=x.dtype, device=x.device)
        _swiglu_forward(x2, out)
        ctx.save_for_backward(x2)
        ctx.shape = shape
        return out.view(*shape[:-1], shape[-1] // 2)

    @staticmethod
    def backward(ctx, output_grad: torch.Tensor):
        (x2,) = ctx.saved_tensors
        g = output_grad.reshape(x2.size(0), -1)
        if g.stride(-1) != 1:
            g = g.contiguous()
        x_grad = torch.empty_like(x2)
        _swiglu_backward(x2, g, x_grad)
        return x_grad.view(ctx.shape)


def swiglu_unchunked_cute(x: torch.Tensor, kernel_backend_forward=None, kernel_backend_backward=None, BLOCK_SIZE_B_forward=None, BLOCK_SIZE_H_forward=None, BLOCK_SIZE_B_backward=None, BLOCK_SIZE_H_backward=None) -> torch.Tensor:
    """SwiGLU on a tensor whose last dimension holds [up | gate]; differentiable.

    The tuning keywords of the reference's function are accepted and ignored.
    """
    return _SwigluUnchunked.apply(x)


# ---- RMSNorm ---------------------------------------------------------------------------------------


def rmsnorm_torch(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """Eager definition (cute_kernels/kernels/rmsnorm/torch_implementation.py:5-6)."""
    return torch.nn.functional.rms_norm(x, (x.size(-1),), weight=weight, eps=eps)


@b200_op("rmsnorm_forward", mutates_args={"output", "rstd"})
def _rmsnorm_forward(x: torch.Tensor, weight: torch.Tensor | None, output: torch.Tensor, rstd: torch.Tensor | None, eps: float) -> None:
    _require_cuda(x, weight, output, rstd)
    check(
        lib().b200moe_rmsnorm_forward(ptr(x), x.stride(0), ptr(weight), ptr(output), output.stride(0), ptr(rstd), x.size(0), x.size(1), eps, dtype_code(x), stream_ptr(x.device)),
        "rmsnorm_forward",
    )


@b200_op("rmsnorm_backward", mutates_args={"x_grad", "weight_grad"})
def _rmsnorm_backward(x: torch.Tensor, weight: torch.Tensor | None, output_grad: torch.Tensor, rstd: torch.Tensor | None, x_grad: torch.Tensor, weight_grad: torch.Tensor | None, eps: float) -> None:
    _require_cuda(x, weight, output_grad, rstd, x_grad, weight_grad)
    ws = None
    nbytes = 0
    if weight_grad is not None:
        nbytes = lib().b200moe_rmsnorm_workspace_bytes(x.size(0), x.size(1), dtype_code(x))
        ws = _workspace(x.device, nbytes)
    check(
        lib().b200moe_rmsnorm_backward(
            ptr(x), x.stride(0), ptr(weight), ptr(output_grad), output_grad.stride(0), ptr(rstd), ptr(x_grad), x_grad.stride(0), ptr(weight_grad),
            ptr(ws), nbytes, x.size(0), x.size(1), eps, dtype_code(x), stream_ptr(x.device),
        ),
        "rmsnorm_backward",
    )


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor | None, eps: float | None, memory_efficient: bool) -> torch.Tensor:
        if weight is not None:
            assert weight.dim() == 1, "weight should be 1D"
            assert weight.size(-1) == x.size(-1), "hidden size for x and weight tensor is different"
            assert weight.dtype == x.dtype, "tensors weight and y should have same dtype"
            weight = weight.contiguous()
        if eps is None:
            eps = torch.finfo(x.dtype).eps
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        out = torch.empty(x2.size(0), x2.size(1), dtype=x.dtype, device=x.device)
        if x2.size(0) == 0:
            ctx.save_for_backward(x2, weight, None)
            ctx.shape, ctx.eps = shape, eps
            return out.view(shape)
        rstd = None if memory_efficient else torch.empty(x2.size(0), dtype=torch.float32, device=x.device)
        _rmsnorm_forward(x2, weight, out, rstd, eps)
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape, ctx.eps = shape, eps
        return out.view(shape)

    @staticmethod
    def backward(ctx, output_grad: torch.Tensor):
        x2, weight, rstd = ctx.saved_tensors
        if x2.size(0) == 0:
            return x2.new_empty(ctx.shape), (torch.zeros_like(weight) if weight is not None and ctx.needs_input_grad[1] else None), None, None
        g = output_grad.reshape(x2.shape)
        if g.stride(-1) != 1:
            g = g.contiguous()
        x_grad = torch.empty_like(x2)
        weight_grad = torch.empty_like(weight) if weight is not None and ctx.needs_input_grad[1] else None
        _rmsnorm_backward(x2, weight, g, rstd, x_grad, weight_grad, ctx.eps)
        return x_grad.view(ctx.shape), weight_grad, None, None


def rmsnorm_cute(x: torch.Tensor, weight: torch.Tensor | None, eps: float | None, memory_efficient: bool = False, kernel_backend_forward=None, kernel_backend_backward=None,
                 BLOCK_SIZE_B_forward=None, BLOCK_SIZE_B_backward=None, BLOCK_SIZE_H_forward=None, BLOCK_SIZE_H_backward=None) -> torch.Tensor:
    """RMSNorm over the last dimension; differentiable in x and weight (cute_kernels/kernels/rmsnorm/__init__.py:88-112).

    `memory_efficient=True` does not keep the per-row inverse RMS for the backward pass (it is recomputed from x).
    The tuning keywords of the reference's function are accepted and ignored.
    """
    return _RMSNorm.apply(x, weight, eps, memory_efficient)
