"""RMSNorm kernels against the CPU oracle and the golden vectors of the reference's eager definition
(cute_kernels/kernels/rmsnorm/torch_implementation.py:5-6; test matrix modelled on tests/kernels/rmsnorm_test.py:18-72:
1-D and 2-D sizes, fp32 and 16-bit, with and without weight, with and without the stored inverse RMS)."""

import os

import numpy as np
import pytest
import torch

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib
from helpers import rel_l2
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
EPS = 1e-5

SIZES = [(7,), (400,), (1, 8), (5, 3, 40), (33, 256), (64, 1000), (130, 1024), (257, 2048), (96, 4096), (40, 7168), (9, 16384), (3, 16392), (50, 7)]


def tol(dtype):
    return 2e-6 if dtype == torch.float32 else 1e-2


@pytest.mark.parametrize("size", SIZES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("has_weight", [True, False])
@pytest.mark.parametrize("memory_efficient", [True, False])
def test_rmsnorm_matches_oracle(size, dtype, has_weight, memory_efficient):
    g = torch.Generator().manual_seed(len(size) * 1000 + size[-1])
    x_cpu = torch.randn(size, generator=g).to(dtype)
    w_cpu = (torch.randn(size[-1], generator=g) * 0.5 + 1).to(dtype) if has_weight else None
    dy_cpu = torch.randn(size, generator=g).to(dtype)
    x = x_cpu.cuda().requires_grad_(True)
    w = w_cpu.cuda().requires_grad_(True) if has_weight else None
    before = _lib.lib().b200moe_launch_count()
    y = kh.rmsnorm_cute(x=x, weight=w, eps=EPS, memory_efficient=memory_efficient)
    y.backward(dy_cpu.cuda())
    assert _lib.lib().b200moe_launch_count() - before == (3 if has_weight else 2)
    xf, wf, dyf = x_cpu.float(), (w_cpu.float() if has_weight else None), dy_cpu.float()
    want_y = orc.rmsnorm(xf, wf, EPS)
    want_dx, want_dw = orc.rmsnorm_backward(xf, wf, dyf, EPS)
    assert y.shape == x.shape and y.dtype == dtype
    assert rel_l2(y, want_y) <= tol(dtype)
    assert rel_l2(x.grad, want_dx) <= tol(dtype)
    if has_weight:
        assert w.grad.shape == w.shape
        assert rel_l2(w.grad, want_dw) <= tol(dtype)


def test_rmsnorm_golden_vectors(golden_dir):
    gold = np.load(os.path.join(golden_dir, "rmsnorm.npz"))
    for tag, has_weight in (("w", True), ("nw", False), ("odd", True)):
        x = torch.from_numpy(gold[f"{tag}_x"]).cuda().requires_grad_(True)
        w = torch.from_numpy(gold[f"{tag}_w"]).cuda().requires_grad_(True) if has_weight else None
        y = kh.rmsnorm_cute(x, w, EPS)
        y.backward(torch.from_numpy(gold[f"{tag}_dy"]).cuda())
        assert rel_l2(y, gold[f"{tag}_y"]) <= 2e-6 and rel_l2(x.grad, gold[f"{tag}_dx"]) <= 2e-6
        if has_weight:
            assert rel_l2(w.grad, gold[f"{tag}_dw"]) <= 2e-6


def test_rmsnorm_default_eps_strided_rows_and_determinism():
    torch.manual_seed(4)
    base = torch.randn(300, 2 * 1024, device="cuda", dtype=torch.bfloat16)
    x = base[:, :1024].detach().requires_grad_(True)  # row stride 2048: no copy is made
    w = torch.randn(1024, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    y = kh.rmsnorm_cute(x, w, None)
    want = kh.rmsnorm_torch(x.float(), w.float(), torch.finfo(torch.bfloat16).eps)
    assert rel_l2(y, want) <= 1e-2
    dy = torch.randn_like(y)
    grads = []
    for _ in range(2):
        x.grad = w.grad = None
        kh.rmsnorm_cute(x, w, None).backward(dy)
        grads.append((x.grad.clone(), w.grad.clone()))
    assert torch.equal(grads[0][0], grads[1][0]) and torch.equal(grads[0][1], grads[1][1])  # fixed summation order


def test_rmsnorm_empty_and_errors():
    x = torch.empty(0, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = kh.rmsnorm_cute(x, w, EPS)
    assert y.shape == (0, 64)
    y.sum().backward()
    assert w.grad.abs().sum().item() == 0
    with pytest.raises(AssertionError):
        kh.rmsnorm_cute(torch.randn(4, 64, device="cuda"), torch.ones(32, device="cuda"), EPS)
    with pytest.raises(RuntimeError):
        kh.rmsnorm_cute(torch.randn(4, 64), None, EPS)  # CPU tensor: no CPU path


def test_rmsnorm_feeds_the_layer_under_compile():
    torch.manual_seed(5)
    moe = kh.MoE_B200(8, 2, 256, 384, kh.swiglu_unchunked_torch, True, False, 0.02).cuda()
    w = torch.ones(256, device="cuda", requires_grad=True)

    def block(x):
        return x + moe(kh.rmsnorm_cute(x, w, EPS))[0]

    x = torch.randn(2, 50, 256, device="cuda", requires_grad=True)
    want = block(x)
    torch._dynamo.reset()
    kh.set_cute_tracing(True)
    try:
        got = torch.compile(block, fullgraph=True)(x)
    finally:
        kh.set_cute_tracing(False)
    assert rel_l2(got, want) <= 1e-5
