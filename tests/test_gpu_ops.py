"""The four reference-signature operators and the row-wise kernels against the CPU oracle, on both
engines (CUDA cores for every dtype, tcgen05 for bf16 / fp16)."""

import os

import numpy as np
import pytest
import torch

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib
from oracle import moe_oracle as orc

from conftest import GOLDEN
from helpers import rel_l2, tolerance

pytestmark = pytest.mark.gpu

ENGINES = [("simt", torch.float32), ("simt", torch.bfloat16), ("umma", torch.bfloat16), ("umma", torch.float16), ("umma1", torch.bfloat16)]


@pytest.fixture(autouse=True)
def _engine_reset():
    yield
    _lib.set_engine(_lib.ENGINE_AUTO)
    _lib.check_status(torch.device("cuda"))


def use_engine(name):
    _lib.set_engine({"simt": _lib.ENGINE_SIMT, "umma": _lib.ENGINE_UMMA, "umma1": _lib.ENGINE_UMMA_1CTA, "gather4": _lib.ENGINE_UMMA_GATHER4, "auto": _lib.ENGINE_AUTO}[name])


def routed(E, k, T, seed, empty_from=None):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    if empty_from is not None:
        ids[ids >= empty_from] = 0
    se, ss, off, cnt = orc.route(ids.numpy(), E)
    return ids, torch.from_numpy(se), torch.from_numpy(ss), torch.from_numpy(off)


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("engine,dtype", ENGINES)
@pytest.mark.parametrize("E,k,T,K,N", [(4, 2, 48, 64, 128), (8, 2, 300, 256, 512), (6, 1, 19, 40, 24), (16, 4, 257, 136, 264), (3, 2, 700, 512, 72)])
@pytest.mark.parametrize("x_grouped,y_grouped", [(False, True), (True, False), (True, True), (False, False)])
def test_scatter2scatter(engine, dtype, E, k, T, K, N, x_grouped, y_grouped):
    use_engine(engine)
    ids, se, ss, off = routed(E, k, T, seed=E + T, empty_from=E - 1 if E > 4 else None)
    M = T * k
    fan_out = 1 if x_grouped else k
    X = rnd((M if x_grouped else T, K), dtype, 1)
    W_stored = rnd((E, N, K), dtype, 2, 0.05)  # (E, out, in) as the module stores it
    for orient in ("k_contiguous", "n_contiguous"):
        if orient == "k_contiguous":
            W = W_stored.permute(0, 2, 1)  # (E, K, N) view with unit stride along K
        else:
            W = W_stored.permute(0, 2, 1).contiguous()  # (E, K, N) with unit stride along N
        ref = orc.scatter2scatter(X.float(), W.float(), se, ss, fan_out, x_grouped, y_grouped)
        out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        Wd = W_stored.cuda().permute(0, 2, 1) if orient == "k_contiguous" else W.cuda()
        kh.scatter2scatter(X.cuda(), Wd, se.cuda(), ss.cuda(), out, fan_out, x_grouped, y_grouped)
        assert torch.isfinite(out).all()
        assert rel_l2(out, ref) < tolerance(dtype), (orient, rel_l2(out, ref))


@pytest.mark.parametrize("engine,dtype", ENGINES)
@pytest.mark.parametrize("E,k,T,K,N", [(4, 2, 48, 64, 128), (8, 2, 300, 256, 512), (6, 1, 19, 40, 24), (16, 4, 257, 136, 264), (2, 2, 1500, 320, 72)])
def test_group_bwd_W(engine, dtype, E, k, T, K, N):
    use_engine(engine)
    ids, se, ss, off = routed(E, k, T, seed=E * 3 + T, empty_from=E - 1 if E > 4 else None)
    M = T * k
    X, DY = rnd((M, K), dtype, 3), rnd((M, N), dtype, 4)
    ref = orc.group_bwd_W(DY.float(), X.float(), off, E)  # (E, K, N)
    # as the autograd function allocates it: strides of the permuted weight view (unit stride along K)
    DW = torch.full((E, N, K), float("nan"), dtype=dtype, device="cuda").permute(0, 2, 1)
    kh.group_bwd_W(DY.cuda(), X.cuda(), off.cuda(), DW, E)
    assert torch.isfinite(DW).all() and rel_l2(DW, ref) < tolerance(dtype), rel_l2(DW, ref)
    DW2 = torch.full((E, K, N), float("nan"), dtype=dtype, device="cuda")
    kh.group_bwd_W(DY.cuda(), X.cuda(), off.cuda(), DW2, E)
    assert torch.isfinite(DW2).all() and rel_l2(DW2, ref) < tolerance(dtype), rel_l2(DW2, ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("k,T,K", [(2, 48, 64), (1, 19, 40), (4, 257, 136), (2, 100, 33)])
def test_group_and_combine(dtype, k, T, K):
    ids, se, ss, off = routed(8, k, T, seed=T)
    M = T * k
    A, coeff = rnd((T, K), dtype, 5), rnd((M,), dtype, 6)
    for c in (None, coeff):
        out = torch.empty(M, K, dtype=dtype, device="cuda")
        kh.group(A.cuda(), ss.cuda(), out, None if c is None else c.cuda(), k)
        ref = orc.group(A.float(), ss, None if c is None else c.float(), k)
        assert rel_l2(out, ref) < (1e-6 if dtype == torch.float32 else 5e-3)
    Y = rnd((M, K), dtype, 7)
    gates = rnd((T, k), dtype, 8)
    for gt in (None, gates):
        out = torch.empty(T, K, dtype=dtype, device="cuda")
        kh.combine(Y.cuda(), None if gt is None else gt.cuda(), out, k)
        y3 = Y.float().view(T, k, K)
        ref = y3.sum(1) if gt is None else torch.bmm(gt.float().unsqueeze(1), y3).squeeze(1)
        assert rel_l2(out, ref) < (1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,h", [(37, 24), (1, 8), (300, 1408), (64, 513), (129, 4096)])
def test_swiglu_unchunked(dtype, rows, h):
    x = rnd((rows, 2 * h), dtype, rows + h).cuda().requires_grad_(True)
    dy = rnd((rows, h), dtype, 9).cuda()
    y = kh.swiglu_unchunked_cute(x)
    y.backward(dy)
    ref = orc.swiglu_unchunked(x.detach().cpu().float())
    ref_dx = orc.swiglu_unchunked_backward(x.detach().cpu().float(), dy.cpu().float())
    tol = 5.5e-6 if dtype == torch.float32 else 5e-3
    assert (y.detach().cpu().float() - ref).abs().max() < (tol if dtype == torch.float32 else 0.1)
    assert rel_l2(y, ref) < tol and rel_l2(x.grad, ref_dx) < tol


def test_swiglu_golden():
    gold = dict(np.load(os.path.join(GOLDEN, "swiglu.npz")))
    x = torch.from_numpy(gold["x"]).cuda().requires_grad_(True)
    y = kh.swiglu_unchunked_cute(x)
    y.backward(torch.from_numpy(gold["dy"]).cuda())
    assert np.abs(y.detach().cpu().numpy() - gold["y"]).max() < 5.5e-6
    assert np.abs(x.grad.cpu().numpy() - gold["dx"]).max() < 5e-6


def test_engine_umma_rejects_fp32():
    use_engine("umma")
    ids, se, ss, off = routed(4, 2, 16, seed=0)
    with pytest.raises(RuntimeError, match="tcgen05"):
        kh.scatter2scatter(torch.zeros(16, 64, device="cuda"), torch.zeros(4, 64, 64, device="cuda"), se.cuda(), ss.cuda(), torch.zeros(32, 64, device="cuda"), 2)


def test_shape_assertions_like_the_reference():
    ids, se, ss, off = routed(4, 2, 16, seed=0)
    with pytest.raises(AssertionError):
        kh.scatter2scatter(torch.zeros(15, 64, device="cuda"), torch.zeros(4, 64, 64, device="cuda"), se.cuda(), ss.cuda(), torch.zeros(32, 64, device="cuda"), 2)
    with pytest.raises(AssertionError):
        kh.group(torch.zeros(15, 64, device="cuda"), ss.cuda(), torch.zeros(32, 64, device="cuda"), None, 2)


@pytest.mark.parametrize("E,k,T,K,N", [(8, 2, 300, 256, 512), (5, 3, 333, 136, 200)])
def test_tma_row_gather_engine(E, k, T, K, N):
    """Operands picked by a row map fetched with TMA row gather (tile::gather4) in the two-CTA kernel: same results as
    the default engine (which gathers with cp.async in the one-CTA kernel), for the gathered forward GEMM and the
    weight gradient with a gathered operand."""
    ids, se, ss, off = routed(E, k, T, seed=11)
    M = T * k
    X = rnd((T, K), torch.bfloat16, 1).cuda()
    W = rnd((E, N, K), torch.bfloat16, 2, 0.05).cuda().permute(0, 2, 1)
    outs = []
    for eng in ("umma", "gather4"):
        use_engine(eng)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        kh.scatter2scatter(X, W, se.cuda(), ss.cuda(), out, k, False, True)
        outs.append(out)
    assert torch.isfinite(outs[1]).all() and torch.equal(outs[0], outs[1])
    from kernel_hyperdrive_b200 import scattermoe as sm

    flat = ids.flatten().cuda()
    _, _, offs, _, row_token, row_slot = kh.route(flat, E, k, False, True)
    cap = row_token.numel()
    Q = rnd((cap, N), torch.bfloat16, 3).cuda()
    Q[row_token < 0] = 0
    grads = []
    for eng in ("umma", "gather4"):
        use_engine(eng)
        dw = torch.full((E, K, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        sm._wgrad(X, row_token, Q, None, offs, dw, cap)
        grads.append(dw)
    assert torch.isfinite(grads[1]).all() and rel_l2(grads[1], grads[0]) < 1e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,k,H", [(1, 1, 8), (333, 2, 512), (64, 6, 2048), (0, 2, 64)])
def test_gate_grad_row_dots(dtype, T, k, H):
    """Gate gradient of the expert-parallel return path: row dots against the bmm of the reference
    (cute_kernels/kernels/scattermoe/triton_implementation/ops.py:204)."""
    from kernel_hyperdrive_b200.ops import gate_grad as _gate_grad

    torch.manual_seed(T + k)
    expanded = torch.randn(T * k, H, device="cuda").to(dtype)
    grad = torch.randn(T, H, device="cuda").to(dtype)
    got = _gate_grad(expanded, grad, k)
    assert got.shape == (T, k) and got.dtype == dtype
    want = torch.bmm(expanded.float().view(T, k, H), grad.float().unsqueeze(2)).squeeze(-1)
    if T:
        assert rel_l2(got, want) <= tolerance(dtype)
