"""Fused router kernel against the eager router (cute_kernels/kernels/scattermoe/torch_implementation.py:120-133,193-199)
and the CPU oracle.

Integer outputs are checked bit-exactly against the kernel's own logits (the selection must be the stable descending
top-k of the logits it stored; counts must be the histogram of its selection); the logits against an fp32 product
rounded to the tensor type; the weights against the eager formula on the selected logits.
"""

import pytest
import torch

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib
from kernel_hyperdrive_b200.router import fused_router
from helpers import rel_l2
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

CASES = [
    # T, H, E, k, dtype, scoring
    (1000, 4096, 8, 2, torch.bfloat16, "softmax"),   # Mixtral-shaped, ragged last tile
    (4096, 2048, 64, 6, torch.bfloat16, "softmax"),
    (777, 2048, 128, 8, torch.bfloat16, "softmax"),
    (300, 7168, 256, 8, torch.bfloat16, "sigmoid"),  # two weight boxes
    (513, 264, 12, 1, torch.float16, "softmax"),     # expert count not a multiple of 8, k = 1, ragged k extent
    (130, 512, 136, 3, torch.float16, "sigmoid"),
    (1, 256, 16, 4, torch.bfloat16, "softmax"),
]


def make(T, H, E, dtype, seed, std=0.02):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(dtype).cuda()
    w = (torch.randn(E, H, generator=g) * std).to(dtype).cuda()
    return x, w


def eager_scores(vals, scoring, dtype):
    if scoring == "sigmoid":
        s = torch.sigmoid(vals.float())
        return (s / s.sum(-1, keepdim=True)).to(dtype)
    return torch.softmax(vals.float(), dim=-1).to(dtype)


@pytest.mark.parametrize("T,H,E,k,dtype,scoring", CASES)
def test_router_forward(T, H, E, k, dtype, scoring):
    x, w = make(T, H, E, dtype, seed=T + E)
    before = _lib.lib().b200moe_launch_count()
    logits, weights, idx, counts = fused_router(x, w, k, scoring)
    torch.cuda.synchronize()
    _lib.check_status(x.device)
    assert _lib.lib().b200moe_launch_count() - before == 1
    assert logits.shape == (T, E) and weights.shape == (T, k) and idx.shape == (T, k) and idx.dtype == torch.int64
    # logits: fp32 product rounded once to the tensor type; summation order may move a value by one unit in the last place
    ref = (x.float() @ w.float().t()).to(dtype)
    same = (ref == logits).float().mean().item()
    assert same >= 0.98, same
    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    assert ((ref.float() - logits.float()).abs() <= ulp * ref.float().abs() + 1e-4).all()  # 1e-4: fp32 summation order
    # selection: bit-exact stable descending top-k of the stored logits
    order = torch.sort(logits.float(), dim=-1, descending=True, stable=True).indices[:, :k]
    assert torch.equal(order, idx)
    # histogram of the selection
    assert torch.equal(counts.long(), torch.bincount(idx.flatten(), minlength=E))
    assert counts.dtype == torch.int32
    # weights: eager formula on the selected logits, one rounding to the tensor type
    want = eager_scores(logits.gather(1, idx), scoring, dtype)
    assert ((want.float() - weights.float()).abs() <= 2 * ulp * want.float().abs() + 1e-7).all()
    assert (weights.float().sum(-1) - 1).abs().max().item() <= 4 * ulp * k


def test_router_against_cpu_oracle():
    # the oracle routes in fp32; where its top-k gap is wider than the 16-bit rounding the selections must agree
    T, H, E, k = 512, 1024, 32, 4
    x, w = make(T, H, E, torch.bfloat16, seed=5, std=0.05)
    logits, weights, idx, _ = fused_router(x, w, k, "softmax")
    o_logits, o_w, o_idx = orc.routing_weights(x.cpu().float(), w.cpu().float(), k)
    assert rel_l2(logits, o_logits) <= 1e-2
    srt = o_logits.sort(dim=-1, descending=True).values
    gaps = (srt[:, :k] - srt[:, 1 : k + 1]).min(dim=-1).values  # smallest gap among the first k + 1 logits
    clear = gaps > 0.02 * srt[:, 0].abs().clamp(min=1.0)
    assert clear.float().mean().item() > 0.2
    assert torch.equal(idx.cpu()[clear], o_idx[clear])
    assert rel_l2(weights.cpu()[clear], o_w[clear]) <= 1e-2


def test_equal_logits_pick_the_lower_expert():
    T, H, E, k = 256, 512, 16, 4
    x, w = make(T, H, E, torch.bfloat16, seed=9)
    w[5] = w[3]
    w[11] = w[3]
    w[0] = w[14]
    logits, _, idx, counts = fused_router(x, w, k, "softmax")
    assert torch.equal(logits[:, 5], logits[:, 3]) and torch.equal(logits[:, 11], logits[:, 3])
    order = torch.sort(logits.float(), dim=-1, descending=True, stable=True).indices[:, :k]
    assert torch.equal(order, idx)
    has3, has5, has11 = (idx == 3).any(-1), (idx == 5).any(-1), (idx == 11).any(-1)
    assert (~has5 | has3).all() and (~has11 | has5).all()  # a copy is selected only after the lower-numbered one
    assert torch.equal(counts.long(), torch.bincount(idx.flatten(), minlength=E))


def test_empty_batch_and_bad_arguments():
    x, w = make(0, 256, 8, torch.bfloat16, seed=1)
    logits, weights, idx, counts = fused_router(x, w, 2, "softmax")
    assert logits.shape == (0, 8) and idx.shape == (0, 2) and counts.sum().item() == 0
    x, w = make(4, 256, 8, torch.float32, seed=1)
    with pytest.raises(RuntimeError, match="16-bit"):
        fused_router(x, w, 2, "softmax")
    x, w = make(4, 256, 8, torch.bfloat16, seed=1)
    with pytest.raises(RuntimeError):
        fused_router(x, w, 9, "softmax")
    x, w = make(4, 260, 8, torch.bfloat16, seed=1)  # rows of 520 bytes: not a multiple of 16
    with pytest.raises(RuntimeError, match="16-byte"):
        fused_router(x, w, 2, "softmax")


@pytest.mark.parametrize("scoring", ["softmax", "sigmoid"])
def test_router_backward_matches_eager(scoring):
    T, H, E, k = 640, 1024, 64, 6
    x, w = make(T, H, E, torch.bfloat16, seed=21, std=0.05)
    x.requires_grad_(True)
    w.requires_grad_(True)
    ga = torch.randn(T, k, device="cuda").to(torch.bfloat16)
    gb = (torch.randn(T, E, device="cuda") * 0.1).to(torch.bfloat16)
    logits, weights, idx, _ = fused_router(x, w, k, scoring)
    ((weights * ga).sum() + (logits * gb).sum()).backward()
    dx, dw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    # eager router in fp32 with the same selection
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lf = xf @ wf.t()
    wts = eager_scores(lf.gather(1, idx), scoring, torch.float32)
    ((wts * ga.float()).sum() + (lf * gb.float()).sum()).backward()
    assert rel_l2(dx, xf.grad) <= 1e-2 and rel_l2(dw, wf.grad) <= 1e-2


def test_layer_with_fused_router():
    torch.manual_seed(3)
    moe = kh.MoE_B200(8, 2, 512, 768, kh.swiglu_unchunked_torch, True, False, 0.05).cuda().to(torch.bfloat16)
    x = torch.randn(4, 200, 512, device="cuda", dtype=torch.bfloat16)
    y_eager, logits_eager = moe(x)
    _, _, sel_eager = moe._compute_routing_weights(x.view(-1, 512))
    moe.fused_router = True
    before = _lib.lib().b200moe_launch_count()
    y_fused, logits_fused = moe(x)
    assert _lib.lib().b200moe_launch_count() - before >= 6  # router + routing sort + expert kernels
    _, _, sel_fused = moe._compute_routing_weights(x.view(-1, 512))
    agree = (sel_eager.sort(-1).values == sel_fused.sort(-1).values).all(-1)
    assert agree.float().mean().item() >= 0.98
    assert rel_l2(logits_fused, logits_eager) <= 1e-2
    assert rel_l2(y_fused.view(-1, 512)[agree], y_eager.view(-1, 512)[agree]) <= 1e-2
    # gradients flow through the fused router to the gate weight
    xg = x.clone().requires_grad_(True)
    y, _ = moe(xg)
    y.float().pow(2).sum().backward()
    assert moe.gate.weight.grad is not None and moe.gate.weight.grad.abs().sum().item() > 0
    assert xg.grad is not None and torch.isfinite(xg.grad).all()


def test_router_backward_with_few_experts_runs_on_the_grouped_gemm_operators():
    """Eight experts: the logit gradient is an (T, 8) operand, a reduction extent far below one k step of the tensor-core
    kernels (the rest of the step reads as zeros)."""
    T, H, E, k = 1111, 4096, 8, 2
    x, w = make(T, H, E, torch.bfloat16, seed=33, std=0.05)
    x.requires_grad_(True)
    w.requires_grad_(True)
    gb = (torch.randn(T, E, device="cuda") * 0.1).to(torch.bfloat16)
    before = _lib.lib().b200moe_launch_count()
    logits, _, _, _ = fused_router(x, w, k, "softmax")
    (logits * gb).sum().backward()
    assert _lib.lib().b200moe_launch_count() - before >= 3  # router, input-gradient GEMM, weight-gradient GEMM (+ index kernels)
    _lib.check_status(x.device)
    assert rel_l2(x.grad, gb.float() @ w.detach().float()) <= 1e-2
    assert rel_l2(w.grad, gb.float().t() @ x.detach().float()) <= 1e-2


def test_unsupported_layouts_take_the_eager_router():
    from kernel_hyperdrive_b200.router import fused_router_supported

    x, w = make(64, 512, 8, torch.bfloat16, seed=2)
    assert fused_router_supported(x, 8, 2, w)
    wide = torch.zeros(64, 520, device="cuda", dtype=torch.bfloat16)
    assert not fused_router_supported(wide[:, 4:516], 8, 2, w)  # rows start 8 bytes off a 16-byte boundary
    assert not fused_router_supported(x, 8, 2, w.float())
    assert not fused_router_supported(x.t().contiguous().t(), 8, 2, w)  # inner stride is not 1
    moe = kh.MoE_B200(8, 2, 512, 256, kh.swiglu_unchunked_torch, True, False, 0.05).cuda().to(torch.bfloat16)
    moe.fused_router = True
    y, _ = moe(wide[:, 4:516].unsqueeze(0).contiguous())  # contiguous copy: supported again
    assert torch.isfinite(y).all()


@pytest.mark.parametrize("T,H,E,k", [(900, 2048, 64, 6), (257, 4096, 8, 2)])
def test_rmsnorm_fused_with_the_gate_projection(T, H, E, k):
    """RMSNorm feeding the layer with its normalisation folded into the router GEMM (per-row factor in the epilogue,
    norm weight folded into the gate weight): against the eager sequence rms_norm -> linear -> top-k -> softmax."""
    from kernel_hyperdrive_b200.router import fused_rmsnorm_router

    dt, eps = torch.bfloat16, 1e-5
    x, w = make(T, H, E, dt, seed=T, std=0.05)
    x = (x * 3).requires_grad_(True)
    w.requires_grad_(True)
    nw = (1 + 0.1 * torch.randn(H, device="cuda")).to(dt).requires_grad_(True)
    gy = torch.randn(T, H, device="cuda").to(dt)
    gl = (torch.randn(T, E, device="cuda") * 0.1).to(dt)
    before = _lib.lib().b200moe_launch_count()
    y, logits, weights, idx, counts = fused_rmsnorm_router(x, nw, w, eps, k)
    assert _lib.lib().b200moe_launch_count() - before == 2  # the norm kernel and the router kernel
    ((y * gy).sum() + (logits * gl).sum()).backward()
    _lib.check_status(x.device)
    got = (y.detach(), logits.detach(), x.grad.clone(), w.grad.clone(), nw.grad.clone())
    # eager, fp32
    xf, wf, nf = (t.detach().float().requires_grad_(True) for t in (x, w, nw))
    yf = torch.nn.functional.rms_norm(xf, (H,), nf, eps)
    lf = yf @ wf.t()
    ((yf * gy.float()).sum() + (lf * gl.float()).sum()).backward()
    for name, a, b in zip(("y", "logits", "dx", "d_gate", "d_norm"), got, (yf, lf, xf.grad, wf.grad, nf.grad)):
        assert rel_l2(a, b) <= 1e-2, (name, rel_l2(a, b))
    # selection: stable top-k of the stored logits, histogram of the selection, weights from the selected logits
    assert torch.equal(torch.sort(logits.float(), dim=-1, descending=True, stable=True).indices[:, :k], idx)
    assert torch.equal(counts.long(), torch.bincount(idx.flatten(), minlength=E))
    assert rel_l2(weights, eager_scores(logits.gather(1, idx), "softmax", dt)) <= 1e-2
