"""Parity at the benchmark's full size (Mixtral-shaped layer: 8 experts, top-2, hidden 4096, intermediate
14336, 16384 tokens, bf16).  The CPU oracle cannot run the whole layer in seconds, so it checks exact
sub-problems that do not depend on the problem size:
  * output and input-gradient rows of sampled tokens (they depend on that token's row only), and
  * sampled intermediate columns of both weight gradients of one expert (they need every row of that
    expert, but only a handful of weight rows / columns).
"""

import pytest
import torch
import torch.nn.functional as F

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib, synthetic
from oracle import moe_oracle as orc

from helpers import rel_l2

pytestmark = pytest.mark.gpu


def test_mixtral_shape_sampled_parity():
    w = synthetic.WORKLOADS["c2"]
    E, k, H, I, T = w.num_experts, w.top_k, w.hidden, w.intermediate, w.tokens
    dev, dt = torch.device("cuda"), torch.bfloat16
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * 2**30:
        pytest.skip("needs 40 GB of free device memory")
    g = torch.Generator(device="cuda").manual_seed(0)
    w_fc = (torch.randn(E, 2 * I, H, device=dev, generator=g) * w.weight_std).to(dt).requires_grad_(True)
    w_proj = (torch.randn(E, H, I, device=dev, generator=g) * w.weight_std).to(dt).requires_grad_(True)
    gate = (torch.randn(E, H, device=dev, generator=g) * w.weight_std).to(dt)
    x = torch.randn(T, H, device=dev, generator=g).to(dt).requires_grad_(True)
    gy = torch.randn(T, H, device=dev, generator=g).to(dt)
    logits = x.detach().float() @ gate.float().t()
    vals, sel = logits.topk(k, dim=-1)
    rw = torch.softmax(vals, -1).to(dt).requires_grad_(True)

    y = kh.fused_swiglu_experts(x, w_fc, w_proj, rw, sel)
    y.backward(gy)
    _lib.check_status(dev)
    for t in (y, x.grad, w_fc.grad, w_proj.grad, rw.grad):
        assert torch.isfinite(t).all()

    # --- sampled tokens: y, dx, d_router_weights -------------------------------------------------
    tok = torch.randperm(T, generator=torch.Generator().manual_seed(1))[:12]
    w1_cpu, w2_cpu = w_fc.detach().cpu().float(), w_proj.detach().cpu().float()
    xs = x.detach()[tok.to(dev)].cpu().float().requires_grad_(True)
    rws = rw.detach()[tok.to(dev)].cpu().float().requires_grad_(True)
    ys = orc.experts_torch_style(xs, w1_cpu, w2_cpu, rws, sel[tok.to(dev)].cpu())
    ys.backward(gy[tok.to(dev)].cpu().float())
    assert rel_l2(y.detach()[tok.to(dev)], ys) < 1e-2
    assert rel_l2(x.grad[tok.to(dev)], xs.grad) < 1e-2
    assert rel_l2(rw.grad[tok.to(dev)], rws.grad) < 1e-2
    del w1_cpu, w2_cpu

    # --- sampled columns of the weight gradients of one expert ------------------------------------
    e = 5
    cols = torch.tensor([0, 77, 8191, I - 1])
    slot_mask = sel == e  # (T, k)
    rows_t, rows_j = slot_mask.nonzero(as_tuple=True)
    X_e = x.detach()[rows_t].cpu().float()
    G_e = gy[rows_t].cpu().float()
    gate_e = rw.detach()[rows_t, rows_j].cpu().float()
    W1u = w_fc.detach()[e, cols.to(dev)].cpu().float()  # (c, H)
    W1g = w_fc.detach()[e, (cols + I).to(dev)].cpu().float()
    W2c = w_proj.detach()[e][:, cols.to(dev)].cpu().float()  # (H, c)
    bf = lambda t: t.to(dt).float()  # the kernels store these intermediates in bf16
    up, gt = bf(X_e @ W1u.t()), bf(X_e @ W1g.t())
    act = bf(up * F.silu(gt))
    da = bf(gate_e[:, None] * (G_e @ W2c))
    sg = torch.sigmoid(gt)
    dh_up, dh_gate = bf(da * gt * sg), bf(da * up * (sg + gt * sg * (1 - sg)))
    ref_dw1_up, ref_dw1_gate = dh_up.t() @ X_e, dh_gate.t() @ X_e
    ref_dw2 = G_e.t() @ bf(gate_e[:, None] * act)
    assert rel_l2(w_fc.grad[e, cols.to(dev)], ref_dw1_up) < 1e-2
    assert rel_l2(w_fc.grad[e, (cols + I).to(dev)], ref_dw1_gate) < 1e-2
    assert rel_l2(w_proj.grad[e][:, cols.to(dev)], ref_dw2) < 1e-2
