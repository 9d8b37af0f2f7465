"""Parity at the benchmark's full sizes (bf16): the Mixtral-shaped layer (8 experts, top-2, hidden 4096, intermediate
14336, 16384 tokens), the fine-grained layer (64 experts, top-6, 2048 / 1408, 32768 tokens), the Zipf-skewed layer (128
experts, top-8, 2048 / 768, 65536 tokens: empty and very heavy experts) and the per-GPU shape of the 256-expert layer on
eight GPUs (32 experts, 131072 rows, 7168 / 2048).  The CPU oracle cannot run a whole layer of these sizes in seconds, so
it checks exact sub-problems that do not depend on the problem size:
  * output, input-gradient and router-weight-gradient rows of sampled tokens (they depend on that token's row only), and
  * sampled intermediate columns of both weight gradients of chosen experts (they need every row of that expert, but
    only a handful of weight rows / columns): the expert with the most rows and one whose row count leaves an odd
    number of 128-row blocks (the second CTA of a pair then idles through the last block).
"""

import pytest
import torch
import torch.nn.functional as F

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib, synthetic
from oracle import moe_oracle as orc

from helpers import rel_l2

pytestmark = pytest.mark.gpu

CASES = {
    "c2": (synthetic.WORKLOADS["c2"], 40),
    "c3": (synthetic.WORKLOADS["c3"], 24),
    "c4": (synthetic.WORKLOADS["c4"], 24),
    # one rank of the 256-expert layer on eight GPUs: its 32 experts see 16384 * 8 rows
    "c5_per_gpu": (synthetic.scaled(synthetic.WORKLOADS["c5"], num_experts=32, tokens=16384, routing="sigmoid"), 30),
}


def _check_expert_columns(e, cols, x, gy, rw, sel, w_fc, w_proj, dt, I):
    dev = x.device
    rows_t, rows_j = (sel == e).nonzero(as_tuple=True)
    X_e = x.detach()[rows_t].cpu().float()
    G_e = gy[rows_t].cpu().float()
    gate_e = rw.detach()[rows_t, rows_j].cpu().float()
    W1u = w_fc.detach()[e, cols.to(dev)].cpu().float()  # (c, H)
    W1g = w_fc.detach()[e, (cols + I).to(dev)].cpu().float()
    W2c = w_proj.detach()[e][:, cols.to(dev)].cpu().float()  # (H, c)
    bf = lambda t: t.to(dt).float()  # the kernels store these intermediates in the tensor type
    up, gt = bf(X_e @ W1u.t()), bf(X_e @ W1g.t())
    act = bf(up * F.silu(gt))
    sG = bf(gate_e[:, None] * G_e)  # the gate-scaled upstream gradient rows (the reference's group(coeff=gates))
    da = bf(sG @ W2c)
    sg = torch.sigmoid(gt)
    dh_up, dh_gate = bf(da * gt * sg), bf(da * up * (sg + gt * sg * (1 - sg)))
    ref_dw1_up, ref_dw1_gate = dh_up.t() @ X_e, dh_gate.t() @ X_e
    ref_dw2 = sG.t() @ act
    assert rel_l2(w_fc.grad[e, cols.to(dev)], ref_dw1_up) < 1e-2, ("d_w_fc up", e)
    assert rel_l2(w_fc.grad[e, (cols + I).to(dev)], ref_dw1_gate) < 1e-2, ("d_w_fc gate", e)
    assert rel_l2(w_proj.grad[e][:, cols.to(dev)], ref_dw2) < 1e-2, ("d_w_proj", e)


@pytest.mark.parametrize("name", list(CASES))
def test_full_size_sampled_parity(name):
    w, need_gb = CASES[name]
    E, k, H, I, T = w.num_experts, w.top_k, w.hidden, w.intermediate, w.tokens
    dev, dt = torch.device("cuda"), torch.bfloat16
    free, _ = torch.cuda.mem_get_info()
    if free < need_gb * 2**30:
        pytest.skip(f"needs {need_gb} GB of free device memory")
    g = torch.Generator(device="cuda").manual_seed(0)
    w_fc = (torch.randn(E, 2 * I, H, device=dev, generator=g) * w.weight_std).to(dt).requires_grad_(True)
    w_proj = (torch.randn(E, H, I, device=dev, generator=g) * w.weight_std).to(dt).requires_grad_(True)
    gate = (torch.randn(E, H, device=dev, generator=g) * w.weight_std).to(dt)
    x = torch.randn(T, H, device=dev, generator=g).to(dt).requires_grad_(True)
    gy = torch.randn(T, H, device=dev, generator=g).to(dt)
    if w.routing == "gate":
        logits = x.detach().float() @ gate.float().t()
        vals, sel = logits.topk(k, dim=-1)
        rw = torch.softmax(vals, -1)
    else:
        rw, sel = synthetic.make_routing(w, torch.zeros(T, 1), torch.zeros(E, 1), seed=7)
        sel = sel.to(dev)
    rw = rw.to(dev, dt).requires_grad_(True)

    y = kh.fused_swiglu_experts(x, w_fc, w_proj, rw, sel)
    y.backward(gy)
    _lib.check_status(dev)
    for t in (y, x.grad, w_fc.grad, w_proj.grad, rw.grad):
        assert torch.isfinite(t).all()

    counts = sel.flatten().bincount(minlength=E).cpu()
    if w.routing == "zipf":
        assert counts.max() > 8 * counts.float().mean()  # the skew the workload is about

    # --- sampled tokens: y, dx, d_router_weights; only the experts those tokens use are brought to the host ----------
    tok = torch.randperm(T, generator=torch.Generator().manual_seed(1))[:12].to(dev)
    used, sel_c = torch.unique(sel[tok], return_inverse=True)
    w1_cpu, w2_cpu = w_fc.detach()[used].cpu().float(), w_proj.detach()[used].cpu().float()
    xs = x.detach()[tok].cpu().float().requires_grad_(True)
    rws = rw.detach()[tok].cpu().float().requires_grad_(True)
    ys = orc.experts_torch_style(xs, w1_cpu, w2_cpu, rws, sel_c.cpu())
    ys.backward(gy[tok].cpu().float())
    assert rel_l2(y.detach()[tok], ys) < 1e-2
    assert rel_l2(x.grad[tok], xs.grad) < 1e-2
    assert rel_l2(rw.grad[tok], rws.grad) < 1e-2
    del w1_cpu, w2_cpu

    # --- sampled columns of the weight gradients: heaviest expert, an odd-block expert, an empty one if there is one ---
    cols = torch.tensor([0, 77, I // 2 + 5, I - 1])
    heavy = int(counts.argmax())
    blocks = (counts + 127) // 128
    odd = [int(e) for e in torch.nonzero((blocks % 2 == 1) & (counts > 0)).flatten().tolist() if int(e) != heavy]
    experts = [heavy] + odd[:1]
    for e in experts:
        _check_expert_columns(e, cols, x, gy, rw, sel, w_fc, w_proj, dt, I)
    for e in torch.nonzero(counts == 0).flatten().tolist()[:2]:
        assert float(w_fc.grad[e].abs().max()) == 0.0 and float(w_proj.grad[e].abs().max()) == 0.0
