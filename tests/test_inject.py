"""Graph-level and module-level injection (`kernel_hyperdrive_b200/inject.py`).

CPU part: the graph rewrite and the module swap are host logic.  GPU part: a compiled function whose SwiGLU was
replaced, and a model whose MoE layers were swapped, agree with the eager torch definitions.
"""

import operator

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.fx import symbolic_trace

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import inject
from helpers import rel_l2


def mlp_act(x):
    up, gate = x.chunk(2, dim=-1)
    return up * F.silu(gate)


def mlp_act_swapped_operands(x):
    parts = torch.chunk(x, 2, dim=-1)
    return torch.mul(F.silu(parts[1]), parts[0]) + 1.0


def not_swiglu_three_chunks(x):
    a, b, c = x.chunk(3, dim=-1)
    return a * F.silu(b) + c


def not_swiglu_first_dim(x):
    up, gate = x.chunk(2, dim=0)
    return up * F.silu(gate)


def not_swiglu_gate_reused(x):
    up, gate = x.chunk(2, dim=-1)
    return up * F.silu(gate) + gate


def not_swiglu_silu_on_up(x):
    up, gate = x.chunk(2, dim=-1)
    return F.silu(up) * gate


def rewrite(fn):
    gm = symbolic_trace(fn)
    changed = sum(bool(inject.replace_swiglu_unchunked(gm, n)) for n in list(gm.graph.nodes) if not n._erased)
    gm.graph.lint()
    gm.recompile()
    return gm, changed


def targets(gm):
    return [n.target for n in gm.graph.nodes if n.op in ("call_function", "call_method")]


@pytest.mark.parametrize("fn", [mlp_act, mlp_act_swapped_operands])
def test_swiglu_pattern_is_replaced(fn):
    gm, changed = rewrite(fn)
    assert changed == 1
    t = targets(gm)
    assert kh.swiglu_unchunked_cute in t
    assert F.silu not in t and "chunk" not in t and torch.chunk not in t and operator.getitem not in t


@pytest.mark.parametrize("fn", [not_swiglu_three_chunks, not_swiglu_first_dim, not_swiglu_gate_reused])
def test_other_patterns_are_left_alone(fn):
    gm, changed = rewrite(fn)
    assert changed == 0
    assert kh.swiglu_unchunked_cute not in targets(gm)
    x = torch.randn(6, 12)
    assert torch.equal(gm(x), fn(x))


def test_silu_on_first_half_is_not_the_fused_operator():
    # silu(up) * gate is a GLU variant with the halves exchanged; the fused operator applies silu to the second half
    gm, changed = rewrite(not_swiglu_silu_on_up)
    assert changed == 0


class Block(nn.Module):
    def __init__(self, moe):
        super().__init__()
        self.norm = nn.LayerNorm(moe.hidden_size)
        self.moe = moe

    def forward(self, x):
        y, logits = self.moe(self.norm(x))
        return x + y, logits


def test_swap_moe_modules_adopts_parameters():
    torch.manual_seed(0)
    model = nn.Sequential()
    model.add_module("a", Block(kh.MoE_Torch(4, 2, 16, 32, kh.swiglu_unchunked_torch, True, False, 0.02)))
    model.add_module("b", Block(kh.MoE_Torch(4, 1, 16, 32, nn.GELU(approximate="tanh"), False, True, 0.02)))
    keys = list(model.state_dict().keys())
    params = {n: p for n, p in model.named_parameters()}
    assert inject.swap_moe_modules(model) == 2
    assert isinstance(model.a.moe, kh.MoE_B200) and isinstance(model.b.moe, kh.MoE_B200)
    assert isinstance(model.a.moe.c_fc, kh.Experts_B200)
    assert list(model.state_dict().keys()) == keys
    for n, p in model.named_parameters():
        assert p is params[n]
    assert model.a.moe.is_glu and not model.b.moe.is_glu
    assert model.b.moe.top_k == 1 and model.b.moe.c_fc.bias is not None
    assert inject.swap_moe_modules(model) == 0  # idempotent


def test_adopt_infers_glu_from_the_projection_width():
    class MoE_Torch(nn.Module):  # a module with the reference's attribute set (no is_glu attribute)
        def __init__(self):
            super().__init__()
            self.num_experts, self.top_k, self.hidden_size, self.intermediate_size = 2, 1, 8, 16
            self.gate = nn.Linear(8, 2, bias=False)
            self.c_fc = kh.Experts_Torch(2, 8, 32, add_bias=False, std=0.02)
            self.act = kh.swiglu_unchunked_torch
            self.c_proj = kh.Experts_Torch(2, 16, 8, add_bias=False, std=0.02)

    old = MoE_Torch()
    new = inject.adopt_moe(old)
    assert new.is_glu and new.router_scoring == "softmax" and new.num_shared_experts == 0
    assert new.c_fc.weight is old.c_fc.weight and new.gate is old.gate


# ---- GPU -------------------------------------------------------------------------------------------


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_compiled_graph_runs_the_fused_operator(dtype):
    from kernel_hyperdrive_b200 import _lib

    torch.manual_seed(1)
    x = torch.randn(4, 33, 256, device="cuda", dtype=dtype, requires_grad=True)
    g = torch.randn(4, 33, 128, device="cuda", dtype=dtype)
    injector = inject.GraphInjector()
    torch._dynamo.reset()
    compiled = torch.compile(mlp_act, backend=injector.compiler, fullgraph=True)
    before = _lib.lib().b200moe_launch_count()
    y = compiled(x)
    y.backward(g)
    assert injector.replaced == 1
    assert _lib.lib().b200moe_launch_count() - before == 2  # forward and backward kernels of the library ran
    dx, x.grad = x.grad, None
    ref = mlp_act(x.float())
    ref.backward(g.float())
    tol = 5e-6 if dtype == torch.float32 else 1e-2
    assert rel_l2(y, ref) <= tol and rel_l2(dx, x.grad) <= tol


@pytest.mark.gpu
def test_swapped_model_matches_the_eager_model():
    torch.manual_seed(2)
    model = Block(kh.MoE_Torch(8, 2, 256, 384, kh.swiglu_unchunked_torch, True, False, 0.02)).cuda()
    x = torch.randn(3, 70, 256, device="cuda", requires_grad=True)
    g = torch.randn_like(x)
    y0, logits0 = model(x)
    y0.backward(g)
    ref = {n: p.grad.clone() for n, p in model.named_parameters()}
    dx0 = x.grad.clone()
    model.zero_grad()
    x.grad = None
    assert inject.swap_moe_modules(model) == 1
    y1, logits1 = model(x)
    y1.backward(g)
    assert torch.equal(logits0, logits1)
    assert rel_l2(y1, y0) <= 1e-5 and rel_l2(x.grad, dx0) <= 1e-5
    for n, p in model.named_parameters():
        assert rel_l2(p.grad, ref[n]) <= 1e-5, n
