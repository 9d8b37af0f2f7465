"""The MoE layer (fused and generic paths) against the CPU oracle and the golden fixtures: output and all
gradients (input, both expert weights, router weights, gate weight)."""

import os

import numpy as np
import pytest
import torch

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib, synthetic
from oracle import moe_oracle as orc

from conftest import GOLDEN
from helpers import make_case, oracle_experts, rel_l2, to_dev, tolerance

pytestmark = pytest.mark.gpu

W = synthetic.WORKLOADS
SMALL = {
    "tiny": W["tiny"],
    "c1": W["c1"],
    "ragged_k1": synthetic.MoEWorkload("ragged", 6, 1, 40, 24, 19, dtype="fp32", routing="normal_logits"),
    "c2_small": synthetic.scaled(W["c2"], hidden=512, intermediate=1024, tokens=1024),
    "c3_small": synthetic.scaled(W["c3"], hidden=256, intermediate=384, tokens=512, shared_experts=0),
    "c4_small": synthetic.scaled(W["c4"], hidden=256, intermediate=128, tokens=1024),
    "c5_small": synthetic.scaled(W["c5"], hidden=512, intermediate=256, tokens=768),
    "odd": synthetic.MoEWorkload("odd", 5, 3, 136, 200, 333, routing="normal_logits"),
}


@pytest.fixture(autouse=True)
def _engine_reset():
    yield
    _lib.set_engine(_lib.ENGINE_AUTO)
    _lib.check_status(torch.device("cuda"))


def run_fused(case_dev, activation="swiglu"):
    x = case_dev["x"].clone().requires_grad_(True)
    w1 = case_dev["w_fc"].clone().requires_grad_(True)
    w2 = case_dev["w_proj"].clone().requires_grad_(True)
    rw = case_dev["rw"].clone().requires_grad_(True)
    y = kh.fused_swiglu_experts(x, w1, w2, rw, case_dev["sel"], activation=activation)
    y.backward(case_dev["g"])
    return dict(y=y.detach(), dx=x.grad, d_w_fc=w1.grad, d_w_proj=w2.grad, d_router_weights=rw.grad)


def check(got, ref, tol, what):
    for key in ("y", "dx", "d_w_fc", "d_w_proj", "d_router_weights"):
        assert torch.isfinite(got[key]).all(), (what, key)
        err = rel_l2(got[key], ref[key])
        assert err < tol, (what, key, err)


@pytest.mark.parametrize("order", [0, 1, 2])
def test_tile_orders_give_identical_results(order):
    """The order in which an expert's tiles are walked (row tiles of a column block first, column blocks of a row tile
    first, blocks of 8 x 8 tiles) changes which cluster computes a tile and when, not the arithmetic of the tile: every
    output and gradient is bit-identical to the default order.  Twelve row-tile pairs and ten column blocks per expert, so
    that the 8 x 8 blocks have ragged edges in both directions."""
    w = synthetic.scaled(W["c2"], hidden=512, intermediate=1280, tokens=12288, routing="normal_logits")
    case = to_dev(make_case(w, seed=3, dtype=torch.bfloat16), torch.bfloat16)
    _lib.set_engine(_lib.ENGINE_UMMA)
    _lib.set_option(_lib.OPT_TILE_VARIANT, _lib.TILE_PAIR_256x256)
    try:
        ref = run_fused(case)
        _lib.set_option(_lib.OPT_TILE_ORDER, order)
        got = run_fused(case)
    finally:
        _lib.set_option(_lib.OPT_TILE_ORDER, -1)
        _lib.set_option(_lib.OPT_TILE_VARIANT, -1)
    for key in ref:
        assert torch.equal(got[key], ref[key]), (order, key)


@pytest.mark.parametrize("engine", ["umma", "umma1"])
def test_sm_limit_keeps_the_results(engine):
    """GEMM launches restricted to part of the SMs (the rest is left to other streams) compute the same tiles with fewer
    CTAs: bit-identical outputs and gradients."""
    w = synthetic.scaled(W["c2"], hidden=512, intermediate=1024, tokens=4096, routing="normal_logits")
    case = to_dev(make_case(w, seed=5, dtype=torch.bfloat16), torch.bfloat16)
    _lib.set_engine({"umma": _lib.ENGINE_UMMA, "umma1": _lib.ENGINE_UMMA_1CTA}[engine])
    try:
        ref = run_fused(case)
        _lib.set_option(_lib.OPT_SM_LIMIT, 101)
        assert _lib.get_option(_lib.OPT_SM_LIMIT) == 101
        got = run_fused(case)
    finally:
        _lib.set_option(_lib.OPT_SM_LIMIT, 0)
    for key in ref:
        assert torch.equal(got[key], ref[key]), key


@pytest.mark.parametrize("name", list(SMALL))
@pytest.mark.parametrize("engine,dtype", [("simt", torch.float32), ("simt", torch.bfloat16), ("umma", torch.bfloat16), ("umma", torch.float16), ("umma1", torch.bfloat16)])
def test_fused_experts_match_oracle(name, engine, dtype):
    w = SMALL[name]
    _lib.set_engine({"simt": _lib.ENGINE_SIMT, "umma": _lib.ENGINE_UMMA, "umma1": _lib.ENGINE_UMMA_1CTA}[engine])
    case = make_case(w, seed=1, dtype=dtype)
    ref = oracle_experts(case)
    got = run_fused(to_dev(case, dtype))
    check(got, ref, tolerance(dtype), (name, engine, dtype))


@pytest.mark.parametrize("name", ["tiny", "c1", "ragged"])
def test_layer_matches_golden_fp32(name):
    """Whole layer in fp32 against the reference module's own outputs (router included): 1e-5."""
    gold = dict(np.load(os.path.join(GOLDEN, f"{name}.npz")))
    w, seed = {"tiny": (W["tiny"], 0), "c1": (W["c1"], 0), "ragged": (synthetic.MoEWorkload("ragged", 6, 1, 40, 24, 19, dtype="fp32"), 3)}[name]
    wt = synthetic.make_weights(w, seed)
    x, g = synthetic.make_tokens(w, seed)
    m = kh.MoE_Triton(w.num_experts, w.top_k, w.hidden, w.intermediate, kh.swiglu_unchunked_torch, True, False, w.weight_std).cuda()
    m.load_state_dict({"gate.weight": wt["gate"], "c_fc.weight": wt["w_fc"], "c_proj.weight": wt["w_proj"]})
    xr = x.cuda().requires_grad_(True)
    y, logits = m(xr)
    y.backward(g.cuda())
    _, _, sel = m._compute_routing_weights(x.cuda())
    assert np.array_equal(sel.cpu().numpy(), gold["selected_experts"])
    sub = lambda t: t.detach().flatten()[::97].cpu().numpy()
    assert rel_l2(y, gold["y"]) < 1e-5 and rel_l2(logits, gold["logits"]) < 1e-5
    assert rel_l2(xr.grad, gold["dx"]) < 1e-5
    assert rel_l2(m.gate.weight.grad, gold["d_gate"]) < 1e-4
    assert rel_l2(sub(m.c_fc.weight.grad), gold["d_w_fc_sub"]) < 1e-5
    assert rel_l2(sub(m.c_proj.weight.grad), gold["d_w_proj_sub"]) < 1e-5
    assert abs(m.c_fc.weight.grad.double().norm().item() - gold["d_w_fc_norm"]) < 1e-5 * gold["d_w_fc_norm"]
    # externally supplied routing through the module seam
    xr2 = x.cuda().requires_grad_(True)
    rw = torch.from_numpy(gold["ext_router_weights"]).cuda().requires_grad_(True)
    m.zero_grad()
    y2 = m._compute_experts(xr2, rw, torch.from_numpy(gold["ext_selected_experts"]).cuda())
    y2.backward(g.cuda())
    assert rel_l2(y2, gold["ext_y"]) < 1e-5 and rel_l2(xr2.grad, gold["ext_dx"]) < 1e-5
    assert rel_l2(rw.grad, gold["ext_d_router_weights"]) < 1e-5
    assert rel_l2(sub(m.c_fc.weight.grad), gold["ext_d_w_fc_sub"]) < 1e-5


@pytest.mark.parametrize("name", ["tiny", "c2_small", "c5_small", "odd"])
@pytest.mark.parametrize("engine,dtype", [("simt", torch.float32), ("umma", torch.bfloat16), ("umma", torch.float16), ("umma1", torch.bfloat16)])
def test_fused_glu_experts_match_oracle(name, engine, dtype):
    """The sigmoid-gated variant of the fused path (torch.nn.GLU between the projections, the activation of the
    reference's module test, tests/test_commons.py:86-87) against the CPU oracle with that activation."""
    w = SMALL[name]
    _lib.set_engine({"simt": _lib.ENGINE_SIMT, "umma": _lib.ENGINE_UMMA, "umma1": _lib.ENGINE_UMMA_1CTA}[engine])
    case = make_case(w, seed=2, dtype=dtype)
    ref = orc.experts_with_grads(case["x"], case["w_fc"], case["w_proj"], case["rw"], case["sel"], case["g"], act=lambda t: torch.nn.functional.glu(t, dim=-1))
    got = run_fused(to_dev(case, dtype), activation="glu")
    check(got, ref, tolerance(dtype), (name, engine, dtype))


def test_glu_module_takes_the_fused_path():
    from kernel_hyperdrive_b200 import scattermoe

    assert scattermoe.fused_activation(torch.nn.GLU()) == "glu" and scattermoe.fused_activation(torch.nn.GLU(dim=0)) is None
    assert scattermoe.fused_activation(kh.swiglu_unchunked_torch) == "swiglu" and scattermoe.fused_activation(torch.tanh) is None
    m = kh.MoE_Triton(8, 2, 256, 512, torch.nn.GLU(), True, False, 0.02).cuda().bfloat16()
    x = torch.randn(300, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    names = []
    scattermoe.set_timing_sink(names)
    try:
        y, _ = m(x)
        y.sum().backward()
    finally:
        scattermoe.set_timing_sink(None)
    gemms = ("up_forward", "down_forward", "down_dgrad", "down_wgrad", "up_wgrad", "up_dgrad")
    assert [n[0] for n in names if n[0] in gemms] == list(gemms)
    # the row passes around them: token gather, un-sort + gate-weighted sum, gradient gather (+ gate gradient), un-sort + slot sum
    assert [n[0] for n in names if n[0] not in gemms] == ["route", "gather_x", "combine_y", "gather_grad", "combine_dx"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act_name,is_glu", [("glu", True), ("glu_callable", True), ("gelu", False), ("swiglu", True)])
def test_generic_path_matches_eager_module(dtype, act_name, is_glu):
    """Any activation callable: same operator sequence as the reference's scatter module; compared with the
    eager torch module on the same device and weights (the reference's own test strategy, many tokens)."""
    act = {"glu": torch.nn.GLU(), "glu_callable": lambda t: torch.nn.functional.glu(t, dim=-1), "gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"), "swiglu": lambda t: kh.swiglu_unchunked_torch(t)}[act_name]
    torch.manual_seed(42)
    E, k, H, I, T = 8, 2, 256, 512, 200
    ref_m = kh.MoE_Torch(E, k, H, I, act, is_glu, False, 0.02).cuda().to(dtype)
    our_m = kh.MoE_Triton(E, k, H, I, act, is_glu, False, 0.02).cuda().to(dtype)
    our_m.load_state_dict(ref_m.state_dict())
    x = torch.randn(4, T // 4, H, device="cuda", dtype=dtype)
    g = torch.randn_like(x)
    outs = []
    for m in (ref_m, our_m):
        xr = x.clone().requires_grad_(True)
        y, logits = m(xr)
        y.backward(g)
        outs.append((y.detach(), xr.grad, m.c_fc.weight.grad, m.c_proj.weight.grad, m.gate.weight.grad))
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2  # both sides round to bf16 here
    for a, b, what in zip(outs[1], outs[0], ("y", "dx", "d_w_fc", "d_w_proj", "d_gate")):
        assert rel_l2(a, b) < (tol if what != "d_gate" else 20 * tol), (what, rel_l2(a, b))


@pytest.mark.parametrize("name", ["tiny", "c2_small", "c4_small", "odd"])
@pytest.mark.parametrize("engine,dtype", [("simt", torch.float32), ("umma", torch.bfloat16), ("umma", torch.float16), ("umma1", torch.bfloat16)])
def test_fused_gelu_experts_match_oracle(name, engine, dtype):
    """Plain (non-GLU) expert layer with the tanh form of GELU, the other activation of the reference's layer test
    (tests/test_commons.py:86-87): fused forward and input-gradient epilogues against the oracle's expert computation
    with the same activation.  The up projection has I output features here (the first I rows of the case's weights)."""
    w = SMALL[name]
    case = make_case(w, seed=2, dtype=dtype)
    case["w_fc"] = case["w_fc"][:, : w.intermediate].contiguous()
    gelu = lambda t: torch.nn.functional.gelu(t, approximate="tanh")
    ref = orc.experts_with_grads(case["x"], case["w_fc"], case["w_proj"], case["rw"], case["sel"], case["g"], act=gelu)
    _lib.set_engine({"simt": _lib.ENGINE_SIMT, "umma": _lib.ENGINE_UMMA, "umma1": _lib.ENGINE_UMMA_1CTA}[engine])
    got = run_fused(to_dev(case, dtype), activation="gelu_tanh")
    check(got, ref, tolerance(dtype), (name, engine, dtype, "gelu_tanh"))


def test_gelu_module_takes_the_fused_path():
    from kernel_hyperdrive_b200 import scattermoe

    assert scattermoe.fused_activation(torch.nn.GELU(approximate="tanh"), is_glu=False) == "gelu_tanh"
    assert scattermoe.fused_activation(torch.nn.GELU(), is_glu=False) is None  # the erf form stays un-fused
    ref_m = kh.MoE_Torch(8, 2, 256, 384, torch.nn.GELU(approximate="tanh"), False, False, 0.02).cuda().bfloat16()
    m = kh.MoE_Triton(8, 2, 256, 384, torch.nn.GELU(approximate="tanh"), False, False, 0.02).cuda().bfloat16()
    m.load_state_dict(ref_m.state_dict())
    x = torch.randn(300, 256, device="cuda", dtype=torch.bfloat16)
    g = torch.randn_like(x)
    names = []
    scattermoe.set_timing_sink(names)
    outs = []
    try:
        for layer in (m, ref_m):
            xr = x.clone().requires_grad_(True)
            y, _ = layer(xr)
            y.backward(g)
            outs.append((y.detach(), xr.grad, layer.c_fc.weight.grad, layer.c_proj.weight.grad))
    finally:
        scattermoe.set_timing_sink(None)
    gemms = ("up_forward", "down_forward", "down_dgrad", "down_wgrad", "up_wgrad", "up_dgrad")
    assert [n[0] for n in names if n[0] in gemms] == list(gemms)  # the eager module launches none of them
    for a, b, what in zip(outs[0], outs[1], ("y", "dx", "d_w_fc", "d_w_proj")):
        assert rel_l2(a, b) < 1.5e-2, (what, rel_l2(a, b))


@pytest.mark.parametrize("dtype,engine", [(torch.float32, "simt"), (torch.bfloat16, "umma")])
def test_slots_without_an_expert_are_left_out(dtype, engine):
    """Negative expert ids (padding tokens, slots dropped by a capacity limit) take no part: same output and gradients as
    the oracle run in which those slots carry a zero gate, and a zero router-weight gradient for them."""
    w = synthetic.MoEWorkload("drop", 8, 3, 128, 256, 300, routing="normal_logits")
    case = make_case(w, seed=4, dtype=dtype)
    drop = torch.rand(case["sel"].shape, generator=torch.Generator().manual_seed(9)) < 0.3
    drop[7] = True  # a token that keeps no expert at all
    ref_case = dict(case)
    ref_case["rw"] = torch.where(drop, torch.zeros_like(case["rw"]), case["rw"])
    ref = oracle_experts(ref_case)
    case["sel"] = torch.where(drop, torch.full_like(case["sel"], -1), case["sel"])
    _lib.set_engine({"simt": _lib.ENGINE_SIMT, "umma": _lib.ENGINE_UMMA}[engine])
    got = run_fused(to_dev(case, dtype))
    keep = ~drop
    tol = tolerance(dtype)
    for key in ("y", "dx", "d_w_fc", "d_w_proj"):
        assert rel_l2(got[key], ref[key]) < tol, (key, rel_l2(got[key], ref[key]))
    assert float(got["y"][7].abs().max()) == 0.0
    assert rel_l2(got["d_router_weights"].cpu()[keep], ref["d_router_weights"][keep]) < tol
    assert float(got["d_router_weights"].cpu()[drop].abs().max()) == 0.0


def test_drop_in_shapes_and_state_dict():
    m = kh.MoE_Triton(8, 2, 256, 512, kh.swiglu_unchunked_torch, True, False, 0.02).cuda().bfloat16()
    x = torch.randn(2, 3, 5, 256, device="cuda", dtype=torch.bfloat16)
    y, logits = m(x)
    assert y.shape == x.shape and logits.shape == (30, 8) and y.dtype == torch.bfloat16
    t = kh.MoE_Torch(8, 2, 256, 512, kh.swiglu_unchunked_torch, True, False, 0.02).cuda().bfloat16()
    t.load_state_dict(m.state_dict())
    y2, _ = t(x)
    assert rel_l2(y, y2) < 1.5e-2


def test_weight_grads_of_empty_experts_are_zero():
    w = synthetic.MoEWorkload("e", 16, 2, 128, 128, 64, routing="normal_logits")
    case = make_case(w, seed=5, dtype=torch.bfloat16)
    case["sel"] = case["sel"] % 5  # experts 5.. receive nothing
    got = run_fused(to_dev(case, torch.bfloat16))
    assert (got["d_w_fc"][5:] == 0).all() and (got["d_w_proj"][5:] == 0).all()
    ref = oracle_experts(case)
    check(got, ref, 1e-2, "empty experts")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shared_experts_and_sigmoid_scoring(dtype):
    """Extensions the benchmark configurations ask for on top of the reference layer: always-on shared experts
    and sigmoid scoring of the selected logits.  Checked against the eager module on the device and against the
    CPU oracle's restatement of both."""
    torch.manual_seed(7)
    E, k, H, I, T, S, I_s = 16, 4, 256, 384, 500, 2, 128
    kw = dict(num_shared_experts=S, shared_intermediate_size=I_s, router_scoring="sigmoid")
    ref_m = kh.MoE_Torch(E, k, H, I, kh.swiglu_unchunked_torch, True, False, 0.05, **kw).cuda().to(dtype)
    our_m = kh.MoE_B200(E, k, H, I, kh.swiglu_unchunked_torch, True, False, 0.05, **kw).cuda().to(dtype)
    our_m.load_state_dict(ref_m.state_dict())
    assert "shared_c_fc.weight" in our_m.state_dict() and our_m.shared_c_fc.weight.shape == (S, 2 * I_s, H)
    x = torch.randn(T, H, device="cuda", dtype=dtype)
    g = torch.randn_like(x)
    outs = []
    for m in (ref_m, our_m):
        xr = x.clone().requires_grad_(True)
        y, _ = m(xr)
        y.backward(g)
        outs.append((y.detach(), xr.grad, m.c_fc.weight.grad, m.shared_c_fc.weight.grad, m.shared_c_proj.weight.grad, m.gate.weight.grad))
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    for a, b, what in zip(outs[1], outs[0], ("y", "dx", "d_w_fc", "d_shared_fc", "d_shared_proj", "d_gate")):
        assert rel_l2(a, b) < (tol if what != "d_gate" else 20 * tol), (what, rel_l2(a, b))
    # oracle: routed part with sigmoid routing + dense shared experts
    xf = x.cpu().float()
    sd = {n: t.detach().cpu().float() for n, t in ref_m.state_dict().items()}
    logits = xf @ sd["gate.weight"].t()
    rw, sel = orc.sigmoid_routing(logits, k)
    _, _, sel_dev = our_m._compute_routing_weights(x)
    if torch.equal(sel, sel_dev.cpu()):  # a 16-bit gate may order near-ties differently; compare only on equal routing
        y_ref = orc.experts_torch_style(xf, sd["c_fc.weight"], sd["c_proj.weight"], rw, sel) + orc.shared_experts(xf, sd["shared_c_fc.weight"], sd["shared_c_proj.weight"])
        assert rel_l2(outs[1][0], y_ref) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("act_name", ["swiglu", "glu"])
def test_torch_compile_fullgraph(act_name):
    """The layer traces under torch.compile(fullgraph=True) like the reference's module in its own test
    (tests/kernels/scattermoe_test.py:92-93): every kernel launch is one opaque custom op in the graph."""
    act = kh.swiglu_unchunked_torch if act_name == "swiglu" else torch.nn.GLU()
    torch.manual_seed(0)
    m = kh.MoE_Triton(8, 2, 256, 512, act, True, False, 0.02).cuda().bfloat16()
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y0, _ = m(x)
    y0.sum().backward()
    g0 = x.grad.clone()
    x.grad = None
    mc = torch.compile(m, fullgraph=True)
    y1, _ = mc(x)
    y1.sum().backward()
    assert rel_l2(y1, y0) < 1e-3 and rel_l2(x.grad, g0) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_empty_batch_and_single_token(dtype):
    """No tokens at all: outputs and input gradient are empty, weight gradients are exact zeros.  One token (the case
    the reference's own module test uses): matches the eager module."""
    torch.manual_seed(1)
    m = kh.MoE_Triton(8, 2, 256, 512, kh.swiglu_unchunked_torch, True, False, 0.02).cuda().to(dtype)
    x0 = torch.zeros(0, 256, device="cuda", dtype=dtype, requires_grad=True)
    y0, logits0 = m(x0)
    assert y0.shape == (0, 256) and logits0.shape == (0, 8)
    y0.sum().backward()
    assert x0.grad.shape == (0, 256)
    assert (m.c_fc.weight.grad == 0).all() and (m.c_proj.weight.grad == 0).all()
    m.zero_grad()
    t = kh.MoE_Torch(8, 2, 256, 512, kh.swiglu_unchunked_torch, True, False, 0.02).cuda().to(dtype)
    t.load_state_dict(m.state_dict())
    x1 = torch.randn(256, device="cuda", dtype=dtype)
    outs = []
    for layer in (t, m):
        xr = x1.clone().requires_grad_(True)
        y, _ = layer(xr)
        y.sum().backward()
        outs.append((y.detach(), xr.grad))
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    assert rel_l2(outs[1][0], outs[0][0]) < tol and rel_l2(outs[1][1], outs[0][1]) < tol
    _lib.check_status(torch.device("cuda"))
