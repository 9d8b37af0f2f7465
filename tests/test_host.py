"""Host-side checks that need no GPU: the C-ABI library loads and exports what include/b200moe.h declares,
size helpers, error behaviour, module parameter layout, the eager torch module against the oracle."""

import os
import re

import numpy as np
import pytest
import torch

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib, synthetic
from oracle import moe_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-zA-Z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200moe.h but not exported"
        assert n in _lib.EXPORTED, f"{n} has no ctypes prototype"
    assert set(_lib.EXPORTED) == set(names)


def test_version_and_error_strings():
    lib = _lib.lib()
    assert lib.b200moe_version() >= 100
    assert lib.b200moe_error_string(0) == b"ok"
    for code in range(-8, 0):
        assert lib.b200moe_error_string(code) != b"unknown error code"


def test_size_helpers():
    lib = _lib.lib()
    for M, E in [(0, 1), (1, 1), (512, 8), (32768, 8), (1 << 20, 256), (127, 3)]:
        cap = lib.b200moe_padded_rows_cap(M, E)
        assert cap == kh.scattermoe.padded_rows_cap(M, E)
        assert cap % 128 == 0
        # worst case: every expert but one holds 1 row
        counts = np.ones(E, dtype=np.int64)
        if M >= E:
            counts[0] = M - (E - 1)
            assert orc.padded_layout(counts)[-1] <= cap
        assert lib.b200moe_route_workspace_bytes(M, E) >= 2 * E * 4
        assert lib.b200moe_scatter2scatter_workspace_bytes(M, E) >= 8 * E + 8 * M


def test_argument_errors_do_not_launch():
    lib = _lib.lib()
    before = lib.b200moe_launch_count()
    assert lib.b200moe_contiguous_count(None, 1, 4, None, 8, None) == -1
    assert b"contiguous_count" in lib.b200moe_last_error_detail()
    assert lib.b200moe_route(None, 10, 100000, 2, None, None, None, None, None, None, 0, None, 0, None, None) == -6
    assert lib.b200moe_set_engine(7) == -1
    assert lib.b200moe_launch_count() == before


def test_argument_errors_of_the_steps_around_the_path():
    """Router, RMSNorm and the gate-gradient kernel: bad arguments come back as codes, nothing is launched."""
    import ctypes

    lib = _lib.lib()
    before = lib.b200moe_launch_count()
    f32 = ctypes.c_float(1e-5)
    # router: fp32 tensors, too many experts, k > 8, missing counts
    assert lib.b200moe_router_forward(None, 64, None, 64, 4, 64, 8, 2, 0, None, 8, None, None, None, _lib.DTYPE_CODE[torch.float32], None, None) == -2
    assert lib.b200moe_router_forward(None, 64, None, 64, 4, 64, 257, 2, 0, None, 257, None, None, None, _lib.DTYPE_CODE[torch.bfloat16], None, None) == -6
    assert lib.b200moe_router_forward(None, 64, None, 64, 4, 64, 8, 9, 0, None, 8, None, None, None, _lib.DTYPE_CODE[torch.bfloat16], None, None) == -6
    assert lib.b200moe_router_forward(None, 64, None, 64, 4, 64, 8, 2, 3, None, 8, None, None, None, _lib.DTYPE_CODE[torch.bfloat16], None, None) == -1
    assert b"router_forward" in lib.b200moe_last_error_detail()
    # rmsnorm: unknown dtype, NULL pointers with rows > 0, weight gradient without weight; the workspace size is positive
    assert lib.b200moe_rmsnorm_forward(None, 64, None, None, 64, None, 4, 64, f32, 9, None) == -2
    assert lib.b200moe_rmsnorm_forward(None, 64, None, None, 64, None, 4, 64, f32, 1, None) == -1
    assert lib.b200moe_rmsnorm_forward(None, 64, None, None, 64, None, 0, 64, f32, 1, None) == 0  # no rows: nothing to do
    assert lib.b200moe_rmsnorm_backward(None, 64, None, None, 64, None, None, 64, ctypes.c_void_p(16), None, 0, 4, 64, f32, 1, None) == -1
    assert lib.b200moe_rmsnorm_workspace_bytes(1000, 4096, 1) >= 4096 * 4
    assert lib.b200moe_rmsnorm_workspace_bytes(-1, 4096, 1) == 0
    # gate gradient
    assert lib.b200moe_ep_gate_grad(None, 64, None, 64, None, 4, 2, 64, 1, None) == -1
    assert lib.b200moe_ep_gate_grad(None, 64, None, 64, None, 0, 2, 64, 1, None) == 0
    assert lib.b200moe_launch_count() == before


def test_ops_refuse_cpu_tensors():
    with pytest.raises(RuntimeError, match="CUDA"):
        kh.contiguous_count_cute(torch.zeros(4, dtype=torch.long), 3)
    x = torch.zeros(4, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        kh.swiglu_unchunked_cute(x)


def test_module_parameters_match_reference_layout():
    m = kh.MoE_Triton(8, 2, 32, 64, kh.swiglu_unchunked_torch, True, False, 0.02)
    sd = m.state_dict()
    assert list(sd) == ["gate.weight", "c_fc.weight", "c_proj.weight"]
    assert sd["gate.weight"].shape == (8, 32) and sd["c_fc.weight"].shape == (8, 128, 32) and sd["c_proj.weight"].shape == (8, 32, 64)
    t = kh.MoE_Torch(8, 2, 32, 64, kh.swiglu_unchunked_torch, True, False, 0.02)
    t.load_state_dict(sd)
    m2 = kh.MoE_Torch(8, 2, 32, 64, torch.nn.functional.gelu, False, True, 0.02)
    assert m2.c_fc.weight.shape == (8, 64, 32) and m2.c_fc.bias.shape == (8, 64)


def test_eager_module_matches_oracle_on_cpu():
    w = synthetic.WORKLOADS["tiny"]
    wt = synthetic.make_weights(w, 0)
    x, g = synthetic.make_tokens(w, 0)
    m = kh.MoE_Torch(w.num_experts, w.top_k, w.hidden, w.intermediate, kh.swiglu_unchunked_torch, True, False, 0.02)
    with torch.no_grad():
        m.gate.weight.copy_(wt["gate"])
        m.c_fc.weight.copy_(wt["w_fc"])
        m.c_proj.weight.copy_(wt["w_proj"])
    xr = x.clone().requires_grad_(True)
    y, logits = m(xr)
    y.backward(g)
    ref = orc.moe_layer(x, wt["gate"], wt["w_fc"], wt["w_proj"], w.top_k, grad_out=g)
    assert orc.rel_l2(y, ref["y"]) < 1e-6 and orc.rel_l2(xr.grad, ref["dx"]) < 1e-6
    assert orc.rel_l2(m.c_fc.weight.grad, ref["d_w_fc"]) < 1e-6 and orc.rel_l2(m.gate.weight.grad, ref["d_gate_weight"]) < 1e-5


def test_workload_table_matches_benchmark_configs():
    W = synthetic.WORKLOADS
    assert (W["c2"].num_experts, W["c2"].top_k, W["c2"].hidden, W["c2"].intermediate, W["c2"].tokens) == (8, 2, 4096, 14336, 16384)
    assert abs(W["c2"].flops_fwd_bwd() - 34.635e12) < 0.01e12
    assert abs(W["c3"].flops_fwd_bwd() - 13.606e12) < 0.01e12
    assert abs(W["c5"].flops_fwd_bwd() - 277.08e12) < 0.1e12
    rw, sel = synthetic.make_routing(synthetic.scaled(W["c4"], tokens=4096), torch.zeros(4096, 8), torch.zeros(128, 8), 0)
    counts = sel.flatten().bincount(minlength=128)
    assert counts.max() > 10 * counts.float().mean() * 0.5 and (sel.sort(-1).values.diff(dim=-1) != 0).all()


def test_options_are_range_checked_and_round_trip():
    """The process-wide switches: unknown options and out-of-range values come back as argument errors and leave the
    stored value alone; valid values can be read back."""
    lib = _lib.lib()
    defaults = {_lib.OPT_DYNAMIC_TILES: 2, _lib.OPT_TILE_VARIANT: -1, _lib.OPT_TILE_ORDER: -1, _lib.OPT_SM_LIMIT: 0}
    for opt, value in defaults.items():
        assert lib.b200moe_get_option(opt) == value
    for opt, bad in [(0, 0), (5, 0), (_lib.OPT_DYNAMIC_TILES, 4), (_lib.OPT_TILE_VARIANT, 2), (_lib.OPT_TILE_ORDER, 3), (_lib.OPT_TILE_ORDER, -2), (_lib.OPT_SM_LIMIT, -1)]:
        assert lib.b200moe_set_option(opt, bad) == -1
    for opt, value in defaults.items():
        assert lib.b200moe_get_option(opt) == value
    try:
        for opt, good in [(_lib.OPT_TILE_ORDER, 2), (_lib.OPT_SM_LIMIT, 132), (_lib.OPT_DYNAMIC_TILES, 0), (_lib.OPT_TILE_VARIANT, _lib.TILE_CTA_128x256)]:
            _lib.set_option(opt, good)
            assert _lib.get_option(opt) == good
    finally:
        for opt, value in defaults.items():
            _lib.set_option(opt, value)


def test_plan_kernel_argument_errors_do_not_launch():
    lib = _lib.lib()
    before = lib.b200moe_launch_count()
    # world * E above the table size, E not divisible by the world size, rank outside the world, NULL tables
    assert lib.b200moe_ep_plan(None, None, 32, 0, 256, 0, None, None, None, None, None, None, None) == -1
    assert lib.b200moe_ep_plan(None, None, 3, 0, 8, 0, None, None, None, None, None, None, None) == -1
    assert lib.b200moe_ep_plan(None, None, 2, 2, 8, 0, None, None, None, None, None, None, None) == -1
    assert lib.b200moe_ep_plan(None, None, 2, 0, 8, 0, None, None, None, None, None, None, None) == -1
    assert b"ep_plan" in lib.b200moe_last_error_detail()
    assert lib.b200moe_launch_count() == before


def test_zipf_placement_from_sampled_counts_balances_the_ranks():
    """The benchmark places the experts of the Zipf-skewed layer by token counts sampled from the routing distribution;
    with them the greedy placement keeps every rank within 2 % of the mean at 2 and 4 ranks (with 8 ranks the largest
    expert alone is 0.95 of a rank's share, so 1.10 is the floor there)."""
    from kernel_hyperdrive_b200.expert_parallel import make_placement

    w = synthetic.WORKLOADS["c4"]
    E = w.num_experts
    _, sample = synthetic.make_routing(synthetic.scaled(w, tokens=16384), torch.zeros(16384, 1), None, 987)
    expected = torch.bincount(sample.flatten(), minlength=E).double().add_(1.0).tolist()
    _, sel = synthetic.make_routing(synthetic.scaled(w, tokens=32768), torch.zeros(32768, 1), None, 0)
    real = torch.bincount(sel.flatten(), minlength=E).double()
    for world, bound in [(2, 1.02), (4, 1.02), (8, 1.12)]:
        slot = make_placement("balanced", E, world, expected)
        assert torch.equal(slot.sort().values, torch.arange(E))
        rank = slot // (E // world)
        loads = torch.stack([real[rank == r].sum() for r in range(world)])
        assert (loads.max() / loads.mean()).item() < bound, (world, loads.tolist())
