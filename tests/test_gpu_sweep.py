"""Seeded sweep over layer shapes for the fused path on the tensor-core engines: expert counts that leave experts
empty, odd numbers of 128-row blocks per expert (the two-CTA kernel then idles one CTA of a pair), hidden and
intermediate sizes that are multiples of 8 but not of the 64 / 128 / 256 tile sizes, k from 1 to 8."""

import random

import pytest
import torch

import kernel_hyperdrive_b200 as kh
from kernel_hyperdrive_b200 import _lib, synthetic

from helpers import make_case, oracle_experts, rel_l2, to_dev

pytestmark = pytest.mark.gpu


def sweep_cases(n=24):
    rng = random.Random(1234)
    cases = []
    for i in range(n):
        E = rng.choice([1, 2, 3, 5, 8, 17, 40])
        k = rng.choice([kk for kk in (1, 2, 3, 4, 8) if kk <= E])
        H = 8 * rng.randint(2, 60)
        I = 8 * rng.randint(2, 70)
        T = rng.choice([1, 7, 130, 257, 600, 1100])
        routing = rng.choice(["normal_logits", "zipf"]) if E >= 3 and k < E else "normal_logits"
        cases.append((i, E, k, H, I, T, routing))
    return cases


@pytest.mark.parametrize("i,E,k,H,I,T,routing", sweep_cases())
@pytest.mark.parametrize("engine", ["umma", "umma1"])
def test_fused_path_shape_sweep(engine, i, E, k, H, I, T, routing):
    _lib.set_engine({"umma": _lib.ENGINE_UMMA, "umma1": _lib.ENGINE_UMMA_1CTA}[engine])
    try:
        w = synthetic.MoEWorkload(f"sweep{i}", E, k, H, I, T, routing=routing, weight_std=0.05)
        case = make_case(w, seed=100 + i, dtype=torch.bfloat16)
        ref = oracle_experts(case)
        d = to_dev(case, torch.bfloat16)
        x = d["x"].clone().requires_grad_(True)
        w1 = d["w_fc"].clone().requires_grad_(True)
        w2 = d["w_proj"].clone().requires_grad_(True)
        rw = d["rw"].clone().requires_grad_(True)
        y = kh.fused_swiglu_experts(x, w1, w2, rw, d["sel"])
        y.backward(d["g"])
        _lib.check_status(torch.device("cuda"))
        got = dict(y=y.detach(), dx=x.grad, d_w_fc=w1.grad, d_w_proj=w2.grad, d_router_weights=rw.grad)
        for key, val in got.items():
            assert torch.isfinite(val).all(), key
            assert rel_l2(val, ref[key]) < 1e-2, (key, rel_l2(val, ref[key]))
    finally:
        _lib.set_engine(_lib.ENGINE_AUTO)
