"""Shared helpers of the GPU parity tests: inputs from the seeded generators, oracle results on CPU."""

import numpy as np
import torch

from kernel_hyperdrive_b200 import synthetic
from oracle import moe_oracle as orc

DT = synthetic.TORCH_DTYPES


def rel_l2(a, b) -> float:
    return orc.rel_l2(torch.as_tensor(a).detach().cpu().float(), torch.as_tensor(b).detach().cpu().float())


def tolerance(dtype: torch.dtype) -> float:
    """The parity bar of the path: fp32 within 1e-5, 16-bit tensors within 1e-2 (relative L2)."""
    return 1e-5 if dtype == torch.float32 else 1e-2


def make_case(w: synthetic.MoEWorkload, seed: int, dtype: torch.dtype):
    """CPU fp32 tensors rounded to `dtype` (so that both sides see identical values) + routing."""
    wt = synthetic.make_weights(w, seed)
    x, g = synthetic.make_tokens(w, seed)
    rnd = lambda t: t.to(dtype).float()
    x, g = rnd(x), rnd(g)
    wt = {k: rnd(v) for k, v in wt.items()}
    rw, sel = synthetic.make_routing(w, x, wt["gate"], seed)
    rw = rnd(rw)
    return dict(x=x, g=g, rw=rw, sel=sel, **wt)


def oracle_experts(case):
    return orc.experts_with_grads(case["x"], case["w_fc"], case["w_proj"], case["rw"], case["sel"], case["g"])


def to_dev(case, dtype, device="cuda"):
    out = {}
    for k, v in case.items():
        if v.is_floating_point():
            out[k] = v.to(device=device, dtype=dtype)
        else:
            out[k] = v.to(device)
    return out


def segments_equal_as_sets(sorted_experts: np.ndarray, idx_a: np.ndarray, idx_b: np.ndarray) -> bool:
    """The order inside one expert's segment is not defined by an unstable sort: compare segment-wise."""
    bounds = np.flatnonzero(np.diff(sorted_experts)) + 1
    for sa, sb in zip(np.split(idx_a, bounds), np.split(idx_b, bounds)):
        if not np.array_equal(np.sort(sa), np.sort(sb)):
            return False
    return True
