"""Generate the golden fixtures in this folder from the reference's own torch module.

Run in a container that has the reference checked out (it is not needed to run the tests):

    REFERENCE_ROOT=/path/to/kernel-hyperdrive python tests/golden/make_golden.py

For each case the unmodified `MoE_Torch` (cute_kernels/kernels/scattermoe/torch_implementation.py:61-199)
runs forward and backward on CPU in fp32 with the SwiGLU of
cute_kernels/kernels/swiglu_unchunked/torch_implementation.py:5-7.  One name of that module is rebound
before use: its histogram `contiguous_count_cute` only has a GPU implementation, and the reference's own
test defines it as `bincount(minlength=size)` (tests/kernels/contiguous_count_test.py:34-37).
Inputs come from `kernel_hyperdrive_b200.synthetic` (numpy RandomState streams), so the fixtures store
outputs only, except for the tiny case which also stores its inputs.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.dont_write_bytecode = True
if "REFERENCE_ROOT" not in os.environ:
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference (kernel-hyperdrive) before running this script")
sys.path.insert(0, os.environ["REFERENCE_ROOT"])

import cute_kernels.kernels.scattermoe.torch_implementation as ref_impl  # noqa: E402
from cute_kernels.kernels.swiglu_unchunked.torch_implementation import swiglu_unchunked_torch  # noqa: E402

from kernel_hyperdrive_b200 import synthetic  # noqa: E402

ref_impl.contiguous_count_cute = lambda x, size: x.bincount(minlength=size).to(torch.int32)


def sub(t: torch.Tensor, stride: int = 97) -> np.ndarray:
    return t.detach().flatten()[::stride].contiguous().numpy()


def run_case(name: str, w, seed: int, store_inputs: bool):
    wt = synthetic.make_weights(w, seed)
    x, g = synthetic.make_tokens(w, seed)
    m = ref_impl.MoE_Torch(w.num_experts, w.top_k, w.hidden, w.intermediate, swiglu_unchunked_torch, True, False, w.weight_std)
    with torch.no_grad():
        m.gate.weight.copy_(wt["gate"])
        m.c_fc.weight.copy_(wt["w_fc"])
        m.c_proj.weight.copy_(wt["w_proj"])
    xr = x.clone().requires_grad_(True)
    y, logits = m(xr)
    y.backward(g)
    _, weights, sel = m._compute_routing_weights(x)
    # the routing integers of the scatter module (triton_implementation/__init__.py:79-81), with a stable sort
    flat = sel.flatten()
    se, ss = flat.sort(stable=True)
    off = flat.bincount(minlength=w.num_experts).cumsum(-1)
    out = dict(
        y=y.detach().numpy(),
        logits=logits.detach().numpy(),
        router_weights=weights.detach().numpy(),
        selected_experts=sel.numpy(),
        sorted_expert_idxs=se.numpy(),
        sorted_scattered_idxs=ss.numpy(),
        expert_offsets=off.numpy(),
        dx=xr.grad.numpy(),
        d_gate=m.gate.weight.grad.numpy(),
        d_w_fc_sub=sub(m.c_fc.weight.grad),
        d_w_proj_sub=sub(m.c_proj.weight.grad),
        d_w_fc_norm=np.float64(m.c_fc.weight.grad.double().norm().item()),
        d_w_proj_norm=np.float64(m.c_proj.weight.grad.double().norm().item()),
    )
    if store_inputs:
        out.update(x=x.numpy(), g=g.numpy(), gate=wt["gate"].numpy(), w_fc=wt["w_fc"].numpy(), w_proj=wt["w_proj"].numpy())
        out.update(d_w_fc=m.c_fc.weight.grad.numpy(), d_w_proj=m.c_proj.weight.grad.numpy())

    # externally supplied routing through the module's own seam (_compute_experts), incl. k=1 style cases
    rw2, sel2 = synthetic.make_routing(synthetic.scaled(w, routing="normal_logits"), x, wt["gate"], seed)
    xr2 = x.clone().requires_grad_(True)
    rwr = rw2.clone().requires_grad_(True)
    m.zero_grad()
    y2 = m._compute_experts(xr2, rwr, sel2)
    y2.backward(g)
    out.update(
        ext_router_weights=rw2.numpy(),
        ext_selected_experts=sel2.numpy(),
        ext_y=y2.detach().numpy(),
        ext_dx=xr2.grad.numpy(),
        ext_d_router_weights=rwr.grad.numpy(),
        ext_d_w_fc_sub=sub(m.c_fc.weight.grad),
        ext_d_w_proj_sub=sub(m.c_proj.weight.grad),
    )
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    print(name, {k: getattr(v, "shape", None) for k, v in out.items()})


def swiglu_case():
    rs = np.random.RandomState(11)
    x = torch.from_numpy(rs.standard_normal((37, 2 * 24)).astype(np.float32)).requires_grad_(True)
    dy = torch.from_numpy(rs.standard_normal((37, 24)).astype(np.float32))
    y = swiglu_unchunked_torch(x)
    y.backward(dy)
    np.savez_compressed(os.path.join(HERE, "swiglu.npz"), x=x.detach().numpy(), dy=dy.numpy(), y=y.detach().numpy(), dx=x.grad.numpy())


def rmsnorm_case():
    # the reference's eager definition (cute_kernels/kernels/rmsnorm/torch_implementation.py:5-6), eps of its test
    from cute_kernels.kernels.rmsnorm.torch_implementation import rmsnorm_torch

    rs = np.random.RandomState(13)
    out = {}
    for tag, shape, has_weight in (("w", (29, 56), True), ("nw", (5, 3, 40), False), ("odd", (17, 7), True)):
        x = torch.from_numpy(rs.standard_normal(shape).astype(np.float32)).requires_grad_(True)
        w = torch.from_numpy(rs.standard_normal(shape[-1]).astype(np.float32)).requires_grad_(True) if has_weight else None
        dy = torch.from_numpy(rs.standard_normal(shape).astype(np.float32))
        y = rmsnorm_torch(x, w, 1e-5)
        y.backward(dy)
        out.update({f"{tag}_x": x.detach().numpy(), f"{tag}_dy": dy.numpy(), f"{tag}_y": y.detach().numpy(), f"{tag}_dx": x.grad.numpy()})
        if has_weight:
            out.update({f"{tag}_w": w.detach().numpy(), f"{tag}_dw": w.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, "rmsnorm.npz"), **out)


if __name__ == "__main__":
    torch.manual_seed(0)
    torch.set_num_threads(8)
    run_case("tiny", synthetic.WORKLOADS["tiny"], seed=0, store_inputs=True)
    run_case("c1", synthetic.WORKLOADS["c1"], seed=0, store_inputs=False)
    # uneven loads, an empty expert and k=1 exercise the split/concat bookkeeping of the reference
    run_case("ragged", synthetic.MoEWorkload("ragged", 6, 1, 40, 24, 19, dtype="fp32"), seed=3, store_inputs=True)
    swiglu_case()
    rmsnorm_case()
