"""Seeded synthetic inputs for the MoE layer workloads.

The reference measures on no dataset; every workload here is random data with the shapes and value
distributions of the benchmark configurations.  numpy's legacy `RandomState` is used for anything
that a committed fixture depends on, because its stream is stable across numpy and torch versions.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np
import torch


@dataclass(frozen=True)
class MoEWorkload:
    name: str
    num_experts: int
    top_k: int
    hidden: int
    intermediate: int
    tokens: int
    dtype: str = "bf16"
    weight_std: float = 0.02
    routing: str = "gate"  # "gate" | "normal_logits" | "zipf" | "sigmoid"
    shared_experts: int = 0

    @property
    def routed_rows(self) -> int:
        return self.tokens * self.top_k

    def flops_fwd_bwd(self) -> float:
        """Routed-expert GEMM work of one forward + backward pass of a GLU expert layer."""
        f = 18.0 * self.tokens * self.top_k * self.hidden * self.intermediate
        f += 18.0 * self.tokens * self.shared_experts * self.hidden * self.intermediate
        return f


WORKLOADS = {
    "tiny": MoEWorkload("tiny", 4, 2, 64, 128, 48, dtype="fp32"),
    "c1": MoEWorkload("c1", 8, 2, 256, 512, 256, dtype="fp32"),
    "c2": MoEWorkload("c2", 8, 2, 4096, 14336, 16384),
    "c3": MoEWorkload("c3", 64, 6, 2048, 1408, 32768, routing="normal_logits", shared_experts=2),
    "c4": MoEWorkload("c4", 128, 8, 2048, 768, 65536, routing="zipf"),
    "c5": MoEWorkload("c5", 256, 8, 7168, 2048, 131072, weight_std=0.006, routing="sigmoid"),
}

TORCH_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def scaled(w: MoEWorkload, **kw) -> MoEWorkload:
    return replace(w, **kw)


def _normal(rs: np.random.RandomState, shape, std=1.0) -> torch.Tensor:
    return torch.from_numpy((rs.standard_normal(size=shape) * std).astype(np.float32))


def make_weights(w: MoEWorkload, seed: int = 0, expert_slice: slice | None = None):
    """fp32 CPU tensors gate (E,H), w_fc (E,2I,H), w_proj (E,H,I) (+ shared), N(0, std).

    Weights are drawn expert by expert so that a rank holding a slice of the experts can draw only
    its own without changing the values.
    """
    E, H, I = w.num_experts, w.hidden, w.intermediate
    gate = _normal(np.random.RandomState(seed * 7919 + 1), (E, H), w.weight_std)
    experts = range(E)[expert_slice] if expert_slice is not None else range(E)
    fc, proj = [], []
    for e in experts:
        rs = np.random.RandomState((seed * 7919 + 1000 + e) % (2**31))
        fc.append(_normal(rs, (2 * I, H), w.weight_std))
        proj.append(_normal(rs, (H, I), w.weight_std))
    out = dict(gate=gate, w_fc=torch.stack(fc), w_proj=torch.stack(proj))
    if w.shared_experts:
        rs = np.random.RandomState(seed * 7919 + 500)
        out["w_fc_shared"] = _normal(rs, (w.shared_experts, 2 * I, H), w.weight_std)
        out["w_proj_shared"] = _normal(rs, (w.shared_experts, H, I), w.weight_std)
    return out


def make_tokens(w: MoEWorkload, seed: int = 0, tokens: int | None = None):
    """x ~ N(0,1) and the upstream gradient g ~ N(0,1), fp32 CPU, (T,H) each."""
    T = w.tokens if tokens is None else tokens
    rs = np.random.RandomState(seed * 7919 + 2)
    return _normal(rs, (T, w.hidden)), _normal(rs, (T, w.hidden))


def make_routing(w: MoEWorkload, x: torch.Tensor, gate: torch.Tensor, seed: int = 0):
    """(router_weights fp32 (T,k), selected_experts int64 (T,k)) for the workload's routing mode.

    "gate": top-k of x @ gate^T, softmax over the selected logits (the reference's own router).
    "normal_logits": logits ~ N(0,1) iid per (token, expert), softmax over the top-k.
    "sigmoid": logits ~ N(0,1), sigmoid scores of the top-k normalised to sum one.
    "zipf": k distinct experts per token drawn without replacement with p ~ rank^-1.2,
            weights = softmax of N(0,1) values.
    """
    T, E, k = x.shape[0], w.num_experts, w.top_k
    g = torch.Generator().manual_seed(seed * 7919 + 3)
    if w.routing == "gate":
        logits = x.float() @ gate.float().t()
        vals, idx = logits.topk(k, dim=-1) if k > 1 else logits.max(-1, keepdim=True)
        return torch.softmax(vals, -1), idx
    if w.routing in ("normal_logits", "sigmoid"):
        logits = torch.randn(T, E, generator=g)
        vals, idx = logits.topk(k, dim=-1)
        if w.routing == "sigmoid":
            s = torch.sigmoid(vals)
            return s / s.sum(-1, keepdim=True), idx
        return torch.softmax(vals, -1), idx
    if w.routing == "zipf":
        p = torch.arange(1, E + 1, dtype=torch.float64).pow(-1.2)
        idx = torch.multinomial((p / p.sum()).expand(T, E), k, replacement=False, generator=g)
        vals = torch.randn(T, k, generator=g)
        return torch.softmax(vals, -1), idx
    raise ValueError(w.routing)
