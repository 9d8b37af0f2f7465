"""Injection of the sm_100a kernels into existing models, at graph level and at module level.

Graph level mirrors the reference's `CuteInductor` (`cute_kernels/cute_inductor/compiler.py:14-49`): a
`torch.compile` backend that walks the captured graph, lets a list of replace functions rewrite it and hands the
graph back.  `replace_swiglu_unchunked` is the counterpart of `cute_kernels/cute_inductor/swiglu_unchunked.py:54-72`:
it finds `up, gate = x.chunk(2, dim=-1); up * F.silu(gate)` and substitutes the fused operator.

Module level: `swap_moe_modules` replaces every MoE layer of the reference's shape (`MoE_Torch` / `MoE_Triton`,
`cute_kernels/kernels/scattermoe/torch_implementation.py:62-99`) inside a model by `MoE_B200`, adopting the existing
parameters (no copy, so optimiser state and `state_dict` keys stay valid).
"""

from __future__ import annotations

import operator
from typing import Callable, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.fx import GraphModule, Node

from .custom_op import set_cute_tracing
from .ops import swiglu_unchunked_cute
from .scattermoe import Experts_B200, MoE_B200

_MUL_TARGETS = (operator.mul, torch.mul)
_SILU_TARGETS = (F.silu, torch.nn.functional.silu)


def _arg(node: Node, position: int, name: str, default=None):
    if name in node.kwargs:
        return node.kwargs[name]
    return node.args[position] if len(node.args) > position else default


def _is_half_split(node: Node) -> bool:
    """`x.chunk(2, dim=-1)` or `torch.chunk(x, 2, dim=-1)`: two halves of the last dimension."""
    if node.op == "call_method" and node.target == "chunk":
        pass
    elif node.op == "call_function" and node.target is torch.chunk:
        pass
    else:
        return False
    if _arg(node, 1, "chunks") != 2:
        return False
    dim = _arg(node, 2, "dim", 0)
    if dim == -1:
        return True
    # a positive dim is the last one only if the rank is known from the captured example value
    val = node.meta.get("example_value", node.meta.get("val"))
    return val is not None and isinstance(val, (tuple, list)) and len(val) == 2 and dim == val[0].dim() - 1


def _halves(node: Node) -> tuple[Node, Node] | None:
    """The two `getitem` users (index 0 = up, index 1 = gate) if they are the split's only users."""
    picks: dict[int, Node] = {}
    for user in node.users:
        if user.op == "call_function" and user.target is operator.getitem and user.args[1] in (0, 1) and user.args[1] not in picks:
            picks[user.args[1]] = user
        else:
            return None
    return (picks[0], picks[1]) if len(picks) == 2 else None


def _only_user(node: Node) -> Node | None:
    return next(iter(node.users)) if len(node.users) == 1 else None


def replace_swiglu_unchunked(gm: GraphModule, node: Node) -> bool:
    """Rewrite one `chunk -> silu -> mul` pattern rooted at `node`; returns whether the graph changed."""
    if not _is_half_split(node):
        return False
    halves = _halves(node)
    if halves is None:
        return False
    up, gate = halves
    silu = _only_user(gate)
    if silu is None or not (
        (silu.op == "call_function" and silu.target in _SILU_TARGETS) or (silu.op == "call_method" and silu.target == "silu")
    ):
        return False
    if silu.kwargs.get("inplace", False):
        return False
    product = _only_user(silu)
    if product is None or _only_user(up) is not product:
        return False
    if not ((product.op == "call_function" and product.target in _MUL_TARGETS) or (product.op == "call_method" and product.target == "mul")):
        return False
    if set(product.all_input_nodes) != {up, silu}:
        return False
    source = _arg(node, 0, "input")
    with gm.graph.inserting_after(node):
        fused = gm.graph.call_function(swiglu_unchunked_cute, args=(source,))
    product.replace_all_uses_with(fused)
    for dead in (product, silu, up, gate, node):
        gm.graph.erase_node(dead)
    return True


class GraphInjector:
    """`torch.compile(model, backend=GraphInjector().compiler)`: apply the replace functions to the captured graph.

    By default the rewritten graph runs as captured (the operators launch the library's kernels directly); with
    `then_inductor=True` it is handed on to torch's inductor the way the reference does.
    """

    def __init__(self, replace_functions: Sequence[Callable[[GraphModule, Node], bool]] = (replace_swiglu_unchunked,), then_inductor: bool = False) -> None:
        self.replace_functions = tuple(replace_functions)
        self.then_inductor = then_inductor
        self.replaced = 0

    def compiler(self, gm: GraphModule, example_inputs: list[torch.Tensor]) -> Callable:
        set_cute_tracing(True)
        try:
            for fn in self.replace_functions:
                for node in list(gm.graph.nodes):
                    if node.graph is gm.graph and not node._erased and fn(gm, node):
                        self.replaced += 1
            gm.graph.lint()
            gm.recompile()
            if self.then_inductor:
                from torch._dynamo import lookup_backend

                return lookup_backend("inductor")(gm, example_inputs)
            return gm.forward
        finally:
            set_cute_tracing(False)


# ---- module level ---------------------------------------------------------------------------------

_MOE_CLASS_NAMES = ("MoE_Torch", "MoE_Triton")


def _looks_like_moe(module: nn.Module) -> bool:
    if isinstance(module, MoE_B200):
        return False
    if type(module).__name__ not in _MOE_CLASS_NAMES:
        return False
    return all(hasattr(module, a) for a in ("gate", "c_fc", "c_proj", "act", "top_k", "num_experts", "hidden_size", "intermediate_size"))


def _adopt_experts(old: nn.Module) -> Experts_B200:
    new = Experts_B200.__new__(Experts_B200)
    nn.Module.__init__(new)
    new.num_experts, new.in_features, new.out_features = old.num_experts, old.in_features, old.out_features
    new.std = getattr(old, "std", None)
    new.weight = old.weight
    new.bias = getattr(old, "bias", None)
    return new


def adopt_moe(old: nn.Module) -> MoE_B200:
    """A `MoE_B200` that owns the very parameters of `old` (an MoE layer with the reference's attributes)."""
    new = MoE_B200.__new__(MoE_B200)
    nn.Module.__init__(new)
    new.num_experts, new.top_k = old.num_experts, old.top_k
    new.hidden_size, new.intermediate_size = old.hidden_size, old.intermediate_size
    new.is_glu = getattr(old, "is_glu", old.c_fc.out_features == 2 * old.intermediate_size)
    new.router_scoring = getattr(old, "router_scoring", "softmax")
    new.num_shared_experts = getattr(old, "num_shared_experts", 0)
    new.gate = old.gate
    new.c_fc = _adopt_experts(old.c_fc)
    new.act = old.act
    new.c_proj = _adopt_experts(old.c_proj)
    if new.num_shared_experts > 0:
        new.shared_c_fc, new.shared_c_proj = old.shared_c_fc, old.shared_c_proj
    new.train(old.training)
    return new


def swap_moe_modules(model: nn.Module) -> int:
    """Replace, in place, every MoE layer named like the reference's by `MoE_B200`; returns how many were swapped.

    Pass the parent model; a bare MoE layer has no parent to re-bind it in, use `adopt_moe` for that.
    """
    swapped = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if _looks_like_moe(child):
                setattr(parent, name, adopt_moe(child))
                swapped += 1
    return swapped
