"""B200-native (sm_100a) implementation of the scattermoe MoE layer path."""

from .custom_op import set_cute_tracing
from .ops import combine, contiguous_count_cute, gate_grad, group, group_bwd_W, rmsnorm_cute, rmsnorm_torch, scatter2scatter, swiglu_unchunked_cute, swiglu_unchunked_torch
from .scattermoe import (
    Experts_B200,
    Experts_Torch,
    Experts_Triton,
    MoE_B200,
    MoE_Torch,
    MoE_Triton,
    fused_swiglu_experts,
    route,
    scattered_experts,
)
from .inject import GraphInjector, adopt_moe, replace_swiglu_unchunked, swap_moe_modules
from .router import fused_rmsnorm_router, fused_router, router_forward
