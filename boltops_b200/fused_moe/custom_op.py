"""``torch.ops.boltops_b200.fused_experts_impl``: the layer as a registered torch custom op
with a fake (meta) implementation, so graphs traced by ``torch.compile`` / FakeTensorMode see
the output shape without running a kernel.  Mirrors the reference's registration of
``boltops::fused_experts_impl`` (boltops/utility/torch_guard.py:34-182 and
boltops/fused_moe/triton/fused_moe.py:727-774,892-898 in the reference project).

Import this module to register the op; ``fused_experts`` itself does not depend on it.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .layer import fused_experts_impl as _impl


@torch.library.custom_op("boltops_b200::fused_experts_impl", mutates_args=("hidden_states",))
def fused_experts_op(
    hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
    topk_ids: torch.Tensor, output_dtype: Optional[torch.dtype] = None, inplace: bool = False,
    activation: str = "silu", is_gated: Optional[bool] = None, b1: Optional[torch.Tensor] = None,
    b2: Optional[torch.Tensor] = None, apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False, use_int8_w8a8: bool = False, per_channel_quant: bool = False,
    global_num_experts: int = -1, expert_map: Optional[torch.Tensor] = None,
    w1_scale: Optional[torch.Tensor] = None, w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None, a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[List[int]] = None, no_combine: bool = False,
    routed_scaling_factor: float = 1.0, gemm1_alpha: Optional[float] = None,
    gemm1_limit: Optional[float] = None, use_ue8m0: bool = False,
) -> torch.Tensor:
    out = _impl(hidden_states, w1, w2, topk_weights, topk_ids, output_dtype=output_dtype,
                inplace=inplace, activation=activation, is_gated=is_gated, b1=b1, b2=b2,
                apply_router_weight_on_input=apply_router_weight_on_input,
                use_fp8_w8a8=use_fp8_w8a8, use_int8_w8a8=use_int8_w8a8,
                per_channel_quant=per_channel_quant, global_num_experts=global_num_experts,
                expert_map=expert_map, w1_scale=w1_scale, w2_scale=w2_scale, a1_scale=a1_scale,
                a2_scale=a2_scale, block_shape=block_shape, no_combine=no_combine,
                routed_scaling_factor=routed_scaling_factor, gemm1_alpha=gemm1_alpha,
                gemm1_limit=gemm1_limit, use_ue8m0=use_ue8m0)
    # a custom op may not return one of its inputs: the in-place variant hands back a view-free copy
    return out.clone() if inplace else out


@fused_experts_op.register_fake
def _fused_experts_fake(hidden_states, w1, w2, topk_weights, topk_ids, output_dtype=None,
                        inplace=False, activation="silu", is_gated=None, b1=None, b2=None,
                        apply_router_weight_on_input=False, use_fp8_w8a8=False,
                        use_int8_w8a8=False, per_channel_quant=False, global_num_experts=-1,
                        expert_map=None, w1_scale=None, w2_scale=None, a1_scale=None,
                        a2_scale=None, block_shape=None, no_combine=False,
                        routed_scaling_factor=1.0, gemm1_alpha=None, gemm1_limit=None,
                        use_ue8m0=False):
    m, topk = topk_ids.shape
    dtype = hidden_states.dtype if output_dtype is None else output_dtype
    shape = (m, topk, w2.shape[1]) if no_combine else (m, w2.shape[1])
    return torch.empty(shape, dtype=dtype, device=hidden_states.device)
