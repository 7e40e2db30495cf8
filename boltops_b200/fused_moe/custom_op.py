"""``torch.ops.boltops_b200.fused_experts_impl``: the layer as a registered torch operator
with a fake (meta) implementation, so graphs traced by ``torch.compile`` / FakeTensorMode see
the output shape without running a kernel.  Mirrors the reference's registration of
``boltops::fused_experts_impl`` (boltops/utility/torch_guard.py:34-182 and
boltops/fused_moe/triton/fused_moe.py:727-774,892-898,1200 in the reference project): the
operator takes every argument of ``fused_experts_impl`` -- the MX recipes and the SITU
activation parameters included -- and, like the reference's, hands back ``hidden_states``
itself when ``inplace=True`` (no copy).

Import this module to register the operator; ``fused_experts`` itself does not depend on it.
"""
from __future__ import annotations

import torch

from .layer import fused_experts_impl as _impl

_SCHEMA = (
    "fused_experts_impl(Tensor(a!) hidden_states, Tensor w1, Tensor w2, Tensor topk_weights, "
    "Tensor topk_ids, ScalarType? output_dtype=None, bool inplace=False, str activation='silu', "
    "bool? is_gated=None, Tensor? b1=None, Tensor? b2=None, "
    "bool apply_router_weight_on_input=False, bool use_fp8_w8a8=False, bool use_int8_w8a8=False, "
    "bool use_int8_w8a16=False, bool use_int4_w4a16=False, bool use_int4_w4a8=False, "
    "bool per_channel_quant=False, int global_num_experts=-1, Tensor? expert_map=None, "
    "Tensor? w1_scale=None, Tensor? w2_scale=None, Tensor? w1_zp=None, Tensor? w2_zp=None, "
    "Tensor? a1_scale=None, Tensor? a2_scale=None, int[]? block_shape=None, "
    "bool no_combine=False, float? routed_scaling_factor=1.0, float? gemm1_alpha=None, "
    "float? gemm1_limit=None, float? activation_situ_beta=None, "
    "float? activation_situ_linear_beta=None, bool use_mxfp4_w4a8=False, bool use_ue8m0=False, "
    "bool use_mxfp8=False, float? gemm1_beta=None) -> Tensor"
)

_lib = torch.library.Library("boltops_b200", "FRAGMENT")
_lib.define(_SCHEMA)


def _fused_experts_cuda(hidden_states, w1, w2, topk_weights, topk_ids, *args, **kwargs):
    return _impl(hidden_states, w1, w2, topk_weights, topk_ids, *args, **kwargs)


def _fused_experts_fake(hidden_states, w1, w2, topk_weights, topk_ids, output_dtype=None,
                        inplace=False, activation="silu", is_gated=None, b1=None, b2=None,
                        apply_router_weight_on_input=False, use_fp8_w8a8=False,
                        use_int8_w8a8=False, use_int8_w8a16=False, use_int4_w4a16=False,
                        use_int4_w4a8=False, per_channel_quant=False, global_num_experts=-1,
                        expert_map=None, w1_scale=None, w2_scale=None, w1_zp=None, w2_zp=None,
                        a1_scale=None, a2_scale=None, block_shape=None, no_combine=False,
                        routed_scaling_factor=1.0, gemm1_alpha=None, gemm1_limit=None,
                        activation_situ_beta=None, activation_situ_linear_beta=None,
                        use_mxfp4_w4a8=False, use_ue8m0=False, use_mxfp8=False, gemm1_beta=None):
    m, topk = topk_ids.shape
    dtype = hidden_states.dtype if output_dtype is None else output_dtype
    shape = (m, topk, w2.shape[1]) if no_combine else (m, w2.shape[1])
    return torch.empty(shape, dtype=dtype, device=hidden_states.device)


_lib.impl("fused_experts_impl", _fused_experts_cuda, "CUDA")
# CPU tensors reach the layer's own "no CPU path" error instead of a dispatcher error
_lib.impl("fused_experts_impl", _fused_experts_cuda, "CPU")
torch.library.register_fake("boltops_b200::fused_experts_impl", _fused_experts_fake, lib=_lib)

fused_experts_op = torch.ops.boltops_b200.fused_experts_impl
