"""Router front-end for the fused-MoE layer.

``fused_topk`` has the signature and semantics of the reference helper of the same name
(boltops/tools/fused_moe_triton_tune/routing.py:10-35 in the reference project): softmax or
sigmoid scores of the gating logits in fp32, top-k, optional renormalisation, int32 ids.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi
from .._cabi import check, dtype_code, ptr, stream_of


def fused_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, topk: int,
               renormalize: bool, topk_ids: Optional[torch.Tensor] = None,
               topk_weights: Optional[torch.Tensor] = None, is_softmax: bool = True):
    assert hidden_states.shape[0] == gating_output.shape[0]
    if not gating_output.is_cuda:
        raise ValueError("boltops_b200 kernels need CUDA tensors (there is no CPU path)")
    lib = _cabi.load()
    m, e = gating_output.shape
    gating_output = gating_output.contiguous()
    dev = gating_output.device
    weights = torch.empty((m, topk), dtype=torch.float32, device=dev)
    ids = torch.empty((m, topk), dtype=torch.int32, device=dev)
    with _cabi.on_device(dev):
        check(lib.bolt_fused_topk(ptr(gating_output), dtype_code(gating_output.dtype), m, e, topk,
                                  int(renormalize), int(is_softmax), ptr(weights), ptr(ids),
                                  stream_of(gating_output)))
    from . import ops
    ops._count()
    if topk_weights is not None:
        topk_weights.copy_(weights)
        weights = topk_weights
    if topk_ids is not None:
        topk_ids.copy_(ids)
        ids = topk_ids
    return weights, ids


def moe_fused_gate(input: torch.Tensor, bias: torch.Tensor, topk_weights: torch.Tensor,
                   topk_ids: torch.Tensor, num_expert_group: int, topk_group: int, topk: int,
                   num_fused_shared_experts: int, routed_scaling_factor: float = 1.0):
    """Grouped gate with optional fused shared expert; same arguments and outputs as the
    reference helper (boltops/tools/fused_moe_triton_tune/routing.py:38-79).  Writes into the
    caller's ``topk_weights`` (fp32) / ``topk_ids`` (int32) and returns them as a list."""
    if not input.is_cuda:
        raise ValueError("boltops_b200 kernels need CUDA tensors (there is no CPU path)")
    assert topk_weights.dtype == torch.float32 and topk_ids.dtype == torch.int32
    assert topk_weights.is_contiguous() and topk_ids.is_contiguous()
    lib = _cabi.load()
    m, e = input.shape
    x = input.contiguous()
    b = bias.float().contiguous()
    with _cabi.on_device(x.device):
        check(lib.bolt_moe_fused_gate(ptr(x), dtype_code(x.dtype), ptr(b), m, e, num_expert_group,
                                      topk_group, topk, num_fused_shared_experts,
                                      float(routed_scaling_factor), ptr(topk_weights),
                                      ptr(topk_ids), stream_of(x)))
    from . import ops
    ops._count()
    return [topk_weights, topk_ids]
