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
    with torch.cuda.device(dev):
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
