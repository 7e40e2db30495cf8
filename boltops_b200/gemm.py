"""Dense block-scaled GEMM on the grouped-GEMM kernel (one "expert").

Same call surface as the reference's ``gemm_a8w8_blockscale``
(boltops/gemm/gemm_a8w8_blockscale.py:10-70 in the reference project) and
``w8a8_triton_block_scaled_mm`` for the recipe the fused-MoE path uses: e4m3 or int8
operands, A scales per row and 128 K elements, B scales per 128x128 block.  It is the
op a DeepSeek-style layer calls next to ``fused_experts`` (shared experts, dense layers).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _cabi
from .fused_moe import ops


def gemm_a8w8_blockscale(x: torch.Tensor, w: torch.Tensor, x_scale: torch.Tensor,
                         w_scale: torch.Tensor, dtype: Optional[torch.dtype] = torch.bfloat16,
                         out: Optional[torch.Tensor] = None, config=None, backend=None):
    """``y[m, n] = sum_kb (x[m, kb] . w[n, kb]) * x_scale[m, kb] * w_scale[n//128, kb]``.

    x [M, K] and w [N, K] e4m3 or int8 (same dtype), x_scale [M, K/128], w_scale
    [N/128, K/128] floating point; K and N multiples of 128.  ``config`` / ``backend``
    are accepted for signature compatibility and ignored (one kernel, one schedule)."""
    if dtype is None:
        dtype = torch.bfloat16
    if not x.is_cuda:
        raise ValueError("boltops_b200 kernels need CUDA tensors (there is no CPU path)")
    if x.dtype != w.dtype or x.dtype not in (torch.float8_e4m3fn, torch.int8):
        raise TypeError("x and w must both be float8_e4m3fn or int8")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or k % 128 or n % 128:
        raise NotImplementedError("K and N must be multiples of 128 (1x128 / 128x128 scale recipe)")
    if tuple(x_scale.shape) != (m, k // 128) or tuple(w_scale.shape) != (n // 128, k // 128):
        raise ValueError("scale shapes do not match the 1x128 / 128x128 recipe")
    kind = _cabi.GEMM_FP8_BLOCK if x.dtype == torch.float8_e4m3fn else _cabi.GEMM_INT8_BLOCK
    dev = x.device
    cap = ops.ceil_to(max(m, 1), 128)
    x = x.contiguous()
    if cap != m:
        xp = torch.zeros((cap, k), dtype=x.dtype, device=dev)
        xp[:m] = x
        x = xp
    a_scale = torch.zeros((k // 128, cap), dtype=torch.float32, device=dev)
    a_scale[:, :m] = x_scale.float().t()
    direct = out is not None and cap == m
    if out is not None:
        assert out.shape == (m, n) and out.dtype == dtype and out.is_contiguous()
    c = out if direct else torch.empty((cap, n), dtype=dtype, device=dev)
    expert_ids = torch.zeros(cap // 128, dtype=torch.int32, device=dev)
    num_valid = torch.full((1,), cap, dtype=torch.int32, device=dev)
    ops.grouped_gemm(kind=kind, epilogue=_cabi.EPI_STORE, a=x, b=w.contiguous().unsqueeze(0), c=c,
                     sorted_expert_ids=expert_ids, num_valid=num_valid, a_scale=a_scale,
                     a_scale_ld=cap, b_scale=w_scale.float().contiguous().unsqueeze(0))
    if direct:
        return out
    if out is not None:
        out.copy_(c[:m])
        return out
    return c[:m]


def w8a8_block_scaled_mm(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                         block_size: Sequence[int], output_dtype: torch.dtype = torch.float16):
    """vLLM/SGLang-style name of the same operation (B is [N, K], ``block_size`` [128, 128])."""
    if list(block_size) != [128, 128]:
        raise NotImplementedError("only block_size [128, 128] is built in boltops_b200")
    return gemm_a8w8_blockscale(A, B, As, Bs, dtype=output_dtype)


w8a8_triton_block_scaled_mm = w8a8_block_scaled_mm
w8a8_block_int8_matmul = w8a8_block_scaled_mm
