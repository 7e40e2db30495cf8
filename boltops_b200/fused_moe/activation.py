"""MoE expert activations: name registry and the ``moe_activation`` entry.

Mirrors the reference's public contract (reference paths relative to its root):
``normalize_moe_activation`` / ``moe_activation_output_size`` /
``moe_activation`` in boltops/fused_moe/triton/moe_activation.py:1335-1525
(same names, argument meaning and error behaviour).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _cabi
from .._cabi import check, dtype_code, ptr, stream_of

_ALIASES = {
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_pytorch_tanh_no_mul": "gelu_tanh_no_mul",
}

# name -> (default gated?, allowed gated modes)
_SPECS = {
    "silu": (True, (False, True)),
    "gelu": (True, (False, True)),
    "gelu_tanh": (True, (False, True)),
    "situ": (True, (True,)),
    "swigluoai": (True, (True,)),
    "swiglustep": (True, (True,)),
    "silu_no_mul": (False, (False,)),
    "gelu_no_mul": (False, (False,)),
    "gelu_tanh_no_mul": (False, (False,)),
    "relu2": (False, (False,)),
    "relu2_no_mul": (False, (False,)),
}


def normalize_moe_activation(activation: str, is_gated: Optional[bool] = None) -> Tuple[str, bool]:
    """Normalise an activation name and resolve whether it is gated."""
    name = _ALIASES.get(activation.lower(), activation.lower())
    spec = _SPECS.get(name)
    if spec is None:
        raise ValueError(f"Unsupported activation: {activation}")
    default_gated, modes = spec
    if is_gated is None:
        is_gated = default_gated
    if is_gated not in modes:
        if modes == (False,):
            raise ValueError(f"Activation '{activation}' is non-gated but is_gated=True")
        raise ValueError(f"Activation '{activation}' requires gated mode")
    return name, is_gated


def moe_activation_output_size(n: int, is_gated: bool) -> int:
    """Last-dimension size produced by an MoE activation."""
    if n <= 0:
        raise ValueError("input last dimension must be greater than zero")
    if is_gated and n % 2:
        raise ValueError("gated input last dimension must be even")
    return n // 2 if is_gated else n


def resolve_kernel(activation: str, is_gated: bool, gemm1_alpha: Optional[float],
                   gemm1_limit: Optional[float], activation_situ_beta: Optional[float] = None,
                   activation_situ_linear_beta: Optional[float] = None):
    """Map a normalised (activation, gated) pair + parameters to
    ``(bolt_activation kind, alpha, limit)`` following the dispatch rules of the
    reference's ``_apply_activation`` (moe_activation.py:1382-1476)."""
    if is_gated:
        if activation == "silu":
            if gemm1_alpha is not None:
                if gemm1_limit is None:
                    raise ValueError("gemm1_limit must be set when gemm1_alpha is set")
                return _cabi.ACT_SWIGLU_OAI, float(gemm1_alpha), float(gemm1_limit)
            if gemm1_limit is not None:
                return _cabi.ACT_SILU_CLAMP, 0.0, float(gemm1_limit)
            return _cabi.ACT_SILU, 0.0, 0.0
        if activation in ("gelu", "gelu_tanh"):
            if gemm1_alpha is not None or gemm1_limit is not None:
                raise ValueError(
                    f"gemm1_alpha/gemm1_limit are not supported for gated {activation.upper()}")
            return (_cabi.ACT_GELU if activation == "gelu" else _cabi.ACT_GELU_TANH), 0.0, 0.0
        if activation == "swiglustep":
            if gemm1_alpha is not None:
                raise ValueError("gemm1_alpha is not supported for swiglustep")
            return _cabi.ACT_SWIGLU_STEP, 0.0, 7.0 if gemm1_limit is None else float(gemm1_limit)
        if activation == "situ":
            if gemm1_alpha is not None or gemm1_limit is not None:
                raise ValueError("gemm1_alpha/gemm1_limit are not supported for SITU")
            if activation_situ_beta is None:
                raise ValueError("SITU requires activation_situ_beta")
            lin = 0.0 if activation_situ_linear_beta is None else float(activation_situ_linear_beta)
            return _cabi.ACT_SITU, float(activation_situ_beta), lin
        if activation == "swigluoai":
            # interleaved [g0, u0, g1, u1, ...] layout, defaults alpha 1.702 / limit 7
            alpha = 1.702 if gemm1_alpha is None else float(gemm1_alpha)
            limit = 7.0 if gemm1_limit is None else float(gemm1_limit)
            return _cabi.ACT_SWIGLU_OAI_INTERLEAVED, alpha, limit
        raise ValueError(f"Unsupported gated activation: {activation}")
    if activation in ("silu", "silu_no_mul"):
        return _cabi.ACT_SILU, 0.0, 0.0
    if activation in ("gelu", "gelu_no_mul"):
        return _cabi.ACT_GELU, 0.0, 0.0
    if activation in ("gelu_tanh", "gelu_tanh_no_mul"):
        return _cabi.ACT_GELU_TANH, 0.0, 0.0
    if activation in ("relu2", "relu2_no_mul"):
        return _cabi.ACT_RELU2, 0.0, 0.0
    raise ValueError(f"Unsupported non-gated activation: {activation}")


def apply_activation(activation: str, is_gated: bool, activated_out: torch.Tensor,
                     ffn1_out_2d: torch.Tensor, gemm1_alpha: Optional[float] = None,
                     gemm1_limit: Optional[float] = None,
                     activation_situ_beta: Optional[float] = None,
                     activation_situ_linear_beta: Optional[float] = None,
                     rows_dev: Optional[torch.Tensor] = None) -> None:
    """Launch the activation kernel (no validation of shapes)."""
    kind, alpha, limit = resolve_kernel(activation, is_gated, gemm1_alpha, gemm1_limit,
                                        activation_situ_beta, activation_situ_linear_beta)
    lib = _cabi.load()
    rows, n_out = activated_out.shape
    with _cabi.on_device(ffn1_out_2d.device):
        check(lib.bolt_moe_activation(ptr(ffn1_out_2d), ptr(activated_out),
                                      dtype_code(ffn1_out_2d.dtype), rows, n_out, kind,
                                      int(is_gated), alpha, limit, ptr(rows_dev),
                                      stream_of(ffn1_out_2d)))
    from . import ops
    ops._count()


def moe_activation(activated_out: torch.Tensor, ffn1_out_2d: torch.Tensor,
                   activation: str = "silu", is_gated: Optional[bool] = None, *,
                   gemm1_alpha: Optional[float] = None, gemm1_limit: Optional[float] = None,
                   activation_situ_beta: Optional[float] = None,
                   activation_situ_linear_beta: Optional[float] = None) -> None:
    """Apply an MoE activation into a caller-owned 2-D output tensor."""
    activation, is_gated = normalize_moe_activation(activation, is_gated)
    if ffn1_out_2d.ndim != 2 or activated_out.ndim != 2:
        raise ValueError("ffn1_out_2d and activated_out must both be 2D")
    if not ffn1_out_2d.is_cuda or not activated_out.is_cuda:
        raise ValueError("moe_activation only supports CUDA/HIP tensors")
    if ffn1_out_2d.device != activated_out.device:
        raise ValueError("activated_out and ffn1_out_2d must be on the same device")
    if not ffn1_out_2d.is_floating_point() or not activated_out.is_floating_point():
        raise TypeError("activation input and output must have floating-point dtypes")
    if not ffn1_out_2d.is_contiguous() or not activated_out.is_contiguous():
        raise ValueError("activation input and output must be contiguous")
    rows, n = ffn1_out_2d.shape
    output_n = moe_activation_output_size(n, is_gated)
    if activated_out.shape != (rows, output_n):
        raise ValueError(
            f"activated_out shape must be {(rows, output_n)}, got {tuple(activated_out.shape)}")
    if activated_out.dtype != ffn1_out_2d.dtype:
        raise TypeError("activation input and output must share a dtype")
    if ffn1_out_2d.numel() == 0:
        return
    apply_activation(activation, is_gated, activated_out, ffn1_out_2d, gemm1_alpha, gemm1_limit,
                     activation_situ_beta, activation_situ_linear_beta)


def activation_quant(ffn1_out_2d: torch.Tensor, activation: str, is_gated: bool,
                     quant_dtype: torch.dtype, row_multiplier: Optional[torch.Tensor] = None,
                     rows_dev: Optional[torch.Tensor] = None):
    """Fused activation + per-token quantisation (reference:
    ``triton_activation_quant``, moe_activation.py:1239-1332).  Returns ``(q, scale[rows,1])``."""
    kind, _, _ = resolve_kernel(activation, is_gated, None, None)
    lib = _cabi.load()
    rows, n = ffn1_out_2d.shape
    n_out = moe_activation_output_size(n, is_gated)
    q = torch.empty((rows, n_out), dtype=quant_dtype, device=ffn1_out_2d.device)
    scale = torch.empty((rows, 1), dtype=torch.float32, device=ffn1_out_2d.device)
    if row_multiplier is not None:
        row_multiplier = row_multiplier.to(torch.float32).contiguous()
    with _cabi.on_device(ffn1_out_2d.device):
        check(lib.bolt_act_quant(ptr(ffn1_out_2d), dtype_code(ffn1_out_2d.dtype), rows, n_out, kind,
                                 int(is_gated), dtype_code(quant_dtype), ptr(row_multiplier),
                                 ptr(q), ptr(scale), ptr(rows_dev), stream_of(ffn1_out_2d)))
    from . import ops
    ops._count()
    return q, scale
