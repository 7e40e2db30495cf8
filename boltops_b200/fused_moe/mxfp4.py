"""MXFP4 (w4a8) experts (`use_mxfp4_w4a8=True`): packed e2m1 weights with one E8M0 byte per
32 K elements, e4m3 activations.

Reference semantics (boltops/fused_moe/triton/fused_moe.py:923-1197 and the CPU statement in
test/fused_moe/test_fused_moe.py:1411-1563 of the reference project).  Two recipes:

* dynamic (``a2_scale is None``): activations quantised per 1 x 128 group with a power-of-two
  scale; GEMM1 rounded to the output dtype; SiLU (rounded through bf16), ``swiglustep`` or ``situ``;
  second quantisation; GEMM2 rounded to the output dtype; the router weights enter in the fp32 sum
  over a token's routes -- or multiply the input when ``apply_router_weight_on_input`` (top-1).
* static (``a1_scale`` and ``a2_scale`` one fp32 value each): ``e4m3(x / a1_scale)``, GEMM1 times
  ``a1_scale`` plus bias, SwiGLU-OAI with ``gemm1_alpha`` / ``gemm1_limit``, times the router weight
  when it is applied on the input, ``e4m3(act / a2_scale)``, GEMM2 times ``a2_scale`` plus bias,
  times the router weight otherwise; fp32 sum.

How it runs here.  The dynamic recipe on 16-bit input runs on the tensor core's block-scaled
kind (``BOLT_GEMM_MXFP4``): the packed weights and their E8M0 bytes are read as stored (a quarter
of the bytes of a decoded copy), the activation codes carry their power-of-two group scale as four
equal E8M0 bytes, and the tensor core applies both scales per 32 K elements.  The other variants
(static scales, pre-quantised input) and ``BOLTOPS_B200_MXFP4=decoded`` use the fact that an e2m1
or e4m3 code times a power of two is exact in bf16 and that products of two such values are exact
in fp32: the K-grouped scaled contraction then equals a bf16 tensor-core GEMM with fp32
accumulation over DECODED operands; weights are decoded once per (weight, scale) pair and cached,
activations by the kernel that quantises them.
"""
from __future__ import annotations

import ctypes as C
import os
import weakref
from typing import Optional

import torch

from .. import _cabi
from .._cabi import check, dtype_code, ptr, stream_of
from . import ops
from .activation import apply_activation

_decoded = {}
_NATIVE = os.environ.get("BOLTOPS_B200_MXFP4", "native") != "decoded"
# native kind, SiLU: the activation and the second quantisation run in GEMM1's epilogue
# (BOLTOPS_B200_MXFP4_FUSED=0: plain GEMM1 + the stand-alone kernel; same codes bit for bit)
_FUSED = os.environ.get("BOLTOPS_B200_MXFP4_FUSED", "1") != "0"


def _decode_weights(w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 [E, N, K/2] + E8M0 bytes [E, N, K/32] -> bf16 [E, N, K]; decoded once per
    (weight, scale) pair and kept while both tensors are alive and unmodified."""
    key = (w.data_ptr(), scale.data_ptr(), tuple(w.shape), w._version, scale._version)
    hit = _decoded.get(key)
    if hit is not None and hit[0]() is w and hit[1]() is scale:
        return hit[2]
    for k in [k for k, v in _decoded.items() if v[0]() is None or v[1]() is None]:
        del _decoded[k]
    e, n, kp = w.shape
    out = torch.empty((e, n, 2 * kp), dtype=torch.bfloat16, device=w.device)
    wc, sc = w.contiguous(), scale.contiguous()
    with _cabi.on_device(w.device):
        check(_cabi.load().bolt_mxfp4_decode(ptr(wc), ptr(sc), e * n, 2 * kp, ptr(out),
                                             _cabi.BF16, stream_of(w)))
    ops._count()
    _decoded[key] = (weakref.ref(w), weakref.ref(scale), out)
    return out


def act_quant(x: torch.Tensor, *, gated: bool = False, limit: Optional[float] = None,
              static_scale: Optional[torch.Tensor] = None, want_codes: bool = False,
              want_deq: bool = True, want_sf: bool = False):
    """Quantise-and-decode ``x`` [rows, cols] (``[rows, 2 * cols]`` = [gate | up] with ``gated``).
    Returns ``(decoded bf16 [rows, cols], codes or None, fp32 scales [rows, cols/128] or None)``;
    with ``want_sf`` a fourth value, the E8M0 byte of every 32 elements ``[rows, cols/32]``."""
    rows = x.shape[0]
    cols = x.shape[1] // 2 if gated else x.shape[1]
    x = x.contiguous()
    deq = torch.empty((rows, cols), dtype=torch.bfloat16, device=x.device) if want_deq else None
    codes = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device) if want_codes else None
    sf = torch.empty((rows, cols // 32), dtype=torch.uint8, device=x.device) if want_sf else None
    static = static_scale is not None or x.dtype == torch.float8_e4m3fn
    scales = None if static or not want_codes else \
        torch.empty((rows, cols // 128), dtype=torch.float32, device=x.device)
    with _cabi.on_device(x.device):
        check(_cabi.load().bolt_mx4_act_quant(
            ptr(x), dtype_code(x.dtype), rows, cols, int(gated), int(limit is not None),
            float(limit or 0.0), int(static), ptr(static_scale), ptr(deq), _cabi.BF16, ptr(codes),
            ptr(scales), ptr(sf), stream_of(x)))
    ops._count()
    if want_sf:
        return deq, codes, scales, sf
    return deq, codes, scales


def group_decode(codes: torch.Tensor, scales: torch.Tensor, group: int) -> torch.Tensor:
    """Pre-quantised activations: e4m3 codes [rows, cols] times fp32 scales [rows, cols/group]."""
    rows, cols = codes.shape
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=codes.device)
    codes, scales = codes.contiguous(), scales.contiguous()
    with _cabi.on_device(codes.device):
        check(_cabi.load().bolt_fp8_group_decode(ptr(codes), ptr(scales), rows, cols, group,
                                                 ptr(out), _cabi.BF16, stream_of(codes)))
    ops._count()
    return out


def _activation_scales_as_float(scale: torch.Tensor, rows: int, cols: int):
    """a1_scale of pre-quantised activations -> (fp32 multipliers [rows, groups], group).  Accepts
    E8M0 bytes or power-of-two fp32 values per 32 or 128 elements, or int32 words packing four
    g128 bytes (the formats boltops/fused_moe/triton/mxfp4.py:159-191 accepts)."""
    if scale is None or scale.ndim != 2:
        raise ValueError("MXFP4 activation scales must be a [rows,groups] tensor")
    groups = (128,) if scale.dtype == torch.int32 else (32, 128)
    for group in groups:
        if cols % group:
            continue
        count = cols // group
        width = (count + 3) // 4 if scale.dtype == torch.int32 else count
        if tuple(scale.shape) == (rows, width):
            if scale.dtype == torch.float32:
                return scale, group
            if scale.dtype == torch.uint8:
                return torch.exp2(scale.float() - 127.0), group
            if scale.dtype == torch.int32:
                b = torch.stack([(scale >> (8 * i)) & 0xFF for i in range(4)], -1)
                return torch.exp2(b.reshape(rows, -1)[:, :count].float() - 127.0), group
            raise ValueError("scales must be UE8M0 bytes, packed int32 or power-of-two FP32")
    raise ValueError("MXFP4 activation scales must describe g128 or unpacked g32")


def validate(hidden_states, w1, w2, topk_ids, w1_scale, w2_scale, a1_scale, a2_scale, b1, b2,
             apply_router_weight_on_input, output_dtype, block_shape, activation, is_gated,
             inplace, no_combine, gemm1_alpha, gemm1_beta) -> bool:
    """The reference's argument checks for this recipe, same order, types and messages
    (fused_moe.py:968-1056).  Returns whether the static recipe is selected."""
    static = a2_scale is not None
    if static:
        for scale in (a1_scale, a2_scale):
            if (scale is None or scale.numel() != 1 or scale.dtype != torch.float32
                    or scale.device != hidden_states.device or not scale.is_contiguous()):
                raise ValueError("static MXFP4 requires a1_scale and a2_scale as one FP32 value "
                                 "on the input device")
    if w1_scale is None or w2_scale is None:
        raise ValueError("MXFP4 requires UE8M0 weight scales and no zero points")
    if block_shape is not None and list(block_shape) != [1, 32]:
        raise ValueError("MXFP4 weight block_shape must be [1, 32]")
    if hidden_states.dtype not in (torch.bfloat16, torch.float16, torch.float8_e4m3fn):
        raise ValueError("MXFP4 experts require BF16/FP16 or prequantized E4M3 activations")
    if not static and (b1 is not None or b2 is not None or gemm1_alpha is not None):
        raise ValueError("dynamic MXFP4 follows DeepGEMM and does not support bias or custom alpha")
    if apply_router_weight_on_input and not static:
        if topk_ids.shape[1] != 1:
            raise ValueError("MXFP4 input routing weights require topk=1, as in vLLM prepare")
        if hidden_states.dtype == torch.float8_e4m3fn:
            raise ValueError("MXFP4 input routing weights must be applied before FP8 quantization; "
                             "provide BF16/FP16 hidden_states")
    if hidden_states.dtype == torch.float8_e4m3fn:
        if a1_scale is None or output_dtype is None:
            raise ValueError("prequantized MXFP4 activations require a1_scale and output_dtype")
    elif a1_scale is not None and not static:
        raise ValueError("a1_scale is only used with prequantized MXFP4 activations")
    resolved = hidden_states.dtype if output_dtype is None else output_dtype
    if resolved not in (torch.bfloat16, torch.float16, torch.float32):
        raise ValueError("MXFP4 output_dtype must be BF16, FP16 or FP32")
    if inplace and resolved != hidden_states.dtype:
        raise ValueError("inplace MXFP4 requires output_dtype to match hidden_states.dtype")
    if hidden_states.dtype == torch.float8_e4m3fn and not static:
        _, group = _activation_scales_as_float(a1_scale, hidden_states.shape[0],
                                               hidden_states.shape[1])
        if group != 128:
            raise ValueError("dynamic MXFP4 fused_experts requires G128 activation scales")
    allowed = ("swigluoai",) if static else ("silu", "swiglustep", "situ")
    if static and gemm1_beta is not None and gemm1_beta != 1.:
        raise ValueError("static MXFP4 SwiGLU-OAI requires gemm1_beta=1")
    if not is_gated or activation not in allowed:
        raise ValueError(f"MXFP4 requires gated {allowed}")
    if gemm1_beta is not None and not static:
        raise ValueError("gemm1_beta requires native MXFP8 or static MXFP4")
    if no_combine:
        assert not inplace, "no_combine + inplace is not supported"
    return static


def fused_experts_mxfp4(hidden_states, w1, w2, topk_weights, topk_ids, *, w1_scale, w2_scale,
                        a1_scale, a2_scale, b1, b2, static: bool, activation: str,
                        output_dtype: Optional[torch.dtype], inplace: bool, no_combine: bool,
                        apply_router_weight_on_input: bool, global_num_experts: int,
                        expert_map: Optional[torch.Tensor], routed_scaling_factor: float,
                        gemm1_alpha, gemm1_limit, activation_situ_beta,
                        activation_situ_linear_beta, chunk: int) -> torch.Tensor:
    if not hidden_states.is_cuda:
        raise ValueError("boltops_b200 kernels need CUDA tensors (there is no CPU path)")
    assert hidden_states.shape[1] == w1.shape[2] * 2, "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.stride(-1) == 1 and w2.stride(-1) == 1, "Stride of last dimension must be 1"
    lib = _cabi.load()
    dev = hidden_states.device
    out_dtype = hidden_states.dtype if output_dtype is None else output_dtype
    num_tokens, hidden = hidden_states.shape
    e_local, n1, _ = w1.shape
    inter = n1 // 2
    model_dim = w2.shape[1]
    topk = topk_ids.shape[1]
    if hidden % 128 or (not static and inter % 128):
        raise NotImplementedError("MXFP4 experts need K dimensions in whole 128-wide groups here")
    if global_num_experts == -1:
        global_num_experts = expert_map.numel() if expert_map is not None else e_local
    if static:
        alpha = 1.702 if gemm1_alpha is None else gemm1_alpha
        limit = 7. if gemm1_limit is None else gemm1_limit
        a1_scale, a2_scale = a1_scale.view(-1), a2_scale.view(-1)
    else:
        limit = 7. if activation == "swiglustep" else gemm1_limit
    native = (_NATIVE and not static and hidden_states.dtype != torch.float8_e4m3fn
              and w1.is_contiguous() and w2.is_contiguous()
              and w1.data_ptr() % 32 == 0 and w2.data_ptr() % 32 == 0)
    if native:
        from .mxfp8 import _tile_weight_scales
        fuse_act = _FUSED and activation == "silu" and inter % 128 == 0
        sfb1 = _tile_weight_scales(w1, w1_scale.contiguous(), gated=fuse_act)
        sfb2 = _tile_weight_scales(w2, w2_scale.contiguous())
    else:
        w1_d = _decode_weights(w1, w1_scale)
        w2_d = _decode_weights(w2, w2_scale)
    expert_mask = (expert_map >= 0).to(torch.int32) if expert_map is not None else None
    ids_all = topk_ids.to(torch.int32)
    wts_all = topk_weights.to(torch.float32)
    needs_weight = not (apply_router_weight_on_input or no_combine)
    b1f = b1.float().contiguous() if b1 is not None else None
    b2f = b2.float().contiguous() if b2 is not None else None

    if inplace:
        out = hidden_states
    elif no_combine:
        out = torch.empty((num_tokens, topk, model_dim), device=dev, dtype=out_dtype)
    else:
        out = torch.empty((num_tokens, model_dim), device=dev, dtype=out_dtype)

    for begin in range(0, num_tokens, chunk):
        end = min(begin + chunk, num_tokens)
        m = end - begin
        x = hidden_states[begin:end]
        ids = ids_all[begin:end].contiguous()
        wts = wts_all[begin:end].contiguous()
        # ---- A1: quantise (or take the caller's codes) and decode -------------------------
        if static:
            a_tok = act_quant(x, static_scale=a1_scale)[0]
        elif x.dtype == torch.float8_e4m3fn:
            s, group = _activation_scales_as_float(a1_scale[begin:end], m, hidden)
            a_tok = group_decode(x, s, group)
        else:
            if apply_router_weight_on_input:
                # multiplied in the input dtype before the quantiser, as the reference prepares it
                x = x * topk_weights[begin:end].to(x.dtype)
            if native:
                _, a_tok, _, a_sf = act_quant(x, want_codes=True, want_deq=False, want_sf=True)
            else:
                a_tok = act_quant(x)[0]
        route_pos = torch.empty((m, topk), device=dev, dtype=torch.int32)
        sorted_ids, sorted_w, expert_ids, num_valid, _, _ = ops.moe_sorting_ck(
            ids, wts, global_num_experts, None, None, ops.SORT_UNIT, expert_mask,
            alloc_moe_buf=False, route_pos=route_pos)
        if expert_map is not None:
            expert_ids = ops.relabel_tiles(expert_ids, expert_map)
        cap = sorted_ids.shape[0]
        a_sorted, _ = ops.gather_rows(a_tok, sorted_ids, num_valid, cap)
        common = dict(kind=_cabi.GEMM_MXFP4 if native else _cabi.GEMM_BF16,
                      sorted_expert_ids=expert_ids, num_valid=num_valid,
                      sorted_ids=sorted_ids, sorted_weights=sorted_w, num_tokens=m, topk=topk)
        if native:
            gemm1 = dict(b=w1, a_scale=ops.mx_sf_layout(a_sf, cap, sorted_ids, num_valid),
                         b_scale=sfb1)
        else:
            gemm1 = dict(b=w1_d)
        # ---- GEMM1, activation, second quantisation ------------------------------------------
        if static:
            g1 = torch.empty((cap, n1), device=dev, dtype=torch.float32)
            ops.grouped_gemm(epilogue=_cabi.EPI_STORE, a=a_sorted, b=w1_d, c=g1, **common)
            act = torch.empty((cap, inter), device=dev, dtype=torch.bfloat16)
            with _cabi.on_device(dev):
                check(lib.bolt_mx4_swiglu_static(
                    ptr(g1), ptr(expert_ids), ptr(num_valid), cap, inter, e_local, ptr(a1_scale),
                    ptr(b1f), float(alpha), float(limit),
                    ptr(sorted_w) if apply_router_weight_on_input else None, ptr(a2_scale),
                    ptr(act), _cabi.BF16, stream_of(g1)))
            ops._count()
        elif native and fuse_act:
            # one kernel: GEMM1, rounding to the output dtype, SiLU(gate) * up through bf16, the
            # 1 x 128 power-of-two quantiser; codes and exponent bytes go straight to GEMM2
            act = torch.empty((cap, inter), device=dev, dtype=torch.float8_e4m3fn)
            act_s = torch.empty((cap, inter // 32), device=dev, dtype=torch.uint8)
            ops.grouped_gemm(epilogue=_cabi.EPI_SILU_MUL_QUANT, a=a_sorted, c=act, c_scale=act_s,
                             c_scale_ld=inter // 32, mid_dtype=out_dtype, act_limit=limit,
                             **gemm1, **common)
            gemm2 = dict(a=act, b=w2, a_scale=ops.mx_sf_layout(act_s, cap), b_scale=sfb2)
        else:
            g1 = torch.empty((cap, n1), device=dev, dtype=out_dtype)
            ops.grouped_gemm(epilogue=_cabi.EPI_STORE, a=a_sorted, c=g1, **gemm1, **common)
            want = dict(want_codes=True, want_deq=False, want_sf=True) if native else {}
            if activation == "silu":
                q2 = act_quant(g1, gated=True, limit=limit, **want)
            else:
                activated = torch.empty((cap, inter), device=dev, dtype=out_dtype)
                apply_activation(activation, True, activated, g1, None, limit,
                                 activation_situ_beta, activation_situ_linear_beta,
                                 rows_dev=num_valid)
                q2 = act_quant(activated, **want)
            if native:
                gemm2 = dict(a=q2[1], b=w2, a_scale=ops.mx_sf_layout(q2[3], cap), b_scale=sfb2)
            else:
                gemm2 = dict(a=q2[0], b=w2_d)
        # ---- GEMM2 and the sum over the routes ------------------------------------------------
        if static:
            g2 = torch.empty((cap, model_dim), device=dev, dtype=torch.float32)
            ops.grouped_gemm(epilogue=_cabi.EPI_STORE, a=act, b=w2_d, c=g2, **common)
            if no_combine:
                routes = out[begin:end].view(m * topk, model_dim)
                if expert_map is not None:
                    routes.zero_()
                dst, scatter = routes, 1
            else:
                dst = torch.empty((cap, model_dim), device=dev, dtype=out_dtype)
                scatter = 0
            with _cabi.on_device(dev):
                check(lib.bolt_mx4_affine_rows(
                    ptr(g2), ptr(expert_ids), ptr(sorted_ids), ptr(num_valid), cap, model_dim,
                    e_local, m, topk, ptr(a2_scale), ptr(b2f),
                    ptr(sorted_w) if needs_weight else None, scatter, ptr(dst),
                    dtype_code(out_dtype), stream_of(g2)))
            ops._count()
            if not no_combine:
                ops.gather_sum(dst, route_pos, out[begin:end], routed_scaling_factor)
        else:
            routes = (torch.zeros if expert_map is not None else torch.empty)(
                (m, topk, model_dim), device=dev, dtype=out_dtype)
            ops.grouped_gemm(epilogue=_cabi.EPI_STORE, c=routes.view(m * topk, model_dim),
                             scatter=True, **gemm2, **common)
            if no_combine:
                out[begin:end].copy_(routes)
            else:
                ops.moe_sum(routes, out[begin:end], routed_scaling_factor,
                            router_weights=wts if needs_weight else None)
    return out
