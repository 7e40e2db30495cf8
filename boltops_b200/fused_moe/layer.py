"""Orchestration of one fused-MoE layer on a B200.

Drop-in for the reference's ``fused_experts`` / ``fused_experts_impl``
(boltops/fused_moe/triton/fused_moe.py:647-724, 1200-1777; reference paths are
relative to the reference project root): same arguments, defaults, error
behaviour and numerics contract; the schedule is B200-native:

    sort (CK format, 128-row units) -> [quantise hidden once per token]
    -> gather (or quantise-and-scatter) rows into the expert-sorted layout
    -> grouped GEMM 1 with SiLU(gate)*up (+ 1x128 re-quantisation) in its epilogue
    -> grouped GEMM 2 with the router weight in its epilogue, rows kept in sorted order
    -> top-k combine that gathers each token's rows through the sort's inverse permutation
       ([M, topk, H] exists only for ``no_combine=True``).

No step synchronises the host; the padded row count stays on the device.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from .. import _cabi
from . import ops
from .activation import apply_activation, normalize_moe_activation

_FLOAT_OUT = (torch.float16, torch.bfloat16, torch.float32)


class StageTimer:
    """Optional per-stage CUDA-event timing of the layer (benchmarks only).

    Assign an instance to ``STAGE_TIMER``; every stage of ``fused_experts_impl`` is
    then bracketed by events on torch's current stream.  ``summary()`` synchronises
    and returns the mean milliseconds per stage."""

    def __init__(self):
        self._events = {}

    def begin(self):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def end(self, name, start):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.setdefault(name, []).append((start, ev))

    def summary(self):
        torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in self._events.items()}


STAGE_TIMER: Optional[StageTimer] = None
# BOLTOPS_B200_ONE_CALL=0 drives the kernels one by one from Python (same results; used by the
# tests to hold the two orchestrations against each other)
_ONE_CALL = os.environ.get("BOLTOPS_B200_ONE_CALL", "1") != "0"
# 16-bit and block-scaled experts: GEMM1 can gather its rows from token order itself (the 16-bit
# input as it is, 8-bit codes written once per token instead of once per route) instead of
# reading a copy in sorted order; same results.  It wins while the sorted layout is mostly tile
# padding and loses once experts have more than a tile of rows (the extra copy instructions slow
# the accumulator promotion down), so it is used up to _GATHER_MAX_AVG_ROWS routes per expert --
# the rule of bolt_moe_layer.  BOLTOPS_B200_GATHER=0 / 1 forces it off / on.
_GATHER = {"0": False, "1": True}.get(os.environ.get("BOLTOPS_B200_GATHER", ""), None)
_GATHER_MAX_AVG_ROWS = 64


def _use_gather(routes: int, experts: int) -> bool:
    if _GATHER is not None:
        return _GATHER
    return routes <= _GATHER_MAX_AVG_ROWS * experts


class _Stage:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        self.t = STAGE_TIMER
        self.start = self.t.begin() if self.t is not None else None

    def __exit__(self, *exc):
        if self.t is not None:
            self.t.end(self.name, self.start)
        return False


def _chunk_size() -> int:
    raw = os.environ.get("BOLTOPS_FUSED_MOE_CHUNK_SIZE",
                         os.environ.get("TRITON_FUSED_MOE_CHUNK_SIZE", "32768"))
    size = int(raw)
    if size <= 0:
        raise ValueError("TRITON_FUSED_MOE_CHUNK_SIZE must be positive")
    return size


def _use_tile_pairs(kind: int, routes: int, experts: int) -> bool:
    """Schedule of the two grouped GEMMs.  In the tile-pair schedule two CTAs of a cluster take
    two row tiles of one expert and share its weight tile (tcgen05 ``cta_group::2``): each CTA
    stages half of the weight tile.  Measured on B200 (same box, same inputs, results bit
    identical): +2-3 % for 16-bit experts with many row tiles per expert (Mixtral shape, 16
    tiles), no change for per-channel 8-bit experts, and slower for the block-scaled kinds,
    whose per-K-block promotion chain now has to wait for the epilogues of two CTAs.  So pairs
    are used for bf16 / fp16 experts from three row tiles per expert on.  The host knows only
    the average (tokens * topk / experts).  ``BOLTOPS_B200_GEMM_SCHEDULE`` = ``tiles`` /
    ``pairs`` overrides the choice."""
    forced = os.environ.get("BOLTOPS_B200_GEMM_SCHEDULE", "auto")
    if forced == "tiles":
        return False
    if forced == "pairs":
        return True
    if kind not in (_cabi.GEMM_BF16, _cabi.GEMM_F16):
        return False
    return routes >= _PAIR_MIN_AVG_ROWS * max(experts, 1)


_PAIR_MIN_AVG_ROWS = 384


def gemm_schedule(kind: int, routes: int, experts: int) -> str:
    """Name of the schedule ``fused_experts`` picks for this problem ("pairs" / "tiles")."""
    return "pairs" if _use_tile_pairs(kind, routes, experts) else "tiles"


def _gemm_kind(w_dtype, use_fp8, use_int8, per_channel, block_shape) -> int:
    if use_fp8:
        return _cabi.GEMM_FP8_CHANNEL if per_channel else _cabi.GEMM_FP8_BLOCK
    if use_int8:
        return _cabi.GEMM_INT8_CHANNEL if per_channel else _cabi.GEMM_INT8_BLOCK
    if w_dtype == torch.bfloat16:
        return _cabi.GEMM_BF16
    if w_dtype == torch.float16:
        return _cabi.GEMM_F16
    raise NotImplementedError(f"unquantised experts in {w_dtype} are not built in boltops_b200")


def fused_experts_impl(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    output_dtype: Optional[torch.dtype] = None,
    inplace: bool = False,
    activation: str = "silu",
    is_gated: Optional[bool] = None,
    b1: Optional[torch.Tensor] = None,
    b2: Optional[torch.Tensor] = None,
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    use_int8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    use_int4_w4a16: bool = False,
    use_int4_w4a8: bool = False,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    expert_map: Optional[torch.Tensor] = None,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    w1_zp: Optional[torch.Tensor] = None,
    w2_zp: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[List[int]] = None,
    no_combine: bool = False,
    routed_scaling_factor: Optional[float] = 1.0,
    gemm1_alpha: Optional[float] = None,
    gemm1_limit: Optional[float] = None,
    activation_situ_beta: Optional[float] = None,
    activation_situ_linear_beta: Optional[float] = None,
    use_mxfp4_w4a8: bool = False,
    use_ue8m0: bool = False,
    use_mxfp8: bool = False,
    gemm1_beta: Optional[float] = None,
    _out_peers=None,
) -> torch.Tensor:
    # ---- variants outside this build -------------------------------------------------
    if use_mxfp4_w4a8 or use_mxfp8:
        name = "MXFP8" if use_mxfp8 else "MXFP4"
        if any((use_fp8_w8a8, use_int8_w8a8, use_int8_w8a16, use_int4_w4a16, use_int4_w4a8,
                per_channel_quant)):
            raise ValueError(f"{name} cannot be combined with other quantization flags")
        if use_mxfp8 and use_mxfp4_w4a8:
            raise ValueError("MXFP8 and MXFP4 are mutually exclusive")
        activation, is_gated = normalize_moe_activation(activation, is_gated)
        if use_mxfp4_w4a8:
            from . import mxfp4
            static = mxfp4.validate(hidden_states, w1, w2, topk_ids, w1_scale, w2_scale, a1_scale,
                                    a2_scale, b1, b2, apply_router_weight_on_input, output_dtype,
                                    block_shape, activation, is_gated, inplace, no_combine,
                                    gemm1_alpha, gemm1_beta)
            return mxfp4.fused_experts_mxfp4(
                hidden_states, w1, w2, topk_weights, topk_ids, w1_scale=w1_scale,
                w2_scale=w2_scale, a1_scale=a1_scale, a2_scale=a2_scale, b1=b1, b2=b2,
                static=static, activation=activation, output_dtype=output_dtype, inplace=inplace,
                no_combine=no_combine, apply_router_weight_on_input=apply_router_weight_on_input,
                global_num_experts=global_num_experts, expert_map=expert_map,
                routed_scaling_factor=1.0 if routed_scaling_factor is None else routed_scaling_factor,
                gemm1_alpha=gemm1_alpha, gemm1_limit=gemm1_limit,
                activation_situ_beta=activation_situ_beta,
                activation_situ_linear_beta=activation_situ_linear_beta, chunk=_chunk_size())
        from . import mxfp8
        mxfp8.validate(hidden_states, w1, w2, w1_scale, w2_scale, a1_scale, a2_scale, b1, b2,
                       apply_router_weight_on_input, output_dtype, block_shape, activation,
                       is_gated, inplace, no_combine)
        return mxfp8.fused_experts_mxfp8(
            hidden_states, w1, w2, topk_weights, topk_ids, w1_scale=w1_scale, w2_scale=w2_scale,
            activation=activation, inplace=inplace, no_combine=no_combine,
            global_num_experts=global_num_experts, expert_map=expert_map,
            routed_scaling_factor=1.0 if routed_scaling_factor is None else routed_scaling_factor,
            gemm1_alpha=gemm1_alpha, gemm1_beta=gemm1_beta, gemm1_limit=gemm1_limit,
            chunk=_chunk_size())
    if use_int8_w8a16 or use_int4_w4a16 or use_int4_w4a8:
        raise NotImplementedError("weight-only / int4 experts are not built in boltops_b200")
    if w1_zp is not None or w2_zp is not None:
        raise NotImplementedError("zero points are not built in boltops_b200")

    # ---- contract checks (same order and exception types as the reference) ------------
    if use_fp8_w8a8:
        e8m0 = getattr(torch, "float8_e8m0fnu", None)
        for name, scale in (("w1_scale", w1_scale), ("w2_scale", w2_scale),
                            ("a1_scale", a1_scale), ("a2_scale", a2_scale)):
            if scale is not None and (not scale.is_floating_point() or scale.dtype == e8m0):
                raise ValueError(
                    f"{name} must be a decoded floating-point multiplier for FP8; "
                    "convert checkpoint UE8M0 scales during weight preparation")
    if use_ue8m0 and (not use_fp8_w8a8 or block_shape is None or per_channel_quant):
        raise ValueError(
            "use_ue8m0 requires use_fp8_w8a8=True, block_shape, and per_channel_quant=False")
    if routed_scaling_factor is None:
        routed_scaling_factor = 1.0
    activation, is_gated = normalize_moe_activation(activation, is_gated)
    if gemm1_beta is not None:
        raise ValueError("gemm1_beta requires native MXFP8 or static MXFP4")
    if output_dtype is None:
        output_dtype = hidden_states.dtype

    assert hidden_states.shape[1] == w1.shape[2], "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    # (rows of pre-quantised or 16-bit input may also sit inside wider records -- the
    # expert-parallel layer hands over rows of its receive buffer in place -- as long as the
    # last dimension is dense; everything else must be contiguous as in the reference)
    assert hidden_states.is_contiguous() or (
        hidden_states.dim() == 2 and hidden_states.stride(1) == 1
        and (hidden_states.stride(0) * hidden_states.element_size()) % 16 == 0
    ), "Hidden_states must be contiguous"
    assert w1.stride(-1) == 1, "Stride of last dimension must be 1"
    assert w2.stride(-1) == 1, "Stride of last dimension must be 1"
    assert hidden_states.dtype in (torch.float32, torch.float16, torch.bfloat16, torch.int8,
                                   torch.float8_e4m3fn)
    assert output_dtype in _FLOAT_OUT, "Unsupported output_dtype"
    if not hidden_states.is_cuda:
        raise ValueError("boltops_b200 kernels need CUDA tensors (there is no CPU path)")

    quantised = use_fp8_w8a8 or use_int8_w8a8
    if quantised and hidden_states.dtype == torch.float32:
        # the reference quantises fp16 / bf16 rows only and hands any other dtype to its 8-bit
        # kernel as it is (fused_moe.py:1486-1492,1524-1529 of the reference); that combination
        # has no defined result, so it is refused here instead of quantised silently
        raise NotImplementedError("w8a8 experts take fp16 / bf16 rows (quantised here) or "
                                  "pre-quantised int8 / e4m3 rows with a1_scale")
    # TMA tiles and 128-bit row accesses need 16-byte rows in every operand and result
    for what, cols, esz in (("hidden size", w1.shape[2], w1.element_size()),
                            ("intermediate size", w2.shape[2], w2.element_size()),
                            ("hidden size", w1.shape[2], hidden_states.element_size()),
                            ("output size", w2.shape[1], torch.empty((), dtype=output_dtype).element_size())):
        if (cols * esz) % 16:
            raise NotImplementedError(
                f"{what} {cols} x {esz} B is not a multiple of 16 bytes: not built in boltops_b200")
    if quantised and not per_channel_quant and block_shape is None:
        raise NotImplementedError("per-tensor quantised experts are not built in boltops_b200")
    if quantised and block_shape is not None and not per_channel_quant:
        if list(block_shape) != [128, 128]:
            raise NotImplementedError("only block_shape [128, 128] is built in boltops_b200")
    block_mode = quantised and not per_channel_quant
    q_dtype = torch.float8_e4m3fn if use_fp8_w8a8 else torch.int8
    kind = _gemm_kind(w1.dtype, use_fp8_w8a8, use_int8_w8a8, per_channel_quant, block_shape)
    if quantised:
        assert w1_scale is not None and w2_scale is not None, "weight scales are required"
        assert w1.dtype == q_dtype and w2.dtype == q_dtype, "weight dtype does not match the flags"
    else:
        assert hidden_states.dtype == w1.dtype, "hidden_states / weight dtype mismatch"
    if not w1.is_contiguous():
        w1 = w1.contiguous()
    if not w2.is_contiguous():
        w2 = w2.contiguous()

    num_tokens, hidden = hidden_states.shape
    e_local, n1, _ = w1.shape
    model_dim = w2.shape[1]
    if global_num_experts == -1:
        global_num_experts = expert_map.numel() if expert_map is not None else e_local
    topk = topk_ids.shape[1]
    act_dim = n1 // 2 if is_gated else n1
    assert w2.shape[2] == act_dim, "w2 inner size does not match the activation output"
    dev = hidden_states.device
    mid_dtype = output_dtype

    if _out_peers is not None:
        # expert parallelism over peer memory: the top-k combine writes every live row straight
        # into the exchange buffer of the rank the token came from (ep.py); nothing is returned
        assert not (no_combine or inplace), "the direct exchange returns combined rows"
        out = None
    elif no_combine:
        assert not inplace, "no_combine + inplace is not supported"
        out = torch.empty((num_tokens, topk, model_dim), device=dev, dtype=output_dtype)
    elif inplace:
        out = hidden_states
    else:
        out = torch.empty((num_tokens, model_dim), device=dev, dtype=output_dtype)
    if num_tokens == 0:
        return out

    if topk_weights.dtype != torch.float32:
        topk_weights = topk_weights.to(torch.float32)
    expert_mask = (expert_map >= 0).to(torch.int32) if expert_map is not None else None
    fused_silu = (is_gated and activation == "silu" and gemm1_alpha is None
                  and gemm1_limit is None)
    needs_router_weight = not (apply_router_weight_on_input or no_combine)
    w1_scale_c = w1_scale.contiguous().float() if quantised else None
    w2_scale_c = w2_scale.contiguous().float() if quantised else None

    chunk = _chunk_size()
    # ---- the whole layer in one native call -------------------------------------------------
    # Same kernels, same order, same arithmetic as the loop below; one foreign call and one
    # workspace instead of one of each per kernel, which is what a decode-sized layer's time is
    # made of.  Used whenever the variant is the common one.
    if (_ONE_CALL and STAGE_TIMER is None and fused_silu and not no_combine
            and _out_peers is None
            and num_tokens <= chunk and not use_ue8m0 and hidden_states.is_contiguous()
            and hidden_states.dtype in (torch.float16, torch.bfloat16)
            and output_dtype == hidden_states.dtype
            and (b1 is None or b2 is None or b1.dtype == b2.dtype)
            and (not quantised or (w1_scale_c.dtype == torch.float32))
            and not _use_tile_pairs(kind, num_tokens * topk, global_num_experts)):
        args = _cabi.LayerArgs()
        args.kind = kind
        args.x_dtype = _cabi.dtype_code(hidden_states.dtype)
        args.out_dtype = _cabi.dtype_code(output_dtype)
        args.num_tokens, args.topk = num_tokens, topk
        args.hidden, args.inter, args.model_dim = hidden, act_dim, model_dim
        args.num_experts, args.global_num_experts = e_local, global_num_experts
        ids32 = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        ids32 = ids32.contiguous()
        wts32 = topk_weights.contiguous()
        bias = b1 if b1 is not None else b2
        b1c = b1.contiguous() if b1 is not None else None
        b2c = b2.contiguous() if b2 is not None else None
        args.hidden_states = hidden_states.data_ptr()
        args.w1, args.w2 = w1.data_ptr(), w2.data_ptr()
        args.w1_scale = _cabi.ptr(w1_scale_c)
        args.w2_scale = _cabi.ptr(w2_scale_c)
        args.b1, args.b2 = _cabi.ptr(b1c), _cabi.ptr(b2c)
        args.bias_dtype = _cabi.dtype_code(bias.dtype) if bias is not None else _cabi.F32
        args.apply_router_weight_on_input = int(apply_router_weight_on_input)
        args.topk_weights, args.topk_ids = wts32.data_ptr(), ids32.data_ptr()
        args.expert_mask = _cabi.ptr(expert_mask)
        args.routed_scaling_factor = float(routed_scaling_factor)
        args.out = out.data_ptr()
        args.status = ops.device_status(dev).data_ptr()
        lib = _cabi.load()
        need = lib.bolt_moe_layer_workspace_bytes(args)
        if need == 0:
            _cabi.check(1)
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        args.workspace, args.workspace_bytes = workspace.data_ptr(), need
        with _cabi.on_device(dev):
            _cabi.check(lib.bolt_moe_layer(args, _cabi.stream_of(hidden_states)))
        ops._count(lib.bolt_moe_layer_kernel_count(args))
        return out

    for begin in range(0, num_tokens, chunk):
        end = min(begin + chunk, num_tokens)
        m = end - begin
        x = hidden_states[begin:end]
        ids = topk_ids[begin:end]
        wts = topk_weights[begin:end]

        # ---- sort -----------------------------------------------------------------------
        # inverse permutation of the sort: the combine gathers through it, and the block
        # quantiser scatters through it
        route_pos = torch.empty((m, topk), device=dev, dtype=torch.int32)
        pairs = _use_tile_pairs(kind, m * topk, global_num_experts)
        segments = num_segments = None
        with _Stage("sort"):
            res = ops.moe_sorting_ck(
                ids, wts, global_num_experts, None, None, ops.SORT_UNIT, expert_mask,
                alloc_moe_buf=False, route_pos=route_pos,
                segment_rows=_cabi.PAIR_SEGMENT_ROWS if pairs else 0)
            sorted_ids, sorted_w, expert_ids, num_valid = res[:4]
            if pairs:
                segments, num_segments = res[6:8]
        cap = sorted_ids.shape[0]

        # ---- A1: quantise once per token, then gather into sorted rows --------------------
        a_scale = None
        gemm1_rows = {}
        if quantised and x.dtype in (torch.float16, torch.bfloat16) and not x.is_contiguous():
            x = x.contiguous()                      # the quantisers read dense rows
        if quantised and block_mode and x.dtype in (torch.float16, torch.bfloat16):
            # quantise each token once and write it straight to its sorted rows
            in_gemm = segments is None and _use_gather(m * topk, global_num_experts)
            with _Stage("quant_a1"):
                a_sorted, a_scale = ops.quant_scatter_rows(
                    x, 128, q_dtype, route_pos, sorted_ids, num_valid, cap,
                    scale_ue8m0=use_ue8m0, token_order=in_gemm)
            if in_gemm:
                gemm1_rows = dict(a_gather=True)   # a_sorted is [m, H] in token order
        elif quantised:
            # per-token scales: quantise, then gather (a row-centric gather writes the sorted rows
            # faster than a token-centric scatter of whole rows; measured 0.131 vs 0.157 ms at
            # 16384 x 2048)
            with _Stage("quant_a1"):
                if x.dtype in (torch.float16, torch.bfloat16):
                    if block_mode:
                        x_q, x_s = ops.per_block_quant(x, 128, q_dtype, scale_ue8m0=use_ue8m0)
                    else:
                        x_q, x_s = ops.per_token_quant(x, quant_dtype=q_dtype)
                else:
                    assert a1_scale is not None, "pre-quantised hidden_states need a1_scale"
                    x_q = x
                    x_s = a1_scale[begin:end] if a1_scale.ndim == 2 else a1_scale
                    x_s = x_s.float()
            with _Stage("gather"):
                a_sorted, a_scale = ops.gather_rows(x_q, sorted_ids, num_valid, cap, x_s)
        elif (segments is None and _use_gather(m * topk, global_num_experts)
              and x.stride(1) == 1 and x.data_ptr() % 16 == 0
              and (x.stride(0) * x.element_size()) % 16 == 0):
            a_sorted, gemm1_rows = x, dict(a_gather=True)   # GEMM1 reads the token rows itself
        else:
            with _Stage("gather"):
                a_sorted, _ = ops.gather_rows(x, sorted_ids, num_valid, cap)

        common = dict(kind=kind, sorted_expert_ids=expert_ids, num_valid=num_valid,
                      sorted_ids=sorted_ids, sorted_weights=sorted_w, num_tokens=m, topk=topk,
                      segments=segments, num_segments=num_segments)

        # ---- GEMM1 (+ activation, + re-quantisation) ---------------------------------------
        act_scale = None
        fuse_quant = fused_silu and block_mode and not use_ue8m0
        if fuse_quant:
            act = torch.empty((cap, act_dim), device=dev, dtype=q_dtype)
            act_scale = torch.empty((act_dim // 128, cap), device=dev, dtype=torch.float32)
            with _Stage("gemm1"):
              ops.grouped_gemm(epilogue=_cabi.EPI_SILU_MUL_QUANT, a=a_sorted, b=w1, c=act,
                             a_scale=a_scale, a_scale_ld=cap, b_scale=w1_scale_c, bias=b1,
                             c_scale=act_scale, c_scale_ld=cap, mid_dtype=mid_dtype,
                             mul_routed_weight=apply_router_weight_on_input, **gemm1_rows,
                             **common)
        else:
            if fused_silu:
                act_f = torch.empty((cap, act_dim), device=dev, dtype=mid_dtype)
                with _Stage("gemm1"):
                  ops.grouped_gemm(epilogue=_cabi.EPI_SILU_MUL, a=a_sorted, b=w1, c=act_f,
                                 a_scale=a_scale, a_scale_ld=cap, b_scale=w1_scale_c, bias=b1,
                                 mid_dtype=mid_dtype,
                                 mul_routed_weight=apply_router_weight_on_input, **gemm1_rows,
                                 **common)
            else:
                c1 = torch.empty((cap, n1), device=dev, dtype=mid_dtype)
                with _Stage("gemm1"):
                  ops.grouped_gemm(epilogue=_cabi.EPI_STORE, a=a_sorted, b=w1, c=c1,
                                 a_scale=a_scale, a_scale_ld=cap, b_scale=w1_scale_c, bias=b1,
                                 mul_routed_weight=apply_router_weight_on_input, **gemm1_rows,
                                 **common)
                act_f = torch.empty((cap, act_dim), device=dev, dtype=mid_dtype)
                apply_activation(activation, is_gated, act_f, c1, gemm1_alpha, gemm1_limit,
                                 activation_situ_beta, activation_situ_linear_beta,
                                 rows_dev=num_valid)
            if quantised:
                with _Stage("quant_a2"):
                    if block_mode:
                        act, act_scale = ops.per_block_quant(       # scales [act_dim/128, cap]
                            act_f, 128, q_dtype, scale_ue8m0=use_ue8m0, group_major=True)
                    else:
                        act, s = ops.per_token_quant(act_f, quant_dtype=q_dtype)
                        act_scale = s.reshape(-1)
            else:
                act = act_f

        # ---- GEMM2 (router weight in the epilogue) + combine --------------------------------
        if _out_peers is not None and "routes" in _out_peers:
            # expert parallelism over peer memory, per-route return: every route's row goes from
            # the epilogue straight to its slot of the [tokens, topk, H] buffer of the rank that
            # owns the token (ep.py); the sum over the routes happens there
            assert begin == 0 and end == num_tokens, "per-route return takes one chunk"
            with _Stage("gemm2"):
                ops.grouped_gemm(epilogue=_cabi.EPI_STORE, a=act, b=w2, c=_out_peers["routes"],
                                 a_scale=act_scale, a_scale_ld=cap, b_scale=w2_scale_c, bias=b2,
                                 scatter=True, mul_routed_weight=needs_router_weight,
                                 scatter_src=_out_peers["src"], scatter_seg_off=_out_peers["seg_off"],
                                 scatter_seg_rows=_out_peers["seg_rows"], **common)
        elif no_combine:
            # the caller wants [m, topk, H]: scatter rows to their route slots
            c3 = out[begin:end]
            if expert_map is not None:
                c3.zero_()
            with _Stage("gemm2"):
                ops.grouped_gemm(epilogue=_cabi.EPI_STORE, a=act, b=w2,
                                 c=c3.view(m * topk, model_dim), a_scale=act_scale,
                                 a_scale_ld=cap, b_scale=w2_scale_c, bias=b2, scatter=True,
                                 mul_routed_weight=needs_router_weight, **common)
        else:
            # rows stay in sorted order; the combine gathers each token's routes through the
            # inverse permutation (k ascending, fp32), so no [m, topk, H] intermediate exists
            c_sorted = torch.empty((cap, model_dim), device=dev, dtype=output_dtype)
            with _Stage("gemm2"):
                ops.grouped_gemm(epilogue=_cabi.EPI_STORE, a=act, b=w2, c=c_sorted,
                                 a_scale=act_scale, a_scale_ld=cap, b_scale=w2_scale_c, bias=b2,
                                 scatter=False, mul_routed_weight=needs_router_weight, **common)
            with _Stage("combine"):
                if _out_peers is not None:
                    ops.gather_sum_to_peers(c_sorted, route_pos, routed_scaling_factor,
                                            first_row=begin, seg_rows=_out_peers["seg_rows"],
                                            seg_ptrs=_out_peers["seg_ptrs"], hdr=_out_peers["hdr"])
                else:
                    ops.gather_sum(c_sorted, route_pos, out[begin:end], routed_scaling_factor)
    return out
