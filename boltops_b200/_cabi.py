"""ctypes binding of ``libboltops_b200.so`` (the C ABI in include/boltops_b200.h).

The library is the only compute path.  If it is missing, loading raises
``RuntimeError`` -- nothing falls back to torch or to the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
_LIB_PATH = Path(os.environ.get("BOLTOPS_B200_LIB", _PKG / "lib" / "libboltops_b200.so"))

BOLT_OK = 0
# enum bolt_dtype
BF16, F16, F32, FP8_E4M3, INT8 = 0, 1, 2, 3, 4
# enum bolt_activation
(ACT_SILU, ACT_GELU, ACT_GELU_TANH, ACT_RELU2, ACT_SWIGLU_OAI, ACT_SWIGLU_STEP, ACT_SILU_CLAMP,
 ACT_SWIGLU_OAI_INTERLEAVED, ACT_SITU) = range(9)
# enum bolt_gemm_kind
GEMM_BF16, GEMM_F16, GEMM_FP8_BLOCK, GEMM_INT8_CHANNEL, GEMM_FP8_CHANNEL, GEMM_INT8_BLOCK, \
    GEMM_MXFP8, GEMM_MXFP4 = range(8)
# enum bolt_gemm_epilogue
EPI_STORE, EPI_SILU_MUL, EPI_SILU_MUL_QUANT = range(3)
# enum bolt_gemm_schedule, BOLT_PAIR_SEGMENT_ROWS
SCHEDULE_ROW_TILES, SCHEDULE_TILE_PAIRS = range(2)
PAIR_SEGMENT_ROWS = 256

_DTYPES = {
    torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32,
    torch.float8_e4m3fn: FP8_E4M3, torch.int8: INT8,
}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


class GemmArgs(C.Structure):
    """struct bolt_gemm_args"""
    _fields_ = [
        ("kind", C.c_int), ("epilogue", C.c_int), ("capacity", C.c_int), ("n", C.c_int),
        ("k", C.c_int), ("num_experts", C.c_int),
        ("a", C.c_void_p), ("b", C.c_void_p), ("a_scale", C.c_void_p), ("a_scale_ld", C.c_int64),
        ("b_scale", C.c_void_p), ("bias", C.c_void_p), ("bias_dtype", C.c_int),
        ("c", C.c_void_p), ("c_dtype", C.c_int), ("mid_dtype", C.c_int), ("c_ld", C.c_int64),
        ("c_scale", C.c_void_p), ("c_scale_ld", C.c_int64),
        ("scatter", C.c_int), ("num_tokens", C.c_int), ("topk", C.c_int),
        ("mul_routed_weight", C.c_int),
        ("sorted_ids", C.c_void_p), ("sorted_weights", C.c_void_p),
        ("sorted_expert_ids", C.c_void_p), ("num_valid_ids", C.c_void_p),
        ("status", C.c_void_p), ("sm_count", C.c_int),
        ("act_alpha", C.c_float), ("act_beta", C.c_float), ("act_limit", C.c_float),
        ("act_has_limit", C.c_int),
        ("schedule", C.c_int), ("max_segments", C.c_int),
        ("segments", C.c_void_p), ("num_segments", C.c_void_p),
        ("a_gather", C.c_int), ("a_rows", C.c_int), ("a_row_bytes", C.c_int64),
        ("scatter_src", C.c_void_p), ("scatter_seg_off", C.c_void_p), ("scatter_seg_rows", C.c_int),
    ]


class LayerArgs(C.Structure):
    """struct bolt_layer_args"""
    _fields_ = [
        ("kind", C.c_int), ("x_dtype", C.c_int), ("out_dtype", C.c_int),
        ("num_tokens", C.c_int), ("topk", C.c_int),
        ("hidden", C.c_int), ("inter", C.c_int), ("model_dim", C.c_int),
        ("num_experts", C.c_int), ("global_num_experts", C.c_int),
        ("hidden_states", C.c_void_p), ("w1", C.c_void_p), ("w2", C.c_void_p),
        ("w1_scale", C.c_void_p), ("w2_scale", C.c_void_p), ("b1", C.c_void_p), ("b2", C.c_void_p),
        ("bias_dtype", C.c_int), ("apply_router_weight_on_input", C.c_int),
        ("topk_weights", C.c_void_p), ("topk_ids", C.c_void_p), ("expert_mask", C.c_void_p),
        ("routed_scaling_factor", C.c_float),
        ("out", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
    ]


_SIGNATURES = {
    "bolt_last_error": (C.c_char_p, []),
    "bolt_abi_version": (C.c_int, []),
    "bolt_moe_sort_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "bolt_moe_sort_ck": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                   C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                   C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "bolt_moe_sort_static_scratch_bytes": (C.c_size_t, []),
    "bolt_moe_sort_ck_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p]),
    "bolt_moe_align_block_size": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_size_t, C.c_void_p]),
    "bolt_fused_topk": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int,
                                  C.c_void_p, C.c_void_p, C.c_void_p]),
    "bolt_moe_fused_gate": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int,
                                      C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p,
                                      C.c_void_p]),
    "bolt_ep_dest_ranks": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_int64, C.c_void_p, C.c_void_p]),
    "bolt_ep_wire_row_bytes": (C.c_int64, [C.c_int, C.c_int, C.c_int]),
    "bolt_ep_pack_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                    C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64,
                                    C.c_void_p, C.c_int64, C.c_void_p]),
    "bolt_quant_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int,
                                  C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "bolt_quant_scatter_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                          C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int,
                                          C.c_void_p]),
    "bolt_mx_quant_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_float,
                                     C.c_float, C.c_int, C.c_float, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_int, C.c_void_p]),
    "bolt_mx_dequant_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p,
                                       C.c_int, C.c_void_p]),
    "bolt_mx_sf_layout": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int64,
                                    C.c_void_p, C.c_void_p]),
    "bolt_mxfp4_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p,
                                    C.c_int, C.c_void_p]),
    "bolt_mx4_act_quant": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int,
                                     C.c_float, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "bolt_fp8_group_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int,
                                        C.c_void_p, C.c_int, C.c_void_p]),
    "bolt_mx4_swiglu_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                         C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_float,
                                         C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "bolt_mx4_affine_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                       C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "bolt_gather_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_int64,
                                   C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                   C.c_void_p, C.c_int64, C.c_void_p]),
    "bolt_moe_activation": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int,
                                      C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p]),
    "bolt_act_quant": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int,
                                 C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p]),
    "bolt_moe_sum": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int,
                               C.c_int, C.c_float, C.c_void_p, C.c_void_p]),
    "bolt_moe_gather_sum": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                      C.c_int64, C.c_int, C.c_int, C.c_float, C.c_void_p]),
    "bolt_grouped_gemm": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p]),
    "bolt_ep_dispatch_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                        C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                        C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_int64,
                                        C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "bolt_ep_unpack_routes": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                                        C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_int64, C.c_void_p, C.c_void_p]),
    "bolt_moe_gather_sum_to_peers": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int,
                                               C.c_int, C.c_float, C.c_int64, C.c_void_p,
                                               C.c_void_p, C.c_int64, C.c_void_p]),
    "bolt_ep_barrier": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_void_p,
                                  C.c_void_p]),
    "bolt_moe_layer_workspace_bytes": (C.c_size_t, [C.POINTER(LayerArgs)]),
    "bolt_moe_layer_kernel_count": (C.c_int, [C.POINTER(LayerArgs)]),
    "bolt_moe_layer": (C.c_int, [C.POINTER(LayerArgs), C.c_void_p]),
}

EXPORTS = tuple(_SIGNATURES)
_lib = None


def lib_path() -> Path:
    return _LIB_PATH


def load() -> C.CDLL:
    """Load the shared library (once) and attach prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} not found: build it with `python -m boltops_b200.build`. "
            "boltops_b200 has no fallback path.")
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.bolt_abi_version() != 3:
        raise RuntimeError("libboltops_b200.so ABI version mismatch")
    _lib = lib
    return lib


class BoltError(RuntimeError):
    pass


def check(status: int) -> None:
    if status != BOLT_OK:
        msg = load().bolt_last_error().decode(errors="replace")
        raise BoltError(f"boltops_b200 status {status}: {msg}")


def ptr(t) -> int | None:
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    """Raw handle of torch's current stream on the tensor's device."""
    return torch.cuda.current_stream(t.device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def on_device(device: torch.device):
    """Context that makes `device` current for a C-ABI call; free when it already is (the
    common case: entering torch.cuda.device costs several microseconds per kernel launch, which
    is most of a decode-sized layer's host time)."""
    index = device.index
    if index is None or index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)
