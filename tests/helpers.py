"""Shared helpers for the test-suite (fixture decoding, tolerances)."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_npz(name: str):
    return np.load(GOLDEN / name)


def bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def fp8(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)


def t(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a))


MX_CASES = {            # case -> activation arguments of the reference's MXFP8 CPU statement
    "default": dict(activation="silu"),
    "silu_alpha": dict(activation="silu", alpha=1.2),
    "swigluoai": dict(activation="swigluoai", alpha=1.2, beta=0.3, limit=0.15),
    "no_combine": dict(activation="silu", no_combine=True),
    "dynamic_fp16": dict(activation="silu"),
}


def load_mx_case(case: str):
    """Inputs and expected output of one case of tests/golden/mxfp8.npz."""
    z = load_npz("mxfp8.npz")
    half = case == "dynamic_fp16"
    dec = (lambda a: t(a)) if half else bf16
    return dict(x=dec(z[f"{case}_x"]), w1=fp8(z[f"{case}_w1"]), w2=fp8(z[f"{case}_w2"]),
                s1=t(z[f"{case}_s1"]), s2=t(z[f"{case}_s2"]), ids=t(z[f"{case}_ids"]),
                weights=t(z[f"{case}_weights"]), expected=dec(z[f"{case}_expected"]))


MXFP4_CASES = (
    "dense", "sparse_routing", "clamp_no_combine", "chunked", "prequantized_chunked",
    "static", "static_bias", "static_clamp", "static_input_router",
    "static_input_router_zero", "static_prequantized_chunked",
    "static_expert_map_chunked", "static_no_combine", "static_input_router_no_combine",
    "prequantized_g128_swiglustep", "prequantized_g128_situ",
    "expert_map_chunked", "swiglustep", "situ",
    "input_router", "input_router_chunked", "input_router_inplace",
    "input_router_no_combine", "input_router_fp16",
    "input_router_zero", "input_router_inplace_chunked",
    "input_router_expert_map_chunked",
)


def load_mxfp4_case(case: str):
    """Inputs, expected output and call arguments of one case of tests/golden/mxfp4.npz (the
    reference's test_public_mxfp4_cpu_reference parametrisation)."""
    z = load_npz("mxfp4.npz")

    def get(name, default=None):
        if f"{case}__{name}__f16" in z.files:
            return t(z[f"{case}__{name}__f16"])
        key = f"{case}__{name}"
        if key not in z.files:
            return default
        a = z[key]
        if a.dtype == np.uint16:
            return bf16(a)
        return t(a)

    static = case.startswith("static")
    clamp = float(z[f"{case}__clamp"])
    c = dict(x=get("x"), w1=get("w1"), w2=get("w2"), s1=get("s1"), s2=get("s2"), ids=get("ids"),
             weights=get("weights"), expected=get("expected"), expert_map=get("expert_map"),
             bias1=get("bias1"), bias2=get("bias2"), static=static,
             static_s1=get("static_s1"), static_s2=get("static_s2"),
             input_q=fp8(z[f"{case}__input_q"]), input_scale=get("input_scale"),
             alpha=float(z[f"{case}__alpha"]), clamp=None if clamp != clamp else clamp,
             chunk=int(z[f"{case}__chunk"]), input_router="input_router" in case,
             no_combine="no_combine" in case, prequantized="prequantized" in case,
             inplace="inplace" in case,
             activation="swigluoai" if static else ("swiglustep" if "swiglustep" in case else
                                                    ("situ" if "situ" in case else "silu")))
    return c
