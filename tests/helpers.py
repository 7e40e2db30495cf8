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
