"""CPU-only checks: the C-ABI library loads and exports every declared symbol,
the ctypes struct matches the C header, host-side argument logic, and oracle
self-consistency.  No compute entry point is called here."""
import ctypes
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from boltops_b200 import build, _cabi
    build.build()
    return _cabi.load()


def test_library_exports_every_declared_symbol(lib):
    from boltops_b200 import _cabi
    header = (ROOT / "include" / "boltops_b200.h").read_text()
    declared = set(re.findall(r"\b(bolt_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_cabi.EXPORTS)
    assert lib.bolt_abi_version() == 3


def test_gemm_args_struct_matches_header(tmp_path):
    from boltops_b200 import _cabi
    fields = [f[0] for f in _cabi.GemmArgs._fields_]
    prog = ['#include <stdio.h>', '#include <stddef.h>',
            f'#include "{ROOT / "include" / "boltops_b200.h"}"', "int main(void){",
            'printf("%zu\\n", sizeof(bolt_gemm_args));']
    prog += [f'printf("%zu\\n", offsetof(bolt_gemm_args, {f}));' for f in fields]
    prog += ["return 0;}"]
    src = tmp_path / "abi.c"
    src.write_text("\n".join(prog))
    exe = tmp_path / "abi"
    subprocess.run(["gcc", str(src), "-o", str(exe)], check=True)
    nums = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True,
                                           check=True).stdout.split()]
    assert nums[0] == ctypes.sizeof(_cabi.GemmArgs)
    for f, off in zip(fields, nums[1:]):
        assert getattr(_cabi.GemmArgs, f).offset == off, f


def test_layer_args_struct_matches_header(tmp_path):
    from boltops_b200 import _cabi
    fields = [f[0] for f in _cabi.LayerArgs._fields_]
    prog = ['#include <stdio.h>', '#include <stddef.h>',
            f'#include "{ROOT / "include" / "boltops_b200.h"}"', "int main(void){",
            'printf("%zu\\n", sizeof(bolt_layer_args));']
    prog += [f'printf("%zu\\n", offsetof(bolt_layer_args, {f}));' for f in fields]
    prog += ["return 0;}"]
    src = tmp_path / "abi_layer.c"
    src.write_text("\n".join(prog))
    exe = tmp_path / "abi_layer"
    subprocess.run(["gcc", str(src), "-o", str(exe)], check=True)
    nums = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True,
                                           check=True).stdout.split()]
    assert nums[0] == ctypes.sizeof(_cabi.LayerArgs)
    for f, off in zip(fields, nums[1:]):
        assert getattr(_cabi.LayerArgs, f).offset == off, f


def test_workspace_query_is_host_only(lib):
    assert lib.bolt_moe_sort_workspace_bytes(64, 2, 8) == 16          # single-CTA path
    big = lib.bolt_moe_sort_workspace_bytes(16384, 8, 128)
    assert big > 128 * 4 and big < (1 << 22)


def test_activation_registry():
    from boltops_b200.fused_moe import (moe_activation_output_size, normalize_moe_activation)
    assert normalize_moe_activation("SiLU") == ("silu", True)
    assert normalize_moe_activation("gelu_pytorch_tanh", False) == ("gelu_tanh", False)
    assert normalize_moe_activation("relu2") == ("relu2", False)
    with pytest.raises(ValueError, match="Unsupported activation"):
        normalize_moe_activation("tanh")
    with pytest.raises(ValueError, match="non-gated"):
        normalize_moe_activation("relu2", True)
    with pytest.raises(ValueError, match="requires gated"):
        normalize_moe_activation("swigluoai", False)
    assert moe_activation_output_size(10, True) == 5
    assert moe_activation_output_size(10, False) == 10
    with pytest.raises(ValueError):
        moe_activation_output_size(0, False)
    with pytest.raises(ValueError):
        moe_activation_output_size(7, True)


def test_public_signatures_match_reference_order():
    """Every public function has the reference's parameters: same names, order, kind and
    defaults (tests/golden/signatures.json is written by make_golden.py from the reference's
    boltops/fused_moe/__init__.py)."""
    import inspect
    import json
    import boltops_b200.fused_moe as pkg
    ref = json.loads((ROOT / "tests" / "golden" / "signatures.json").read_text())
    assert set(ref) == {"fused_experts", "moe_activation", "normalize_moe_activation",
                        "moe_activation_output_size"}
    assert len(ref["fused_experts"]) == 37
    for fn_name, params in ref.items():
        sig = inspect.signature(getattr(pkg, fn_name))
        got = []
        for name, prm in sig.parameters.items():
            kind = "keyword_only" if prm.kind is inspect.Parameter.KEYWORD_ONLY else "positional"
            default = None if prm.default is inspect.Parameter.empty else repr(prm.default)
            got.append([name, kind, default])
        assert got == params, f"{fn_name}: {got} != {params}"


def test_no_cpu_fallback():
    from boltops_b200.fused_moe import fused_experts, moe_activation
    hid = torch.zeros(2, 128, dtype=torch.bfloat16)
    w1 = torch.zeros(2, 256, 128, dtype=torch.bfloat16)
    w2 = torch.zeros(2, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        fused_experts(hid, w1, w2, torch.ones(2, 1), torch.zeros(2, 1, dtype=torch.int32))
    with pytest.raises(ValueError, match="CUDA"):
        moe_activation(torch.zeros(2, 64), torch.zeros(2, 128), "silu")


def test_product_does_not_import_oracle():
    for path in (ROOT / "boltops_b200").rglob("*.py"):
        text = path.read_text()
        assert "oracle" not in text, f"{path} mentions the oracle"


@pytest.mark.parametrize("tokens,E,topk,unit,use_mask", [(1, 8, 2, 16, False), (50, 16, 4, 8, True),
                                                         (200, 64, 8, 32, True), (3, 4, 4, 128, False)])
def test_oracle_sort_vectorised_equals_loops(tokens, E, topk, unit, use_mask):
    rng = np.random.default_rng(tokens + E)
    ids = np.argsort(rng.random((tokens, E)), axis=1)[:, :topk].astype(np.int32)
    w = rng.random((tokens, topk), dtype=np.float32)
    mask = None
    if use_mask:
        mask = np.ones(E, np.int32)
        mask[1::4] = 0
    a = O.sort_ck_loops(torch.from_numpy(ids), torch.from_numpy(w), E, unit, mask)
    b = O.sort_ck_numpy(ids, w, E, unit, mask)
    assert (b["sorted_ids"].astype(np.int64) & 0xFFFFFFFF).tolist() == a[0]
    assert b["sorted_weights"].tolist() == a[1]
    assert b["expert_ids"].tolist() == a[2]
    assert b["counts"].tolist() == a[3]


def test_oracle_kernel_quantiser_matches_clamped_oracle_on_benign_inputs():
    torch.manual_seed(0)
    x = torch.randn(32, 256).bfloat16()
    q1, s1 = O.quant_rows_kernel(x, O.FP8, 128)
    q2, s2 = O.group_quant_fp8_native(x, 128)
    assert torch.equal(s1, s2)
    assert (q1.float() - q2.float()).abs().max() <= 32     # at most one e4m3 step at the top binade
    assert (q1.view(torch.uint8) != q2.view(torch.uint8)).float().mean() < 0.02


def test_custom_op_fake_impl_shapes():
    """The registered torch op reports output shapes under FakeTensorMode without a kernel
    (the reference checks its meta function the same way, test_fused_moe.py:1715-1769)."""
    import boltops_b200.fused_moe.custom_op  # noqa: F401  (registers the op)
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        hid = torch.empty(5, 128, dtype=torch.bfloat16)
        w1 = torch.empty(4, 256, 128, dtype=torch.bfloat16)
        w2 = torch.empty(4, 128, 128, dtype=torch.bfloat16)
        wts = torch.empty(5, 2)
        ids = torch.empty(5, 2, dtype=torch.int32)
        out = torch.ops.boltops_b200.fused_experts_impl(hid, w1, w2, wts, ids)
        assert out.shape == (5, 128) and out.dtype == torch.bfloat16
        out = torch.ops.boltops_b200.fused_experts_impl(hid, w1, w2, wts, ids, no_combine=True,
                                                        output_dtype=torch.float16)
        assert out.shape == (5, 2, 128) and out.dtype == torch.float16


@pytest.mark.parametrize("case", ["block128", "fp32_scale", "packed_scale", "bias", "input_router",
                                  "prequantized", "output_dtype"])
def test_mxfp8_rejections_match_reference(case):
    """Same ValueErrors, raised before any device work, as the reference's
    test_public_mxfp8_rejects_non_native_recipe / ..._unsupported_native_options."""
    import torch
    from boltops_b200.fused_moe import fused_experts
    x = torch.zeros(1, 128, dtype=torch.bfloat16)
    if case == "prequantized":
        x = x.to(torch.float8_e4m3fn)
    w1 = torch.zeros(1, 256, 128, dtype=torch.float8_e4m3fn)
    w2 = torch.zeros(1, 128, 128, dtype=torch.float8_e4m3fn)
    scale_dtype = {"fp32_scale": torch.float32, "packed_scale": torch.int32}.get(case, torch.uint8)
    match = "native MXFP8 requires" if case in ("block128", "fp32_scale", "packed_scale") \
        else "native MXFP8"
    with pytest.raises(ValueError, match=match):
        fused_experts(
            x, w1, w2, torch.ones(1, 1), torch.zeros(1, 1, dtype=torch.int32), use_mxfp8=True,
            block_shape=[128, 128] if case == "block128" else [1, 32],
            b1=torch.zeros(1, 256) if case == "bias" else None,
            apply_router_weight_on_input=case == "input_router",
            output_dtype=torch.float32 if case == "output_dtype" else None,
            w1_scale=torch.ones(1, 256, 4, dtype=scale_dtype),
            w2_scale=torch.ones(1, 128, 4, dtype=scale_dtype))


def test_gathered_row_operand_rule_and_layer_kernel_count(monkeypatch):
    """The rule that picks the gathered row operand is the same on both sides of the C ABI (up
    to 64 routes per expert), and the one-call layer reports the kernels it would launch (host
    arithmetic only: nothing runs on a device)."""
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import layer
    monkeypatch.setattr(layer, "_GATHER", None)
    assert layer._use_gather(64 * 256, 256) and not layer._use_gather(64 * 256 + 1, 256)
    monkeypatch.setattr(layer, "_GATHER", False)
    assert not layer._use_gather(8, 256)
    lib = _cabi.load()

    def count(kind, tokens):
        a = _cabi.LayerArgs()
        a.kind, a.x_dtype, a.out_dtype = kind, _cabi.BF16, _cabi.BF16
        a.num_tokens, a.topk = tokens, 8
        a.hidden, a.inter, a.model_dim = 1024, 512, 1024
        a.num_experts = a.global_num_experts = 32
        a.w1_scale = a.w2_scale = 1          # non-null: only checked for presence here
        return lib.bolt_moe_layer_kernel_count(a)

    import os
    if os.environ.get("BOLTOPS_B200_GATHER") is None:
        small = 32 * 64 // 8                 # 64 routes per expert
        assert count(_cabi.GEMM_BF16, small) == count(_cabi.GEMM_BF16, small + 1) - 1
    fp8 = count(_cabi.GEMM_FP8_BLOCK, 16)
    assert fp8 >= 5 and count(_cabi.GEMM_INT8_CHANNEL, 16) == fp8 + 2
    bad = _cabi.LayerArgs()
    assert lib.bolt_moe_layer_kernel_count(bad) == -1
