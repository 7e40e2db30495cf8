"""Generate golden fixtures by RUNNING the reference's own Python reference
functions on seeded inputs.

Usage (in a checkout that has the reference project available)::

    python tests/golden/make_golden.py /path/to/reference

The reference's oracle functions live in modules that import its device
backend at import time, so the modules cannot be imported on a machine without
that backend.  The functions themselves are plain torch; this script pulls the
individual ``def`` nodes out of the source files with ``ast`` and executes them
unchanged in a namespace that only holds torch.  Nothing from the reference is
written into this repository except the *numeric outputs* (``.npz`` files).
"""

from __future__ import annotations

import ast
import os
import sys
import textwrap
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent


def load_defs(path: Path, names, extra=None):
    """Execute selected top-level function definitions of ``path``."""
    tree = ast.parse(path.read_text(encoding="utf-8"))
    picked = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in picked}
    if missing:
        raise SystemExit(f"{path}: missing {sorted(missing)}")
    for n in picked:
        n.decorator_list = []
    ns = {"torch": torch, "F": F, "Optional": __import__("typing").Optional}
    ns.update(extra or {})
    module = ast.Module(body=picked, type_ignores=[])
    exec(compile(module, str(path), "exec"), ns)  # noqa: S102 - trusted local tree
    return ns


def t2n(t: torch.Tensor) -> np.ndarray:
    """Tensor -> numpy, bit-preserving for bf16/fp8 (stored as uint16/uint8)."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def make_mxfp8(ref: Path) -> None:
    """Native MXFP8 layer: the CPU statement inside test_public_mxfp8_cpu_reference
    (everything from the seed down to the line that forms `expected`; the device half of the
    test follows that line and is not executed)."""
    text = (ref / "test/fused_moe/test_fused_moe.py").read_text().splitlines()
    start = next(i for i, l in enumerate(text) if l.strip() == "torch.manual_seed(673)")
    stop = next(i for i in range(start, len(text))
                if text[i].startswith("    expected = (expected if case"))
    body = textwrap.dedent("\n".join(text[start:stop + 1]))
    mx = {}
    for case in ("default", "silu_alpha", "swigluoai", "no_combine", "dynamic_fp16"):
        ns = {"torch": torch, "case": case, "monkeypatch": None}
        exec(compile(body, "mxfp8_cpu_reference", "exec"), ns)
        for name in ("x", "w1", "w2", "s1", "s2", "ids", "weights", "expected"):
            v = ns[name]
            if v.dtype == torch.float8_e4m3fn:
                v = v.view(torch.uint8)
            mx[f"{case}_{name}"] = t2n(v)
    np.savez_compressed(HERE / "mxfp8.npz", **mx)


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


def make_mxfp4(ref: Path) -> None:
    """MXFP4 (w4a8) layer: the CPU statement inside test_public_mxfp4_cpu_reference for every
    case of its parametrisation (from `static = ...` down to the line that forms `expected`),
    plus the pre-quantised inputs the test derives with its own quantiser.  The device half of
    the test is not executed."""
    path = ref / "test/fused_moe/test_fused_moe.py"
    text = path.read_text().splitlines()
    start = next(i for i, l in enumerate(text) if l.strip() == "static = case.startswith('static')")
    stop = next(i for i in range(start, len(text))
                if text[i].startswith("        expected = (combined * 1.25).to(x.dtype)"))
    body = textwrap.dedent("\n".join(text[start:stop + 1]))
    helpers = load_defs(path, ["_quantize_mxfp4_reference", "_decode_mxfp4_reference",
                               "_mxfp4_reference_gemm"])

    class _Env:                      # the test sets the chunk size through monkeypatch
        def __init__(self):
            self.env = {}

        def setenv(self, k, v):
            self.env[k] = v

    out = {}
    for case in MXFP4_CASES:
        mp = _Env()
        ns = dict(helpers)
        ns.update(torch=torch, case=case, monkeypatch=mp)
        exec(compile(body, "mxfp4_cpu_reference", "exec"), ns)
        group = ns["group_size"]
        q, qs = helpers["_quantize_mxfp4_reference"](ns["x"], return_scales=True, group_size=group)
        if ns["static"]:
            q = (ns["x"].float() / ns["static_s1"]).to(torch.float8_e4m3fn)
            qs = ns["static_s1"]
        rec = dict(x=ns["x"], w1=ns["w1"], w2=ns["w2"], s1=ns["s1"], s2=ns["s2"], ids=ns["ids"],
                   weights=ns["weights"], expected=ns["expected"], input_q=q, input_scale=qs,
                   static_s1=ns["static_s1"], static_s2=ns["static_s2"],
                   alpha=torch.tensor(float(ns["alpha"])),
                   clamp=torch.tensor(float("nan") if ns["clamp"] is None else float(ns["clamp"])),
                   chunk=torch.tensor(int(mp.env.get("TRITON_FUSED_MOE_CHUNK_SIZE", 0))))
        for name in ("expert_map", "bias1", "bias2"):
            if ns.get(name) is not None:
                rec[name] = ns[name]
        for name, v in rec.items():
            if v.dtype == torch.float8_e4m3fn:
                v = v.view(torch.uint8)
            key = f"{case}__{name}"
            if v.dtype == torch.float16:
                out[key + "__f16"] = v.numpy()
            else:
                out[key] = t2n(v)
    np.savez_compressed(HERE / "mxfp4.npz", **out)


def make_signatures(ref: Path) -> None:
    """Parameter lists of the public functions (name, kind, default as source text), read from
    the reference's package file with ``ast`` -- the drop-in signature contract."""
    import json
    tree = ast.parse((ref / "boltops/fused_moe/__init__.py").read_text(encoding="utf-8"))
    out = {}
    for node in tree.body:
        if not isinstance(node, ast.FunctionDef) or node.name.startswith("_"):
            continue
        a = node.args
        params = []
        pos = a.posonlyargs + a.args
        defaults = [None] * (len(pos) - len(a.defaults)) + list(a.defaults)
        for arg, d in zip(pos, defaults):
            params.append([arg.arg, "positional", None if d is None else ast.unparse(d)])
        for arg, d in zip(a.kwonlyargs, a.kw_defaults):
            params.append([arg.arg, "keyword_only", None if d is None else ast.unparse(d)])
        out[node.name] = params
    lines = [f' "{name}": [\n' + ",\n".join("  " + json.dumps(q) for q in params) + "\n ]"
             for name, params in out.items()]
    (HERE / "signatures.json").write_text("{\n" + ",\n".join(lines) + "\n}\n")


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    tdir = ref / "test" / "fused_moe"
    tune = ref / "boltops" / "tools" / "fused_moe_triton_tune"

    # ---- sorter: the reference test's own cases and seed --------------------
    srt = load_defs(tdir / "test_moe_sorting_hipc.py", ["_reference"])
    sort_cases = {}
    for tokens, experts, topk, unit, use_mask in [
        (1, 8, 2, 16, False), (17, 8, 2, 32, True),
        (128, 64, 8, 32, False), (512, 64, 8, 32, True),
        (5, 6, 3, 4, False), (5, 6, 3, 4, True),
    ]:
        torch.manual_seed(20260720)
        if tokens == 5:
            # worked example of the sorter's header comment
            ids = torch.tensor([[0, 3, 5], [2, 3, 5], [1, 3, 5], [1, 2, 3], [1, 3, 5]],
                               dtype=torch.int32)
        else:
            ids = torch.rand((tokens, experts)).topk(topk, dim=-1).indices.to(torch.int32)
        w = torch.rand((tokens, topk), dtype=torch.float32)
        mask = None
        if use_mask:
            mask = torch.ones(experts, dtype=torch.int32)
            if tokens == 5:
                mask[1] = 0
                mask[4] = 0
            else:
                mask[1::4] = 0
        o_ids, o_w, o_e, counts, starts = srt["_reference"](ids, w, experts, unit, mask)
        key = f"t{tokens}_e{experts}_k{topk}_u{unit}_m{int(use_mask)}"
        sort_cases[key + "/topk_ids"] = ids.numpy()
        sort_cases[key + "/topk_weights"] = w.numpy()
        sort_cases[key + "/mask"] = (mask.numpy() if mask is not None
                                     else np.zeros(0, np.int32))
        sort_cases[key + "/sorted_ids"] = np.asarray(o_ids, dtype=np.int64)
        sort_cases[key + "/sorted_weights"] = np.asarray(o_w, dtype=np.float32)
        sort_cases[key + "/expert_ids"] = np.asarray(o_e, dtype=np.int32)
        sort_cases[key + "/counts"] = np.asarray(counts, dtype=np.int32)
        sort_cases[key + "/starts"] = np.asarray(starts, dtype=np.int32)
    np.savez_compressed(HERE / "sort_ck.npz", **sort_cases)

    # ---- vLLM-format routing helper ----------------------------------------
    sk = load_defs(tdir / "test_moe_single_k.py", ["_cpu_moe_routing"])
    torch.manual_seed(7)
    ids = torch.randint(0, 6, (19, 3), dtype=torch.int32)
    s_ids, e_ids, total = sk["_cpu_moe_routing"](ids, 6, 8)
    np.savez_compressed(HERE / "align_vllm.npz", topk_ids=ids.numpy(),
                        sorted_ids=s_ids.numpy(), expert_ids=e_ids.numpy(),
                        total=total.numpy())

    # ---- routing -------------------------------------------------------------
    rt = load_defs(tune / "routing.py", ["fused_topk"])
    torch.manual_seed(11)
    logits = torch.randn(13, 16)
    wts, tid = rt["fused_topk"](torch.zeros(13, 4), logits, 4, True)
    np.savez_compressed(HERE / "routing.npz", logits=logits.numpy(),
                        weights=wts.numpy(), ids=tid.numpy())

    # ---- grouped gate ----------------------------------------------------------------
    gt = load_defs(tune / "routing.py", ["moe_fused_gate"])
    torch.manual_seed(12)
    glog = torch.randn(11, 64)
    gbias = torch.randn(64) * 0.1
    gate = {"logits": glog.numpy(), "bias": gbias.numpy()}
    for shared in (0, 1):
        k = 6 + shared
        gw = torch.empty(11, k)
        gi = torch.empty(11, k, dtype=torch.int32)
        gt["moe_fused_gate"](glog, gbias, gw, gi, 4, 2, k, shared, 2.5)
        gate[f"w{shared}"] = gw.numpy()
        gate[f"i{shared}"] = gi.numpy()
    np.savez_compressed(HERE / "gate.npz", **gate)

    # ---- bf16 layer ------------------------------------------------------------
    tf = load_defs(tdir / "test_fused_moe.py",
                   ["_torch_moe", "_dynamic_group_quant_int8",
                    "_block_scaled_int8_matmul", "_torch_w8a8_moe"],
                   extra={"DEVICE": "cpu"})
    torch.manual_seed(1)
    m, h, i, e, k = 24, 64, 32, 4, 2
    hidden = (torch.randn(m, h) / 10).bfloat16()
    w1 = (torch.randn(e, 2 * i, h) / 10).bfloat16()
    w2 = (torch.randn(e, h, i) / 10).bfloat16()
    wts, tid = rt["fused_topk"](hidden, torch.randn(m, e), k, True)
    out = tf["_torch_moe"](hidden, w1, w2, wts, tid)
    np.savez_compressed(HERE / "layer_bf16.npz", hidden=t2n(hidden), w1=t2n(w1),
                        w2=t2n(w2), topk_weights=wts.numpy(), topk_ids=tid.numpy(),
                        out=t2n(out))

    # ---- int8 block layer (block 32x32 keeps the fixture small) --------------
    torch.manual_seed(3)
    m, h, i, e, k, blk = 16, 64, 32, 4, 2, (32, 32)
    hidden = (torch.randn(m, h) / 10).half()
    w1 = torch.randint(-127, 128, (e, 2 * i, h), dtype=torch.int8)
    w2 = torch.randint(-127, 128, (e, h, i), dtype=torch.int8)
    w1_s = torch.rand(e, 2 * i // blk[0], h // blk[1]) * 1e-2
    w2_s = torch.rand(e, h // blk[0], i // blk[1]) * 1e-2
    wts, tid = rt["fused_topk"](hidden, torch.randn(m, e), k, True)
    out = tf["_torch_w8a8_moe"](hidden, w1, w2, w1_s, w2_s, wts, tid, blk)
    np.savez_compressed(HERE / "layer_int8_block.npz", hidden=hidden.numpy(),
                        w1=w1.numpy(), w2=w2.numpy(), w1_s=w1_s.numpy(),
                        w2_s=w2_s.numpy(), topk_weights=wts.numpy(),
                        topk_ids=tid.numpy(), out=out.numpy(),
                        block=np.asarray(blk))

    # ---- fp8 block layer ------------------------------------------------------
    cm = load_defs(tune / "common.py", ["apply_activation_ref"])
    fp = load_defs(tune / "tune_moe_fp8.py",
                   ["native_per_token_group_quant_fp8", "native_w8a8_block_fp8_matmul",
                    "torch_w8a8_block_fp8_moe_expert_mask"],
                   extra={"apply_activation_ref": cm["apply_activation_ref"],
                          "ACTIVATION_NAME": "silu", "IS_GATED": True})
    torch.manual_seed(5)
    m, h, i, e, k, blk = 16, 64, 32, 4, 2, [32, 32]
    hidden = (torch.randn(m, h) / 10).bfloat16()
    w1 = (torch.randn(e, 2 * i, h) * 40).clamp(-448, 448).to(torch.float8_e4m3fn)
    w2 = (torch.randn(e, h, i) * 40).clamp(-448, 448).to(torch.float8_e4m3fn)
    w1_s = torch.rand(e, 2 * i // blk[0], h // blk[1]) * 1e-2
    w2_s = torch.rand(e, h // blk[0], i // blk[1]) * 1e-2
    wts, tid = rt["fused_topk"](hidden, torch.randn(m, e), k, True)
    out = fp["torch_w8a8_block_fp8_moe_expert_mask"](
        hidden, w1, w2, w1_s, w2_s, wts, tid.long(), blk)
    q, s = fp["native_per_token_group_quant_fp8"](hidden, 32)
    mm = fp["native_w8a8_block_fp8_matmul"](q, w1[0], s, w1_s[0], blk,
                                             output_dtype=torch.bfloat16)
    np.savez_compressed(HERE / "layer_fp8_block.npz", hidden=t2n(hidden), w1=t2n(w1),
                        w2=t2n(w2), w1_s=w1_s.numpy(), w2_s=w2_s.numpy(),
                        topk_weights=wts.numpy(), topk_ids=tid.numpy(), out=t2n(out),
                        quant_q=t2n(q), quant_s=s.numpy(), matmul0=t2n(mm),
                        block=np.asarray(blk))

    # ---- per-channel int8 layer ---------------------------------------------
    compat = load_defs(ref / "boltops" / "fused_moe" / "triton" / "moe_compat.py",
                       ["pertoken_quant"])

    def _per_token_quant(x, quant_dtype=torch.int8):
        return compat["pertoken_quant"](x, quant_dtype=quant_dtype)

    ch = load_defs(tune / "tune_moe_int8_channel.py",
                   ["native_w8a8_per_token_matmul", "torch_w8a8_per_column_moe_expert_mask"],
                   extra={"apply_activation_ref": cm["apply_activation_ref"],
                          "ACTIVATION_NAME": "silu", "IS_GATED": True,
                          "per_token_quant_triton": _per_token_quant})
    torch.manual_seed(9)
    m, h, i, e, k = 16, 64, 32, 4, 2
    hidden = (torch.randn(m, h) / 10).bfloat16()
    w1 = torch.randint(-127, 128, (e, 2 * i, h), dtype=torch.int8)
    w2 = torch.randint(-127, 128, (e, h, i), dtype=torch.int8)
    w1_s = torch.rand(e, 2 * i) * 1e-2
    w2_s = torch.rand(e, h) * 1e-2
    wts, tid = rt["fused_topk"](hidden, torch.randn(m, e), k, True)
    out = ch["torch_w8a8_per_column_moe_expert_mask"](
        hidden, w1, w2, w1_s, w2_s, wts, tid.long())
    np.savez_compressed(HERE / "layer_int8_channel.npz", hidden=t2n(hidden),
                        w1=w1.numpy(), w2=w2.numpy(), w1_s=w1_s.numpy(),
                        w2_s=w2_s.numpy(), topk_weights=wts.numpy(),
                        topk_ids=tid.numpy(), out=t2n(out))

    # ---- activations -----------------------------------------------------------
    torch.manual_seed(13)
    x = torch.randn(9, 48).bfloat16()
    acts = {"x": t2n(x)}
    for name, gated in [("silu", True), ("gelu", True), ("gelu_tanh", True),
                        ("swigluoai", True), ("swiglustep", True),
                        ("silu", False), ("gelu", False), ("gelu_tanh", False),
                        ("relu2", False)]:
        y = cm["apply_activation_ref"](x.float(), activation_name=name, is_gated=gated)
        acts[f"{name}_{int(gated)}"] = y.numpy()
    np.savez_compressed(HERE / "activations.npz", **acts)

    make_mxfp8(ref)
    make_mxfp4(ref)
    make_signatures(ref)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2 and "BOLTOPS_REFERENCE" not in os.environ:
        raise SystemExit("usage: make_golden.py <path of the reference project checkout> "
                         "(or set BOLTOPS_REFERENCE)")
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ["BOLTOPS_REFERENCE"]
    if len(sys.argv) > 2 and sys.argv[2] == "mxfp8":      # only one fixture
        make_mxfp8(Path(root))
    elif len(sys.argv) > 2 and sys.argv[2] == "mxfp4":
        make_mxfp4(Path(root))
    elif len(sys.argv) > 2 and sys.argv[2] == "signatures":
        make_signatures(Path(root))
    else:
        main(root)
