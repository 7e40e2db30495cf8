"""Pin the CPU oracle against outputs of the reference's own reference
functions (tests/golden/*.npz, produced by tests/golden/make_golden.py) and
against the known-answer vectors written in the reference's tests."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import bf16, fp8, load_npz, t

SORT_KEYS = ["t1_e8_k2_u16_m0", "t17_e8_k2_u32_m1", "t128_e64_k8_u32_m0",
             "t512_e64_k8_u32_m1", "t5_e6_k3_u4_m0", "t5_e6_k3_u4_m1"]


@pytest.mark.parametrize("key", SORT_KEYS)
def test_sort_ck_matches_reference_output(key):
    z = load_npz("sort_ck.npz")
    ids, w = z[key + "/topk_ids"], z[key + "/topk_weights"]
    mask = z[key + "/mask"]
    mask = None if mask.size == 0 else mask
    _, e, k, u, _ = key.split("_")
    E, unit = int(e[1:]), int(u[1:])
    for impl in ("loops", "numpy"):
        if impl == "loops":
            o_ids, o_w, o_e, counts, starts = O.sort_ck_loops(
                torch.from_numpy(ids), torch.from_numpy(w), E, unit, mask)
        else:
            r = O.sort_ck_numpy(ids, w, E, unit, mask)
            o_ids = (r["sorted_ids"].astype(np.int64) & 0xFFFFFFFF).tolist()
            o_w, o_e, counts = r["sorted_weights"].tolist(), r["expert_ids"].tolist(), r["counts"].tolist()
            starts = r["starts"].tolist()
        assert list(o_ids) == z[key + "/sorted_ids"].tolist()
        assert np.array_equal(np.asarray(o_w, np.float32), z[key + "/sorted_weights"])
        assert list(o_e) == z[key + "/expert_ids"].tolist()
        ref_counts, ref_starts = z[key + "/counts"], z[key + "/starts"]
        for ex in range(E):
            if mask is None or mask[ex]:
                assert counts[ex] == ref_counts[ex]
            if ref_starts[ex] >= 0:
                assert starts[ex] == ref_starts[ex]


def test_sort_ck_header_worked_example():
    # moe_sorting_kernel.h:26-88 (E=6, topk=3, unit=4, 5 tokens)
    ids = torch.tensor([[0, 3, 5], [2, 3, 5], [1, 3, 5], [1, 2, 3], [1, 3, 5]], dtype=torch.int32)
    w = torch.arange(15, dtype=torch.float32).reshape(5, 3)
    o_ids, o_w, o_e, _, _ = O.sort_ck_loops(ids, w, 6, 4, None)
    assert o_e == [0, 1, 2, 3, 3, 5] and len(o_ids) == 24
    assert [i & 0xFFFFFF for i in o_ids] == [0, 5, 5, 5, 2, 3, 4, 5, 1, 3, 5, 5,
                                            0, 1, 2, 3, 4, 5, 5, 5, 0, 1, 2, 4]
    mask = torch.tensor([1, 0, 1, 1, 0, 1])
    o_ids, _, o_e, _, _ = O.sort_ck_loops(ids, w, 6, 4, mask)
    assert o_e == [0, 1, 2, 2, 3] and len(o_ids) == 20


def test_align_block_size_docstring_example_and_fixture():
    # boltops/fused_moe/triton/fused_moe.py:362-375 (expert ids run 1..4 => E=5)
    ids = np.array([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=np.int32)
    s, e, total = O.align_block_size_loops(ids, 4, 5)
    assert s[:total].tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert e[: total // 4].tolist() == [1, 2, 3, 4] and total == 16
    z = load_npz("align_vllm.npz")
    s, e, total = O.align_block_size_loops(z["topk_ids"], 8, 6)
    assert total == int(z["total"][0])
    assert s[:total].tolist() == z["sorted_ids"].tolist()
    assert e[: total // 8].tolist() == z["expert_ids"].tolist()


def test_routing_fixture():
    z = load_npz("routing.npz")
    w, ids = O.fused_topk(t(z["logits"]), 4, True)
    assert torch.equal(ids, t(z["ids"]))
    assert torch.equal(w, t(z["weights"]))


def test_layer_bf16_fixture():
    z = load_npz("layer_bf16.npz")
    out = O.moe_bf16(bf16(z["hidden"]), bf16(z["w1"]), bf16(z["w2"]),
                     t(z["topk_weights"]), t(z["topk_ids"]))
    assert torch.equal(out, bf16(z["out"]))


def test_layer_int8_block_fixture():
    z = load_npz("layer_int8_block.npz")
    out = O.moe_block_int8(t(z["hidden"]), t(z["w1"]), t(z["w2"]), t(z["w1_s"]), t(z["w2_s"]),
                           t(z["topk_weights"]), t(z["topk_ids"]), tuple(z["block"]))
    assert torch.equal(out, t(z["out"]))


def test_layer_fp8_block_fixture():
    z = load_npz("layer_fp8_block.npz")
    blk = tuple(int(b) for b in z["block"])
    hidden = bf16(z["hidden"])
    q, s = O.group_quant_fp8_native(hidden, blk[1])
    assert torch.equal(q.view(torch.uint8), fp8(z["quant_q"]).view(torch.uint8))
    assert torch.equal(s, t(z["quant_s"]))
    mm = O.block_scaled_matmul(q, fp8(z["w1"])[0], s, t(z["w1_s"])[0], blk, torch.bfloat16)
    assert torch.equal(mm, bf16(z["matmul0"]))
    out = O.moe_block_fp8(hidden, fp8(z["w1"]), fp8(z["w2"]), t(z["w1_s"]), t(z["w2_s"]),
                          t(z["topk_weights"]), t(z["topk_ids"]), blk)
    assert torch.equal(out, bf16(z["out"]))


def test_layer_int8_channel_fixture():
    z = load_npz("layer_int8_channel.npz")
    out = O.moe_per_channel(bf16(z["hidden"]), t(z["w1"]), t(z["w2"]), t(z["w1_s"]),
                            t(z["w2_s"]), t(z["topk_weights"]), t(z["topk_ids"]))
    assert torch.equal(out, bf16(z["out"]))


@pytest.mark.parametrize("name,gated", [("silu", True), ("gelu", True), ("gelu_tanh", True),
                                        ("swigluoai", True), ("swiglustep", True),
                                        ("silu", False), ("gelu", False),
                                        ("gelu_tanh", False), ("relu2", False)])
def test_activation_fixture(name, gated):
    z = load_npz("activations.npz")
    y = O.activation_ref(bf16(z["x"]), name, gated)
    torch.testing.assert_close(y, t(z[f"{name}_{int(gated)}"]), rtol=1e-6, atol=1e-6)


# ---- known-answer vectors transcribed from the reference's tests ------------
@pytest.mark.parametrize("qdtype", [O.FP8, torch.int8])
def test_quant_zero_rows(qdtype):
    # test/fused_moe/test_quant.py:39-72
    torch.manual_seed(20)
    x = torch.randn(257, 128).bfloat16()
    x[[0, 128, 256]] = 0
    q, s = O.quant_rows_kernel(x, qdtype)
    dmax = 448.0 if qdtype == O.FP8 else 127.0
    expect = torch.tensor(1.0e-10 / dmax, dtype=torch.float32)
    assert torch.isfinite(s).all() and torch.isfinite(q.float()).all()
    torch.testing.assert_close(s[[0, 128, 256], 0], expect.expand(3))
    assert (q[[0, 128, 256]].float() == 0).all()


def test_quant_int8_half_even_and_fp8_fractions():
    # test/fused_moe/test_quant.py:94-142
    v = torch.zeros(2, 8, dtype=torch.float16)
    v[:, :6] = torch.tensor([0.5, -0.5, 1.5, -1.5, 126.5, 127.0], dtype=torch.float16)
    q, s = O.quant_rows_kernel(v, torch.int8)
    assert torch.equal(s, torch.ones_like(s))
    assert q[0, :6].tolist() == [0, 0, 2, -2, 126, 127]
    v = torch.tensor([[0.5, 1.5, 2.5, 448.0]], dtype=torch.float16)
    q, s = O.quant_rows_kernel(v, O.FP8)
    assert torch.equal(s, torch.ones_like(s))
    assert torch.equal(q.float(), v.float())


def test_quant_power2_scales():
    # test/fused_moe/test_quant.py:359-379
    exps = torch.arange(-33, 128, dtype=torch.float32)
    x = torch.zeros(len(exps) + 2, 128)
    x[:-2, 0] = torch.exp2(exps)
    x[:-2, 1] = -torch.exp2(exps)
    x[-1, 0] = torch.finfo(torch.float32).tiny
    _, s = O.group_quant_fp8_power2(x)
    expect = torch.cat((torch.exp2(exps - 8), torch.full((2,), 2.0 ** -42)))
    assert torch.equal(s[:, 0], expect)


@pytest.mark.parametrize("width", [128, 137])
def test_moe_sum_known_answer(width):
    # test/fused_moe/test_fused_moe.py:1359-1377
    x = (torch.arange(3 * 2 * width).reshape(3, 2, width).float() / 256).bfloat16()
    expect = ((x[:, 0].float() + x[:, 1].float()) * 1.25).bfloat16()
    assert torch.equal(O.moe_sum(x, 1.25), expect)


@pytest.mark.parametrize("shared", [0, 1])
def test_grouped_gate_fixture(shared):
    z = load_npz("gate.npz")
    k = 6 + shared
    w, i = O.fused_gate(t(z["logits"]), t(z["bias"]), 4, 2, k, shared, 2.5)
    ref_w, ref_i = t(z[f"w{shared}"]), t(z[f"i{shared}"])
    # the reference does not sort the routed experts when no shared expert is fused
    for row in range(w.shape[0]):
        got = sorted(zip(i[row].tolist(), w[row].tolist()))
        exp = sorted(zip(ref_i[row].tolist(), ref_w[row].tolist()))
        assert [a for a, _ in got] == [a for a, _ in exp]
        assert all(abs(a - b) <= 1e-6 for (_, a), (_, b) in zip(got, exp))


@pytest.mark.parametrize("case", ["default", "silu_alpha", "swigluoai", "no_combine", "dynamic_fp16"])
def test_mxfp8_layer_fixture(case):
    """The oracle's MXFP8 layer reproduces the reference's own CPU statement bit for bit."""
    from tests.helpers import MX_CASES, load_mx_case
    c = load_mx_case(case)
    out = O.moe_mxfp8(c["x"], c["w1"], c["w2"], c["s1"], c["s2"], c["weights"], c["ids"],
                      **MX_CASES[case])
    assert out.dtype == c["expected"].dtype
    assert torch.equal(out.float(), c["expected"].float())


@pytest.mark.parametrize("case", __import__("tests.helpers", fromlist=["MXFP4_CASES"]).MXFP4_CASES)
def test_mxfp4_layer_fixture(case):
    """The oracle's MXFP4 layer reproduces the reference's CPU statement bit for bit on every
    case of test_public_mxfp4_cpu_reference (fixture written by make_golden.py)."""
    from tests.helpers import load_mxfp4_case
    c = load_mxfp4_case(case)
    got = O.moe_mxfp4(
        c["x"], c["w1"], c["w2"], c["s1"], c["s2"], c["weights"], c["ids"],
        activation=c["activation"], expert_map=c["expert_map"],
        a1_scale=c["static_s1"] if c["static"] else None,
        a2_scale=c["static_s2"] if c["static"] else None, b1=c["bias1"], b2=c["bias2"],
        alpha=c["alpha"] if c["static"] else None, limit=c["clamp"],
        apply_router_weight_on_input=c["input_router"], no_combine=c["no_combine"],
        routed_scaling_factor=1.25)
    assert got.dtype == c["expected"].dtype and got.shape == c["expected"].shape
    assert torch.equal(got, c["expected"])
    # the test's pre-quantised inputs are the oracle quantiser's codes and scales
    if not c["static"]:
        q, scale, _ = O.mxfp4_quant_g128(c["x"])
        assert torch.equal(q.view(torch.uint8), c["input_q"].view(torch.uint8))
        assert torch.equal(scale, c["input_scale"])
