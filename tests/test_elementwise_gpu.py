"""Quantisers, activations and the combine vs the CPU oracle."""
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import bf16, load_npz, t

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _bits(x):
    return x.view(torch.uint8) if x.dtype == FP8 else x


@pytest.mark.parametrize("shape,group", [((2, 128), None), ((257, 128), None), ((1281, 1232), None),
                                         ((64, 7168), 128), ((33, 2048), 128), ((5, 4096), None),
                                         ((3, 20000), None), ((7, 100), None), ((16, 512), 64)])
@pytest.mark.parametrize("qdtype", [FP8, torch.int8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quant_rows_bit_exact(shape, group, qdtype, dtype):
    from boltops_b200.fused_moe import ops
    torch.manual_seed(20)
    x = (torch.randn(shape) * 3).to(dtype)
    x[0] = 0
    x[shape[0] // 2, : shape[1] // 2] = 0
    q_ref, s_ref = O.quant_rows_kernel(x, qdtype, group)
    q, s = ops.quant_rows(x.cuda(), qdtype, group)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(_bits(q.cpu()), _bits(q_ref))


def test_quant_known_answers():
    from boltops_b200.fused_moe import ops
    v = torch.zeros(256, 128, dtype=torch.float16)
    v[:, :6] = torch.tensor([0.5, -0.5, 1.5, -1.5, 126.5, 127.0], dtype=torch.float16)
    q, s = ops.per_token_quant(v.cuda(), quant_dtype=torch.int8)
    assert torch.equal(s.cpu(), torch.ones(256, 1))
    assert q.cpu()[0, :6].tolist() == [0, 0, 2, -2, 126, 127]
    v = torch.tensor([[0.5, 1.5, 2.5, 448.0]], dtype=torch.float16)
    q, s = ops.per_token_quant(v.cuda(), quant_dtype=FP8)
    assert torch.equal(s.cpu(), torch.ones(1, 1))
    assert torch.equal(q.cpu().float(), v.float())
    z = torch.zeros(4, 256, dtype=torch.bfloat16)
    for qd, dmax in ((FP8, 448.0), (torch.int8, 127.0)):
        q, s = ops.per_token_quant(z.cuda(), quant_dtype=qd)
        assert torch.equal(s.cpu(), torch.full((4, 1), 1.0e-10, dtype=torch.float32) / dmax)
        assert (q.cpu().float() == 0).all()


@pytest.mark.parametrize("width", [32, 128, 256])
def test_quant_power2(width):
    from boltops_b200.fused_moe import ops
    torch.manual_seed(225)
    x = torch.randn(19, width)
    x[0].zero_()
    bounds = torch.tensor([448 * 2.0 ** e for e in range(-9, 8)])
    x[1:18] *= 0.01
    x[1:18, 0] = bounds
    x[18, 0] = torch.nextafter(bounds[8], torch.tensor(float("inf")))
    q_ref, s_ref = O.group_quant_fp8_power2(x)
    q, s = ops.quant_rows(x.cuda(), FP8, None, scale_ue8m0=True)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(_bits(q.cpu()), _bits(q_ref))


@pytest.mark.parametrize("name,gated,kw", [
    ("silu", True, {}), ("gelu", True, {}), ("gelu_tanh", True, {}), ("swiglustep", True, {}),
    ("silu", False, {}), ("gelu", False, {}), ("gelu_tanh", False, {}), ("relu2", False, {}),
    ("silu", True, {"gemm1_limit": 4.0}),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,n", [(9, 48), (64, 3072), (3, 1000), (1, 6)])
def test_moe_activation(name, gated, kw, dtype, rows, n):
    from boltops_b200.fused_moe import moe_activation
    torch.manual_seed(13)
    x = torch.randn(rows, n).to(dtype)
    n_out = n // 2 if gated else n
    out = torch.empty(rows, n_out, dtype=dtype, device="cuda")
    moe_activation(out, x.cuda(), name, gated, **kw)
    ref = O.activation_ref(x, name, gated, limit=kw.get("gemm1_limit")).to(dtype)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    if name == "silu" and gated and not kw:
        # same formula, same rounding: at most 1 ulp of the storage type apart
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2 ** -7, atol=1e-6)


def test_moe_activation_fixture_and_errors():
    from boltops_b200.fused_moe import moe_activation
    z = load_npz("activations.npz")
    x = bf16(z["x"])
    out = torch.empty(9, 24, dtype=torch.bfloat16, device="cuda")
    moe_activation(activated_out=out, ffn1_out_2d=x.cuda(), activation="silu")
    torch.testing.assert_close(out.cpu().float(), t(z["silu_1"]).bfloat16().float(),
                               rtol=2 ** -7, atol=1e-6)
    with pytest.raises(ValueError):
        moe_activation(out, x.cuda(), "nope")
    with pytest.raises(ValueError):
        moe_activation(out[:, :5], x.cuda(), "silu")
    with pytest.raises(ValueError):
        moe_activation(out, x, "silu")
    with pytest.raises(TypeError):
        moe_activation(out.to(torch.int32), x.cuda().to(torch.int32), "silu")


@pytest.mark.parametrize("qdtype", [FP8, torch.int8])
def test_activation_quant_matches_unfused(qdtype):
    from boltops_b200.fused_moe import ops
    from boltops_b200.fused_moe.activation import activation_quant, apply_activation
    torch.manual_seed(3)
    x = torch.randn(37, 1536, dtype=torch.bfloat16, device="cuda")
    act = torch.empty(37, 768, dtype=torch.bfloat16, device="cuda")
    apply_activation("silu", True, act, x)
    q_ref, s_ref = ops.per_token_quant(act, quant_dtype=qdtype)
    q, s = activation_quant(x, "silu", True, qdtype)
    assert torch.equal(s, s_ref) and torch.equal(_bits(q), _bits(q_ref))
    mult = torch.rand(37, device="cuda")
    q2, s2 = activation_quant(x, "silu", True, qdtype, row_multiplier=mult)
    assert torch.equal(_bits(q2), _bits(q)) and torch.equal(s2, s * mult[:, None])


@pytest.mark.parametrize("width", [128, 137, 7168])
@pytest.mark.parametrize("weighted", [False, True])
def test_moe_sum(width, weighted):
    from boltops_b200.fused_moe import ops
    x = (torch.arange(3 * 2 * width).reshape(3, 2, width).float() / 256).bfloat16()
    w = torch.tensor([[0.2, 0.8], [0.7, 0.3], [0.4, 0.6]]) if weighted else None
    out = torch.empty(3, width, dtype=torch.bfloat16, device="cuda")
    ops.moe_sum(x.cuda(), out, 1.25, None if w is None else w.cuda())
    assert torch.equal(out.cpu(), O.moe_sum(x, 1.25, weights=w))


def test_moe_sum_topk8_random():
    from boltops_b200.fused_moe import ops
    torch.manual_seed(0)
    x = torch.randn(100, 8, 2048).bfloat16()
    out = torch.empty(100, 2048, dtype=torch.bfloat16, device="cuda")
    ops.moe_sum(x.cuda(), out, 2.5)
    assert torch.equal(out.cpu(), O.moe_sum(x, 2.5))
    out32 = torch.empty(100, 2048, dtype=torch.float32, device="cuda")
    ops.moe_sum(x.cuda(), out32, 1.0)
    assert torch.equal(out32.cpu(), O.moe_sum(x, 1.0, out_dtype=torch.float32))


def test_moe_activation_swigluoai_interleaved_and_situ():
    from boltops_b200.fused_moe import moe_activation
    torch.manual_seed(21)
    x = (torch.randn(33, 512) * 3).bfloat16()
    out = torch.empty(33, 256, dtype=torch.bfloat16, device="cuda")
    moe_activation(out, x.cuda(), "swigluoai")
    ref = O.activation_ref(x, "swigluoai", True, interleaved=True).bfloat16()
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    moe_activation(out, x.cuda(), "swigluoai", gemm1_alpha=1.2, gemm1_limit=3.0)
    ref = O.activation_ref(x, "swigluoai", True, limit=3.0, alpha=1.2, interleaved=True).bfloat16()
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    for lin in (None, 5.0):
        moe_activation(out, x.cuda(), "situ", activation_situ_beta=6.0,
                       activation_situ_linear_beta=lin)
        ref = O.activation_ref(x, "situ", True, situ_beta=6.0, situ_linear_beta=lin).bfloat16()
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    with pytest.raises(ValueError):
        moe_activation(out, x.cuda(), "situ")


@pytest.mark.parametrize("m,e,k,softmax,renorm,dtype", [
    (13, 16, 4, True, True, torch.float32), (4096, 256, 8, True, True, torch.float32),
    (300, 128, 8, True, False, torch.bfloat16), (77, 8, 2, False, True, torch.float32),
    (1, 384, 6, True, True, torch.float16),
])
def test_fused_topk(m, e, k, softmax, renorm, dtype):
    from boltops_b200.fused_moe.routing import fused_topk
    g = torch.Generator().manual_seed(m + e)
    logits = torch.randn(m, e, generator=g).to(dtype)
    w_ref, i_ref = O.fused_topk(logits, k, renorm, softmax)
    w, i = fused_topk(torch.zeros(m, 4), logits.cuda(), k, renorm, is_softmax=softmax)
    assert i.dtype == torch.int32 and w.dtype == torch.float32
    torch.testing.assert_close(w.cpu(), w_ref, rtol=1e-5, atol=1e-7)
    # ids: identical unless logits tie (16-bit logits tie often; either expert is a valid pick):
    # the chosen experts must carry exactly the reference's scores, without repeats
    scores = torch.softmax(logits.float(), -1) if softmax else logits.float().sigmoid()
    picked = scores.gather(1, i.cpu().long())
    torch.testing.assert_close(picked, scores.gather(1, i_ref.long()), rtol=1e-6, atol=0)
    assert all(len(set(row)) == k for row in i.cpu().tolist())
    if dtype == torch.float32:
        assert torch.equal(i.cpu(), i_ref)


@pytest.mark.parametrize("m,e,groups,topk_group,topk,shared", [
    (64, 256, 8, 4, 8, 0), (33, 256, 8, 4, 9, 1), (7, 64, 4, 2, 6, 0), (5, 16, 1, 1, 4, 0),
])
def test_moe_fused_gate(m, e, groups, topk_group, topk, shared):
    from boltops_b200.fused_moe.routing import moe_fused_gate
    g = torch.Generator().manual_seed(m + e)
    logits = torch.randn(m, e, generator=g)
    bias = torch.randn(e, generator=g) * 0.1
    w_ref, i_ref = O.fused_gate(logits, bias, groups, topk_group, topk, shared, 2.5)
    w = torch.empty(m, topk, dtype=torch.float32, device="cuda")
    i = torch.empty(m, topk, dtype=torch.int32, device="cuda")
    out = moe_fused_gate(logits.cuda(), bias.cuda(), w, i, groups, topk_group, topk, shared, 2.5)
    assert out[0] is w and out[1] is i
    # the reference leaves the order of the routed experts unspecified unless a shared expert
    # is fused; compare as sets of (id, weight) pairs, the shared slot stays last
    for t_ in range(m):
        got = sorted(zip(i[t_].tolist(), w[t_].tolist()))
        exp = sorted(zip(i_ref[t_].tolist(), w_ref[t_].tolist()))
        assert [a for a, _ in got] == [a for a, _ in exp]
        for (_, a), (_, b) in zip(got, exp):
            assert abs(a - b) <= 1e-5 * max(1.0, abs(b))
    if shared:
        assert (i[:, -1] == e).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("q_dtype", [torch.float8_e4m3fn, torch.int8])
@pytest.mark.parametrize("group", [128, 512])      # 1 x 128 blocks / one scale per token
def test_quant_scatter_equals_quant_then_gather(dtype, q_dtype, group):
    """The fused quantise+scatter writes the same bytes as quantising and gathering, and zeros
    in the rows that only pad a tile."""
    from boltops_b200.fused_moe import ops
    torch.manual_seed(5)
    m, h, e, k = 77, 512, 8, 3
    x = (torch.randn(m, h) * 3).to(dtype).cuda()
    _, ids = O.make_routing(m, e, k, 11)
    ids[3, 1] = -1                                   # a masked route
    ids = ids.cuda()
    w = torch.rand(m, k).cuda()
    pos = torch.empty((m, k), dtype=torch.int32, device="cuda")
    s_ids, _, _, nv, _, _ = ops.moe_sorting_ck(ids, w, e, None, None, 128, None,
                                               alloc_moe_buf=False, route_pos=pos)
    cap = s_ids.shape[0]
    x_q, x_s = ops.per_block_quant(x, group, q_dtype)
    ref, ref_s = ops.gather_rows(x_q, s_ids, nv, cap, x_s)
    ref_s = ref_s.reshape(h // group, cap)
    got, got_s = ops.quant_scatter_rows(x, group, q_dtype, pos, s_ids, nv, cap)
    n = int(nv.item())
    assert torch.equal(got[:n].view(torch.uint8).cpu(), ref[:n].view(torch.uint8).cpu())
    assert torch.equal(got_s[:, :n].cpu(), ref_s[:, :n].cpu())
    pad = ((s_ids[:n] & 0xFFFFFF) >= m).cpu()
    assert pad.any()
    assert (got[:n].view(torch.uint8).cpu()[pad] == 0).all()
    assert (got_s[:, :n].cpu()[:, pad] == 0).all()
