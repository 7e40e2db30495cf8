"""Full fused_experts layer vs the CPU oracle (through the public API)."""
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import bf16, fp8, load_npz, t

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _dev(*xs):
    return [x.cuda() if isinstance(x, torch.Tensor) else x for x in xs]


def _finish(out):
    from boltops_b200.fused_moe import ops
    torch.cuda.synchronize()
    ops.check_device_status(out.device)
    return out.cpu()


def test_layer_bf16_golden_fixture():
    from boltops_b200.fused_moe import fused_experts
    z = load_npz("layer_bf16.npz")
    args = _dev(bf16(z["hidden"]), bf16(z["w1"]), bf16(z["w2"]), t(z["topk_weights"]), t(z["topk_ids"]))
    out = _finish(fused_experts(*args))
    expect = bf16(z["out"])
    assert O.rel_l2(out, expect) <= 1e-2
    torch.testing.assert_close(out.float(), expect.float(), rtol=3e-2, atol=2e-2)


@pytest.mark.parametrize("m", [1, 64, 333])
def test_layer_bf16_config1(m):
    """E=8, top-2, H=1024, I=512 (the CPU-runnable benchmark configuration)."""
    from boltops_b200.fused_moe import fused_experts
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn(m, 1024, generator=g).bfloat16()
    w1 = (torch.randn(8, 1024, 1024, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(8, 1024, 512, generator=g) * 0.02).bfloat16()
    wts, ids = O.make_routing(m, 8, 2, 1)
    out = _finish(fused_experts(*_dev(hidden, w1, w2, wts, ids)))
    expect = O.moe_bf16(hidden, w1, w2, wts, ids)
    assert out.shape == hidden.shape and out.dtype == hidden.dtype
    assert O.rel_l2(out, expect) <= 1e-2


def test_layer_bf16_reference_test_shape_topk1():
    """hidden 336 (not a multiple of the K tile), as in the reference's top-1 test."""
    from boltops_b200.fused_moe import fused_experts
    torch.manual_seed(4)
    m, h, i, e = 32, 336, 512, 4
    hidden = (torch.randn(m, h) / 10).bfloat16()
    w1 = (torch.randn(e, 2 * i, h) / 10).bfloat16()
    w2 = (torch.randn(e, h, i) / 10).bfloat16()
    ids = (torch.arange(m)[:, None] % e).to(torch.int32)
    wts = torch.ones(m, 1)
    out = _finish(fused_experts(*_dev(hidden, w1, w2, wts, ids), activation="silu", is_gated=True,
                                global_num_experts=e))
    expect = O.moe_bf16(hidden, w1, w2, wts, ids)
    torch.testing.assert_close(out.float(), expect.float(), rtol=3e-2, atol=2e-2)


def _fp8_block_case(m, e, topk, h, i, seed):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(m, h, generator=g).bfloat16()
    w1q, w1s = O.quantize_weight_block_fp8(torch.randn(e, 2 * i, h, generator=g) * 0.02)
    w2q, w2s = O.quantize_weight_block_fp8(torch.randn(e, h, i, generator=g) * 0.02)
    wts, ids = O.make_routing(m, e, topk, seed + 1)
    return hidden, w1q, w2q, w1s, w2s, wts, ids


@pytest.mark.parametrize("m,e,topk,h,i", [(48, 8, 2, 512, 256), (130, 16, 4, 1024, 384)])
def test_layer_fp8_block(m, e, topk, h, i):
    from boltops_b200.fused_moe import fused_experts
    hidden, w1q, w2q, w1s, w2s, wts, ids = _fp8_block_case(m, e, topk, h, i, 3)
    out = _finish(fused_experts(*_dev(hidden, w1q, w2q, wts, ids), use_fp8_w8a8=True,
                                w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128]))
    expect = O.moe_block_fp8(hidden, w1q, w2q, w1s, w2s, wts, ids, (128, 128))
    assert O.rel_l2(out, expect) <= 2e-2


def test_layer_fp8_block_ue8m0_unfused_path():
    from boltops_b200.fused_moe import fused_experts
    hidden, w1q, w2q, w1s, w2s, wts, ids = _fp8_block_case(40, 8, 2, 512, 256, 8)
    out = _finish(fused_experts(*_dev(hidden, w1q, w2q, wts, ids), use_fp8_w8a8=True,
                                w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128],
                                use_ue8m0=True))
    expect = O.moe_block_fp8(hidden, w1q, w2q, w1s, w2s, wts, ids, (128, 128), power2=True)
    assert O.rel_l2(out, expect) <= 2e-2


def test_layer_int8_block():
    from boltops_b200.fused_moe import fused_experts
    torch.manual_seed(3)
    m, e, topk, h, i = 64, 8, 2, 512, 256
    hidden = (torch.randn(m, h) / 10).half()
    w1 = torch.randint(-127, 128, (e, 2 * i, h), dtype=torch.int8)
    w2 = torch.randint(-127, 128, (e, h, i), dtype=torch.int8)
    w1s = torch.rand(e, 2 * i // 128, h // 128) * 1e-2
    w2s = torch.rand(e, h // 128, i // 128) * 1e-2
    wts, ids = O.make_routing(m, e, topk, 2)
    out = _finish(fused_experts(*_dev(hidden, w1, w2, wts, ids), use_int8_w8a8=True,
                                w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128],
                                output_dtype=hidden.dtype))
    expect = O.moe_block_int8(hidden, w1, w2, w1s, w2s, wts, ids, (128, 128))
    err = (out.float() - expect.float()).abs().mean() / expect.float().abs().mean()
    assert err < 0.02 and O.rel_l2(out, expect) <= 2e-2


@pytest.mark.parametrize("qdtype", [torch.int8, FP8])
def test_layer_per_channel(qdtype):
    from boltops_b200.fused_moe import fused_experts
    g = torch.Generator().manual_seed(9)
    m, e, topk, h, i = 100, 16, 4, 512, 384
    hidden = torch.randn(m, h, generator=g).bfloat16()
    if qdtype == torch.int8:
        w1, w1s = O.quantize_weight_channel_int8(torch.randn(e, 2 * i, h, generator=g) * 0.02)
        w2, w2s = O.quantize_weight_channel_int8(torch.randn(e, h, i, generator=g) * 0.02)
        flags = dict(use_int8_w8a8=True)
    else:
        m1 = torch.randn(e, 2 * i, h, generator=g) * 0.02
        m2 = torch.randn(e, h, i, generator=g) * 0.02
        w1s = m1.abs().amax(-1) / 448
        w2s = m2.abs().amax(-1) / 448
        w1 = (m1 / w1s[..., None]).to(FP8)
        w2 = (m2 / w2s[..., None]).to(FP8)
        flags = dict(use_fp8_w8a8=True)
    wts, ids = O.make_routing(m, e, topk, 4)
    out = _finish(fused_experts(*_dev(hidden, w1, w2, wts, ids), per_channel_quant=True,
                                w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), **flags))
    expect = O.moe_per_channel(hidden, w1, w2, w1s, w2s, wts, ids, qdtype)
    assert O.rel_l2(out, expect) <= 2e-2


def test_layer_golden_quantised_fixtures():
    """int8 per-channel fixture produced by the reference's own torch path."""
    from boltops_b200.fused_moe import fused_experts
    z = load_npz("layer_int8_channel.npz")
    hidden, w1, w2 = bf16(z["hidden"]), t(z["w1"]), t(z["w2"])
    out = _finish(fused_experts(*_dev(hidden, w1, w2, t(z["topk_weights"]), t(z["topk_ids"])),
                                use_int8_w8a8=True, per_channel_quant=True,
                                w1_scale=t(z["w1_s"]).cuda(), w2_scale=t(z["w2_s"]).cuda()))
    assert O.rel_l2(out, bf16(z["out"])) <= 2e-2


def test_layer_variants_no_combine_inplace_expert_map_scaling():
    from boltops_b200.fused_moe import fused_experts
    g = torch.Generator().manual_seed(5)
    m, e, topk, h, i = 50, 8, 2, 256, 128
    hidden = torch.randn(m, h, generator=g).bfloat16()
    w1 = (torch.randn(e, 2 * i, h, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(e, h, i, generator=g) * 0.05).bfloat16()
    wts, ids = O.make_routing(m, e, topk, 6)
    base = O.moe_bf16(hidden, w1, w2, wts, ids)
    d = _dev(hidden, w1, w2, wts, ids)
    # routed scaling factor
    out = _finish(fused_experts(*d, routed_scaling_factor=2.5))
    assert O.rel_l2(out, O.moe_bf16(hidden, w1, w2, wts, ids, 2.5)) <= 1e-2
    # no_combine returns unweighted per-route rows
    nc = _finish(fused_experts(*d, no_combine=True))
    assert nc.shape == (m, topk, h)
    comb = (nc.float() * wts[:, :, None]).sum(1)
    assert O.rel_l2(comb, base) <= 1e-2
    # expert-parallel masking: two ranks' partial sums add up to the full layer
    parts = []
    for rank in range(2):
        emap = torch.full((e,), -1, dtype=torch.int32)
        emap[rank * 4:(rank + 1) * 4] = torch.arange(4, dtype=torch.int32)
        sl = slice(rank * 4, rank * 4 + 4)
        parts.append(_finish(fused_experts(hidden.cuda(), w1[sl].cuda(), w2[sl].cuda(), wts.cuda(),
                                           ids.cuda(), expert_map=emap.cuda(),
                                           global_num_experts=e)).float())
    assert O.rel_l2(parts[0] + parts[1], base) <= 1.5e-2
    # inplace returns the input tensor itself
    hid_dev = hidden.cuda()
    ret = fused_experts(hid_dev, d[1], d[2], d[3], d[4], inplace=True)
    assert ret.data_ptr() == hid_dev.data_ptr()
    assert O.rel_l2(_finish(ret), base) <= 1e-2


def test_layer_non_fused_activation_and_bias():
    from boltops_b200.fused_moe import fused_experts
    g = torch.Generator().manual_seed(12)
    m, e, topk, h, i = 40, 4, 2, 256, 128
    hidden = torch.randn(m, h, generator=g).bfloat16()
    w1 = (torch.randn(e, 2 * i, h, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(e, h, i, generator=g) * 0.05).bfloat16()
    b1 = (torch.randn(e, 2 * i, generator=g) * 0.1).bfloat16()
    b2 = (torch.randn(e, h, generator=g) * 0.1).bfloat16()
    wts, ids = O.make_routing(m, e, topk, 13)
    out = _finish(fused_experts(*_dev(hidden, w1, w2, wts, ids), activation="gelu",
                                b1=b1.cuda(), b2=b2.cuda()))
    rep = hidden[:, None, :].expand(m, topk, h).reshape(-1, h)
    flat = ids.reshape(-1)
    routed = torch.zeros(m * topk, h)
    for ex in range(e):
        sel = flat == ex
        c1 = (rep[sel].float() @ w1[ex].float().t() + b1[ex].float()).bfloat16()
        act = O.activation_ref(c1, "gelu", True).bfloat16()
        routed[sel] = (act.float() @ w2[ex].float().t() + b2[ex].float())
    expect = (routed.view(m, topk, h) * wts[:, :, None]).sum(1)
    assert O.rel_l2(out, expect) <= 1.5e-2


def test_layer_argument_errors():
    from boltops_b200.fused_moe import fused_experts
    hid = torch.zeros(1, 128, dtype=torch.bfloat16, device="cuda")
    w1 = torch.zeros(1, 256, 128, dtype=torch.bfloat16, device="cuda")
    w2 = torch.zeros(1, 128, 128, dtype=torch.bfloat16, device="cuda")
    wts = torch.ones(1, 1, device="cuda")
    ids = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError):
        fused_experts(hid, w1, w2, wts, ids, use_ue8m0=True)
    with pytest.raises(ValueError):
        fused_experts(hid, w1, w2, wts, ids, gemm1_beta=1.0)
    with pytest.raises(ValueError):
        fused_experts(hid, w1, w2, wts, ids, activation="nope")
    with pytest.raises(AssertionError):
        fused_experts(hid, w1, w2, wts[:, :0], ids)
    with pytest.raises(NotImplementedError):
        fused_experts(hid, w1, w2, wts, ids, use_int4_w4a16=True)


def test_layer_is_cuda_graph_capturable():
    """No step of the layer synchronises the host, so it captures into a CUDA graph
    (the reference benchmarks its layer under graphs, test/fused_moe/test_fused_moe.py:1317-1324)."""
    from boltops_b200.fused_moe import fused_experts
    hidden, w1q, w2q, w1s, w2s, wts, ids = _fp8_block_case(64, 8, 2, 512, 256, 21)
    d = _dev(hidden, w1q, w2q, wts, ids)
    kw = dict(use_fp8_w8a8=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128])
    eager = _finish(fused_experts(*d, **kw))
    static_in = d[0].clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fused_experts(static_in, d[1], d[2], d[3], d[4], **kw)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = fused_experts(static_in, d[1], d[2], d[3], d[4], **kw)
    graph.replay()
    assert torch.equal(_finish(static_out), eager)
    static_in.copy_(d[0] * 0.5)            # new input, same graph
    graph.replay()
    again = _finish(static_out)
    expect = _finish(fused_experts(d[0] * 0.5, d[1], d[2], d[3], d[4], **kw))
    assert torch.equal(again, expect)


def test_layer_edge_cases_empty_single_duplicates_chunks(monkeypatch):
    from boltops_b200.fused_moe import fused_experts
    g = torch.Generator().manual_seed(31)
    e, topk, h, i = 16, 4, 256, 128
    w1 = (torch.randn(e, 2 * i, h, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(e, h, i, generator=g) * 0.05).bfloat16()
    d1, d2 = w1.cuda(), w2.cuda()
    # empty batch
    out = fused_experts(torch.empty(0, h, dtype=torch.bfloat16, device="cuda"), d1, d2,
                        torch.empty(0, topk, device="cuda"),
                        torch.empty(0, topk, dtype=torch.int32, device="cuda"))
    assert out.shape == (0, h)
    # one token: most experts receive nothing
    hidden = torch.randn(1, h, generator=g).bfloat16()
    wts, ids = O.make_routing(1, e, topk, 5)
    out = _finish(fused_experts(hidden.cuda(), d1, d2, wts.cuda(), ids.cuda()))
    assert O.rel_l2(out, O.moe_bf16(hidden, w1, w2, wts, ids)) <= 1e-2
    # a token that lists the same expert twice, and all tokens on one expert
    m = 40
    hidden = torch.randn(m, h, generator=g).bfloat16()
    wts, ids = O.make_routing(m, e, topk, 6)
    ids[:, 1] = ids[:, 0]
    ids[m // 2:] = 3
    out = _finish(fused_experts(hidden.cuda(), d1, d2, wts.cuda(), ids.cuda()))
    assert O.rel_l2(out, O.moe_bf16(hidden, w1, w2, wts, ids)) <= 1e-2
    # token chunking (the reference's TRITON_FUSED_MOE_CHUNK_SIZE loop), ragged last chunk
    monkeypatch.setenv("BOLTOPS_FUSED_MOE_CHUNK_SIZE", "17")
    wts, ids = O.make_routing(m, e, topk, 7)
    out = _finish(fused_experts(hidden.cuda(), d1, d2, wts.cuda(), ids.cuda()))
    assert O.rel_l2(out, O.moe_bf16(hidden, w1, w2, wts, ids)) <= 1e-2
    monkeypatch.setenv("BOLTOPS_FUSED_MOE_CHUNK_SIZE", "0")
    with pytest.raises(ValueError):
        fused_experts(hidden.cuda(), d1, d2, wts.cuda(), ids.cuda())


def test_layer_apply_router_weight_on_input_topk1_and_prequantised_input():
    from boltops_b200.fused_moe import fused_experts, ops
    g = torch.Generator().manual_seed(41)
    m, e, h, i = 48, 8, 256, 128
    hidden = torch.randn(m, h, generator=g).bfloat16()
    w1 = (torch.randn(e, 2 * i, h, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(e, h, i, generator=g) * 0.05).bfloat16()
    wts, ids = O.make_routing(m, e, 1, 9)
    wts = torch.rand(m, 1, generator=g) + 0.5
    out = _finish(fused_experts(*_dev(hidden, w1, w2, wts, ids), apply_router_weight_on_input=True))
    # weight applied to GEMM1's output (before the activation), nothing after GEMM2
    rows = []
    for t_ in range(m):
        ex = int(ids[t_, 0])
        c1 = ((hidden[t_].float() @ w1[ex].float().t()) * wts[t_, 0]).bfloat16()
        act = O.activation_ref(c1[None], "silu", True).bfloat16()
        rows.append((act.float() @ w2[ex].float().t()).bfloat16())
    assert O.rel_l2(out, torch.cat(rows)) <= 1e-2
    # pre-quantised fp8 hidden with a1_scale equals the layer quantising by itself
    hq, w1q, w2q, w1s, w2s, wts, ids = _fp8_block_case(32, 8, 2, 512, 256, 17)
    kw = dict(use_fp8_w8a8=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128])
    ref = _finish(fused_experts(*_dev(hq, w1q, w2q, wts, ids), **kw))
    x_q, x_s = ops.per_block_quant(hq.cuda(), 128, FP8)
    out = _finish(fused_experts(x_q, w1q.cuda(), w2q.cuda(), wts.cuda(), ids.cuda(), a1_scale=x_s,
                                output_dtype=torch.bfloat16, **kw))
    assert torch.equal(out, ref)


def test_layer_special_values_stay_in_their_rows():
    """A token with NaN / Inf inputs poisons only its own output row (rows are independent in
    every stage), and denormal / signed-zero inputs give finite results."""
    from boltops_b200.fused_moe import fused_experts
    g = torch.Generator().manual_seed(51)
    m, e, topk, h, i = 130, 8, 2, 256, 128
    hidden = torch.randn(m, h, generator=g).bfloat16()
    w1 = (torch.randn(e, 2 * i, h, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(e, h, i, generator=g) * 0.05).bfloat16()
    wts, ids = O.make_routing(m, e, topk, 52)
    clean = _finish(fused_experts(*_dev(hidden, w1, w2, wts, ids)))
    bad = hidden.clone()
    bad[3, 5] = float("nan")
    bad[77, 0] = float("inf")
    bad[10, :] = 0.0
    bad[10, 1] = -0.0
    bad[11, :] = 1e-40          # flushes to a bf16 denormal / zero
    out = _finish(fused_experts(*_dev(bad, w1, w2, wts, ids)))
    assert torch.isnan(out[3]).any() and not torch.isfinite(out[77]).all()
    ok_rows = [r for r in range(m) if r not in (3, 77, 10, 11)]
    assert torch.equal(out[ok_rows], clean[ok_rows])
    assert torch.isfinite(out[10].float()).all() and (out[10] == 0).all()
    assert torch.isfinite(out[11].float()).all()


@pytest.mark.parametrize("kind", ["bf16", "fp8_block", "int8_channel"])
def test_layer_tile_pair_schedule(monkeypatch, kind):
    """The layer with the tile-pair GEMM schedule forced (experts with one to five row tiles,
    expert parallel mask included): equal to the single-tile schedule bit for bit, and within
    the tolerance of the oracle."""
    from boltops_b200.fused_moe import fused_experts
    m, e, topk, h, i = 1200, 8, 2, 512, 256
    g = torch.Generator().manual_seed(21)
    hidden = torch.randn(m, h, generator=g).bfloat16()
    m1 = torch.randn(e, 2 * i, h, generator=g) * 0.05
    m2 = torch.randn(e, h, i, generator=g) * 0.05
    wts, ids = O.make_routing(m, e, topk, 8)
    if kind == "bf16":
        w1, w2, kw, tol = m1.bfloat16(), m2.bfloat16(), {}, 1e-2
        expect = O.moe_bf16(hidden, w1, w2, wts, ids)
    elif kind == "fp8_block":
        w1, w1s = O.quantize_weight_block_fp8(m1)
        w2, w2s = O.quantize_weight_block_fp8(m2)
        kw, tol = dict(use_fp8_w8a8=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(),
                       block_shape=[128, 128]), 2e-2
        expect = O.moe_block_fp8(hidden, w1, w2, w1s, w2s, wts, ids, (128, 128))
    else:
        w1, w1s = O.quantize_weight_channel_int8(m1)
        w2, w2s = O.quantize_weight_channel_int8(m2)
        kw, tol = dict(use_int8_w8a8=True, per_channel_quant=True, w1_scale=w1s.cuda(),
                       w2_scale=w2s.cuda()), 2e-2
        expect = O.moe_per_channel(hidden, w1, w2, w1s, w2s, wts, ids, torch.int8)
    args = _dev(hidden, w1, w2, wts, ids)
    outs = {}
    for sched in ("tiles", "pairs"):
        monkeypatch.setenv("BOLTOPS_B200_GEMM_SCHEDULE", sched)
        outs[sched] = _finish(fused_experts(*args, **kw))
    assert torch.equal(outs["pairs"], outs["tiles"])
    assert O.rel_l2(outs["pairs"], expect) <= tol
    # expert-parallel mask: two ranks' partial outputs add up to the full layer
    monkeypatch.setenv("BOLTOPS_B200_GEMM_SCHEDULE", "pairs")
    total = torch.zeros(m, h)
    for lo in (0, 4):
        emap = torch.full((e,), -1, dtype=torch.int32)
        emap[lo:lo + 4] = torch.arange(4, dtype=torch.int32)
        loc = dict(kw)
        for name in ("w1_scale", "w2_scale"):
            if name in loc:
                loc[name] = loc[name][lo:lo + 4]
        part = fused_experts(args[0], args[1][lo:lo + 4], args[2][lo:lo + 4], args[3], args[4],
                             expert_map=emap.cuda(), global_num_experts=e, **loc)
        total += _finish(part).float()
    assert O.rel_l2(total, outs["pairs"].float()) <= 1e-2


@pytest.mark.parametrize("kind", ["bf16", "fp8_block", "int8_block", "int8_channel", "fp8_channel"])
def test_layer_one_call_equals_kernel_by_kernel(monkeypatch, kind):
    """The native one-call layer (sort, row placement, both GEMMs and the combine enqueued by one
    C-ABI call) and the kernel-by-kernel Python orchestration give bit-identical outputs: plain
    call, biases + expert mask, router weight on the input (top-1), in place."""
    from boltops_b200.fused_moe import fused_experts, layer, ops
    m, e, topk, h, i = 77, 8, 2, 512, 256
    g = torch.Generator().manual_seed(31)
    hidden = torch.randn(m, h, generator=g).bfloat16()
    m1 = torch.randn(e, 2 * i, h, generator=g) * 0.05
    m2 = torch.randn(e, h, i, generator=g) * 0.05
    wts, ids = O.make_routing(m, e, topk, 12)
    if kind == "bf16":
        w1, w2, kw = m1.bfloat16(), m2.bfloat16(), {}
    elif kind == "fp8_block":
        w1, w1s = O.quantize_weight_block_fp8(m1)
        w2, w2s = O.quantize_weight_block_fp8(m2)
        kw = dict(use_fp8_w8a8=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128])
    elif kind == "int8_block":
        def qi(wm):
            v = wm.view(wm.shape[0], wm.shape[1] // 128, 128, wm.shape[2] // 128, 128)
            s = v.abs().amax(dim=(2, 4), keepdim=True).clamp(min=1e-10) / 127.0
            return ((v / s).round().clamp(-128, 127).to(torch.int8).view_as(wm),
                    s.view(wm.shape[0], wm.shape[1] // 128, wm.shape[2] // 128))
        w1, w1s = qi(m1)
        w2, w2s = qi(m2)
        kw = dict(use_int8_w8a8=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128])
    else:
        w1, w1s = O.quantize_weight_channel_int8(m1)
        w2, w2s = O.quantize_weight_channel_int8(m2)
        if kind == "fp8_channel":
            w1, w2 = (w1.float() * 3).to(FP8), (w2.float() * 3).to(FP8)
            kw = dict(use_fp8_w8a8=True, per_channel_quant=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda())
        else:
            kw = dict(use_int8_w8a8=True, per_channel_quant=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda())
    args = _dev(hidden, w1, w2, wts, ids)
    emap = torch.full((e,), -1, dtype=torch.int32)
    emap[2:6] = torch.arange(4, dtype=torch.int32)
    b1 = (torch.randn(4, 2 * i, generator=g) / 4).bfloat16().cuda()
    b2 = (torch.randn(4, h, generator=g) / 4).bfloat16().cuda()
    loc = {k: (v[2:6] if k.endswith("_scale") else v) for k, v in kw.items()}
    variants = [
        (args, kw),
        ((args[0], args[1][2:6], args[2][2:6], args[3], args[4]),
         dict(loc, expert_map=emap.cuda(), global_num_experts=e, b1=b1, b2=b2,
              routed_scaling_factor=2.5)),
        ((args[0], args[1], args[2], args[3][:, :1].contiguous(), args[4][:, :1].contiguous()),
         dict(kw, apply_router_weight_on_input=True)),
    ]
    for a, k in variants:
        outs = []
        for one_call in (True, False):
            monkeypatch.setattr(layer, "_ONE_CALL", one_call)
            before = ops.launch_count()
            outs.append(_finish(fused_experts(*a, **k)))
            assert ops.launch_count() - before >= 4
        assert torch.equal(outs[0], outs[1])
    monkeypatch.setattr(layer, "_ONE_CALL", True)
    x = args[0].clone()
    out = fused_experts(x, *args[1:], inplace=True, **kw)
    assert out.data_ptr() == x.data_ptr()
    monkeypatch.setattr(layer, "_ONE_CALL", False)
    assert torch.equal(_finish(out), _finish(fused_experts(*args, **kw)))
