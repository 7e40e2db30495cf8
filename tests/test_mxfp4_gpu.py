"""MXFP4 (w4a8) experts through the public API against the reference's CPU statement: every
case of the reference's test_public_mxfp4_cpu_reference (fixture written by
tests/golden/make_golden.py), with the reference's tolerance, plus the element-wise kernels
against the oracle and the argument contract."""
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import MXFP4_CASES, load_mxfp4_case

FP8 = torch.float8_e4m3fn


@pytest.mark.gpu
@pytest.mark.parametrize("path", ["native", "decoded"])
@pytest.mark.parametrize("case", MXFP4_CASES)
def test_public_mxfp4_matches_reference_cpu_statement(monkeypatch, case, path):
    """path: the tensor core's block-scaled kind on the packed weights (taken by the dynamic recipe
    on 16-bit input; the other cases run the decoded form either way), or decoded operands."""
    from boltops_b200.fused_moe import fused_experts, mxfp4, ops
    monkeypatch.setattr(mxfp4, "_NATIVE", path == "native")
    c = load_mxfp4_case(case)
    if c["chunk"]:
        monkeypatch.setenv("TRITON_FUSED_MOE_CHUNK_SIZE", str(c["chunk"]))
    static, x = c["static"], c["x"]
    device_x = (c["input_q"] if c["prequantized"] else x).cuda()
    a1 = None
    if c["prequantized"]:
        a1 = c["input_scale"].cuda()
    elif static:
        a1 = c["static_s1"].cuda()
    before = ops.launch_count()
    actual = fused_experts(
        device_x, c["w1"].cuda(), c["w2"].cuda(), c["weights"].cuda(), c["ids"].cuda(),
        a1_scale=a1, a2_scale=c["static_s2"].cuda() if static else None,
        b1=None if c["bias1"] is None else c["bias1"].cuda(),
        b2=None if c["bias2"] is None else c["bias2"].cuda(),
        gemm1_alpha=c["alpha"] if static else None, output_dtype=x.dtype, inplace=c["inplace"],
        apply_router_weight_on_input=c["input_router"], activation=c["activation"],
        activation_situ_beta=1.5 if c["activation"] == "situ" else None,
        activation_situ_linear_beta=2.0 if c["activation"] == "situ" else None,
        expert_map=None if c["expert_map"] is None else c["expert_map"].cuda(),
        use_mxfp4_w4a8=True, use_ue8m0=True, w1_scale=c["s1"].cuda(), w2_scale=c["s2"].cuda(),
        block_shape=[1, 32], gemm1_limit=c["clamp"], no_combine=c["no_combine"],
        routed_scaling_factor=1.25)
    torch.cuda.synchronize()
    ops.check_device_status(actual.device)
    assert ops.launch_count() > before
    if c["inplace"]:
        assert actual.data_ptr() == device_x.data_ptr()
    assert actual.dtype == c["expected"].dtype
    torch.testing.assert_close(actual.cpu(), c["expected"], rtol=.03, atol=.003)


@pytest.mark.gpu
def test_mxfp4_weight_decode_and_quantiser_bit_exact():
    from boltops_b200.fused_moe import mxfp4
    g = torch.Generator().manual_seed(5)
    w = torch.randint(0, 256, (3, 40, 64), dtype=torch.uint8, generator=g)
    s = torch.randint(110, 140, (3, 40, 4), dtype=torch.uint8, generator=g)
    dec = mxfp4._decode_weights(w.cuda(), s.cuda())
    assert torch.equal(dec.float().cpu(), O.mxfp4_decode(w, s))
    x = (torch.randn(37, 384, generator=g) * 3).bfloat16()
    x[5] = 0                                                   # an all-zero group: scale floor
    deq, codes, scales = mxfp4.act_quant(x.cuda(), want_codes=True)
    q_ref, s_ref, d_ref = O.mxfp4_quant_g128(x)
    assert torch.equal(codes.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(scales.cpu(), s_ref)
    assert torch.equal(deq.float().cpu(), d_ref)
    # gated: SiLU(gate) * up with clamp, rounded through bf16, then the same quantiser
    g1 = (torch.randn(20, 512, generator=g) * 2).bfloat16()
    gate, up = g1.float().chunk(2, -1)
    gate, up = gate.clamp(max=.25), up.clamp(-.25, .25)
    act = (up * gate / (1 + torch.exp(-gate))).bfloat16()
    deq = mxfp4.act_quant(g1.cuda(), gated=True, limit=.25)[0]
    ref = O.mxfp4_quant_g128(act)[2]
    # expf on the device and torch.exp on the host may differ in the last place before the
    # bf16 rounding: nearly all decoded values are identical, the rest one quantisation step
    same = (deq.float().cpu() == ref)
    assert same.float().mean() > 0.995
    torch.testing.assert_close(deq.float().cpu(), ref, rtol=0.13, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(300, 1024, 512, 768, 8, 4), (64, 7168, 256, 7168, 16, 8)])
def test_mxfp4_packed_weights_on_the_tensor_core_equal_decoded_operands(monkeypatch, shape):
    """The block-scaled kind on packed e2m1 weights against the 16-bit kind on decoded operands:
    the same exact products summed in fp32, so the layer outputs agree to accumulation order;
    the quantiser's four equal E8M0 bytes are the power-of-two group scale."""
    from boltops_b200.fused_moe import fused_experts, mxfp4
    m, hidden, inter, model_dim, experts, topk = shape
    g = torch.Generator().manual_seed(31)
    x = (torch.randn(m, hidden, generator=g)).bfloat16().cuda()
    w1 = torch.randint(0, 256, (experts, 2 * inter, hidden // 2), dtype=torch.uint8, generator=g).cuda()
    w2 = torch.randint(0, 256, (experts, model_dim, inter // 2), dtype=torch.uint8, generator=g).cuda()
    s1 = torch.randint(116, 122, (experts, 2 * inter, hidden // 32), dtype=torch.uint8, generator=g).cuda()
    s2 = torch.randint(116, 122, (experts, model_dim, inter // 32), dtype=torch.uint8, generator=g).cuda()
    logits = torch.randn(m, experts, generator=g)
    wts, ids = torch.topk(torch.softmax(logits, -1), topk)
    outs = {}
    for path in ("native", "decoded"):
        monkeypatch.setattr(mxfp4, "_NATIVE", path == "native")
        outs[path] = fused_experts(x, w1, w2, wts.cuda(), ids.int().cuda(), use_mxfp4_w4a8=True,
                                   w1_scale=s1, w2_scale=s2, block_shape=[1, 32]).float()
    torch.cuda.synchronize()
    from boltops_b200.fused_moe import ops
    ops.check_device_status(x.device)
    assert torch.isfinite(outs["native"]).all()
    err = (outs["native"] - outs["decoded"]).norm() / outs["decoded"].norm()
    assert err < 2e-3, float(err)
    # the activation + quantiser fused into GEMM1's epilogue against the stand-alone kernel: the
    # same operations in the same order on the same accumulators, so every output bit agrees
    monkeypatch.setattr(mxfp4, "_NATIVE", True)
    monkeypatch.setattr(mxfp4, "_FUSED", False)
    unfused = fused_experts(x, w1, w2, wts.cuda(), ids.int().cuda(), use_mxfp4_w4a8=True,
                            w1_scale=s1, w2_scale=s2, block_shape=[1, 32], gemm1_limit=0.75).float()
    monkeypatch.setattr(mxfp4, "_FUSED", True)
    fused = fused_experts(x, w1, w2, wts.cuda(), ids.int().cuda(), use_mxfp4_w4a8=True,
                          w1_scale=s1, w2_scale=s2, block_shape=[1, 32], gemm1_limit=0.75).float()
    torch.cuda.synchronize()
    ops.check_device_status(x.device)
    assert torch.equal(fused, unfused)
    _, codes, scales, sf = mxfp4.act_quant(x, want_codes=True, want_deq=False, want_sf=True)
    assert torch.equal(torch.exp2(sf.float() - 127.0),
                       scales.repeat_interleave(4, dim=1))


def test_mxfp4_argument_contract_matches_reference_messages():
    """The rejections of the reference's test_public_mxfp4_prequantized_contract and
    test_mxfp4_input_router_rejects_unsupported_preparation, raised before any device work."""
    from boltops_b200.fused_moe import fused_experts
    w1 = torch.zeros(1, 256, 64, dtype=torch.uint8)
    w2 = torch.zeros(1, 128, 64, dtype=torch.uint8)
    sc = dict(w1_scale=torch.full((1, 256, 4), 127, dtype=torch.uint8),
              w2_scale=torch.full((1, 128, 4), 127, dtype=torch.uint8))
    xq = torch.zeros(1, 128).to(FP8)
    one = (torch.ones(1, 1), torch.zeros(1, 1, dtype=torch.int32))
    for kw, match in [
        (dict(a1_scale=None, output_dtype=torch.bfloat16), "require a1_scale and output_dtype"),
        (dict(a1_scale=torch.ones(1, 1), output_dtype=None), "require a1_scale and output_dtype"),
        (dict(a1_scale=torch.ones(1, 1), output_dtype=torch.bfloat16, a2_scale=torch.ones(1, 1)),
         "MXFP4 requires gated"),
        (dict(a1_scale=torch.ones(1, 1), output_dtype=torch.bfloat16, inplace=True),
         "inplace MXFP4 requires output_dtype"),
    ]:
        with pytest.raises(ValueError, match=match):
            fused_experts(xq, w1, w2, *one, use_mxfp4_w4a8=True, **kw, **sc)
    x = torch.zeros(1, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="require topk=1"):
        fused_experts(x, w1, w2, torch.ones(1, 2), torch.zeros(1, 2, dtype=torch.int32),
                      use_mxfp4_w4a8=True, apply_router_weight_on_input=True, **sc)
    with pytest.raises(ValueError, match="before FP8 quantization"):
        fused_experts(xq, w1, w2, *one, use_mxfp4_w4a8=True, apply_router_weight_on_input=True,
                      a1_scale=torch.ones(1, 1), output_dtype=torch.bfloat16, **sc)
    with pytest.raises(ValueError, match="cannot be combined"):
        fused_experts(x, w1, w2, *one, use_mxfp4_w4a8=True, use_fp8_w8a8=True, **sc)
