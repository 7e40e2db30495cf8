"""Native-MXFP8 experts on the GPU against the oracle (which is pinned to the reference's own
CPU statement of this layer by tests/test_oracle_golden.py::test_mxfp8_layer_fixture)."""
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import MX_CASES, load_mx_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("gated", [False, True])
def test_mx_quantiser_matches_oracle(dtype, gated):
    from boltops_b200.fused_moe import ops
    torch.manual_seed(3)
    rows, cols = 37, 96
    x = torch.randn(rows, 2 * cols if gated else cols) * 3
    x[5] = 0                                           # an all-zero row: exponent byte 0
    x[6, :32] *= 1e-6
    x = x.to(dtype)
    kw = dict(alpha=1.2, beta=0.3, limit=2.5) if gated else {}
    ref_in = O.mx_gated_activation(x, "swigluoai", **kw) if gated else x
    q_ref, s_ref, d_ref = O.mx_quant(ref_in)
    q, s, d = ops.mx_quant_rows(x.cuda(), gated=gated, deq_dtype=torch.float32, **kw)
    if gated:
        # the activation runs in fp32 on both sides but with different exp/sigmoid routines:
        # compare the dequantised values within one e4m3 step of the group's scale
        step = torch.exp2(s_ref.float() - 127).repeat_interleave(32, -1) * 32
        assert ((d.cpu() - d_ref).abs() <= step + 1e-30).all()
        assert (s.cpu().int() - s_ref.int()).abs().max() <= 1
    else:
        assert torch.equal(s.cpu(), s_ref)
        assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
        assert torch.equal(d.cpu(), d_ref)
    back = ops.mx_dequant_rows(q, s, torch.float32)
    assert torch.equal(back.cpu(), d.cpu())


@pytest.mark.parametrize("case", ["default", "silu_alpha", "swigluoai", "no_combine", "dynamic_fp16"])
def test_mxfp8_layer_reference_cases(case):
    """The five CPU-statement cases of the reference's own test, with its tolerances."""
    from boltops_b200.fused_moe import fused_experts
    c = load_mx_case(case)
    kw = dict(MX_CASES[case])
    act = kw.pop("activation")
    out = fused_experts(c["x"].cuda(), c["w1"].cuda(), c["w2"].cuda(), c["weights"].cuda(),
                        c["ids"].cuda(), activation=act, gemm1_alpha=kw.get("alpha"),
                        gemm1_beta=kw.get("beta"), gemm1_limit=kw.get("limit"), use_mxfp8=True,
                        w1_scale=c["s1"].cuda(), w2_scale=c["s2"].cuda(), block_shape=[1, 32],
                        output_dtype=c["x"].dtype, no_combine=kw.get("no_combine", False))
    torch.testing.assert_close(out.cpu().float(), c["expected"].float(), rtol=.025, atol=.003)


def _random_mx_weights(e, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(e, n, k, generator=g) * 2).to(torch.float8_e4m3fn)
    s = torch.randint(118, 124, (e, n, k // 32), dtype=torch.uint8, generator=g)
    return w, s


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("inter", [128, 96])   # 128: tensor-core MX kind; 96: dequantised 16-bit kind
def test_mxfp8_layer_random_vs_oracle(masked, inter):
    from boltops_b200.fused_moe import fused_experts
    m, e, k, h = 150, 8, 2, 256
    w1, s1 = _random_mx_weights(e, 2 * inter, h, 1)
    w2, s2 = _random_mx_weights(e, h, inter, 2)
    x = (torch.randn(m, h, generator=torch.Generator().manual_seed(4)) * 0.5).bfloat16()
    wts, ids = O.make_routing(m, e, k, 9)
    emap = None
    if masked:                      # experts 0..3 local, the rest on "another rank"
        emap = torch.tensor([0, 1, 2, 3, -1, -1, -1, -1], dtype=torch.int32)
    ref = O.moe_mxfp8(x, w1[:4] if masked else w1, w2[:4] if masked else w2,
                      s1[:4] if masked else s1, s2[:4] if masked else s2, wts, ids,
                      expert_map=emap)
    out = fused_experts(x.cuda(), (w1[:4] if masked else w1).cuda(),
                        (w2[:4] if masked else w2).cuda(), wts.cuda(), ids.cuda(), use_mxfp8=True,
                        w1_scale=(s1[:4] if masked else s1).cuda(),
                        w2_scale=(s2[:4] if masked else s2).cuda(), block_shape=[1, 32],
                        expert_map=None if emap is None else emap.cuda(),
                        global_num_experts=e)
    assert O.rel_l2(out.cpu(), ref) <= 2e-2


@pytest.mark.parametrize("m,e,topk,n,k", [(150, 4, 2, 512, 256), (40, 3, 1, 384, 128), (600, 8, 2, 256, 1024)])
@pytest.mark.parametrize("c_dtype", [torch.float32, torch.bfloat16])
def test_mx_grouped_gemm_kind(m, e, topk, n, k, c_dtype):
    """The tensor-core block-scaled kind against an fp32 matmul over the dequantised operands."""
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    torch.manual_seed(m + n)
    x = (torch.randn(m, k) * 0.7).bfloat16().cuda()
    w, ws = _random_mx_weights(e, n, k, 5)
    wts, ids = O.make_routing(m, e, topk, 21)
    pos = torch.empty((m, topk), dtype=torch.int32, device="cuda")
    s_ids, s_w, s_e, nv, _, _ = ops.moe_sorting_ck(ids.cuda(), wts.cuda(), e, None, None, 128, None,
                                                   alloc_moe_buf=False, route_pos=pos)
    cap = s_ids.shape[0]
    q, sc, deq = ops.mx_quant_rows(x, deq_dtype=torch.float32)
    a_sorted, _ = ops.gather_rows(q, s_ids, nv, cap)
    sfa = ops.mx_sf_layout(sc, cap, s_ids, nv)
    n_pad = (n + 127) // 128 * 128
    ws_pad = torch.zeros(e, n_pad, k // 32, dtype=torch.uint8)
    ws_pad[:, :n] = ws
    sfb = ops.mx_sf_layout(ws_pad.view(e * n_pad, k // 32).cuda(), e * n_pad)
    c = torch.full((cap, n), -7.0, dtype=c_dtype, device="cuda")
    ops.grouped_gemm(kind=_cabi.GEMM_MXFP8, epilogue=_cabi.EPI_STORE, a=a_sorted, b=w.cuda(), c=c,
                     a_scale=sfa, b_scale=sfb, sorted_expert_ids=s_e, num_valid=nv,
                     sorted_ids=s_ids, sorted_weights=s_w, num_tokens=m, topk=topk,
                     mul_routed_weight=True)
    torch.cuda.synchronize()
    ops.check_device_status(torch.device("cuda"))
    wd = O.mx_dequant_weight(w, ws)
    deq = deq.cpu()
    pos = pos.cpu()
    got = c.cpu().float()
    worst = 0.0
    for t in range(m):
        for j in range(topk):
            r = int(pos[t, j])
            ref = (deq[t] @ wd[int(ids[t, j])].T) * wts[t, j]
            if c_dtype != torch.float32:
                ref = ref.to(c_dtype).float()
            err = (got[r] - ref).abs().max() / ref.abs().max().clamp_min(1e-6)
            worst = max(worst, float(err))
    assert worst <= (1e-5 if c_dtype == torch.float32 else 1e-2), worst


def test_mxfp8_layer_chunked_scaled_inplace(monkeypatch):
    """Token chunking, routed_scaling_factor and inplace go through the MX path unchanged."""
    from boltops_b200.fused_moe import fused_experts
    m, e, k, h, inter = 200, 4, 2, 128, 128
    w1, s1 = _random_mx_weights(e, 2 * inter, h, 7)
    w2, s2 = _random_mx_weights(e, h, inter, 8)
    x = (torch.randn(m, h, generator=torch.Generator().manual_seed(1)) * 0.5).bfloat16()
    wts, ids = O.make_routing(m, e, k, 2)
    ref = (O.moe_mxfp8(x, w1, w2, s1, s2, wts, ids).float() * 2.0)
    args = (w1.cuda(), w2.cuda(), wts.cuda(), ids.cuda())
    kw = dict(use_mxfp8=True, w1_scale=s1.cuda(), w2_scale=s2.cuda(), block_shape=[1, 32],
              routed_scaling_factor=2.0)
    whole = fused_experts(x.cuda(), *args, **kw)
    monkeypatch.setenv("BOLTOPS_FUSED_MOE_CHUNK_SIZE", "64")
    xin = x.cuda().clone()
    out = fused_experts(xin, *args, inplace=True, **kw)
    assert out.data_ptr() == xin.data_ptr()
    assert torch.equal(out.cpu(), whole.cpu())          # rows are independent of the chunking
    assert O.rel_l2(out.cpu().float(), ref) <= 2e-2
