"""Benchmark-sized cases: every configuration of the benchmark at its own shape
(Mixtral-8x7B bf16, DeepSeek-V3 fp8 block, Qwen3-30B int8 per-channel, Qwen3-235B fp8 block
with Zipf routing), including the end points of the token sweeps.

Full CPU oracles of these layers take minutes, so parity is checked through
size-independent properties plus an oracle spot check on a few tokens:
run-to-run bit-identity, no_combine consistency, sort invariants at 32768 routes
over 256 experts, bit-exact quantisation, and the oracle on the routes of four
tokens (only their experts are copied to the host)."""
import numpy as np
import pytest
import torch

import bench as B
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _finish(dev):
    from boltops_b200.fused_moe import ops
    torch.cuda.synchronize()
    ops.check_device_status(dev)


@pytest.fixture(scope="module")
def dsv3():
    cfg = dict(B.WORKLOADS["deepseek_v3_fp8_block"])
    dev = torch.device("cuda")
    w1, w2, w1s, w2s = B.make_weights(cfg, dev, list(range(cfg["E"])), 0)
    hidden, wts, ids = B.make_tokens(cfg, 4096, 0)
    return cfg, (w1, w2, w1s, w2s), (hidden, wts, ids)


def test_dsv3_sort_invariants_and_oracle(dsv3):
    from boltops_b200.fused_moe import ops
    cfg, _, (hidden, wts, ids) = dsv3
    pos = torch.empty(ids.shape, dtype=torch.int32, device="cuda")
    s_ids, s_w, s_e, nv, cnt, _ = ops.moe_sorting_ck(ids.cuda(), wts.cuda(), cfg["E"], None, None,
                                                     128, None, route_pos=pos)
    torch.cuda.synchronize()
    ref = O.sort_ck_numpy(ids.numpy(), wts.numpy(), cfg["E"], 128, None)
    n = int(nv.item())
    assert n == ref["num_valid"] and n % 128 == 0
    assert np.array_equal(s_ids.cpu().numpy()[:n], ref["sorted_ids"])
    assert np.array_equal(s_w.cpu().numpy()[:n].view(np.uint32), ref["sorted_weights"].view(np.uint32))
    e = s_e.cpu().numpy()[: n // 128]
    assert np.array_equal(e, ref["expert_ids"]) and (np.diff(e) >= 0).all()      # sortedness
    assert np.array_equal(cnt.cpu().numpy()[: cfg["E"]], np.bincount(ids.numpy().ravel(), minlength=cfg["E"]))
    p = pos.cpu().numpy().ravel()
    assert len(np.unique(p)) == p.size and p.min() >= 0 and p.max() < n          # a permutation


def test_dsv3_activation_quant_bit_exact(dsv3):
    from boltops_b200.fused_moe import ops
    _, _, (hidden, _, _) = dsv3
    q, s = ops.per_block_quant(hidden.cuda(), 128, FP8)
    q_ref, s_ref = O.quant_rows_kernel(hidden, FP8, 128)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


def test_dsv3_layer_properties_and_spot_oracle(dsv3):
    from boltops_b200.fused_moe import fused_experts
    cfg, (w1, w2, w1s, w2s), (hidden, wts, ids) = dsv3
    dev = w1.device
    kw = dict(use_fp8_w8a8=True, w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
    h, w, i = hidden.cuda(), wts.cuda(), ids.cuda()
    out1 = fused_experts(h, w1, w2, w, i, **kw)
    out2 = fused_experts(h, w1, w2, w, i, **kw)
    _finish(dev)
    assert torch.equal(out1, out2)                                   # run-to-run bit identity
    assert torch.isfinite(out1.float()).all()
    # no_combine rows, weighted and summed on the host, reproduce the combined output
    sub = slice(0, 512)
    nc = fused_experts(h[sub], w1, w2, w[sub], i[sub], no_combine=True, **kw)
    _finish(dev)
    comb = (nc.float() * w[sub][:, :, None]).sum(1)
    assert O.rel_l2(out1[sub].cpu(), comb.cpu()) <= 5e-3
    # routed_scaling_factor is linear
    out3 = fused_experts(h[sub], w1, w2, w[sub], i[sub], routed_scaling_factor=2.0, **kw)
    _finish(dev)
    assert O.rel_l2(out3.cpu(), out1[sub].float().cpu() * 2.0) <= 5e-3
    # oracle on four tokens: copy only their experts to the host
    toks = [0, 1777, 2048, 4095]
    used = sorted(set(ids[toks].reshape(-1).tolist()))
    remap = {e: j for j, e in enumerate(used)}
    sel = torch.tensor(used, device=dev)
    c_w1, c_w2 = w1[sel].cpu(), w2[sel].cpu()
    c_w1s, c_w2s = w1s[sel].cpu(), w2s[sel].cpu()
    loc_ids = torch.tensor([[remap[int(e)] for e in row] for row in ids[toks]], dtype=torch.int32)
    expect = O.moe_block_fp8(hidden[toks], c_w1, c_w2, c_w1s, c_w2s, wts[toks], loc_ids, (128, 128))
    assert O.rel_l2(out1[toks].cpu(), expect) <= 2e-2


def test_qwen3_int8_channel_full_shape_spot_oracle():
    from boltops_b200.fused_moe import fused_experts
    cfg = dict(B.WORKLOADS["qwen3_30b_int8_channel"])
    dev = torch.device("cuda")
    w1, w2, w1s, w2s = B.make_weights(cfg, dev, list(range(cfg["E"])), 1)
    hidden, wts, ids = B.make_tokens(cfg, 16384, 1)
    kw = dict(use_int8_w8a8=True, per_channel_quant=True, w1_scale=w1s, w2_scale=w2s)
    out = fused_experts(hidden.cuda(), w1, w2, wts.cuda(), ids.cuda(), **kw)
    _finish(dev)
    toks = [0, 5000, 16383]
    expect = O.moe_per_channel(hidden[toks], w1.cpu(), w2.cpu(), w1s.cpu(), w2s.cpu(), wts[toks],
                               ids[toks], torch.int8)
    assert O.rel_l2(out[toks].cpu(), expect) <= 2e-2


def _spot_block_fp8(out, toks, hidden, wts, ids, w1, w2, w1s, w2s):
    """Oracle on the listed tokens: only the experts they use are copied to the host."""
    used = sorted(set(ids[toks].reshape(-1).tolist()))
    remap = {e: j for j, e in enumerate(used)}
    sel = torch.tensor(used, device=w1.device)
    loc_ids = torch.tensor([[remap[int(e)] for e in row] for row in ids[toks]], dtype=torch.int32)
    expect = O.moe_block_fp8(hidden[toks], w1[sel].cpu(), w2[sel].cpu(), w1s[sel].cpu(),
                             w2s[sel].cpu(), wts[toks], loc_ids, (128, 128))
    return O.rel_l2(out[toks].cpu(), expect)


@pytest.mark.parametrize("m,toks", [(1, [0]), (8192, [0, 4097, 8191])])
def test_dsv3_sweep_end_points_spot_oracle(dsv3, m, toks):
    """The DeepSeek-V3 layer at both ends of its token sweep (one token: eight experts, one
    live row each; 8192 tokens: two and three row tiles per expert)."""
    from boltops_b200.fused_moe import fused_experts
    cfg, (w1, w2, w1s, w2s), _ = dsv3
    hidden, wts, ids = B.make_tokens(cfg, m, 5 + m)
    out = fused_experts(hidden.cuda(), w1, w2, wts.cuda(), ids.cuda(), use_fp8_w8a8=True,
                        w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
    _finish(w1.device)
    assert torch.isfinite(out.float()).all()
    assert _spot_block_fp8(out, toks, hidden, wts, ids, w1, w2, w1s, w2s) <= 2e-2


@pytest.fixture(scope="module")
def mixtral():
    cfg = dict(B.WORKLOADS["mixtral_8x7b_bf16"])
    w1, w2, _, _ = B.make_weights(cfg, torch.device("cuda"), list(range(cfg["E"])), 2)
    return cfg, w1, w2


@pytest.mark.parametrize("m,toks", [(1, [0]), (8192, [3, 8191])])
def test_mixtral_bf16_full_shape_spot_oracle(mixtral, m, toks):
    """Mixtral-8x7B shape (16 row tiles per expert at 8192 tokens, 224 K blocks in the down
    GEMM) against the bf16 oracle on a few tokens."""
    from boltops_b200.fused_moe import fused_experts
    cfg, w1, w2 = mixtral
    hidden, wts, ids = B.make_tokens(cfg, m, 11 + m)
    out = fused_experts(hidden.cuda(), w1, w2, wts.cuda(), ids.cuda())
    _finish(w1.device)
    assert torch.isfinite(out.float()).all()
    used = sorted(set(ids[toks].reshape(-1).tolist()))
    remap = {e: j for j, e in enumerate(used)}
    sel = torch.tensor(used, device=w1.device)
    loc_ids = torch.tensor([[remap[int(e)] for e in row] for row in ids[toks]], dtype=torch.int32)
    expect = O.moe_bf16(hidden[toks], w1[sel].cpu(), w2[sel].cpu(), wts[toks], loc_ids)
    assert O.rel_l2(out[toks].cpu(), expect) <= 1e-2


@pytest.fixture(scope="module")
def qwen235():
    cfg = dict(B.WORKLOADS["qwen3_235b_fp8_block_zipf"])
    w = B.make_weights(cfg, torch.device("cuda"), list(range(cfg["E"])), 3)
    return cfg, w


@pytest.mark.parametrize("m", [1, 16, 256])
def test_qwen3_235b_zipf_full_shape_spot_oracle(qwen235, m):
    """Decode-skew case: Zipf(1.2) routing puts many rows on a few experts and none on others."""
    from boltops_b200.fused_moe import fused_experts
    cfg, (w1, w2, w1s, w2s) = qwen235
    hidden, wts, ids = B.make_tokens(cfg, m, 23 + m)
    counts = torch.bincount(ids.flatten().long(), minlength=cfg["E"])
    if m == 256:
        assert counts.max() >= 4 * counts.float().mean() and (counts == 0).any()   # skewed
    out = fused_experts(hidden.cuda(), w1, w2, wts.cuda(), ids.cuda(), use_fp8_w8a8=True,
                        w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
    out2 = fused_experts(hidden.cuda(), w1, w2, wts.cuda(), ids.cuda(), use_fp8_w8a8=True,
                         w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
    _finish(w1.device)
    assert torch.equal(out, out2) and torch.isfinite(out.float()).all()
    toks = list(range(m)) if m <= 16 else [0, 100, 255, int(ids[:, 0].argmax())]
    assert _spot_block_fp8(out, toks, hidden, wts, ids, w1, w2, w1s, w2s) <= 2e-2
