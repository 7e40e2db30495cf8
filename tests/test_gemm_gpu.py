"""Grouped GEMM (tcgen05) vs fp32 CPU references, called through the C ABI."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _routing(m, e, topk, seed):
    w, ids = O.make_routing(m, e, topk, seed)
    return w, ids


def _sorted_problem(m, e, topk, seed):
    """Sort on the GPU, return device handles + host copies of the layout."""
    from boltops_b200.fused_moe import ops
    w, ids = _routing(m, e, topk, seed)
    s_ids, s_w, s_e, nv, _, _ = ops.moe_sorting_ck(ids.cuda(), w.cuda(), e, None, None, 128, None)
    torch.cuda.synchronize()
    return dict(w=w, ids=ids, s_ids=s_ids, s_w=s_w, s_e=s_e, nv=nv, cap=s_ids.shape[0],
                nvi=int(nv.item()), h_ids=s_ids.cpu(), h_w=s_w.cpu(), h_e=s_e.cpu())


def _reference_rows(pr, a_tokens_f32, b_f32):
    """fp32 C[row] = A[token(row)] @ B[expert(row)]^T for all valid, non-pad rows."""
    m = a_tokens_f32.shape[0]
    out = {}
    for row in range(pr["nvi"]):
        tok = int(pr["h_ids"][row]) & 0xFFFFFF
        if tok >= m:
            continue
        e = int(pr["h_e"][row // 128])
        out[row] = (a_tokens_f32[tok] @ b_f32[e].t(), tok, (int(pr["h_ids"][row]) >> 24) & 0xFF)
    return out


@pytest.mark.parametrize("m,e,topk,n,k,dtype", [
    (64, 8, 2, 512, 256, torch.bfloat16),
    (200, 4, 2, 384, 336, torch.bfloat16),      # n tail (384 = 256 + 128), k tail (336 % 64 != 0)
    (33, 16, 4, 256, 1024, torch.float16),
    (700, 8, 2, 1024, 512, torch.bfloat16),     # several row tiles per expert
])
def test_gemm_16bit_store_sorted(m, e, topk, n, k, dtype):
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    torch.manual_seed(m + n)
    pr = _sorted_problem(m, e, topk, 11)
    x = (torch.randn(m, k) / 4).to(dtype)
    b = (torch.randn(e, n, k) / 8).to(dtype)
    a_sorted, _ = ops.gather_rows(x.cuda(), pr["s_ids"], pr["nv"], pr["cap"])
    c = torch.full((pr["cap"], n), -123.0, dtype=dtype, device="cuda")
    kind = _cabi.GEMM_BF16 if dtype == torch.bfloat16 else _cabi.GEMM_F16
    ops.grouped_gemm(kind=kind, epilogue=_cabi.EPI_STORE, a=a_sorted, b=b.cuda(), c=c,
                     sorted_expert_ids=pr["s_e"], num_valid=pr["nv"], sorted_ids=pr["s_ids"],
                     sorted_weights=pr["s_w"], num_tokens=m, topk=topk)
    torch.cuda.synchronize()
    ops.check_device_status(c.device)
    got = c.cpu().float()
    ref = _reference_rows(pr, x.float(), b.float())
    assert ref
    for row, (val, _, _) in ref.items():
        torch.testing.assert_close(got[row], val.to(dtype).float(), rtol=2e-2, atol=2e-2)
    # pad rows and rows beyond num_valid keep the sentinel
    live = torch.zeros(pr["cap"], dtype=torch.bool)
    live[list(ref)] = True
    assert (got[~live] == -123.0).all()


def test_gemm_bf16_scatter_weighted_and_fused_silu():
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    torch.manual_seed(2)
    m, e, topk, inter, k = 96, 8, 2, 256, 512
    pr = _sorted_problem(m, e, topk, 3)
    x = (torch.randn(m, k) / 4).bfloat16()
    w1 = (torch.randn(e, 2 * inter, k) / 8).bfloat16()
    a_sorted, _ = ops.gather_rows(x.cuda(), pr["s_ids"], pr["nv"], pr["cap"])
    common = dict(kind=_cabi.GEMM_BF16, sorted_expert_ids=pr["s_e"], num_valid=pr["nv"],
                  sorted_ids=pr["s_ids"], sorted_weights=pr["s_w"], num_tokens=m, topk=topk)
    # fused SiLU-and-mul epilogue, sorted output
    act = torch.full((pr["cap"], inter), -123.0, dtype=torch.bfloat16, device="cuda")
    ops.grouped_gemm(epilogue=_cabi.EPI_SILU_MUL, a=a_sorted, b=w1.cuda(), c=act,
                     mid_dtype=torch.bfloat16, **common)
    # plain store, scattered to route rows, router weight applied
    c3 = torch.full((m * topk, 2 * inter), -123.0, dtype=torch.bfloat16, device="cuda")
    ops.grouped_gemm(epilogue=_cabi.EPI_STORE, a=a_sorted, b=w1.cuda(), c=c3, scatter=True,
                     mul_routed_weight=True, **common)
    torch.cuda.synchronize()
    ops.check_device_status(act.device)
    ref = _reference_rows(pr, x.float(), w1.float())
    got_act, got_c3 = act.cpu().float(), c3.cpu().float()
    for row, (val, tok, slot) in ref.items():
        c1 = val.bfloat16()
        expect = O.silu_and_mul(c1[None])[0].float()
        torch.testing.assert_close(got_act[row], expect, rtol=3e-2, atol=2e-2)
        wgt = float(pr["h_w"][row])
        torch.testing.assert_close(got_c3[tok * topk + slot], (val * wgt).bfloat16().float(),
                                   rtol=2e-2, atol=2e-2)
    assert (got_c3 != -123.0).all()   # every route row written exactly once


@pytest.mark.parametrize("qdtype", [FP8, torch.int8])
def test_gemm_block_scaled(qdtype):
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    torch.manual_seed(4)
    m, e, topk, inter, k = 80, 8, 2, 256, 512
    pr = _sorted_problem(m, e, topk, 5)
    x = (torch.randn(m, k) / 2).bfloat16()
    if qdtype == FP8:
        w1 = (torch.randn(e, 2 * inter, k) * 40).clamp(-448, 448).to(FP8)
        kind = _cabi.GEMM_FP8_BLOCK
    else:
        w1 = torch.randint(-127, 128, (e, 2 * inter, k), dtype=torch.int8)
        kind = _cabi.GEMM_INT8_BLOCK
    w1_s = torch.rand(e, 2 * inter // 128, k // 128) * 1e-2
    x_q, x_s = ops.per_block_quant(x.cuda(), 128, qdtype)
    a_sorted, a_scale = ops.gather_rows(x_q, pr["s_ids"], pr["nv"], pr["cap"], x_s)
    common = dict(kind=kind, sorted_expert_ids=pr["s_e"], num_valid=pr["nv"], a=a_sorted,
                  b=w1.cuda(), a_scale=a_scale, a_scale_ld=pr["cap"], b_scale=w1_s.cuda(),
                  sorted_ids=pr["s_ids"], sorted_weights=pr["s_w"], num_tokens=m, topk=topk)
    c1 = torch.full((pr["cap"], 2 * inter), -123.0, dtype=torch.bfloat16, device="cuda")
    ops.grouped_gemm(epilogue=_cabi.EPI_STORE, c=c1, **common)
    act = torch.full((pr["cap"], inter), -123.0, dtype=torch.bfloat16, device="cuda")
    ops.grouped_gemm(epilogue=_cabi.EPI_SILU_MUL, c=act, mid_dtype=torch.bfloat16, **common)
    act_q = torch.zeros((pr["cap"], inter), dtype=qdtype, device="cuda")
    act_s = torch.zeros((inter // 128, pr["cap"]), dtype=torch.float32, device="cuda")
    ops.grouped_gemm(epilogue=_cabi.EPI_SILU_MUL_QUANT, c=act_q, c_scale=act_s,
                     c_scale_ld=pr["cap"], mid_dtype=torch.bfloat16, **common)
    torch.cuda.synchronize()
    ops.check_device_status(c1.device)
    xq_h, xs_h = x_q.cpu(), x_s.cpu()
    got_c1, got_act = c1.cpu(), act.cpu()
    got_q, got_s = act_q.cpu(), act_s.cpu()
    for row in range(pr["nvi"]):
        tok = int(pr["h_ids"][row]) & 0xFFFFFF
        if tok >= m:
            continue
        ex = int(pr["h_e"][row // 128])
        ref = O.block_scaled_matmul(xq_h[tok:tok + 1], w1[ex], xs_h[tok:tok + 1], w1_s[ex],
                                    (128, 128), torch.bfloat16)
        torch.testing.assert_close(got_c1[row:row + 1].float(), ref.float(), rtol=2e-2, atol=2e-2)
        ref_act = O.silu_and_mul(got_c1[row:row + 1])          # from the kernel's own C1 rounding
        torch.testing.assert_close(got_act[row:row + 1].float(), ref_act.float(),
                                   rtol=2 ** -6, atol=1e-3)
        q_ref, s_ref = O.quant_rows_kernel(got_act[row:row + 1], qdtype, 128)
        assert torch.equal(got_s[:, row], s_ref[0])
        assert torch.equal(got_q[row].view(torch.uint8), q_ref[0].view(torch.uint8))


@pytest.mark.parametrize("qdtype", [torch.int8, FP8])
def test_gemm_per_channel(qdtype):
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    torch.manual_seed(6)
    m, e, topk, n, k = 70, 8, 2, 512, 384
    pr = _sorted_problem(m, e, topk, 7)
    x = (torch.randn(m, k) / 2).bfloat16()
    if qdtype == torch.int8:
        w = torch.randint(-127, 128, (e, n, k), dtype=torch.int8)
        kind = _cabi.GEMM_INT8_CHANNEL
    else:
        w = (torch.randn(e, n, k) * 40).clamp(-448, 448).to(FP8)
        kind = _cabi.GEMM_FP8_CHANNEL
    w_s = torch.rand(e, n) * 1e-2
    x_q, x_s = ops.per_token_quant(x.cuda(), quant_dtype=qdtype)
    a_sorted, a_scale = ops.gather_rows(x_q, pr["s_ids"], pr["nv"], pr["cap"], x_s)
    c = torch.full((pr["cap"], n), -123.0, dtype=torch.bfloat16, device="cuda")
    ops.grouped_gemm(kind=kind, epilogue=_cabi.EPI_STORE, a=a_sorted, b=w.cuda(), c=c,
                     a_scale=a_scale, b_scale=w_s.cuda(), sorted_expert_ids=pr["s_e"],
                     num_valid=pr["nv"], sorted_ids=pr["s_ids"], sorted_weights=pr["s_w"],
                     num_tokens=m, topk=topk)
    torch.cuda.synchronize()
    ops.check_device_status(c.device)
    got = c.cpu()
    xq_h, xs_h = x_q.cpu(), x_s.cpu()
    for row in range(pr["nvi"]):
        tok = int(pr["h_ids"][row]) & 0xFFFFFF
        if tok >= m:
            continue
        ex = int(pr["h_e"][row // 128])
        ref = O.per_token_matmul(xq_h[tok:tok + 1], w[ex], xs_h[tok:tok + 1], w_s[ex], torch.bfloat16)
        if qdtype == torch.int8:
            torch.testing.assert_close(got[row:row + 1].float(), ref.float(), rtol=2 ** -7, atol=1e-6)
        else:
            torch.testing.assert_close(got[row:row + 1].float(), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("m,n,k,qdtype", [(300, 512, 1024, FP8), (128, 256, 384, torch.int8),
                                          (1, 128, 128, FP8)])
def test_dense_block_scaled_gemm(m, n, k, qdtype):
    from boltops_b200.fused_moe import ops
    from boltops_b200.gemm import gemm_a8w8_blockscale, w8a8_block_scaled_mm
    torch.manual_seed(m + n)
    x = (torch.randn(m, k) / 2).bfloat16()
    if qdtype == FP8:
        w = (torch.randn(n, k) * 40).clamp(-448, 448).to(FP8)
    else:
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8)
    w_s = torch.rand(n // 128, k // 128) * 1e-2
    x_q, x_s = ops.per_block_quant(x.cuda(), 128, qdtype)
    y = gemm_a8w8_blockscale(x_q, w.cuda(), x_s, w_s.cuda())
    torch.cuda.synchronize()
    ops.check_device_status(y.device)
    ref = O.block_scaled_matmul(x_q.cpu(), w, x_s.cpu(), w_s, (128, 128), torch.bfloat16)
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    torch.testing.assert_close(y.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    y2 = w8a8_block_scaled_mm(x_q, w.cuda(), x_s, w_s.cuda(), [128, 128], torch.float16)
    assert y2.dtype == torch.float16
    torch.testing.assert_close(y2.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)


# ---------------------------------------------------------------------------
# tile-pair schedule (two CTAs of a cluster share the weight tile of two row tiles)
# ---------------------------------------------------------------------------
def _pair_problem(m, e, topk, seed, mask=None):
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    w, ids = _routing(m, e, topk, seed)
    pos = torch.empty(ids.shape, dtype=torch.int32, device="cuda")
    res = ops.moe_sorting_ck(ids.cuda(), w.cuda(), e, None, None, 128,
                             None if mask is None else mask.cuda(), route_pos=pos,
                             segment_rows=_cabi.PAIR_SEGMENT_ROWS)
    torch.cuda.synchronize()
    return dict(w=w, ids=ids, s_ids=res[0], s_w=res[1], s_e=res[2], nv=res[3], segs=res[6],
                nseg=res[7], cap=res[0].shape[0], pos=pos, nvi=int(res[3].item()),
                h_ids=res[0].cpu(), h_e=res[2].cpu())


def test_sort_segments_are_pairs_of_row_tiles():
    """Segment list of the sort: per enabled expert, runs of at most 256 live rows."""
    import numpy as np
    m, e, topk = 900, 8, 2
    mask = torch.ones(e, dtype=torch.int32)
    mask[2] = 0
    pr = _pair_problem(m, e, topk, 13, mask)
    counts = np.bincount(pr["ids"].numpy().ravel(), minlength=e)
    expect, start, label = [], 0, 0
    for ex in range(e):
        if mask[ex] == 0:
            continue
        c = int(counts[ex])
        for r in range(0, c, 256):
            expect.append([label, start + r, min(256, c - r), 0])
        start += (c + 127) // 128 * 128
        label += 1
    n = int(pr["nseg"].item())
    assert n == len(expect)
    assert np.array_equal(pr["segs"].cpu().numpy()[:n], np.array(expect, dtype=np.int32))


@pytest.mark.parametrize("kind_name", ["bf16", "fp8_block", "int8_block", "int8_channel"])
@pytest.mark.parametrize("m,e,topk", [(1500, 8, 2), (700, 4, 1), (300, 16, 4)])
def test_gemm_tile_pairs_equal_single_tiles(kind_name, m, e, topk):
    """Same tiles, same arithmetic, other CTA-to-tile mapping: every epilogue of the tile-pair
    schedule reproduces the single-tile schedule bit for bit (experts with one, two, three and
    more row tiles, i.e. full pairs and pairs whose second CTA idles), and untouched rows stay
    untouched."""
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    torch.manual_seed(m + e)
    inter, k = 256, 512
    pr = _pair_problem(m, e, topk, 3 + m)
    x = (torch.randn(m, k) / 2).bfloat16()
    extra = {}
    if kind_name == "bf16":
        kind = _cabi.GEMM_BF16
        w1 = (torch.randn(e, 2 * inter, k) / 8).bfloat16()
        a_sorted, _ = ops.gather_rows(x.cuda(), pr["s_ids"], pr["nv"], pr["cap"])
    elif kind_name in ("fp8_block", "int8_block"):
        qd = FP8 if kind_name == "fp8_block" else torch.int8
        kind = _cabi.GEMM_FP8_BLOCK if qd == FP8 else _cabi.GEMM_INT8_BLOCK
        w1 = ((torch.randn(e, 2 * inter, k) * 40).clamp(-448, 448).to(FP8) if qd == FP8
              else torch.randint(-127, 128, (e, 2 * inter, k), dtype=torch.int8))
        a_sorted, a_scale = ops.quant_scatter_rows(x.cuda(), 128, qd, pr["pos"], pr["s_ids"],
                                                   pr["nv"], pr["cap"])
        extra = dict(a_scale=a_scale, a_scale_ld=pr["cap"],
                     b_scale=(torch.rand(e, 2 * inter // 128, k // 128) * 1e-2 + 1e-3).cuda())
    else:
        kind = _cabi.GEMM_INT8_CHANNEL
        w1 = torch.randint(-127, 128, (e, 2 * inter, k), dtype=torch.int8)
        xq, xs = ops.per_token_quant(x.cuda(), quant_dtype=torch.int8)
        a_sorted, a_scale = ops.gather_rows(xq, pr["s_ids"], pr["nv"], pr["cap"], xs)
        extra = dict(a_scale=a_scale, b_scale=(torch.rand(e, 2 * inter) * 1e-2 + 1e-3).cuda())
    bias = (torch.randn(e, 2 * inter) / 4).bfloat16().cuda()
    common = dict(kind=kind, sorted_expert_ids=pr["s_e"], num_valid=pr["nv"], a=a_sorted,
                  b=w1.cuda(), sorted_ids=pr["s_ids"], sorted_weights=pr["s_w"], num_tokens=m,
                  topk=topk, **extra)
    pairs = dict(segments=pr["segs"], num_segments=pr["nseg"])
    sentinel = -12345.0   # exactly representable in bf16 / fp32

    def run(sched, shape, dtype=torch.bfloat16, **kw):
        c = torch.full(shape, sentinel, dtype=dtype, device="cuda") if dtype.is_floating_point \
            and dtype not in (FP8,) else torch.zeros(shape, dtype=dtype, device="cuda")
        cs = kw.pop("c_scale_shape", None)
        if cs is not None:
            kw["c_scale"] = torch.full(cs, sentinel, dtype=torch.float32, device="cuda")
            kw["c_scale_ld"] = cs[1]
        ops.grouped_gemm(c=c, **kw, **common, **sched)
        torch.cuda.synchronize()
        ops.check_device_status(c.device)
        return c, kw.get("c_scale")

    cap = pr["cap"]
    cases = [
        dict(epilogue=_cabi.EPI_STORE, bias=bias, shape=(cap, 2 * inter)),
        dict(epilogue=_cabi.EPI_STORE, scatter=True, mul_routed_weight=True,
             shape=(m * topk, 2 * inter)),
        dict(epilogue=_cabi.EPI_STORE, shape=(cap, 2 * inter), dtype=torch.float32),
        dict(epilogue=_cabi.EPI_SILU_MUL, bias=bias, mid_dtype=torch.bfloat16, shape=(cap, inter)),
    ]
    if kind_name in ("fp8_block", "int8_block"):
        cases.append(dict(epilogue=_cabi.EPI_SILU_MUL_QUANT, mid_dtype=torch.bfloat16,
                          shape=(cap, inter), dtype=FP8 if kind_name == "fp8_block" else torch.int8,
                          c_scale_shape=(inter // 128, cap)))
    for case in cases:
        shape = case.pop("shape")
        dtype = case.pop("dtype", torch.bfloat16)
        c1, s1 = run({}, shape, dtype, **dict(case))
        c2, s2 = run(pairs, shape, dtype, **dict(case))
        v1 = c1.view(torch.uint8) if dtype in (FP8, torch.int8) else c1
        v2 = c2.view(torch.uint8) if dtype in (FP8, torch.int8) else c2
        assert torch.equal(v1, v2), f"{kind_name} {case.get('epilogue')} differs"
        if s1 is not None:
            assert torch.equal(s1, s2)
        if dtype == torch.bfloat16 and not case.get("scatter"):
            assert (c2 != sentinel).any()


@pytest.mark.parametrize("kind_name", ["bf16", "fp8_block", "int8_channel"])
@pytest.mark.parametrize("m,e,topk,wide", [(1500, 8, 2, False), (33, 16, 4, True), (300, 16, 4, False)])
def test_gemm_rows_gathered_by_the_kernel_equal_sorted_rows(kind_name, m, e, topk, wide):
    """The row operand read from TOKEN order through the sorted ids (16-byte asynchronous copies
    by two warps of the kernel, padding positions zero-filled) against the same rows copied into
    sorted order first: the
    tiles in shared memory must be identical, so every output bit is.  `wide`: token rows that
    are slices of a wider buffer (a_row_bytes)."""
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    torch.manual_seed(m + e)
    inter, k = 256, 512
    pr = _pair_problem(m, e, topk, 5 + m)
    x = (torch.randn(m, k) / 2).bfloat16().cuda()

    def token_order(t):
        """the token rows, optionally as slices of a wider buffer"""
        if not wide:
            return t
        buf = torch.zeros((m, k + 64), dtype=torch.uint8 if t.element_size() == 1
                          else t.dtype, device="cuda")
        view = buf[:, :k]
        view[:m] = t.view(buf.dtype) if t.element_size() == 1 else t
        return view.view(t.dtype) if t.element_size() == 1 else view

    extra = {}
    if kind_name == "bf16":
        kind = _cabi.GEMM_BF16
        w1 = (torch.randn(e, 2 * inter, k) / 8).bfloat16()
        a_sorted, _ = ops.gather_rows(x, pr["s_ids"], pr["nv"], pr["cap"])
        a_tok = token_order(x)
    elif kind_name == "fp8_block":
        kind = _cabi.GEMM_FP8_BLOCK
        w1 = (torch.randn(e, 2 * inter, k) * 40).clamp(-448, 448).to(FP8)
        a_sorted, a_scale = ops.quant_scatter_rows(x, 128, FP8, pr["pos"], pr["s_ids"], pr["nv"],
                                                   pr["cap"])
        xq, _ = ops.per_block_quant(x, 128, FP8)
        a_tok = token_order(xq)
        extra = dict(a_scale=a_scale, a_scale_ld=pr["cap"],
                     b_scale=(torch.rand(e, 2 * inter // 128, k // 128) * 1e-2 + 1e-3).cuda())
    else:
        kind = _cabi.GEMM_INT8_CHANNEL
        w1 = torch.randint(-127, 128, (e, 2 * inter, k), dtype=torch.int8)
        xq, xs = ops.per_token_quant(x, quant_dtype=torch.int8)
        a_sorted, a_scale = ops.gather_rows(xq, pr["s_ids"], pr["nv"], pr["cap"], xs)
        a_tok = token_order(xq)
        extra = dict(a_scale=a_scale, b_scale=(torch.rand(e, 2 * inter) * 1e-2 + 1e-3).cuda())
    common = dict(kind=kind, sorted_expert_ids=pr["s_e"], num_valid=pr["nv"], b=w1.cuda(),
                  sorted_ids=pr["s_ids"], sorted_weights=pr["s_w"], num_tokens=m, topk=topk,
                  **extra)
    cap = pr["cap"]
    for case in [dict(epilogue=_cabi.EPI_STORE, shape=(cap, 2 * inter)),
                 dict(epilogue=_cabi.EPI_SILU_MUL, mid_dtype=torch.bfloat16, shape=(cap, inter)),
                 dict(epilogue=_cabi.EPI_STORE, scatter=True, mul_routed_weight=True,
                      shape=(m * topk, 2 * inter))]:
        shape = case.pop("shape")
        outs = []
        for a, kw in ((a_sorted, {}), (a_tok, dict(a_gather=True))):
            c = torch.full(shape, -12345.0, dtype=torch.bfloat16, device="cuda")
            ops.grouped_gemm(a=a, c=c, **kw, **case, **common)
            torch.cuda.synchronize()
            ops.check_device_status(c.device)
            outs.append(c)
        assert (outs[1] != -12345.0).any()
        assert torch.equal(outs[0], outs[1]), f"{kind_name} {case['epilogue']} differs"


def test_gemm_gathered_rows_with_reduction_and_column_tails():
    """k = 336 (not a multiple of the 64-element K block) and n = 384: the gathered copies must
    zero-fill the reduction tail exactly as the box copy does."""
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    m, e, topk, n, k = 200, 4, 2, 384, 336
    torch.manual_seed(9)
    pr = _sorted_problem(m, e, topk, 11)
    x = (torch.randn(m, k) / 4).bfloat16().cuda()
    b = (torch.randn(e, n, k) / 8).bfloat16().cuda()
    a_sorted, _ = ops.gather_rows(x, pr["s_ids"], pr["nv"], pr["cap"])
    outs = []
    for a, kw in ((a_sorted, {}), (x, dict(a_gather=True))):
        c = torch.full((pr["cap"], n), -12345.0, dtype=torch.bfloat16, device="cuda")
        ops.grouped_gemm(kind=_cabi.GEMM_BF16, epilogue=_cabi.EPI_STORE, a=a, b=b, c=c,
                         sorted_expert_ids=pr["s_e"], num_valid=pr["nv"], sorted_ids=pr["s_ids"],
                         sorted_weights=pr["s_w"], num_tokens=m, topk=topk, **kw)
        torch.cuda.synchronize()
        ops.check_device_status(c.device)
        outs.append(c)
    assert torch.equal(outs[0], outs[1])
