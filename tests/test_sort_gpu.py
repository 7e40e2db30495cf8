"""Sort kernels vs the CPU oracle: bit-exact on every output."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import load_npz

pytestmark = pytest.mark.gpu


def _run_ck(ids, w, E, unit, mask):
    from boltops_b200.fused_moe import ops
    dev = "cuda"
    t_ids = torch.from_numpy(np.ascontiguousarray(ids)).to(dev)
    t_w = torch.from_numpy(np.ascontiguousarray(w)).to(dev)
    t_mask = None if mask is None else torch.from_numpy(np.ascontiguousarray(mask)).to(dev)
    s_ids, s_w, s_e, nv, pos, _ = ops.moe_sorting_ck(t_ids, t_w, E, None, None, unit, t_mask)
    torch.cuda.synchronize()
    return s_ids.cpu().numpy(), s_w.cpu().numpy(), s_e.cpu().numpy(), int(nv.item()), pos.cpu().numpy()


def _check_ck(ids, w, E, unit, mask):
    ref = O.sort_ck_numpy(ids, w, E, unit, mask)
    s_ids, s_w, s_e, nv, pos = _run_ck(ids, w, E, unit, mask)
    assert nv == ref["num_valid"]
    assert np.array_equal(s_ids[:nv], ref["sorted_ids"])
    assert np.array_equal(s_w[:nv].view(np.uint32), ref["sorted_weights"].view(np.uint32))
    assert np.array_equal(s_e[: nv // unit], ref["expert_ids"])
    on = np.ones(E, bool) if mask is None else np.asarray(mask) != 0
    assert np.array_equal(pos[:E], ref["counts"])
    assert np.array_equal(pos[E:][on], ref["starts"][on])
    assert (pos[E:][~on] == -1).all()


@pytest.mark.parametrize("key", ["t1_e8_k2_u16_m0", "t17_e8_k2_u32_m1", "t128_e64_k8_u32_m0",
                                 "t512_e64_k8_u32_m1", "t5_e6_k3_u4_m0", "t5_e6_k3_u4_m1"])
def test_sort_ck_golden(key):
    z = load_npz("sort_ck.npz")
    mask = z[key + "/mask"]
    mask = None if mask.size == 0 else mask
    _, e, k, u, _ = key.split("_")
    E, unit = int(e[1:]), int(u[1:])
    s_ids, s_w, s_e, nv, pos = _run_ck(z[key + "/topk_ids"], z[key + "/topk_weights"], E, unit, mask)
    gold = z[key + "/sorted_ids"]
    assert nv == gold.size
    assert (s_ids[:nv].astype(np.int64) & 0xFFFFFFFF).tolist() == gold.tolist()
    assert np.array_equal(s_w[:nv], z[key + "/sorted_weights"])
    assert s_e[: len(z[key + "/expert_ids"])].tolist() == z[key + "/expert_ids"].tolist()
    for ex in range(E):
        if mask is None or mask[ex]:
            assert pos[ex] == z[key + "/counts"][ex]
        if z[key + "/starts"][ex] >= 0:
            assert pos[E + ex] == z[key + "/starts"][ex]


@pytest.mark.parametrize("tokens,E,topk,unit,use_mask", [
    (1, 8, 2, 128, False), (64, 8, 2, 128, False), (300, 256, 8, 128, False),
    (511, 128, 8, 128, True), (513, 128, 8, 64, False),          # around the single-CTA limit
    (4096, 256, 8, 128, False), (8192, 8, 2, 128, False), (16384, 128, 8, 128, True),
    (1000, 1, 1, 128, False), (777, 384, 6, 32, True),
])
def test_sort_ck_random(tokens, E, topk, unit, use_mask):
    rng = np.random.default_rng(tokens * 131 + E)
    ids = np.argsort(rng.random((tokens, E)), axis=1)[:, :topk].astype(np.int32)
    w = rng.random((tokens, topk), dtype=np.float32)
    mask = None
    if use_mask:
        mask = np.ones(E, np.int32)
        mask[1::4] = 0
    _check_ck(ids, w, E, unit, mask)


def test_sort_ck_skewed_and_empty_experts():
    rng = np.random.default_rng(5)
    ids = np.zeros((3000, 4), np.int32)
    ids[:, 0] = 7
    ids[:, 1:] = 8 + np.argsort(rng.random((3000, 24)), axis=1)[:, :3]
    w = rng.random((3000, 4), dtype=np.float32)
    _check_ck(ids, w, 64, 128, None)


def test_sort_ck_deterministic_across_runs():
    rng = np.random.default_rng(9)
    ids = np.argsort(rng.random((6000, 128)), axis=1)[:, :8].astype(np.int32)
    w = rng.random((6000, 8), dtype=np.float32)
    first = _run_ck(ids, w, 128, 128, None)
    for _ in range(3):
        again = _run_ck(ids, w, 128, 128, None)
        nv = first[3]
        assert again[3] == nv and np.array_equal(first[0][:nv], again[0][:nv])


@pytest.mark.parametrize("numel_shape,E,block,use_map", [
    ((4, 3), 5, 4, False), ((19, 3), 6, 8, False), ((700, 8), 64, 16, True),
    ((5000, 8), 256, 128, False), ((3, 2), 8, 64, True),
])
def test_align_block_size(numel_shape, E, block, use_map):
    from boltops_b200.fused_moe import ops
    rng = np.random.default_rng(sum(numel_shape) + E)
    if numel_shape == (4, 3):
        ids = np.array([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], np.int32)
    else:
        ids = rng.integers(-1, E + 1, size=numel_shape).astype(np.int32)  # incl. out-of-range ids
    emap = None
    if use_map:
        emap = np.full(E, -1, np.int32)
        emap[::2] = np.arange((E + 1) // 2)
    ref_ids, ref_e, total = O.align_block_size_loops(ids, block, E, emap)
    t_map = None if emap is None else torch.from_numpy(emap).cuda()
    s, e, n = ops.moe_align_block_size(torch.from_numpy(ids).cuda(), block, E, t_map)
    torch.cuda.synchronize()
    assert int(n.item()) == total
    assert np.array_equal(s.cpu().numpy(), ref_ids)
    assert np.array_equal(e.cpu().numpy(), ref_e)


@pytest.mark.parametrize("tokens,E,topk,use_mask", [(64, 8, 2, False), (3000, 128, 8, True)])
def test_sort_ck_route_positions_are_the_inverse_permutation(tokens, E, topk, use_mask):
    from boltops_b200.fused_moe import ops
    rng = np.random.default_rng(tokens)
    ids = np.argsort(rng.random((tokens, E)), axis=1)[:, :topk].astype(np.int32)
    w = rng.random((tokens, topk), dtype=np.float32)
    mask = None
    if use_mask:
        mask = np.ones(E, np.int32)
        mask[1::4] = 0
    pos = torch.full((tokens, topk), 12345, dtype=torch.int32, device="cuda")
    s_ids, _, _, nv, _, _ = ops.moe_sorting_ck(
        torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), E, None, None, 128,
        None if mask is None else torch.from_numpy(mask).cuda(), route_pos=pos)
    torch.cuda.synchronize()
    pos_h, ids_h = pos.cpu().numpy(), s_ids.cpu().numpy().astype(np.int64) & 0xFFFFFFFF
    on = np.ones(E, bool) if mask is None else mask != 0
    live = on[ids]
    assert (pos_h[~live] == -1).all()
    assert (pos_h[live] >= 0).all() and (pos_h[live] < int(nv.item())).all()
    tok, slot = np.nonzero(live)
    packed = ids_h[pos_h[tok, slot]]
    assert np.array_equal(packed & 0xFFFFFF, tok) and np.array_equal(packed >> 24, slot)
