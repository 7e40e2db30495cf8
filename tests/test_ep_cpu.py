"""Expert-parallel dispatch/combine logic on CPU ranks (gloo, world_size 2 and 4).

The local expert computation is injected (the CPU oracle in masked mode), so these
tests exercise exactly the host-side plumbing that also runs on GPUs: planning,
count exchange, the two all-to-alls, the deterministic gather-sum order, and the
error path for an expert count that does not shard."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _local_oracle(hidden, w1, w2, wts, ids, expert_map=None, global_num_experts=-1, **kw):
    flat = expert_map.long()[ids.long()]                      # -1 for experts of other ranks
    masked = torch.where(flat >= 0, flat, torch.full_like(flat, -1)).to(torch.int32)
    return O.moe_bf16(hidden, w1, w2, wts, masked)


def _cpu_gather_sum(src, pos, out):
    acc = torch.zeros(out.shape, dtype=torch.float32)
    for j in range(pos.shape[1]):
        p = pos[:, j].long()
        sel = p >= 0
        acc[sel] += src[p[sel]].float()
    out.copy_(acc.to(out.dtype))
    return out


def _worker(rank, world, port, E, K, H, I, M, zipf, ret, chunks=1):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from boltops_b200.fused_moe.ep import ExpertParallelMoE
        g = torch.Generator().manual_seed(0)
        w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16()
        w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
        per = E // world
        gh = torch.Generator().manual_seed(100 + rank)
        hidden = torch.randn(M, H, generator=gh).bfloat16()
        wts, ids = O.make_routing(M, E, K, 200 + rank, zipf)
        if rank == 1:
            ids[0, 0] = -1                                   # an out-of-range id is ignored
        ep = ExpertParallelMoE(dist.group.WORLD, E, "cpu", local_fn=_local_oracle,
                               combine_fn=_cpu_gather_sum)
        if chunks > 1:                                       # the pipelined exchange, in chunks
            ep.pipeline_chunks, ep.pipeline_min_tokens = chunks, 0
            ep.pipeline_rows_per_expert = 0
            if rank == world - 1:
                ids[:] = ids % (E // world)                  # this rank sends to rank 0 only ...
            else:
                ids[:] = ids % (E - E // world)              # ... and nobody sends to the last rank
        out = ep.forward(hidden, w1[rank * per:(rank + 1) * per], w2[rank * per:(rank + 1) * per],
                         wts, ids)
        expect = O.moe_bf16(hidden, w1, w2, wts, ids)
        err = O.rel_l2(out, expect)
        stats = ep.last_stats
        assert stats["rows_sent"] <= stats["routes"]
        assert stats["chunks"] == min(chunks, M)
        if chunks > 1 and rank == world - 1:
            assert stats["rows_received"] == 0               # a rank without any work
        ret[rank] = (err, stats["rows_sent"], stats["routes"])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,E,K,zipf", [(2, 8, 2, None), (4, 16, 4, 1.2)])
def test_ep_dispatch_combine_matches_single_rank(world, E, K, zipf):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), E, K, 64, 32, 37, zipf, ret), nprocs=world,
             join=True)
    assert len(ret) == world
    for rank in range(world):
        err, sent, routes = ret[rank]
        assert err <= 1e-2, f"rank {rank}: rel-L2 {err}"
        assert 0 < sent <= routes


@pytest.mark.parametrize("world,chunks,M", [(2, 2, 37), (4, 3, 50), (2, 4, 3)])
def test_ep_chunked_exchange_matches_single_rank(world, chunks, M):
    """Token chunks of the pipelined exchange: ragged last chunk (37 = 19 + 18, 50 = 17 + 17 +
    16), more chunks than tokens allow (3 tokens, 4 chunks), a rank that receives nothing."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), 4 * world, 2, 64, 32, M, None, ret, chunks),
             nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        err, sent, routes = ret[rank]
        assert err <= 1e-2, f"rank {rank}: rel-L2 {err}"


def test_ep_chunked_plan_orders_by_chunk_rank_token():
    from boltops_b200.fused_moe.ep import ExpertParallelMoE
    ep = ExpertParallelMoE.__new__(ExpertParallelMoE)
    ep.world, ep.rank, ep.num_experts, ep.per_rank = 2, 0, 4, 2
    ids = torch.tensor([[0, 3], [2, 3], [1, 0], [0, 2]], dtype=torch.int32)
    tok, counts, pos = ep.plan(ids, chunks=2)                # chunks: tokens {0,1} and {2,3}
    assert counts.tolist() == [1, 2, 2, 1]                   # (c0,r0) (c0,r1) (c1,r0) (c1,r1)
    assert tok.tolist() == [0, 0, 1, 2, 3, 3]
    assert pos.tolist() == [[0, 1], [-1, 2], [3, -1], [4, 5]]


def _replicated_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from boltops_b200.fused_moe.ep import ExpertParallelMoE
        E, K, H, I, M = 8, 2, 64, 32, 5
        g = torch.Generator().manual_seed(0)
        w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16()
        w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
        per = E // world
        hidden = torch.randn(M, H, generator=torch.Generator().manual_seed(100 + rank)).bfloat16()
        wts, ids = O.make_routing(M, E, K, 200 + rank)
        ep = ExpertParallelMoE(dist.group.WORLD, E, "cpu", local_fn=_local_oracle,
                               combine_fn=_cpu_gather_sum)
        ep.replicate_below = 64          # 5 tokens x 2 ranks: the small-batch path
        out = ep.forward(hidden, w1[rank * per:(rank + 1) * per], w2[rank * per:(rank + 1) * per],
                         wts, ids)
        assert ep.last_stats.get("mode") == "replicated"
        ep.replicate_below = 0
        ref = ep.forward(hidden, w1[rank * per:(rank + 1) * per], w2[rank * per:(rank + 1) * per],
                         wts, ids)
        expect = O.moe_bf16(hidden, w1, w2, wts, ids)
        ret[rank] = (O.rel_l2(out, expect), O.rel_l2(out, ref))
    finally:
        dist.destroy_process_group()


def test_ep_replicated_small_batch_matches_dispatch_and_single_rank():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_replicated_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert len(ret) == 2
    for rank in range(2):
        err, err_vs_dispatch = ret[rank]
        assert err <= 1e-2 and err_vs_dispatch <= 1e-2, (rank, err, err_vs_dispatch)


def _bad_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from boltops_b200.fused_moe.ep import ExpertParallelMoE
        try:
            ExpertParallelMoE(dist.group.WORLD, 7, "cpu", local_fn=_local_oracle,
                              combine_fn=_cpu_gather_sum)
            ret[rank] = "no error"
        except ValueError as exc:
            ret[rank] = str(exc)
    finally:
        dist.destroy_process_group()


def test_ep_rejects_uneven_sharding():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_bad_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert all("do not shard evenly" in ret[r] for r in range(2))


def test_ep_plan_is_deterministic_and_dedups():
    """plan() needs no process group state beyond sizes: check it on a fake 4-rank layout."""
    from boltops_b200.fused_moe.ep import ExpertParallelMoE
    ep = ExpertParallelMoE.__new__(ExpertParallelMoE)
    ep.world, ep.rank, ep.num_experts, ep.per_rank = 4, 0, 16, 4
    ids = torch.tensor([[0, 1, 5], [15, 14, 13], [3, 7, 11], [4, 4, 4]], dtype=torch.int32)
    tok, counts, pos = ep.plan(ids)
    assert counts.tolist() == [2, 3, 1, 1]
    assert tok.tolist() == [0, 2, 0, 2, 3, 2, 1]
    assert pos.tolist() == [[0, 2, -1, -1], [-1, -1, -1, 6], [1, 3, 5, -1], [-1, 4, -1, -1]]


def test_direct_exchange_buffer_layout():
    """Layout arithmetic of the peer-memory exchange buffer (host only): regions do not
    overlap, are 256-byte aligned, hold what the kernels address, and depend only on the
    configuration (every rank must compute the same offsets)."""
    import torch
    from boltops_b200.fused_moe.ep import DirectExchange, wire_layout
    o_scale, o_ids, o_w, wire = wire_layout(7168, 56, 8)
    assert (o_scale, o_ids, o_w, wire) == (7168, 7168 + 224, 7168 + 224 + 32, 7168 + 224 + 64)
    exs = [DirectExchange(8, r, 256, 4096, 7168, 56, 8, 7168, torch.bfloat16, "cpu",
                          torch.float8_e4m3fn) for r in (0, 5)]
    a, b = exs
    assert a.key() == b.key() and a.total_bytes == b.total_bytes
    assert (a.hdr_off, a.flag_off, a.recv_off, a.back_off) == (b.hdr_off, b.flag_off, b.recv_off,
                                                               b.back_off)
    assert a.hdr_off == 0 and a.flag_off >= 8 * 8 and a.recv_off >= a.flag_off + 9 * 4
    assert a.back_off >= a.recv_off + 8 * 4096 * wire
    assert all(off % 256 == 0 for off in (a.flag_off, a.recv_off, a.back_off, a.total_bytes))
    assert a.back_rows == 4096 * 8 and a.total_bytes >= a.back_off + a.back_rows * 7168 * 2
    assert b.expert_map.tolist() == [-1] * 160 + list(range(32)) + [-1] * 64
    # per-route return: the wire row carries the token's index, the return region has topk slots
    c = DirectExchange(2, 1, 64, 100, 1024, 8, 4, 1024, torch.bfloat16, "cpu", torch.float8_e4m3fn,
                       per_route=True)
    base = wire_layout(1024, 8, 4)[3]
    assert (c.o_src, c.wire_bytes, c.back_rows) == (base, base + 16, 100 * 4)
    assert c.key() != DirectExchange(2, 1, 64, 100, 1024, 8, 4, 1024, torch.bfloat16, "cpu",
                                     torch.float8_e4m3fn).key()
    # fewer ranks than top-k: a token cannot go to more ranks than there are
    assert DirectExchange(2, 0, 64, 100, 1024, 0, 8, 512, torch.bfloat16, "cpu",
                          torch.bfloat16).back_rows == 200
