"""Expert parallelism over NCCL on >= 2 GPUs: the EP layer equals the single-GPU layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import bench as B
        from boltops_b200.fused_moe import fused_experts, ops
        from boltops_b200.fused_moe.ep import ExpertParallelMoE
        from oracle import moe_oracle as O
        cfg = dict(kind="fp8_block", E=16, K=4, H=512, I=256)
        per = cfg["E"] // world
        mine = list(range(rank * per, (rank + 1) * per))
        w1, w2, w1s, w2s = B.make_weights(cfg, dev, mine, 0)
        hidden, wts, ids = B.make_tokens(cfg, 200, 50 + rank)
        ep = ExpertParallelMoE(dist.group.WORLD, cfg["E"], dev)
        out = ep.forward(hidden.to(dev), w1, w2, wts.to(dev), ids.to(dev), use_fp8_w8a8=True,
                         w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
        torch.cuda.synchronize()
        ops.check_device_status(dev)
        # single-GPU layer over all experts on this rank's tokens
        fw1, fw2, fw1s, fw2s = B.make_weights(cfg, dev, list(range(cfg["E"])), 0)
        full = fused_experts(hidden.to(dev), fw1, fw2, wts.to(dev), ids.to(dev), use_fp8_w8a8=True,
                             w1_scale=fw1s, w2_scale=fw2s, block_shape=[128, 128])
        torch.cuda.synchronize()
        # pipelined exchange in three token chunks on a second stream: same result
        ep.pipeline_chunks, ep.pipeline_min_tokens, ep.pipeline_rows_per_expert = 3, 0, 0
        piped = ep.forward(hidden.to(dev), w1, w2, wts.to(dev), ids.to(dev), use_fp8_w8a8=True,
                           w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
        torch.cuda.synchronize()
        assert ep.last_stats["chunks"] == 3
        assert torch.equal(piped, out), "chunked exchange changed the result"
        ep.pipeline_chunks = 1
        # small-batch path: replicated tokens + reduce-scatter instead of the dispatch
        ep.replicate_below = 4096
        rep = ep.forward(hidden.to(dev), w1, w2, wts.to(dev), ids.to(dev), use_fp8_w8a8=True,
                         w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
        torch.cuda.synchronize()
        assert ep.last_stats.get("mode") == "replicated"
        err = max(O.rel_l2(out.cpu(), full.cpu()), O.rel_l2(rep.cpu(), full.cpu()))
        # the MXFP8 recipe through the same dispatch (rows travel in 16 bits, experts quantise)
        ep.replicate_below = 0
        mcfg = dict(cfg, kind="mxfp8")
        mw1, mw2, ms1, ms2 = B.make_weights(mcfg, dev, mine, 0)
        mx = ep.forward(hidden.to(dev), mw1, mw2, wts.to(dev), ids.to(dev), use_mxfp8=True,
                        w1_scale=ms1, w2_scale=ms2, block_shape=[1, 32])
        fw1, fw2, fs1, fs2 = B.make_weights(mcfg, dev, list(range(cfg["E"])), 0)
        mfull = fused_experts(hidden.to(dev), fw1, fw2, wts.to(dev), ids.to(dev), use_mxfp8=True,
                              w1_scale=fs1, w2_scale=fs2, block_shape=[1, 32])
        torch.cuda.synchronize()
        # exchange over peer memory: same kernels in the local layer, same summation order in the
        # combine, so the result equals the all-to-all path bit for bit; twice, to cross the
        # hazards between steps
        ep.direct_max_tokens = 256
        for returned, want in (("partials", out), ("routes", full)):
            ep.direct_return = returned
            for _ in range(2):
                direct = ep.forward(hidden.to(dev), w1, w2, wts.to(dev), ids.to(dev),
                                    use_fp8_w8a8=True, w1_scale=w1s, w2_scale=w2s,
                                    block_shape=[128, 128])
                torch.cuda.synchronize()
                ops.check_device_status(dev)
                assert ep._direct_failed is None, ep._direct_failed
                assert ep.last_stats.get("mode") == "direct"
                # partial rows: the all-to-all path's arithmetic; per-route rows: the single-GPU
                # layer's own sum over the routes
                assert torch.equal(direct, want), f"exchange over peer memory ({returned})"
        out = full
        # no host-side state in a step: captured once in a CUDA graph, replayed three times
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ep.forward(hidden.to(dev), w1, w2, wts.to(dev), ids.to(dev), use_fp8_w8a8=True,
                       w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        hd, wd, idd = hidden.to(dev), wts.to(dev), ids.to(dev)
        with torch.cuda.graph(graph):
            replayed = ep.forward(hd, w1, w2, wd, idd, use_fp8_w8a8=True, w1_scale=w1s,
                                  w2_scale=w2s, block_shape=[128, 128])
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        ops.check_device_status(dev)
        assert torch.equal(replayed, out), "graph replay of the peer-memory step changed the result"
        ret[rank] = max(err, O.rel_l2(mx.cpu(), mfull.cpu()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep_two_gpus_matches_single_gpu_layer():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for rank in range(world):
        # per-rank partial sums are rounded to bf16 before they cross the link
        assert ret[rank] <= 1e-2, f"rank {rank}: {ret[rank]}"


def test_ep_plan_cuda_equals_torch_plan():
    """The sort-based planner (no host sync) and the torch planner agree exactly."""
    from boltops_b200.fused_moe.ep import ExpertParallelMoE
    from oracle import moe_oracle as O
    for world, e, k, m in [(8, 256, 8, 4096), (4, 16, 4, 37), (2, 8, 2, 1)]:
        ep = ExpertParallelMoE.__new__(ExpertParallelMoE)
        ep.world, ep.rank, ep.num_experts, ep.per_rank = world, 0, e, e // world
        _, ids = O.make_routing(m, e, k, 3 + m)
        if m > 5:
            ids[5, 0] = -1
        d_ids = ids.cuda()
        tok_a, cnt_a, pos_a = ep._plan_torch(d_ids)
        tok_b, cnt_b, pos_b = ep._plan_cuda(d_ids)
        n = int(cnt_a.sum())
        assert torch.equal(cnt_a.cpu(), cnt_b.cpu())
        assert torch.equal(tok_a.cpu(), tok_b[:n].cpu())
        assert torch.equal(pos_a.cpu(), pos_b.cpu())


@pytest.mark.parametrize("per_route", [False, True])
@pytest.mark.parametrize("kind,world,shape", [
    ("fp8_block", 4, dict(E=16, K=4, H=512, I=256)),
    ("bf16", 4, dict(E=16, K=4, H=512, I=256)),
    ("int8_channel", 4, dict(E=16, K=4, H=512, I=256)),
    ("fp8_block", 8, dict(E=64, K=8, H=1024, I=512)),       # eight ranks, top-8: the 8-GPU index space
])
def test_direct_exchange_phases_with_emulated_ranks(kind, world, shape, per_route):
    """The three phases of the exchange over peer memory for four ranks held by ONE process on
    one GPU (every "peer" buffer is a local tensor, ranks run phase by phase, no rank ever waits
    for another): headers, segment addressing, masking of unused rows and the combine are those
    of the real thing.  Expected, bit for bit: with partial rows coming back, the sum over ranks,
    in rank order, of the masked local layer on the same tokens, each partial rounded to the output
    dtype; with per-route rows coming back (the owners' down projection writes every route's row
    into the token owner's [tokens, topk, H] region), the single-GPU layer over all experts."""
    import bench as B
    from boltops_b200.fused_moe import fused_experts, ops
    from boltops_b200.fused_moe.ep import DirectExchange
    dev = torch.device("cuda", 0)
    m_max = 40 + 17 * (world - 1)
    cfg = dict(kind=kind, **shape)
    per = cfg["E"] // world
    if kind == "fp8_block":
        kw = dict(use_fp8_w8a8=True, block_shape=[128, 128])
        code, groups = torch.float8_e4m3fn, cfg["H"] // 128
        quant = lambda x: ops.per_block_quant(x, 128, torch.float8_e4m3fn)
    elif kind == "int8_channel":
        kw = dict(use_int8_w8a8=True, per_channel_quant=True)
        code, groups = torch.int8, 1
        quant = lambda x: ops.per_token_quant(x, quant_dtype=torch.int8)
    else:
        kw, code, groups, quant = {}, torch.bfloat16, 0, None
    ranks, toks, weights = [], [], []
    for r in range(world):
        ex = DirectExchange(world, r, cfg["E"], m_max, cfg["H"] * (2 if groups == 0 else 1), groups,
                            cfg["K"], cfg["H"], torch.bfloat16, dev, code, per_route)
        ranks.append(ex)
        hidden, wts, ids = B.make_tokens(cfg, 40 + 17 * r, 70 + r)       # ragged batch sizes
        toks.append((hidden.to(dev), wts.to(dev), ids.to(dev)))
        w1, w2, w1s, w2s = B.make_weights(cfg, dev, list(range(r * per, (r + 1) * per)), 0)
        weights.append((w1, w2, dict(kw, w1_scale=w1s, w2_scale=w2s) if w1s is not None else dict(kw)))
    bufs = [torch.full((ex.total_bytes,), 0x7B, dtype=torch.uint8, device=dev) for ex in ranks]
    for ex, buf in zip(ranks, bufs):
        buf[:ex.recv_off].zero_()
        ex.attach(buf, [b.data_ptr() for b in bufs])
    full = None
    if per_route:
        fw1, fw2, fw1s, fw2s = B.make_weights(cfg, dev, list(range(cfg["E"])), 0)
        full = (fw1, fw2, dict(kw, w1_scale=fw1s, w2_scale=fw2s) if fw1s is not None else dict(kw))
    for step in range(2):                                   # twice: stale rows of step one remain
        pos = [ex.dispatch(h, w, i, quant) for ex, (h, w, i) in zip(ranks, toks)]
        for ex, (w1, w2, k) in zip(ranks, weights):
            ex.experts(w1, w2, routed_scaling_factor=1.5, **k)
        for r, ex in enumerate(ranks):
            h, w, i = toks[r]
            out = torch.empty_like(h)
            if per_route:
                ex.combine_routes(i, out, 1.5)
                want = fused_experts(h, full[0], full[1], w, i, routed_scaling_factor=1.5, **full[2])
            else:
                ex.combine(pos[r], out, ops.gather_sum)
                acc = torch.zeros(h.shape, dtype=torch.float32, device=dev)
                for q, (w1, w2, k) in enumerate(weights):
                    emap = torch.full((cfg["E"],), -1, dtype=torch.int32, device=dev)
                    emap[q * per:(q + 1) * per] = torch.arange(per, dtype=torch.int32, device=dev)
                    acc += fused_experts(h, w1, w2, w, i, expert_map=emap, global_num_experts=cfg["E"],
                                         routed_scaling_factor=1.5, **k).float()
                want = acc.to(out.dtype)
            torch.cuda.synchronize()
            ops.check_device_status(dev)
            assert torch.equal(out, want), f"rank {r}, step {step}"
            sent = int((pos[r] >= 0).sum())
            assert int(ex.hdr[:, 0].sum()) == sum(int((p[:, r] >= 0).sum()) for p in pos)
            assert sent <= ex.back_rows


def test_exchange_barrier_gives_up_when_a_rank_never_arrives():
    """Failure detection without a fault: a meeting in which one "rank" never sets its flag
    (its buffer is a local tensor nothing writes to).  The wait runs out after about a second,
    the kernel returns, the status word reports it and the context stays usable; a meeting in
    which the flag is there returns at once."""
    import time
    from boltops_b200 import _cabi
    from boltops_b200.fused_moe import ops
    dev = torch.device("cuda", 0)
    mine = torch.zeros(64, dtype=torch.int32, device=dev)
    absent = torch.zeros(64, dtype=torch.int32, device=dev)
    peers = torch.tensor([mine.data_ptr(), absent.data_ptr()], dtype=torch.int64, device=dev)
    ops.device_status(dev).zero_()
    mine[1] = 1                                   # the other rank has "arrived" at epoch 1
    ops.ep_barrier(peers, 0, 0)                   # (my own epoch counter, slot 2, goes 0 -> 1)
    torch.cuda.synchronize()
    ops.check_device_status(dev)                  # healthy
    assert int(absent[0].item()) == 1             # and this rank told it so
    t0 = time.time()
    ops.ep_barrier(peers, 0, 0)                   # epoch 2: nobody ever writes it into `mine`
    torch.cuda.synchronize()
    assert 0.2 < time.time() - t0 < 10.0
    with pytest.raises(_cabi.BoltError, match="code 20"):
        ops.check_device_status(dev)
    ops.check_device_status(dev)                  # cleared; the context still works
    assert int((mine + 1)[5].item()) == 1         # (slot 5 is not a flag anybody wrote)
