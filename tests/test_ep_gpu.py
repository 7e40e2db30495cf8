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
