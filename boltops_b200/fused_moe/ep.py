"""Expert parallelism for the fused-MoE layer on one NVLink/NVSwitch box.

Experts are sharded contiguously over the ranks of a process group (rank r owns
experts ``[r*E/R, (r+1)*E/R)``; weights never move); every rank brings its own
tokens.  One exchange each way:

* dispatch: a token row travels once to every rank that owns at least one of its
  top-k experts (not once per route), together with its full top-k ids/weights;
* the owning rank runs the local layer in the reference's masked mode
  (``expert_map``; boltops/fused_moe/triton/fused_moe.py:1374-1377,1439-1443 in
  the reference project) and returns ONE partial row per received token;
* combine: the source rank adds the partial rows of a token in ascending rank
  order with an fp32 accumulator (``bolt_moe_gather_sum``).

The reference has no collective of its own: it leaves the cross-rank reduction to
the caller.  The exchange here is ``all_to_all_single`` (NCCL over NVLink on GPUs,
gloo in the CPU tests); index construction is device-agnostic torch so the same
code runs under both.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


class ExpertParallelMoE:
    """Dispatch → local experts → combine for one process group.

    ``local_fn(hidden, w1, w2, topk_weights, topk_ids, expert_map=..., global_num_experts=...,
    **kw)`` computes the masked local layer (default: ``fused_experts``);
    ``combine_fn(src, pos, out)`` the gather-sum (default: the CUDA kernel).
    """

    def __init__(self, group, num_experts: int, device,
                 local_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not shard evenly over {self.world} ranks")
        self.num_experts = num_experts
        self.per_rank = num_experts // self.world
        self.device = torch.device(device)
        emap = torch.full((num_experts,), -1, dtype=torch.int32)
        lo = self.rank * self.per_rank
        emap[lo:lo + self.per_rank] = torch.arange(self.per_rank, dtype=torch.int32)
        self.expert_map = emap.to(self.device)
        if local_fn is None:
            from . import fused_experts as local_fn
        if combine_fn is None:
            from .ops import gather_sum as combine_fn
        self.local_fn = local_fn
        self.combine_fn = combine_fn
        self.last_stats = {}
        self.profile = False      # set True to fill last_stats["ms"] with CUDA-event stage times
        self.quantize_dispatch = True   # w8a8 experts: send 8-bit codes + scales, not 16-bit rows
        # Small batches (decode): when every rank brings the SAME number of tokens and
        # tokens * world <= replicate_below, skip the dispatch (two host round trips and two
        # variable all-to-alls) and use the reference's replicated-token scheme instead:
        # all-gather the tokens, run the masked local layer on all of them, reduce-scatter
        # the partial outputs.  0 = never (the caller must guarantee equal token counts).
        self.replicate_below = 0

    # -- index construction ---------------------------------------------------------------
    def plan(self, topk_ids: torch.Tensor):
        """Which token goes to which rank.  Returns ``(tok_idx [S], send_counts [R],
        pos [M, R])``: rows to send ordered by (rank, token); ``pos[m, r]`` = row of token
        m's partial result in the returned buffer, -1 if rank r owns none of its experts."""
        if topk_ids.is_cuda and self.world <= 255:
            return self._plan_cuda(topk_ids)
        return self._plan_torch(topk_ids)

    def _plan_cuda(self, topk_ids: torch.Tensor):
        """Same result as :meth:`_plan_torch` without a host synchronisation: "token m goes
        to rank r" is a route of token m to "expert" r, so the layer's own stable sort (unit
        1, ranks as experts) yields the (rank, token) order, the per-rank counts and, as its
        inverse permutation, ``pos``."""
        from . import ops
        m = topk_ids.shape[0]
        routes = ops.ep_dest_ranks(topk_ids, self.num_experts, self.per_rank, self.world)
        dummy_w = torch.empty((m, self.world), dtype=torch.float32, device=topk_ids.device)
        pos = torch.empty((m, self.world), dtype=torch.int32, device=topk_ids.device)
        sorted_ids, _, _, _, counts, _ = ops.moe_sorting_ck(
            routes, dummy_w, self.world, None, None, 1, None, alloc_moe_buf=False, route_pos=pos)
        send_counts = counts[:self.world].long()
        # rows beyond the number of sent rows are cut by the caller once the counts are on the host
        tok_idx = (sorted_ids & 0xFFFFFF).long()
        return tok_idx, send_counts, pos

    def _plan_torch(self, topk_ids: torch.Tensor):
        m = topk_ids.shape[0]
        dest = torch.div(topk_ids.long(), self.per_rank, rounding_mode="floor")
        valid = (topk_ids >= 0) & (topk_ids < self.num_experts)
        hit = torch.zeros((m, self.world + 1), dtype=torch.bool, device=topk_ids.device)
        hit.scatter_(1, torch.where(valid, dest, torch.full_like(dest, self.world)), True)
        hit = hit[:, :self.world]
        rank_idx, tok_idx = hit.t().nonzero(as_tuple=True)          # sorted by rank, then token
        send_counts = hit.sum(dim=0)
        pos = torch.full((m, self.world), -1, dtype=torch.int32, device=topk_ids.device)
        pos[tok_idx, rank_idx] = torch.arange(tok_idx.numel(), dtype=torch.int32,
                                              device=topk_ids.device)
        return tok_idx, send_counts, pos

    def _exchange_counts(self, send_counts: torch.Tensor):
        both = torch.empty((2, send_counts.numel()), dtype=send_counts.dtype,
                           device=send_counts.device)
        both[0].copy_(send_counts)
        dist.all_to_all_single(both[1], both[0], group=self.group)
        send_split, recv_split = both.tolist()          # one host synchronisation for both
        if both.is_cuda:
            # the host has just synchronised with the device anyway: a good moment to notice a
            # bounded device-side wait that expired in an earlier layer
            from . import ops
            ops.check_device_status(both.device)
        return send_split, recv_split

    # -- small batches: replicated tokens, no dispatch ---------------------------------------
    def forward_replicated(self, hidden_states, w1_local, w2_local, topk_weights, topk_ids,
                           **kwargs):
        """All ranks hold the same number of tokens.  Partial rows leave the local layer in the
        output dtype (as in the dispatch path), are summed over the ranks in fp32 and rounded
        once.  No host synchronisation."""
        m, h = hidden_states.shape
        world = self.world
        dev = hidden_states.device
        out_dtype = kwargs.get("output_dtype") or hidden_states.dtype

        def gather(t):
            t = t.contiguous()
            full = torch.empty((world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype,
                               device=dev)
            dist.all_gather_into_tensor(full, t, group=self.group)
            return full

        all_h = gather(hidden_states)
        all_w = gather(topk_weights.to(torch.float32))
        all_i = gather(topk_ids.to(torch.int32))
        partial = self.local_fn(all_h, w1_local, w2_local, all_w, all_i,
                                expert_map=self.expert_map,
                                global_num_experts=self.num_experts, **kwargs)
        partial = partial.to(torch.float32)
        if partial.is_cuda:
            mine = torch.empty((m, h), dtype=torch.float32, device=dev)
            dist.reduce_scatter_tensor(mine, partial, group=self.group)
        else:   # gloo has no reduce-scatter
            dist.all_reduce(partial, group=self.group)
            mine = partial[self.rank * m:(self.rank + 1) * m]
        self.last_stats = dict(mode="replicated", tokens=m * world)
        return mine.to(out_dtype)

    # -- the layer ----------------------------------------------------------------------------
    def forward(self, hidden_states, w1_local, w2_local, topk_weights, topk_ids, **kwargs):
        m, h = hidden_states.shape
        if self.replicate_below and m * self.world <= self.replicate_below \
                and not kwargs.get("no_combine"):
            return self.forward_replicated(hidden_states, w1_local, w2_local, topk_weights,
                                           topk_ids, **kwargs)
        k = topk_ids.shape[1]
        marks = []

        def mark(name):
            if self.profile and hidden_states.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        tok_idx, send_counts, pos = self.plan(topk_ids)
        send_split, recv_split = self._exchange_counts(send_counts)
        n_recv = int(sum(recv_split))
        tok_idx = tok_idx[: int(sum(send_split))]
        mark("plan+counts")

        # Quantise before the wire when the experts are w8a8: the rows then cross NVLink as
        # 8-bit codes + scales instead of 16-bit values, and the local layer takes them as
        # pre-quantised input (same codes it would have produced itself).
        out_dtype = kwargs.get("output_dtype") or hidden_states.dtype
        x, x_scale = hidden_states, None
        w8a8 = kwargs.get("use_fp8_w8a8") or kwargs.get("use_int8_w8a8")
        if (self.quantize_dispatch and w8a8 and hidden_states.is_cuda
                and hidden_states.dtype in (torch.float16, torch.bfloat16)
                and not kwargs.get("use_ue8m0")):
            from . import ops
            qd = torch.float8_e4m3fn if kwargs.get("use_fp8_w8a8") else torch.int8
            if kwargs.get("per_channel_quant"):
                x, x_scale = ops.per_token_quant(hidden_states, quant_dtype=qd)
            elif kwargs.get("block_shape") is not None:
                x, x_scale = ops.per_block_quant(hidden_states, kwargs["block_shape"][1], qd)
        dev = hidden_states.device
        meta_cols = [topk_ids.to(torch.int32), topk_weights.to(torch.float32).view(torch.int32)]
        if x_scale is not None:
            meta_cols.append(x_scale.reshape(m, -1).view(torch.int32))
        meta = torch.cat(meta_cols, dim=1)
        send_meta = meta.index_select(0, tok_idx)
        send_x = x.view(torch.uint8).index_select(0, tok_idx) if x_scale is not None \
            else x.index_select(0, tok_idx)
        recv_x = torch.empty((n_recv, send_x.shape[1]), dtype=send_x.dtype, device=dev)
        recv_meta = torch.empty((n_recv, meta.shape[1]), dtype=torch.int32, device=dev)
        dist.all_to_all_single(recv_x, send_x, recv_split, send_split, group=self.group)
        dist.all_to_all_single(recv_meta, send_meta, recv_split, send_split, group=self.group)
        mark("dispatch")

        r_ids = recv_meta[:, :k].contiguous()
        r_w = recv_meta[:, k:2 * k].contiguous().view(torch.float32)
        local_kwargs = dict(kwargs)
        if x_scale is not None:
            recv_x = recv_x.view(x.dtype)
            local_kwargs["a1_scale"] = recv_meta[:, 2 * k:].contiguous().view(torch.float32)
            local_kwargs["output_dtype"] = out_dtype
        if n_recv:
            partial = self.local_fn(recv_x, w1_local, w2_local, r_w, r_ids,
                                    expert_map=self.expert_map,
                                    global_num_experts=self.num_experts, **local_kwargs)
        else:
            partial = torch.empty((0, h), dtype=out_dtype, device=dev)
        mark("experts")
        back = torch.empty((tok_idx.numel(), h), dtype=out_dtype, device=dev)
        dist.all_to_all_single(back, partial.contiguous(), send_split, recv_split,
                               group=self.group)
        mark("return")
        out = torch.empty((m, h), dtype=out_dtype, device=dev)
        self.combine_fn(back, pos, out)
        mark("combine")
        self.last_stats = dict(rows_sent=int(sum(send_split)), rows_received=n_recv,
                               routes=m * k)
        if marks:
            torch.cuda.synchronize()
            self.last_stats["ms"] = {b[0]: a[1].elapsed_time(b[1])
                                     for a, b in zip(marks[:-1], marks[1:])}
        return out
