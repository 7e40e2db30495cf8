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
the caller.  Two exchanges are built.  On GPUs with peer access the rows travel by
plain stores into buffers that every rank can address (:class:`DirectExchange`:
the dispatch kernel writes into the owners' receive regions, the local layer's
combine writes partial rows into the senders' return regions, ranks meet at a
bounded flag barrier; no host synchronisation, replayable from a CUDA graph).
Otherwise, and for CPU ranks in the tests, the exchange is ``all_to_all_single``
(NCCL or gloo) with device-agnostic index construction in torch.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def _a16(n: int) -> int:
    return (n + 15) // 16 * 16


def _a256(n: int) -> int:
    return (n + 255) // 256 * 256


def wire_layout(row_bytes: int, groups: int, topk: int):
    """Byte offsets of the parts of a wire row: scales, ids, weights; total size."""
    o_scale = _a16(row_bytes)
    o_ids = o_scale + _a16(groups * 4)
    o_w = o_ids + _a16(topk * 4)
    return o_scale, o_ids, o_w, o_w + _a16(topk * 4)


class DirectExchange:
    """One rank's side of the exchange over peer memory (CUDA only, one process per GPU).

    Every rank owns a buffer of the same layout that all ranks can address::

        header  int32 [world][2]   {rows rank s sent me, first row of s's return region for me}
        flags   int32 [world + 1]  epochs of the barrier (every rank's flag, then my own counter)
        receive world segments of seg_rows wire rows; segment s is written by rank s
        return  partial output rows of MY tokens, in my send order, written by the experts' ranks

    A step is three phases with a meeting of all ranks between them: ``dispatch`` (quantise,
    write my wire rows into the owners' receive regions), ``experts`` (masked local layer over
    everything received; its top-k combine writes each partial row straight into the sender's
    return region), ``combine`` (sum a token's partial rows in ascending rank order).  Nothing
    in a step reads device data on the host: counts and offsets stay in device memory, the
    local layer always takes ``world * seg_rows`` rows and ignores those no rank sent.

    Hazards between steps are covered by the two meetings of a step: a receive region is
    rewritten only after every rank has passed the second meeting of the previous step (its
    local layer is done), a return region only after the first meeting of this step (its
    owner's final combine of the previous step is done).
    """

    def __init__(self, world: int, rank: int, num_experts: int, seg_rows: int, row_bytes: int,
                 groups: int, topk: int, hidden: int, out_dtype: torch.dtype, device,
                 code_dtype: torch.dtype, per_route: bool = False):
        self.world, self.rank, self.num_experts = world, rank, num_experts
        self.per_rank = num_experts // world
        self.seg_rows, self.row_bytes, self.groups, self.topk = seg_rows, row_bytes, groups, topk
        self.hidden, self.out_dtype, self.code_dtype = hidden, out_dtype, code_dtype
        self.device = torch.device(device)
        self.o_scale, self.o_ids, self.o_w, self.wire_bytes = wire_layout(row_bytes, groups, topk)
        # per_route: the owners' down projection writes every ROUTE's row straight into this rank's
        # [tokens, topk, H] return region (instead of one partial row per token and rank written by
        # their combine), so the wire row also carries the token's index here
        self.per_route = per_route
        self.o_src = self.wire_bytes
        if per_route:
            self.wire_bytes += 16
        self.back_rows = seg_rows * (topk if per_route else min(world, topk))
        self.hdr_off = 0
        self.flag_off = _a256(world * 8)
        self.recv_off = self.flag_off + _a256((world + 1) * 4)
        self.back_off = self.recv_off + _a256(world * seg_rows * self.wire_bytes)
        self.total_bytes = self.back_off + _a256(
            self.back_rows * hidden * torch.empty((), dtype=out_dtype).element_size())
        self.buf = None
        emap = torch.full((num_experts,), -1, dtype=torch.int32)
        emap[rank * self.per_rank:(rank + 1) * self.per_rank] = torch.arange(self.per_rank,
                                                                            dtype=torch.int32)
        self.expert_map = emap.to(self.device)

    def key(self):
        return (self.seg_rows, self.row_bytes, self.groups, self.topk, self.hidden, self.out_dtype,
                self.per_route)

    def attach(self, buf: torch.Tensor, peer_ptrs) -> None:
        """``buf``: this rank's exchange buffer (uint8, ``total_bytes``, zeroed header and
        flags); ``peer_ptrs``: base address of every rank's buffer, in rank order."""
        assert buf.dtype == torch.uint8 and buf.numel() >= self.total_bytes and buf.is_cuda
        assert buf.data_ptr() % 256 == 0 and len(peer_ptrs) == self.world
        self.buf = buf
        dev = self.device
        self.peers = torch.tensor(list(peer_ptrs), dtype=torch.int64, device=dev)
        self.back_ptrs = self.peers + self.back_off
        esz = torch.empty((), dtype=self.out_dtype).element_size()
        # every rank's return region, as an element offset from my own
        self.back_seg_off = torch.tensor([(int(p) - int(peer_ptrs[self.rank])) // esz
                                          for p in peer_ptrs], dtype=torch.int64, device=dev)
        self.hdr = buf[self.hdr_off:self.hdr_off + self.world * 8].view(torch.int32).view(
            self.world, 2)
        self.recv = buf[self.recv_off:self.recv_off + self.world * self.seg_rows
                        * self.wire_bytes].view(self.world * self.seg_rows, self.wire_bytes)
        esz = torch.empty((), dtype=self.out_dtype).element_size()
        self.back = buf[self.back_off:self.back_off + self.back_rows * self.hidden * esz].view(
            self.out_dtype).view(self.back_rows, self.hidden)

    # -- the three phases ---------------------------------------------------------------------
    def dispatch(self, hidden_states, topk_weights, topk_ids, quant):
        """Plan, quantise (``quant(x) -> (codes, scales)`` or None) and write the wire rows.
        Returns ``pos`` [M, world]: row of every partial result in the return region."""
        from . import ops
        m = hidden_states.shape[0]
        assert m <= self.seg_rows, "more tokens than the exchange buffers were sized for"
        routes = ops.ep_dest_ranks(topk_ids, self.num_experts, self.per_rank, self.world, 0)
        dummy_w = torch.empty((m, self.world), dtype=torch.float32, device=self.device)
        pos = torch.empty((m, self.world), dtype=torch.int32, device=self.device)
        sorted_ids, _, _, _, counts, _ = ops.moe_sorting_ck(
            routes, dummy_w, self.world, None, None, 1, None, alloc_moe_buf=False, route_pos=pos)
        x, x_scale = quant(hidden_states) if quant is not None else (hidden_states, None)
        ops.ep_dispatch_rows(x.contiguous(), x_scale, topk_ids.to(torch.int32).contiguous(),
                             topk_weights.to(torch.float32).contiguous(), sorted_ids,
                             counts[:self.world], self.rank, self.seg_rows, self.peers,
                             self.hdr_off, self.recv_off, self.wire_bytes)
        return pos

    def experts(self, w1_local, w2_local, **kwargs):
        """Masked local layer over every row of the receive region; partial rows go straight to
        the return regions of the ranks that sent the tokens."""
        from . import layer, ops
        if self.per_route:
            r_ids, r_w, src = ops.ep_unpack_routes(self.recv, self.o_ids, self.o_w, self.topk,
                                                   self.seg_rows, self.world, self.hdr, self.o_src)
            out_peers = dict(routes=self.back, src=src, seg_off=self.back_seg_off,
                             seg_rows=self.seg_rows)
            kwargs.pop("routed_scaling_factor", None)     # applied by the owner's final sum
        else:
            r_ids, r_w = ops.ep_unpack_routes(self.recv, self.o_ids, self.o_w, self.topk,
                                              self.seg_rows, self.world, self.hdr)
            out_peers = dict(seg_rows=self.seg_rows, seg_ptrs=self.back_ptrs, hdr=self.hdr)
        r_x = self.recv[:, :self.row_bytes].view(self.code_dtype)
        if self.groups:
            kwargs["a1_scale"] = self.recv[:, self.o_scale:self.o_scale + 4 * self.groups].view(
                torch.float32)
            kwargs["output_dtype"] = self.out_dtype
        else:
            r_x = r_x.contiguous()
        kwargs["activation"] = kwargs.get("activation") or "silu"
        layer.fused_experts_impl(
            r_x, w1_local, w2_local, r_w, r_ids, expert_map=self.expert_map,
            global_num_experts=self.num_experts, _out_peers=out_peers, **kwargs)

    def combine(self, pos, out, combine_fn):
        combine_fn(self.back, pos, out)
        return out

    def combine_routes(self, topk_ids, out, scale: float = 1.0):
        """Per-route return: ``out[m] = cast(scale * sum_k f32(back[m * topk + k]))`` over the
        routes with a valid expert id, k ascending -- the single-GPU layer's own sum."""
        from . import ops
        m, k = topk_ids.shape
        slot = torch.arange(m * k, dtype=torch.int32, device=self.device).view(m, k)
        valid = (topk_ids >= 0) & (topk_ids < self.num_experts)
        pos = torch.where(valid, slot, torch.full_like(slot, -1))
        ops.gather_sum(self.back, pos.contiguous(), out, scale)
        return out

    def barrier(self) -> None:
        from . import ops
        ops.ep_barrier(self.peers, self.rank, self.flag_off)


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
        # Pipelined all-to-all exchange: batches of at least pipeline_min_tokens tokens are cut
        # into pipeline_chunks token chunks; the all-to-alls of neighbouring chunks run on a second
        # stream under the expert GEMMs of the current one.  The GEMMs then leave comm_sms SMs
        # to the exchange kernels (a persistent GEMM on every SM would keep them waiting).
        # Off by default (1 chunk): measured on 4 GPUs every chunk streams the local experts'
        # weights again and runs on fewer SMs, which costs more than the overlap hides.
        self.pipeline_chunks = 1
        self.pipeline_min_tokens = 1024
        self.pipeline_rows_per_expert = 384   # expected rows per local expert and chunk, at least
        self.topk_hint = 0                    # set by forward() from topk_ids
        self.comm_sms = 16
        self._comm = None
        # Exchange over peer memory (DirectExchange): used for CUDA batches of at most
        # direct_max_tokens tokens per rank (0 = off; every rank must set the same value, it sizes
        # the exchange buffers).  Falls back to the all-to-all path when the buffers cannot be
        # mapped into all ranks.
        self.direct_max_tokens = 0
        # what comes back: "routes" = every route's row, written by the owners' down projection
        # into [tokens, topk, H] here and summed here in the single-GPU order; "partials" = one
        # partial row per token and rank, written by the owners' top-k combine
        self.direct_return = "routes"
        self._direct = {}
        self._direct_failed = None

    # -- index construction ---------------------------------------------------------------
    def plan(self, topk_ids: torch.Tensor, chunks: int = 1):
        """Which token goes to which rank.  Returns ``(tok_idx [S], send_counts [chunks * R],
        pos [M, R])``: rows to send ordered by (token chunk, rank, token); ``pos[m, r]`` = row
        of token m's partial result in the returned buffer, -1 if rank r owns none of its
        experts.  Token chunk c holds tokens ``[c * ceil(M / chunks), ...)``."""
        if topk_ids.is_cuda and self.world * chunks <= 255:
            return self._plan_cuda(topk_ids, chunks)
        return self._plan_torch(topk_ids, chunks)

    @staticmethod
    def chunk_tokens(m: int, chunks: int) -> int:
        return max((m + chunks - 1) // chunks, 1)

    def _plan_cuda(self, topk_ids: torch.Tensor, chunks: int = 1):
        """Same result as :meth:`_plan_torch` without a host synchronisation: "token m goes
        to rank r" is a route of token m to "expert" (chunk, r), so the layer's own stable sort
        (unit 1) yields the (chunk, rank, token) order, the counts and, as its inverse
        permutation, ``pos``."""
        from . import ops
        m = topk_ids.shape[0]
        routes = ops.ep_dest_ranks(topk_ids, self.num_experts, self.per_rank, self.world,
                                   self.chunk_tokens(m, chunks) if chunks > 1 else 0)
        dummy_w = torch.empty((m, self.world), dtype=torch.float32, device=topk_ids.device)
        pos = torch.empty((m, self.world), dtype=torch.int32, device=topk_ids.device)
        sorted_ids, _, _, _, counts, _ = ops.moe_sorting_ck(
            routes, dummy_w, self.world * chunks, None, None, 1, None, alloc_moe_buf=False,
            route_pos=pos)
        send_counts = counts[:self.world * chunks].long()
        # rows beyond the number of sent rows are cut by the caller once the counts are on the host
        tok_idx = (sorted_ids & 0xFFFFFF).long()
        return tok_idx, send_counts, pos

    def _plan_torch(self, topk_ids: torch.Tensor, chunks: int = 1):
        m = topk_ids.shape[0]
        dest = torch.div(topk_ids.long(), self.per_rank, rounding_mode="floor")
        valid = (topk_ids >= 0) & (topk_ids < self.num_experts)
        hit = torch.zeros((m, self.world + 1), dtype=torch.bool, device=topk_ids.device)
        hit.scatter_(1, torch.where(valid, dest, torch.full_like(dest, self.world)), True)
        hit = hit[:, :self.world]
        ct = self.chunk_tokens(m, chunks)
        chunk_of = torch.div(torch.arange(m, device=topk_ids.device), ct, rounding_mode="floor")
        # key (chunk, rank) per (token, rank) pair; a stable sort keeps tokens ascending
        tok, rank = hit.nonzero(as_tuple=True)
        key = chunk_of[tok] * self.world + rank
        order = torch.sort(key, stable=True).indices
        tok_idx, rank_idx, key = tok[order], rank[order], key[order]
        send_counts = torch.bincount(key, minlength=self.world * chunks)[:self.world * chunks]
        pos = torch.full((m, self.world), -1, dtype=torch.int32, device=topk_ids.device)
        pos[tok_idx, rank_idx] = torch.arange(tok_idx.numel(), dtype=torch.int32,
                                              device=topk_ids.device)
        return tok_idx, send_counts, pos

    def _exchange_counts(self, send_counts: torch.Tensor, chunks: int = 1):
        """All ranks learn how many rows every peer sends them per chunk.  Returns
        ``(send_split, recv_split)``: lists ``[chunk][rank]``.  One small all-to-all and the
        one host synchronisation of the dispatch."""
        world = self.world
        both = torch.empty((2, world, chunks), dtype=send_counts.dtype, device=send_counts.device)
        both[0].copy_(send_counts.view(chunks, world).t())      # grouped by destination rank
        dist.all_to_all_single(both[1], both[0], group=self.group)
        send_rc, recv_rc = both.tolist()                        # the host synchronisation
        send_split = [[send_rc[r][c] for r in range(world)] for c in range(chunks)]
        recv_split = [[recv_rc[r][c] for r in range(world)] for c in range(chunks)]
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

    # -- exchange over peer memory -------------------------------------------------------------
    def _quantiser(self, hidden_states, kwargs):
        """The quantiser the dispatch applies before the wire (None: rows travel as they are)."""
        w8a8 = kwargs.get("use_fp8_w8a8") or kwargs.get("use_int8_w8a8")
        if not (self.quantize_dispatch and w8a8 and hidden_states.is_cuda
                and hidden_states.dtype in (torch.float16, torch.bfloat16)
                and not kwargs.get("use_ue8m0")):
            return None, hidden_states.dtype, 0
        from . import ops
        qd = torch.float8_e4m3fn if kwargs.get("use_fp8_w8a8") else torch.int8
        if kwargs.get("per_channel_quant"):
            return (lambda x: ops.per_token_quant(x, quant_dtype=qd)), qd, 1
        if kwargs.get("block_shape") is not None:
            bn = kwargs["block_shape"][1]
            return (lambda x: ops.per_block_quant(x, bn, qd)), qd, hidden_states.shape[1] // bn
        return None, hidden_states.dtype, 0

    def _direct_exchange(self, hidden_states, topk, code_dtype, groups, out_dtype):
        """The exchange buffers for this configuration, mapped into all ranks on first use."""
        h = hidden_states.shape[1]
        row_bytes = h * torch.empty((), dtype=code_dtype).element_size()
        from .layer import _chunk_size
        # per-route return needs the local layer to take everything received as one chunk
        per_route = (self.direct_return == "routes"
                     and self.world * self.direct_max_tokens <= _chunk_size())
        hit = self._direct.get((self.direct_max_tokens, row_bytes, groups, topk, h, out_dtype,
                                per_route))
        if hit is not None:
            return hit
        ex = DirectExchange(self.world, self.rank, self.num_experts, self.direct_max_tokens,
                            row_bytes, groups, topk, h, out_dtype, hidden_states.device, code_dtype,
                            per_route)
        import torch.distributed._symmetric_memory as symm_mem
        buf = symm_mem.empty(ex.total_bytes, dtype=torch.uint8, device=hidden_states.device)
        handle = symm_mem.rendezvous(buf, self.group)
        buf[:ex.recv_off].zero_()
        ex.attach(buf, [int(p) for p in handle.buffer_ptrs])
        ex.handle = handle
        torch.cuda.synchronize(hidden_states.device)
        dist.barrier(group=self.group)        # every rank's header and flags are zero from here on
        self._direct[ex.key()] = ex
        return ex

    def forward_direct(self, hidden_states, w1_local, w2_local, topk_weights, topk_ids, **kwargs):
        """One step over peer memory; see :class:`DirectExchange`.  No host synchronisation."""
        m, h = hidden_states.shape
        out_dtype = kwargs.get("output_dtype") or hidden_states.dtype
        quant, code_dtype, groups = self._quantiser(hidden_states, kwargs)
        ex = self._direct_exchange(hidden_states, topk_ids.shape[1], code_dtype, groups, out_dtype)
        marks = []

        def mark(name):
            if self.profile:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        pos = ex.dispatch(hidden_states, topk_weights, topk_ids, quant)
        mark("dispatch")
        ex.barrier()
        mark("meet 1")
        ex.experts(w1_local, w2_local, **kwargs)
        mark("experts+return")
        ex.barrier()
        mark("meet 2")
        out = torch.empty((m, h), dtype=out_dtype, device=hidden_states.device)
        if ex.per_route:
            ex.combine_routes(topk_ids, out, float(kwargs.get("routed_scaling_factor") or 1.0))
        else:
            ex.combine(pos, out, self.combine_fn)
        mark("combine")
        self.last_stats = dict(mode="direct", routes=m * topk_ids.shape[1],
                               exchange_bytes=ex.total_bytes,
                               returned="routes" if ex.per_route else "partial rows")
        if marks:
            torch.cuda.synchronize()
            self.last_stats["ms"] = {b[0]: a[1].elapsed_time(b[1])
                                     for a, b in zip(marks[:-1], marks[1:])}
        return out

    # -- wire format -------------------------------------------------------------------------
    _a16 = staticmethod(_a16)

    def _wire_layout(self, row_bytes: int, groups: int, topk: int):
        """Byte offsets of the parts of a wire row: data, scales, ids, weights; total size."""
        return wire_layout(row_bytes, groups, topk)

    def _pack(self, x, x_scale, ids32, w32, tok_idx, send_ids, first, rows, wire):
        """Send buffer of one chunk: one wire row per (token, destination rank)."""
        row_bytes = x.shape[1] * x.element_size()
        groups = 0 if x_scale is None else x_scale.shape[1]
        o_scale, o_ids, o_w, total = wire
        out = torch.empty((rows, total), dtype=torch.uint8, device=x.device)
        if rows == 0:
            return out
        if x.is_cuda:
            from . import ops
            ops.ep_pack_rows(x, x_scale, ids32, w32, send_ids, first, rows, out)
            return out
        sel = tok_idx[first:first + rows]            # CPU ranks (tests): same bytes with torch ops
        out.zero_()
        out[:, :row_bytes] = x.index_select(0, sel).view(torch.uint8).reshape(rows, row_bytes)
        if groups:
            out[:, o_scale:o_scale + groups * 4] = \
                x_scale.index_select(0, sel).contiguous().view(torch.uint8).reshape(rows, -1)
        k = ids32.shape[1]
        out[:, o_ids:o_ids + 4 * k] = ids32.index_select(0, sel).view(torch.uint8).reshape(rows, -1)
        out[:, o_w:o_w + 4 * k] = w32.index_select(0, sel).view(torch.uint8).reshape(rows, -1)
        return out

    # -- the layer ----------------------------------------------------------------------------
    def num_chunks(self, m: int) -> int:
        """Token chunks of the pipelined exchange: chunk i+1 travels to the experts and chunk
        i-1 travels back while chunk i is computed."""
        if self.pipeline_chunks <= 1 or m < self.pipeline_min_tokens:
            return 1
        chunks = min(self.pipeline_chunks, 255 // self.world, m)
        if self.pipeline_rows_per_expert > 0 and self.topk_hint > 0:
            # every chunk streams the local expert weights once more, which only pays while the
            # GEMMs are bound by the tensor cores: keep enough rows per local expert per chunk
            rows = m * self.topk_hint * self.world // self.num_experts
            chunks = min(chunks, rows // self.pipeline_rows_per_expert)
        return max(1, chunks)

    def forward(self, hidden_states, w1_local, w2_local, topk_weights, topk_ids, **kwargs):
        m, h = hidden_states.shape
        if (self.direct_max_tokens and hidden_states.is_cuda and m <= self.direct_max_tokens
                and self._direct_failed is None and not kwargs.get("no_combine")
                and not kwargs.get("use_mxfp8") and not kwargs.get("use_mxfp4_w4a8")):
            try:
                self._direct_exchange(hidden_states, topk_ids.shape[1],
                                      *self._quantiser(hidden_states, kwargs)[1:],
                                      kwargs.get("output_dtype") or hidden_states.dtype)
            except Exception as exc:           # no peer mapping on this box: all-to-all path
                self._direct_failed = repr(exc)
            else:
                return self.forward_direct(hidden_states, w1_local, w2_local, topk_weights,
                                           topk_ids, **kwargs)
        # (the exchange over peer memory comes first: measured on 2 GPUs it is as fast as the
        # replicated-token path at 16 tokens per rank and 4-9 % faster from 256 on, and its
        # traffic does not grow with the number of ranks)
        if self.replicate_below and m * self.world <= self.replicate_below \
                and not kwargs.get("no_combine"):
            return self.forward_replicated(hidden_states, w1_local, w2_local, topk_weights,
                                           topk_ids, **kwargs)
        k = topk_ids.shape[1]
        world = self.world
        dev = hidden_states.device
        cuda = hidden_states.is_cuda
        self.topk_hint = k
        chunks = self.num_chunks(m)
        marks = []

        def mark(name):
            if self.profile and cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        tok_idx, send_counts, pos = self.plan(topk_ids, chunks)
        send_ids = tok_idx.to(torch.int32) if cuda else None

        # Quantise before the wire when the experts are w8a8: the rows then cross NVLink as
        # 8-bit codes + scales instead of 16-bit values, and the local layer takes them as
        # pre-quantised input (same codes it would have produced itself).  Enqueued before the
        # counts are read back, so the device works while the host waits for them.
        out_dtype = kwargs.get("output_dtype") or hidden_states.dtype
        x, x_scale = hidden_states, None
        w8a8 = kwargs.get("use_fp8_w8a8") or kwargs.get("use_int8_w8a8")
        if (self.quantize_dispatch and w8a8 and cuda
                and hidden_states.dtype in (torch.float16, torch.bfloat16)
                and not kwargs.get("use_ue8m0")):
            from . import ops
            qd = torch.float8_e4m3fn if kwargs.get("use_fp8_w8a8") else torch.int8
            if kwargs.get("per_channel_quant"):
                x, x_scale = ops.per_token_quant(hidden_states, quant_dtype=qd)
            elif kwargs.get("block_shape") is not None:
                x, x_scale = ops.per_block_quant(hidden_states, kwargs["block_shape"][1], qd)
        if x_scale is not None:
            x_scale = x_scale.reshape(m, -1)
        x = x.contiguous()
        ids32 = topk_ids.to(torch.int32).contiguous()
        w32 = topk_weights.to(torch.float32).contiguous()
        row_bytes = x.shape[1] * x.element_size()
        groups = 0 if x_scale is None else x_scale.shape[1]
        wire = self._wire_layout(row_bytes, groups, k)
        o_scale, o_ids, o_w, wire_bytes = wire

        send_split, recv_split = self._exchange_counts(send_counts, chunks)
        mark("plan+counts")

        n_send = [sum(v) for v in send_split]
        n_recv = [sum(v) for v in recv_split]
        first = [sum(n_send[:c]) for c in range(chunks)]
        total_send = sum(n_send)
        back = torch.empty((total_send, h), dtype=out_dtype, device=dev)
        main = torch.cuda.current_stream(dev) if cuda else None
        comm = self._comm_stream(dev) if cuda and chunks > 1 else None
        keep = []                                   # buffers shared between the two streams

        def exchange(dst, src, dst_split, src_split, after):
            """All-to-all of one chunk; on GPUs with several chunks it runs on the exchange
            stream once `after` (an event of the main stream) has happened."""
            keep.extend((dst, src))
            if comm is None:
                dist.all_to_all_single(dst, src, dst_split, src_split, group=self.group)
                return None
            with torch.cuda.stream(comm):
                comm.wait_event(after)
                work = dist.all_to_all_single(dst, src, dst_split, src_split, group=self.group,
                                              async_op=True)
            return work

        def event():
            ev = torch.cuda.Event()
            ev.record(main)
            return ev

        # ---- dispatch of every chunk is enqueued first: chunk c + 1 crosses the wire while
        # chunk c is computed
        recv_bufs, d_work = [], []
        for c in range(chunks):
            send_buf = self._pack(x, x_scale, ids32, w32, tok_idx, send_ids, first[c], n_send[c],
                                  wire)
            recv_buf = torch.empty((n_recv[c], wire_bytes), dtype=torch.uint8, device=dev)
            d_work.append(exchange(recv_buf, send_buf, recv_split[c], send_split[c],
                                   event() if comm is not None else None))
            recv_bufs.append(recv_buf)
        mark("dispatch")

        local_kwargs = dict(kwargs)
        if x_scale is not None:
            local_kwargs["output_dtype"] = out_dtype
        r_work = []
        limit_sms = comm is not None and self.comm_sms > 0
        if limit_sms:
            from . import ops
            ops.set_gemm_sm_reserve(self.comm_sms)   # leave SMs to the exchange kernels
        try:
            for c in range(chunks):
                if d_work[c] is not None:
                    d_work[c].wait()                 # main stream waits for chunk c's rows
                rb = recv_bufs[c]
                if n_recv[c]:
                    r_x = rb[:, :row_bytes].view(x.dtype)
                    r_ids = rb[:, o_ids:o_ids + 4 * k].view(torch.int32)
                    r_w = rb[:, o_w:o_w + 4 * k].view(torch.float32)
                    r_ids, r_w = r_ids.contiguous(), r_w.contiguous()
                    if x_scale is None or not cuda:
                        # 16-bit rows are quantised (or used) by kernels that read dense rows;
                        # pre-quantised rows are gathered from the receive buffer in place
                        r_x = r_x.contiguous()
                    if x_scale is not None:
                        local_kwargs["a1_scale"] = rb[:, o_scale:o_scale + 4 * groups].view(
                            torch.float32)
                    partial = self.local_fn(r_x, w1_local, w2_local, r_w, r_ids,
                                            expert_map=self.expert_map,
                                            global_num_experts=self.num_experts, **local_kwargs)
                else:
                    partial = torch.empty((0, h), dtype=out_dtype, device=dev)
                r_work.append(exchange(back[first[c]:first[c] + n_send[c]], partial.contiguous(),
                                       send_split[c], recv_split[c],
                                       event() if comm is not None else None))
        finally:
            if limit_sms:
                ops.set_gemm_sm_reserve(0)
        mark("experts")
        for w in r_work:
            if w is not None:
                w.wait()
        mark("return")
        out = torch.empty((m, h), dtype=out_dtype, device=dev)
        self.combine_fn(back, pos, out)
        mark("combine")
        if comm is not None:
            comm.wait_stream(main)      # buffers handed to the exchange stream die in order
        self.last_stats = dict(rows_sent=total_send, rows_received=sum(n_recv), routes=m * k,
                               chunks=chunks)
        if marks:
            torch.cuda.synchronize()
            self.last_stats["ms"] = {b[0]: a[1].elapsed_time(b[1])
                                     for a, b in zip(marks[:-1], marks[1:])}
        return out

    def _comm_stream(self, device):
        if self._comm is None:
            self._comm = torch.cuda.Stream(device=device)
        return self._comm
