"""Python faces of the C-ABI kernels (allocation, argument checks, stream lookup).

Names and return conventions follow the reference helpers they replace
(reference paths are relative to the reference project root):

* ``moe_sorting_ck``        -- boltops/fused_moe/triton/fused_moe.py:441-485
* ``moe_align_block_size``  -- boltops/fused_moe/triton/fused_moe.py:330-439
* ``per_token_quant`` / ``per_block_quant`` -- boltops/fused_moe/triton/moe_compat.py:55-106
* ``moe_sum``               -- boltops/fused_moe/triton/fused_moe.py:134-188
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from .. import _cabi
from .._cabi import check, dtype_code, ptr, stream_of

SORT_UNIT = 128  # row-tile of the grouped GEMM == padding unit of the sort

_launches = 0   # kernels launched through this module (bookkeeping for benchmarks)


def launch_count() -> int:
    """Number of CUDA kernels this module has launched so far in this process."""
    return _launches


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("boltops_b200 kernels need CUDA tensors (there is no CPU path)")


def sort_launches(lib, m: int, topk: int, num_experts: int) -> int:
    """Kernels one sort launches: one CTA does everything for small inputs, three kernels else."""
    return 1 if lib.bolt_moe_sort_workspace_bytes(m, topk, num_experts) <= 16 else 3


def ceil_to(x: int, m: int) -> int:
    return (x + m - 1) // m * m


# ---------------------------------------------------------------------------
# sort
# ---------------------------------------------------------------------------
def moe_sorting_ck(topk_ids: torch.Tensor, topk_weights: torch.Tensor, num_experts: int,
                   model_dim: Optional[int] = None, moebuf_dtype: Optional[torch.dtype] = None,
                   block_size: int = 32, expert_mask: Optional[torch.Tensor] = None,
                   alloc_moe_buf: bool = True, route_pos: Optional[torch.Tensor] = None,
                   segment_rows: int = 0):
    """CK-format sort.  Returns ``(sorted_ids, sorted_weights, sorted_expert_ids,
    num_valid_ids, tokens_positions_per_expert, moe_buf)`` like the reference.

    ``sorted_ids``/``sorted_weights`` are allocated with the capacity rounded up to
    a multiple of ``block_size`` so that the last row tile is always addressable.
    ``route_pos`` (optional int32 ``[tokens, topk]``) receives every route's position in
    the sorted order (-1 for routes to masked experts).  With ``segment_rows > 0`` the tuple
    gains ``(segments [S, 4] int32, num_segments [1] int32)``: every expert's live rows cut
    into runs of at most ``segment_rows`` rows (``{expert, first row, rows, 0}``), the work
    list of the tile-pair GEMM schedule (``segment_rows`` = two row tiles).
    """
    _require_cuda(topk_ids, topk_weights, expert_mask)
    if topk_ids.dim() != 2 or topk_weights.shape != topk_ids.shape:
        raise AssertionError("topk shape mismatch")
    if topk_weights.dtype != torch.float32:
        raise AssertionError("topk_weights must be float32")
    lib = _cabi.load()
    dev = topk_ids.device
    m, topk = topk_ids.shape
    if topk_ids.dtype != torch.int32:
        topk_ids = topk_ids.to(torch.int32)
    topk_ids = topk_ids.contiguous()
    topk_weights = topk_weights.contiguous()
    if expert_mask is not None:
        expert_mask = expert_mask.to(torch.int32).contiguous()
    cap = m * topk + num_experts * block_size - topk
    cap_alloc = ceil_to(max(cap, 0), block_size)
    blocks = cap_alloc // block_size
    # one allocation for every int32 / fp32 output and the scratch (a decode-sized layer is bound
    # by host time per call; each separate allocation costs microseconds)
    ws_bytes = lib.bolt_moe_sort_workspace_bytes(m, topk, num_experts)
    max_segments = (min(num_experts, m * topk) + (m * topk) // segment_rows) if segment_rows > 0 else 0
    n_blocks = max(blocks, 1)
    sizes = (cap_alloc, cap_alloc, n_blocks, 2 * num_experts, 4, 4 * max(max_segments, 1) if
             segment_rows > 0 else 0, 4 if segment_rows > 0 else 0, (ws_bytes + 3) // 4)
    offs = [0]
    for n in sizes:
        offs.append(offs[-1] + ceil_to(n, 4))                 # 16-byte aligned parts
    buf = torch.empty(offs[-1], dtype=torch.int32, device=dev)
    sorted_ids = buf[offs[0]:offs[0] + cap_alloc]
    sorted_weights = buf[offs[1]:offs[1] + cap_alloc].view(torch.float32)
    sorted_expert_ids = buf[offs[2]:offs[2] + n_blocks]
    positions = buf[offs[3]:offs[3] + 2 * num_experts]
    num_valid = buf[offs[4]:offs[4] + 1]
    segments = num_segments = None
    if segment_rows > 0:
        segments = buf[offs[5]:offs[5] + 4 * max(max_segments, 1)].view(-1, 4)
        num_segments = buf[offs[6]:offs[6] + 1]
    ws = buf[offs[7]:offs[7] + (ws_bytes + 3) // 4]
    moe_buf = None
    if alloc_moe_buf and model_dim is not None and moebuf_dtype is not None:
        moe_buf = torch.empty((m, model_dim), dtype=moebuf_dtype, device=dev)
    with _cabi.on_device(dev):
        check(lib.bolt_moe_sort_ck(
            ptr(topk_ids), ptr(topk_weights), ptr(expert_mask), m, topk, num_experts, block_size,
            ptr(sorted_ids), ptr(sorted_weights), ptr(sorted_expert_ids), ptr(positions),
            ptr(num_valid), ptr(route_pos), ptr(segments), ptr(num_segments), segment_rows,
            ptr(moe_buf), 0 if moe_buf is None else moe_buf.numel() * moe_buf.element_size(),
            ptr(ws), ws_bytes, stream_of(topk_ids)))
    _count(1 if ws_bytes <= 16 else 3)
    if segment_rows > 0:
        return (sorted_ids, sorted_weights, sorted_expert_ids, num_valid, positions, moe_buf,
                segments, num_segments)
    return sorted_ids, sorted_weights, sorted_expert_ids, num_valid, positions, moe_buf


def relabel_tiles(sorted_expert_ids: torch.Tensor, expert_map: torch.Tensor) -> torch.Tensor:
    """Per-tile expert ids of a masked CK sort -> local expert ids under an ARBITRARY
    ``expert_map``.  The masked sort numbers the enabled experts densely in ascending global
    order; a map such as ``[1, -1, 0]`` (the MX paths of the reference take any map, through
    ``moe_align_block_size``: boltops/fused_moe/triton/fused_moe.py:1116-1117,436-437) stores
    them in another order.  Entries of tiles beyond the padded total are arbitrary and stay
    harmless (clamped before the look-up).  No host synchronisation."""
    emap = expert_map.to(torch.int32)
    order = torch.argsort((emap < 0).to(torch.int8), stable=True)      # enabled experts first
    local_of_label = emap[order]
    idx = sorted_expert_ids.clamp(0, emap.numel() - 1).long()
    return local_of_label[idx].contiguous()


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int,
                         expert_map: Optional[torch.Tensor] = None
                         ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """vLLM-format sort: ``(sorted_token_ids, expert_ids, num_tokens_post_padded)``."""
    _require_cuda(topk_ids, expert_map)
    lib = _cabi.load()
    dev = topk_ids.device
    ids = topk_ids.to(torch.int32).contiguous()
    numel = ids.numel()
    cap = numel + num_experts * (block_size - 1)
    blocks = (cap + block_size - 1) // block_size
    sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(blocks, dtype=torch.int32, device=dev)
    num_post = torch.empty(1, dtype=torch.int32, device=dev)
    if expert_map is not None:
        expert_map = expert_map.to(torch.int32).contiguous()
    ws_bytes = lib.bolt_moe_sort_workspace_bytes(numel, 1, num_experts)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with _cabi.on_device(dev):
        check(lib.bolt_moe_align_block_size(
            ptr(ids), numel, num_experts, block_size, ptr(expert_map), ptr(sorted_ids),
            ptr(expert_ids), ptr(num_post), ptr(ws), ws_bytes, stream_of(ids)))
    _count(1 if ws_bytes <= 16 else 3)
    return sorted_ids, expert_ids, num_post


# ---------------------------------------------------------------------------
# quantisation
# ---------------------------------------------------------------------------
def quant_rows(x: torch.Tensor, quant_dtype: torch.dtype, group: Optional[int] = None,
               scale_ue8m0: bool = False, group_major: bool = False
               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dynamic quantisation of a 2-D tensor per row (``group=None``) or per
    ``1 x group`` block.  Returns ``(q, scales[rows, cols/group])``, or with ``group_major``
    ``(q, scales[cols/group, rows])`` -- the layout the grouped GEMM reads per K block."""
    _require_cuda(x)
    if x.dim() != 2:
        raise ValueError("quant_rows expects a 2-D tensor")
    assert x.is_contiguous(), "x_in must be contiguous"
    lib = _cabi.load()
    rows, cols = x.shape
    g = cols if group is None else group
    q = torch.empty((rows, cols), dtype=quant_dtype, device=x.device)
    shape = (cols // g, rows) if group_major else (rows, cols // g)
    scales = torch.empty(shape, dtype=torch.float32, device=x.device)
    with _cabi.on_device(x.device):
        check(lib.bolt_quant_rows(ptr(x), dtype_code(x.dtype), rows, cols, g,
                                  dtype_code(quant_dtype), int(scale_ue8m0), ptr(q), ptr(scales),
                                  rows if group_major else 0, stream_of(x)))
    _count()
    return q, scales


def per_token_quant(x: torch.Tensor, scale: Optional[torch.Tensor] = None,
                    quant_dtype: torch.dtype = torch.int8, scale_ue8m0: bool = False):
    """Per-token dynamic quantisation; scale has shape ``[*x.shape[:-1], 1]``."""
    if scale is not None:
        raise ValueError("unsupported: static per token quant")
    shape = x.shape
    q, s = quant_rows(x.reshape(-1, shape[-1]), quant_dtype, None, scale_ue8m0)
    return q.view(shape), s.view(*shape[:-1], 1)


def per_block_quant(x: torch.Tensor, block_n: int = 128, quant_dtype: torch.dtype = torch.int8,
                    scale_ue8m0: bool = False, group_major: bool = False):
    """1 x ``block_n`` group quantisation of a 2-D tensor: ``(q[m,n], s[m,n/block_n])``
    (``s[n/block_n, m]`` with ``group_major``)."""
    assert x.shape[-1] % block_n == 0, f"block size {block_n} not match {x.shape[-1]}"
    return quant_rows(x, quant_dtype, block_n, scale_ue8m0, group_major)


# ---------------------------------------------------------------------------
# gather / combine
# ---------------------------------------------------------------------------
def gather_rows(src: torch.Tensor, sorted_ids: torch.Tensor, num_valid: torch.Tensor,
                capacity: int, src_scale: Optional[torch.Tensor] = None):
    """Copy token rows into the expert-sorted padded layout.

    Returns ``(dst[capacity, cols], dst_scale)`` where ``dst_scale`` is ``None``,
    ``[capacity]`` (one scale per row) or ``[groups, capacity]`` (group-major)."""
    lib = _cabi.load()
    m, cols = src.shape
    row_bytes = cols * src.element_size()
    # rows (and their scales) may sit inside wider records: only the last dimension must be dense
    assert src.stride(1) == 1, "gather_rows: the last dimension of src must be contiguous"
    src_stride = src.stride(0) * src.element_size() if m > 1 else row_bytes
    dst = torch.empty((capacity, cols), dtype=src.dtype, device=src.device)
    dst_scale = None
    groups = 0
    ld = 0
    scale_stride = 0
    if src_scale is not None:
        if src_scale.dim() != 2 or src_scale.shape[0] != m or src_scale.stride(1) != 1:
            src_scale = src_scale.reshape(m, -1).contiguous()
        groups = src_scale.shape[1]
        scale_stride = src_scale.stride(0) if m > 1 else groups
        if groups == 1:
            dst_scale = torch.empty(capacity, dtype=torch.float32, device=src.device)
            ld = capacity
        else:
            dst_scale = torch.empty((groups, capacity), dtype=torch.float32, device=src.device)
            ld = capacity
    with _cabi.on_device(src.device):
        check(lib.bolt_gather_rows(ptr(src), m, row_bytes, src_stride, ptr(src_scale),
                                   scale_stride, groups, ptr(sorted_ids), ptr(num_valid),
                                   capacity, ptr(dst), ptr(dst_scale), ld, stream_of(src)))
    _count()
    return dst, dst_scale


def quant_scatter_rows(x: torch.Tensor, group: int, q_dtype: torch.dtype, route_pos: torch.Tensor,
                       sorted_ids: torch.Tensor, num_valid: torch.Tensor, capacity: int,
                       scale_ue8m0: bool = False, token_order: bool = False):
    """Quantise ``x`` [M, cols] per 1 x ``group`` block and write every token to the sorted rows
    ``route_pos[m, k] >= 0`` in one pass.  Returns ``(dst [capacity, cols], dst_scale
    [cols/group, capacity])``; tile-padding rows are zero.  ``token_order``: for a GEMM that
    gathers its rows itself -- ``dst`` is ``[M, cols]``, every token once in token order; the
    scales still go to the sorted positions."""
    _require_cuda(x, route_pos, sorted_ids, num_valid)
    lib = _cabi.load()
    x = x.contiguous()
    m, cols = x.shape
    assert route_pos.dtype == torch.int32 and route_pos.is_contiguous() and route_pos.shape[0] == m
    dst = torch.empty((m if token_order else capacity, cols), dtype=q_dtype, device=x.device)
    dst_scale = torch.empty((cols // group, capacity), dtype=torch.float32, device=x.device)
    with _cabi.on_device(x.device):
        check(lib.bolt_quant_scatter_rows(ptr(x), dtype_code(x.dtype), m, cols, group,
                                          dtype_code(q_dtype), int(scale_ue8m0), ptr(route_pos),
                                          route_pos.shape[1], ptr(sorted_ids), ptr(num_valid),
                                          capacity, ptr(dst), ptr(dst_scale), capacity,
                                          int(token_order), stream_of(x)))
    _count()
    return dst, dst_scale


def mx_quant_rows(x: torch.Tensor, *, gated: bool = False, alpha: float = 1.0, beta: float = 0.0,
                  limit: Optional[float] = None, want_codes: bool = True,
                  deq_dtype: Optional[torch.dtype] = None):
    """MX e4m3 quantisation of ``x`` [rows, cols] (or [rows, 2*cols] = [gate | up] with the split
    gated activation fused in front).  Returns ``(q, scales, deq)``: e4m3 codes, E8M0 bytes
    [rows, cols/32], and the dequantised values in ``deq_dtype`` (each ``None`` if not asked for)."""
    _require_cuda(x)
    lib = _cabi.load()
    x = x.contiguous()
    rows = x.shape[0]
    cols = x.shape[1] // 2 if gated else x.shape[1]
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device) if want_codes else None
    s = torch.empty((rows, cols // 32), dtype=torch.uint8, device=x.device) if want_codes else None
    deq = torch.empty((rows, cols), dtype=deq_dtype, device=x.device) if deq_dtype is not None else None
    with _cabi.on_device(x.device):
        check(lib.bolt_mx_quant_rows(ptr(x), dtype_code(x.dtype), rows, cols, int(gated),
                                     float(alpha), float(beta), int(limit is not None),
                                     float(limit or 0.0), ptr(q), ptr(s), ptr(deq),
                                     dtype_code(deq_dtype) if deq_dtype is not None else _cabi.BF16,
                                     stream_of(x)))
    _count()
    return q, s, deq


def mx_dequant_rows(q: torch.Tensor, scales: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``q`` [..., cols] e4m3 with E8M0 bytes [..., cols/32] → floats ``q * 2^(byte-127)``."""
    _require_cuda(q, scales)
    lib = _cabi.load()
    q = q.contiguous()
    scales = scales.contiguous()
    cols = q.shape[-1]
    rows = q.numel() // cols
    assert scales.dtype == torch.uint8 and scales.numel() == rows * (cols // 32)
    out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
    with _cabi.on_device(q.device):
        check(lib.bolt_mx_dequant_rows(ptr(q), ptr(scales), rows, cols, ptr(out),
                                       dtype_code(out_dtype), stream_of(q)))
    _count()
    return out


def mx_sf_layout(scales: torch.Tensor, dst_rows: int, row_ids: Optional[torch.Tensor] = None,
                 num_valid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """E8M0 bytes [rows, K/32] → 512-byte tiles [dst_rows/128, K/128, 512] for the MX GEMM kind
    (optionally gathering rows through the sorted ids)."""
    _require_cuda(scales)
    lib = _cabi.load()
    scales = scales.contiguous()
    rows, sf_cols = scales.shape
    assert scales.dtype == torch.uint8 and sf_cols % 4 == 0 and dst_rows % 128 == 0
    dst = torch.empty((dst_rows // 128, sf_cols // 4, 512), dtype=torch.uint8, device=scales.device)
    with _cabi.on_device(scales.device):
        check(lib.bolt_mx_sf_layout(ptr(scales), rows, sf_cols, ptr(row_ids), ptr(num_valid),
                                    dst_rows, ptr(dst), stream_of(scales)))
    _count()
    return dst


def moe_sum(input_tensor: torch.Tensor, output_tensor: torch.Tensor,
            routed_scaling_factor: float = 1.0,
            router_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``output[m] = cast(scale * sum_k f32(input[m, k]) [* router_weights[m, k]])``."""
    _require_cuda(input_tensor, output_tensor)
    m, topk, n = input_tensor.shape
    assert output_tensor.dtype in (torch.float16, torch.bfloat16, torch.float32)
    assert input_tensor.is_contiguous()
    assert output_tensor.is_contiguous()
    assert input_tensor.shape[0] == output_tensor.shape[0]
    assert input_tensor.shape[2] == output_tensor.shape[1]
    if router_weights is not None:
        router_weights = router_weights.to(torch.float32).contiguous()
    lib = _cabi.load()
    with _cabi.on_device(input_tensor.device):
        check(lib.bolt_moe_sum(ptr(input_tensor), dtype_code(input_tensor.dtype),
                               ptr(output_tensor), dtype_code(output_tensor.dtype), m, topk, n,
                               float(routed_scaling_factor), ptr(router_weights),
                               stream_of(input_tensor)))
    _count()
    return output_tensor


def gather_sum(src: torch.Tensor, pos: torch.Tensor, out: torch.Tensor,
               scale: float = 1.0) -> torch.Tensor:
    """``out[m] = cast(scale * sum_j f32(src[pos[m, j]]))`` over ``pos[m, j] >= 0`` (j ascending)."""
    _require_cuda(src, pos, out)
    lib = _cabi.load()
    m, slots = pos.shape
    assert pos.dtype == torch.int32 and pos.is_contiguous()
    assert src.is_contiguous() and out.is_contiguous()
    with _cabi.on_device(out.device):
        check(lib.bolt_moe_gather_sum(ptr(src), dtype_code(src.dtype), ptr(pos), ptr(out),
                                      dtype_code(out.dtype), m, slots, out.shape[1], float(scale),
                                      stream_of(out)))
    _count()
    return out


def gather_sum_to_peers(src: torch.Tensor, pos: torch.Tensor, scale: float, *, seg_rows: int,
                        seg_ptrs: torch.Tensor, hdr: torch.Tensor, first_row: int = 0) -> None:
    """``gather_sum`` whose row ``first_row + i`` (segment ``s = row // seg_rows``, ``q = row %
    seg_rows``) goes to row ``hdr[s, 1] + q`` of the region at address ``seg_ptrs[s]`` -- possibly
    another rank's memory -- and is skipped when ``q >= hdr[s, 0]``."""
    _require_cuda(src, pos, seg_ptrs, hdr)
    lib = _cabi.load()
    m, slots = pos.shape
    assert pos.dtype == torch.int32 and pos.is_contiguous() and src.is_contiguous()
    assert seg_ptrs.dtype == torch.int64 and hdr.dtype == torch.int32 and hdr.is_contiguous()
    with _cabi.on_device(src.device):
        check(lib.bolt_moe_gather_sum_to_peers(ptr(src), dtype_code(src.dtype), ptr(pos), m, slots,
                                               src.shape[1], float(scale), seg_rows, ptr(seg_ptrs),
                                               ptr(hdr), first_row, stream_of(src)))
    _count()


def ep_dispatch_rows(data: torch.Tensor, scales: Optional[torch.Tensor], topk_ids: torch.Tensor,
                     topk_weights: torch.Tensor, send_ids: torch.Tensor, counts: torch.Tensor,
                     me: int, seg_rows: int, peers: torch.Tensor, hdr_off: int, recv_off: int,
                     wire_bytes: int) -> None:
    """Write this rank's wire rows (send order ``send_ids``, per-destination ``counts``, both on
    the device) into segment ``me`` of every destination's receive region and the
    ``{count, first return row}`` pair into its header (``bolt_ep_dispatch_rows``)."""
    _require_cuda(data, topk_ids, topk_weights, send_ids, counts, peers)
    lib = _cabi.load()
    assert data.is_contiguous() and topk_ids.is_contiguous() and topk_weights.is_contiguous()
    assert topk_ids.dtype == torch.int32 and topk_weights.dtype == torch.float32
    assert send_ids.dtype == torch.int32 and counts.dtype == torch.int32
    assert peers.dtype == torch.int64
    groups = 0
    if scales is not None:
        scales = scales.reshape(data.shape[0], -1).contiguous()
        groups = scales.shape[1]
    world = peers.numel()
    max_rows = data.shape[0] * min(world, topk_ids.shape[1])
    with _cabi.on_device(data.device):
        check(lib.bolt_ep_dispatch_rows(ptr(data), data.shape[1] * data.element_size(), ptr(scales),
                                        groups, ptr(topk_ids), ptr(topk_weights), topk_ids.shape[1],
                                        ptr(send_ids), ptr(counts), world, me, max_rows, seg_rows,
                                        ptr(peers), hdr_off, recv_off, wire_bytes,
                                        ptr(device_status(data.device)), stream_of(data)))
    _count()


def ep_unpack_routes(recv: torch.Tensor, ids_off: int, wts_off: int, topk: int, seg_rows: int,
                     nseg: int, hdr: torch.Tensor, src_off: Optional[int] = None):
    """Dense ``(topk_ids, topk_weights)`` of all ``nseg * seg_rows`` rows of a receive region
    (``recv`` uint8 ``[nseg * seg_rows, wire_bytes]``); rows a segment does not hold get id -1.
    With ``src_off`` a third tensor: every row's token index on the rank it came from."""
    _require_cuda(recv, hdr)
    lib = _cabi.load()
    assert recv.dtype == torch.uint8 and recv.is_contiguous() and hdr.dtype == torch.int32
    rows = nseg * seg_rows
    ids = torch.empty((rows, topk), dtype=torch.int32, device=recv.device)
    wts = torch.empty((rows, topk), dtype=torch.float32, device=recv.device)
    src = torch.empty((rows,), dtype=torch.int32, device=recv.device) if src_off is not None else None
    with _cabi.on_device(recv.device):
        check(lib.bolt_ep_unpack_routes(ptr(recv), recv.shape[1], ids_off, wts_off, topk, seg_rows,
                                        nseg, ptr(hdr), ptr(ids), ptr(wts), src_off or 0, ptr(src),
                                        stream_of(recv)))
    _count()
    return (ids, wts, src) if src_off is not None else (ids, wts)


def ep_barrier(peers: torch.Tensor, me: int, flag_off: int) -> None:
    """All ranks of the exchange meet on the current stream (bounded wait; see
    ``bolt_ep_barrier``).  One process per GPU only."""
    _require_cuda(peers)
    lib = _cabi.load()
    with _cabi.on_device(peers.device):
        check(lib.bolt_ep_barrier(ptr(peers), peers.numel(), me, flag_off,
                                  ptr(device_status(peers.device)), stream_of(peers)))
    _count()


def ep_dest_ranks(topk_ids: torch.Tensor, num_experts: int, experts_per_rank: int,
                  world: int, chunk_tokens: int = 0) -> torch.Tensor:
    """``routes[t, r] = r`` if one of token t's experts lives on rank r, else -1 (int32 [M, world]);
    with ``chunk_tokens`` the value is ``(t // chunk_tokens) * world + r``."""
    _require_cuda(topk_ids)
    lib = _cabi.load()
    ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
    ids = ids.contiguous()
    m, k = ids.shape
    routes = torch.empty((m, world), dtype=torch.int32, device=ids.device)
    with _cabi.on_device(ids.device):
        check(lib.bolt_ep_dest_ranks(ptr(ids), m, k, num_experts, experts_per_rank, world,
                                     chunk_tokens, ptr(routes), stream_of(ids)))
    _count()
    return routes


def ep_wire_row_bytes(row_bytes: int, groups: int, topk: int) -> int:
    """Bytes of one expert-parallel wire row: data, scales, top-k ids, top-k weights (each part
    padded to 16 bytes)."""
    return int(_cabi.load().bolt_ep_wire_row_bytes(row_bytes, groups, topk))


def ep_pack_rows(data: torch.Tensor, scales: Optional[torch.Tensor], topk_ids: torch.Tensor,
                 topk_weights: torch.Tensor, send_ids: torch.Tensor, first: int, rows: int,
                 out: torch.Tensor) -> None:
    """Fill ``out[:rows]`` (uint8 ``[*, wire_row_bytes]``) with the wire rows of the tokens
    ``send_ids[first:first+rows] & 0xFFFFFF``: one kernel for the send buffer of a chunk."""
    _require_cuda(data, scales, topk_ids, topk_weights, send_ids, out)
    lib = _cabi.load()
    assert data.is_contiguous() and topk_ids.is_contiguous() and topk_weights.is_contiguous()
    assert topk_ids.dtype == torch.int32 and topk_weights.dtype == torch.float32
    assert out.dtype == torch.uint8 and out.stride(1) == 1
    groups = 0
    if scales is not None:
        scales = scales.reshape(data.shape[0], -1).contiguous()
        groups = scales.shape[1]
    with _cabi.on_device(data.device):
        check(lib.bolt_ep_pack_rows(ptr(data), data.shape[1] * data.element_size(), ptr(scales),
                                    groups, ptr(topk_ids), ptr(topk_weights), topk_ids.shape[1],
                                    ptr(send_ids), first, rows, ptr(out), out.stride(0),
                                    stream_of(data)))
    _count()


# ---------------------------------------------------------------------------
# grouped GEMM
# ---------------------------------------------------------------------------
_status_words = {}
_gemm_sm_reserve = 0


def set_gemm_sm_reserve(sms: int) -> None:
    """Number of SMs the grouped GEMMs leave free (0 = none).  The expert-parallel layer sets it
    while exchange kernels run next to the GEMMs: a persistent GEMM with one CTA on every SM would
    make a concurrently launched collective wait for it."""
    global _gemm_sm_reserve
    _gemm_sm_reserve = max(int(sms), 0)



def device_status(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that the grouped GEMM and the expert-parallel exchange kernels set
    when a bounded device-side wait expired (0 = healthy).  Reading it synchronises; kernels
    never do."""
    key = torch.device(device).index or 0
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


def check_device_status(device: torch.device) -> None:
    code = int(device_status(device).item())
    if code != 0:
        device_status(device).zero_()
        raise _cabi.BoltError(f"a kernel reported an expired device-side wait (code {code}: 1-5 grouped "
                              f"GEMM, 20 exchange barrier, 21 exchange segment overflow)")


def grouped_gemm(*, kind: int, epilogue: int, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
                 sorted_expert_ids: torch.Tensor, num_valid: torch.Tensor,
                 a_scale: Optional[torch.Tensor] = None, a_scale_ld: int = 0,
                 b_scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                 c_scale: Optional[torch.Tensor] = None, c_scale_ld: int = 0,
                 mid_dtype: Optional[torch.dtype] = None, scatter: bool = False,
                 num_tokens: int = 0, topk: int = 1, mul_routed_weight: bool = False,
                 sorted_ids: Optional[torch.Tensor] = None,
                 sorted_weights: Optional[torch.Tensor] = None, sm_count: int = 0,
                 act_alpha: float = 1.0, act_beta: float = 0.0,
                 act_limit: Optional[float] = None, segments: Optional[torch.Tensor] = None,
                 num_segments: Optional[torch.Tensor] = None,
                 a_gather: bool = False, scatter_src: Optional[torch.Tensor] = None,
                 scatter_seg_off: Optional[torch.Tensor] = None, scatter_seg_rows: int = 0) -> None:
    """One grouped expert GEMM launch (see ``bolt_grouped_gemm``).  With ``segments`` (from
    ``moe_sorting_ck(..., segment_rows=PAIR_SEGMENT_ROWS)``) the tile-pair schedule runs.  With
    ``a_gather`` the row operand ``a`` is in TOKEN order and the kernel gathers its rows through
    ``sorted_ids`` (padding positions read zeros).  ``scatter_src`` / ``scatter_seg_off`` /
    ``scatter_seg_rows``: scattered rows go to per-segment regions (see ``bolt_gemm_args``)."""
    lib = _cabi.load()
    args = _cabi.GemmArgs()
    args.kind = kind
    args.epilogue = epilogue
    if a_gather:
        assert a.stride(1) == 1 and sorted_ids is not None
        args.a_gather = 1
        args.a_rows = a.shape[0]
        args.a_row_bytes = a.stride(0) * a.element_size()
        args.capacity = sorted_ids.shape[0]
    else:
        args.capacity = a.shape[0]
    args.n = b.shape[1]
    args.k = a.shape[1]            # (packed 4-bit weights hold two K elements per byte)
    args.num_experts = b.shape[0]
    args.a = ptr(a)
    args.b = ptr(b)
    args.a_scale = ptr(a_scale)
    args.a_scale_ld = a_scale_ld
    args.b_scale = ptr(b_scale)
    args.bias = ptr(bias)
    args.bias_dtype = dtype_code(bias.dtype) if bias is not None else _cabi.F32
    args.c = ptr(c)
    args.c_dtype = dtype_code(c.dtype)
    args.mid_dtype = dtype_code(mid_dtype) if mid_dtype is not None else _cabi.F32
    args.c_ld = c.stride(-2) if c.dim() >= 2 else c.shape[-1]
    args.c_scale = ptr(c_scale)
    args.c_scale_ld = c_scale_ld
    args.scatter = int(scatter)
    args.num_tokens = num_tokens
    args.topk = topk
    args.mul_routed_weight = int(mul_routed_weight)
    args.sorted_ids = ptr(sorted_ids)
    args.sorted_weights = ptr(sorted_weights)
    args.sorted_expert_ids = ptr(sorted_expert_ids)
    args.num_valid_ids = ptr(num_valid)
    args.status = ptr(device_status(a.device))
    if sm_count == 0 and _gemm_sm_reserve > 0:
        total = torch.cuda.get_device_properties(a.device).multi_processor_count
        sm_count = max(total - _gemm_sm_reserve, 1)
    args.sm_count = sm_count
    args.act_alpha = float(act_alpha)
    args.act_beta = float(act_beta)
    args.act_limit = float(act_limit or 0.0)
    args.act_has_limit = int(act_limit is not None)
    if scatter_src is not None:
        assert scatter and scatter_src.dtype == torch.int32 and scatter_seg_off.dtype == torch.int64
        args.scatter_src = ptr(scatter_src)
        args.scatter_seg_off = ptr(scatter_seg_off)
        args.scatter_seg_rows = scatter_seg_rows
    if segments is not None:
        args.schedule = _cabi.SCHEDULE_TILE_PAIRS
        args.max_segments = segments.shape[0]
        args.segments = ptr(segments)
        args.num_segments = ptr(num_segments)
    with _cabi.on_device(a.device):
        check(lib.bolt_grouped_gemm(C.byref(args), stream_of(a)))
    _count()
