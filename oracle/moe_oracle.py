"""CPU restatement of the reference's fused-MoE arithmetic. TEST INFRASTRUCTURE.

This module is the parity checker: plain torch-on-CPU / numpy restatements of
the reference's own torch reference functions and sort contracts.  It is never
imported by the shipped package.  Each function cites the reference file:line
it follows (paths relative to the reference project root).

Parity status: PINNED.  ``tests/golden/*.npz`` holds outputs of the reference's
own Python reference functions executed in the build container (generator:
``tests/golden/make_golden.py``), plus the hand-transcribed known-answer
vectors from the reference's tests; ``tests/test_oracle_golden.py`` checks this
module against all of them.
"""

from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
INT8_MAX = 127.0


# ---------------------------------------------------------------------------
# Routing  (boltops/tools/fused_moe_triton_tune/routing.py:10-35)
# ---------------------------------------------------------------------------
def fused_topk(gating_output: torch.Tensor, topk: int, renormalize: bool = True,
               is_softmax: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """scores = softmax|sigmoid(logits.float()); top-k; optional renormalise."""
    logits = gating_output.float()
    scores = torch.softmax(logits, dim=-1) if is_softmax else logits.sigmoid()
    weights, ids = torch.topk(scores, k=topk, dim=-1)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return weights, ids.to(torch.int32)


def fused_gate(logits: torch.Tensor, bias: torch.Tensor, num_expert_group: int, topk_group: int,
               topk: int, num_fused_shared_experts: int = 0, routed_scaling_factor: float = 1.0):
    """Grouped gate (boltops/tools/fused_moe_triton_tune/routing.py:38-79)."""
    scores = logits.float().sigmoid()
    choice = scores + bias.float()[None]
    m, e = scores.shape
    gscore = choice.view(m, num_expert_group, -1).topk(2, dim=-1).values.sum(-1)
    groups = gscore.topk(topk_group, dim=-1).indices
    gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, groups, True)
    emask = gmask[:, :, None].expand(m, num_expert_group, e // num_expert_group).reshape(m, e)
    sel = choice.masked_fill(~emask, float("-inf")).topk(topk, dim=-1).indices
    w = scores.gather(1, sel)
    if num_fused_shared_experts:
        sel[:, -1] = e
        w[:, -1] = w[:, :-1].sum(-1) / routed_scaling_factor
        den = w[:, :-1].sum(-1, keepdim=True)
    else:
        den = w.sum(-1, keepdim=True)
    return w / den, sel.to(torch.int32)


# ---------------------------------------------------------------------------
# Sort contracts
# ---------------------------------------------------------------------------
def sort_ck_loops(topk_ids, topk_weights, num_experts: int, unit_size: int,
                  mask=None):
    """CK-format sort, pure-Python loops (small cases only).

    Follows test/fused_moe/test_moe_sorting_hipc.py:69-98 and the layout notes
    in moe_sorting_hipc/csrc/moe_sorting_kernel.h:26-88: id = token | slot<<24,
    pad id = tokens | topk<<24 with weight 0, zero-token experts get no block,
    masked experts get no block and enabled experts are renumbered densely.
    Returns (ids, weights, expert_ids, counts, starts); starts[e] == -1 when
    expert e has no block.
    """
    tokens, topk = topk_ids.shape
    pad = tokens | (topk << 24)
    out_ids, out_w, out_e, counts = [], [], [], []
    starts = [-1] * num_experts
    dense_id = 0
    ids_l = topk_ids.tolist()
    w_l = topk_weights.tolist()
    for e in range(num_experts):
        hits = [(t | (s << 24), float(w_l[t][s]))
                for t in range(tokens) for s in range(topk) if ids_l[t][s] == e]
        counts.append(len(hits))
        on = mask is None or int(mask[e]) != 0
        if on and hits:
            starts[e] = len(out_ids)
            npad = -len(hits) % unit_size
            out_ids += [h[0] for h in hits] + [pad] * npad
            out_w += [h[1] for h in hits] + [0.0] * npad
            out_e += [dense_id if mask is not None else e] * ((len(hits) + npad) // unit_size)
        if on:
            dense_id += 1
    return out_ids, out_w, out_e, counts, starts


def sort_ck_numpy(topk_ids, topk_weights, num_experts: int, unit_size: int,
                  mask=None):
    """Vectorised CK-format sort (same contract as :func:`sort_ck_loops`).

    Returns a dict of numpy arrays: sorted_ids (int32, length num_valid),
    sorted_weights (float32), expert_ids (int32), counts (int32 [E]),
    starts (int32 [E], padded start offset for enabled experts, -1 for masked
    ones), num_valid (int).
    """
    ids = np.asarray(topk_ids, dtype=np.int64)
    w = np.asarray(topk_weights, dtype=np.float32)
    tokens, topk = ids.shape
    flat = ids.reshape(-1)
    inrange = (flat >= 0) & (flat < num_experts)
    counts = np.bincount(flat[inrange], minlength=num_experts).astype(np.int64)
    on = np.ones(num_experts, dtype=bool) if mask is None else (np.asarray(mask) != 0)
    padded = np.where(on, -(-counts // unit_size) * unit_size, 0)
    start = np.concatenate([[0], np.cumsum(padded)])[:-1]
    total = int(padded.sum())
    out_ids = np.full(total, tokens | (topk << 24), dtype=np.int64)
    out_w = np.zeros(total, dtype=np.float32)
    order = np.argsort(np.where(inrange, flat, num_experts), kind="stable")
    order = order[: int(inrange.sum())]
    e_sorted = flat[order]
    rank = np.arange(order.size) - np.concatenate([[0], np.cumsum(counts)])[:-1][e_sorted]
    keep = on[e_sorted]
    dst = start[e_sorted] + rank
    tok = order // topk
    slot = order % topk
    out_ids[dst[keep]] = (tok | (slot << 24))[keep]
    out_w[dst[keep]] = w.reshape(-1)[order][keep]
    dense = np.cumsum(on) - on  # enabled experts before e
    label = dense if mask is not None else np.arange(num_experts)
    expert_ids = np.repeat(label, padded // unit_size).astype(np.int32)
    starts = np.where(on, start, -1).astype(np.int32)
    return dict(sorted_ids=out_ids.astype(np.uint32).view(np.int32)
                if out_ids.size else out_ids.astype(np.int32),
                sorted_weights=out_w, expert_ids=expert_ids,
                counts=counts.astype(np.int32), starts=starts, num_valid=total)


def align_block_size_loops(topk_ids, block_size: int, num_experts: int,
                           expert_map=None):
    """vLLM-format sort (boltops/fused_moe/triton/fused_moe.py:194-276,330-439).

    sorted ids are flat route indices ``m*topk+k`` ascending within an expert,
    pad value = numel over the whole capacity ``numel + E*(block-1)``; ids
    outside [0, E) are ignored; zero-token experts get no block; expert_ids is
    zero-filled beyond the used blocks and mapped through ``expert_map`` last.
    Same per-expert listing as test/fused_moe/test_moe_single_k.py:307-317.
    """
    flat = np.asarray(topk_ids).reshape(-1).tolist()
    numel = len(flat)
    cap = numel + num_experts * (block_size - 1)
    nblk = -(-cap // block_size)
    sorted_ids = [numel] * cap
    expert_ids = [0] * nblk
    pos = 0
    for e in range(num_experts):
        sel = [i for i, x in enumerate(flat) if x == e]
        for j, r in enumerate(sel):
            sorted_ids[pos + j] = r
        padded = -(-len(sel) // block_size) * block_size
        for b in range(pos // block_size, (pos + padded) // block_size):
            expert_ids[b] = e
        pos += padded
    expert_ids = np.asarray(expert_ids, dtype=np.int32)
    if expert_map is not None:
        expert_ids = np.asarray(expert_map, dtype=np.int32)[expert_ids]
    return (np.asarray(sorted_ids, dtype=np.int32), expert_ids, pos)


# ---------------------------------------------------------------------------
# Quantisers
# ---------------------------------------------------------------------------
def _dtype_max(qdtype) -> float:
    return FP8_MAX if qdtype == FP8 else INT8_MAX


def quant_rows_kernel(x: torch.Tensor, qdtype, group: Optional[int] = None):
    """The reference *kernel's* dynamic quantiser arithmetic.

    boltops/fused_moe/triton/quant.py:145-264 (+ :19-23): per row, or per
    ``group`` consecutive columns (moe_compat.py:87-106 views the input as
    ``[-1, group]``): amax taken in the input dtype, ``scale = max(f32(amax),
    1e-10) / dtype_max``, ``q = f32(x) * (1/scale)``; int8 rounds to nearest
    even then casts, fp8 casts (round-to-nearest-even) with no clamp.
    Returns (q [rows, cols], scale fp32 [rows, cols/group]).
    """
    rows, cols = x.shape
    g = cols if group is None else group
    xv = x.reshape(-1, g)
    amax = xv.abs().amax(dim=-1, keepdim=True).float()
    scale = torch.clamp(amax, min=1.0e-10) / _dtype_max(qdtype)
    y = xv.float() * (1.0 / scale)
    if qdtype == torch.int8:
        q = torch.round(y).clamp(-128, 127).to(torch.int8)
    else:
        q = y.to(FP8)
    return q.reshape(rows, cols), scale.reshape(rows, cols // g)


def group_quant_fp8_native(x: torch.Tensor, group: int, eps: float = 1e-10):
    """Tune-script oracle quantiser (tune_moe_fp8.py:157-179): clamp variant."""
    xv = x.reshape(-1, group)
    amax = xv.abs().max(dim=-1, keepdim=True)[0].clamp(min=eps).to(torch.float32)
    s = amax / FP8_MAX
    q = (xv / s).clamp(min=-FP8_MAX, max=FP8_MAX).to(FP8)
    return q.reshape(x.shape), s.reshape(x.shape[:-1] + (x.shape[-1] // group,))


def group_quant_int8_native(x: torch.Tensor, group: int):
    """test/fused_moe/test_fused_moe.py:223-237: round + clamp(-128,127)."""
    xv = x.reshape(-1, group)
    amax = xv.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10).float()
    s = amax / INT8_MAX
    q = (xv.float() / s).round().clamp(-128, 127).to(torch.int8)
    return q.reshape_as(x), s.reshape(*x.shape[:-1], x.shape[-1] // group)


def pertoken_quant_torch(x: torch.Tensor, qdtype=torch.int8):
    """boltops/fused_moe/triton/moe_compat.py:35-52 (torch per-token quant)."""
    v = x.float()
    s = v.abs().amax(dim=-1, keepdim=True) / _dtype_max(qdtype)
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = v / s
    if qdtype == torch.int8:
        q = q.round()
    return q.to(qdtype), s.float()


def group_quant_fp8_power2(x: torch.Tensor, group: Optional[int] = None):
    """Power-of-two (UE8M0-compatible) scales, quant.py:636-661 and its pin in
    test/fused_moe/test_quant.py:340-357: ``scale = 2^ceil(log2(amax/448))``,
    ``q = clamp(x/scale, +-448)``."""
    rows, cols = x.shape
    g = cols if group is None else group
    xv = x.reshape(-1, g).float()
    amax = xv.abs().amax(-1).clamp_min(1.0e-10)
    raw = amax * (1.0 / 448.0)
    scale = torch.exp2(torch.ceil(torch.log2(raw)))
    q = (xv / scale[:, None]).clamp(-448, 448).to(FP8)
    return q.reshape(rows, cols), scale.reshape(rows, cols // g)


# ---------------------------------------------------------------------------
# Activations (test/fused_moe/test_moe_activation.py:44-72, tools common.py:122-175,
# kernel math boltops/fused_moe/triton/moe_activation.py:70-128)
# ---------------------------------------------------------------------------
def activation_ref(x: torch.Tensor, activation: str = "silu", is_gated: bool = True,
                   limit: Optional[float] = None, alpha: Optional[float] = None,
                   situ_beta: Optional[float] = None, situ_linear_beta: Optional[float] = None,
                   interleaved: bool = False):
    """fp32 math on the [gate | up] chunked layout (``interleaved``: [g0,u0,g1,u1,...], the
    layout of the reference's swigluoai kernel, moe_activation.py:869-925); caller casts."""
    xf = x.float()
    if is_gated:
        if interleaved:
            gate, up = xf[..., 0::2], xf[..., 1::2]
        else:
            gate, up = xf.chunk(2, dim=-1)
        if activation == "situ":
            # moe_activation.py:958-1010 / tools common.py:139-150
            act = situ_beta * torch.tanh(gate / situ_beta) * torch.sigmoid(gate)
            if situ_linear_beta is not None:
                up = situ_linear_beta * torch.tanh(up / situ_linear_beta)
            return act * up
        if activation == "silu":
            if limit is not None and alpha is None:
                gate = gate.clamp(max=limit)
                up = up.clamp(min=-limit, max=limit)
            return F.silu(gate) * up
        if activation == "gelu":
            return F.gelu(gate, approximate="none") * up
        if activation == "gelu_tanh":
            return F.gelu(gate, approximate="tanh") * up
        if activation == "swigluoai":
            a = 1.702 if alpha is None else alpha
            lim = 7.0 if limit is None else limit
            g = gate.clamp(max=lim)
            u = up.clamp(min=-lim, max=lim)
            return g * torch.sigmoid(a * g) * (u + 1.0)
        if activation == "swiglustep":
            lim = 7.0 if limit is None else limit
            return F.silu(gate).clamp(max=lim) * up.clamp(min=-lim, max=lim)
        raise ValueError(activation)
    if activation in ("silu", "silu_no_mul"):
        return F.silu(xf)
    if activation in ("gelu", "gelu_no_mul"):
        return F.gelu(xf, approximate="none")
    if activation in ("gelu_tanh", "gelu_tanh_no_mul"):
        return F.gelu(xf, approximate="tanh")
    if activation in ("relu2", "relu2_no_mul"):
        return F.relu(xf).square()
    raise ValueError(activation)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """out = silu(gate) * up in fp32, stored in the input dtype."""
    return activation_ref(x, "silu", True).to(x.dtype)


# ---------------------------------------------------------------------------
# Combine (boltops/fused_moe/triton/fused_moe.py:72-131; pinned by
# test/fused_moe/test_fused_moe.py:1359-1377)
# ---------------------------------------------------------------------------
def moe_sum(x: torch.Tensor, scale: float = 1.0, out_dtype=None,
            weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m] = cast(scale * sum_k f32(x[m,k]) [* w[m,k]]), k ascending, fp32."""
    acc = torch.zeros(x.shape[0], x.shape[2], dtype=torch.float32)
    for k in range(x.shape[1]):
        v = x[:, k].float()
        if weights is not None:
            v = v * weights[:, k, None].float()
        acc = acc + v
    acc = acc * scale
    return acc.to(x.dtype if out_dtype is None else out_dtype)


# ---------------------------------------------------------------------------
# Scaled matmuls
# ---------------------------------------------------------------------------
def block_scaled_matmul(a_q, b_q, a_s, b_s, block: Sequence[int], out_dtype):
    """C[:, nb] += (A[:, kb] @ B[nb, kb]^T) * (a_s[:, kb] * b_s[nb, kb]), fp32,
    cast at the end (tune_moe_fp8.py:182-234; test_fused_moe.py:240-266)."""
    bn, bk = block
    a = a_q.float()
    b = b_q.float()
    m, k = a.shape
    n = b.shape[0]
    c = torch.zeros(m, n, dtype=torch.float32)
    for kb in range(-(-k // bk)):
        ks = slice(kb * bk, min((kb + 1) * bk, k))
        for nb in range(-(-n // bn)):
            ns = slice(nb * bn, min((nb + 1) * bn, n))
            s = a_s[:, kb:kb + 1] * b_s[nb][kb]
            c[:, ns] += (a[:, ks] @ b[ns, ks].t()) * s
    return c.to(out_dtype)


def per_token_matmul(a_q, b_q, a_s, b_s, out_dtype):
    """C = a_s * (A @ B^T) * b_s[None, :] (tune_moe_int8_channel.py:145-165)."""
    c = a_q.float() @ b_q.float().t()
    c = a_s.reshape(-1, 1) * c * b_s.reshape(1, -1)
    return c.to(out_dtype)


# ---------------------------------------------------------------------------
# Full layers
# ---------------------------------------------------------------------------
def _repeat_rows(x, topk):
    m, h = x.shape
    return x[:, None, :].expand(m, topk, h).reshape(-1, h).contiguous()


def moe_bf16(hidden, w1, w2, topk_weights, topk_ids,
             routed_scaling_factor: float = 1.0):
    """Unquantised gated-SiLU layer with per-stage casts.

    test/fused_moe/test_fused_moe.py:123-157: fp32 matmul -> cast; fp32
    silu(gate)*up -> cast; fp32 matmul -> cast; fp32 weighted sum -> cast.
    """
    m, h = hidden.shape
    k = topk_ids.shape[1]
    rep = _repeat_rows(hidden, k)
    flat = topk_ids.reshape(-1)
    routed = torch.zeros(m * k, w2.shape[1], dtype=hidden.dtype)
    for e in range(w1.shape[0]):
        sel = flat == e
        if not sel.any():
            continue
        c1 = (rep[sel].float() @ w1[e].float().t()).to(hidden.dtype)
        act = activation_ref(c1, "silu", True).to(hidden.dtype)
        routed[sel] = (act.float() @ w2[e].float().t()).to(hidden.dtype)
    out = (routed.view(m, k, -1).float() * topk_weights[:, :, None].float()).sum(dim=1)
    return (out * routed_scaling_factor).to(hidden.dtype)


def moe_block_fp8(hidden, w1, w2, w1_s, w2_s, topk_weights, topk_ids, block,
                  expert_map=None, power2: bool = False):
    """fp8 [bn,bk]-block-scaled layer (tune_moe_fp8.py:237-287): quantise the
    repeated rows per 1xbk group, block matmul -> activation dtype, gated SiLU
    (tools common.py:122-135: computed in the activation dtype), re-quantise,
    block matmul, weighted sum in the activation dtype.  ``power2`` swaps in the
    power-of-two-scale quantiser (the ``use_ue8m0`` recipe, quant.py:636-661)."""
    m, h = hidden.shape
    k = topk_ids.shape[1]
    rep = _repeat_rows(hidden, k)
    out = torch.zeros(m * k, w2.shape[1], dtype=hidden.dtype)
    flat = topk_ids.reshape(-1).long()
    if expert_map is not None:
        flat = expert_map.long()[flat]
    quant = group_quant_fp8_power2 if power2 else group_quant_fp8_native
    a_q, a_s = quant(rep, block[1])
    for e in range(w1.shape[0]):
        sel = flat == e
        if not sel.any():
            continue
        c1 = block_scaled_matmul(a_q[sel], w1[e], a_s[sel], w1_s[e], block, hidden.dtype)
        gate, up = torch.chunk(c1, 2, dim=-1)
        act = F.silu(gate) * up
        act_q, act_s = quant(act.contiguous(), block[1])
        out[sel] = block_scaled_matmul(act_q, w2[e], act_s, w2_s[e], block, hidden.dtype)
    return (out.view(m, k, -1) * topk_weights.reshape(m, k, 1).to(out.dtype)).sum(dim=1)


def moe_block_int8(hidden, w1, w2, w1_s, w2_s, topk_weights, topk_ids, block):
    """int8 block-scaled layer (test/fused_moe/test_fused_moe.py:355-408)."""
    m, h = hidden.shape
    k = topk_ids.shape[1]
    rep = _repeat_rows(hidden, k)
    a_q, a_s = group_quant_int8_native(rep, block[1])
    flat = topk_ids.reshape(-1)
    routed = torch.zeros(m * k, w2.shape[1], dtype=hidden.dtype)
    for e in range(w1.shape[0]):
        sel = flat == e
        if not sel.any():
            continue
        c1 = block_scaled_matmul(a_q[sel], w1[e], a_s[sel], w1_s[e], block, hidden.dtype)
        act = activation_ref(c1, "silu", True).to(hidden.dtype).contiguous()
        act_q, act_s = group_quant_int8_native(act, block[1])
        routed[sel] = block_scaled_matmul(act_q, w2[e], act_s, w2_s[e], block, hidden.dtype)
    out = (routed.view(m, k, -1).float() * topk_weights[:, :, None].float()).sum(dim=1)
    return out.to(hidden.dtype)


def moe_per_channel(hidden, w1, w2, w1_s, w2_s, topk_weights, topk_ids,
                    qdtype=torch.int8, expert_map=None):
    """Per-token activation / per-output-channel weight scaled layer
    (tune_moe_int8_channel.py:168-218 with the torch quantiser
    moe_compat.py:35-52 in place of its device quantiser)."""
    m, h = hidden.shape
    k = topk_ids.shape[1]
    a_q, a_s = pertoken_quant_torch(hidden, qdtype)
    a_q = _repeat_rows(a_q, k)
    a_s = a_s.view(m, 1, 1).expand(m, k, 1).reshape(-1, 1)
    out = torch.zeros(m * k, w2.shape[1], dtype=hidden.dtype)
    flat = topk_ids.reshape(-1).long()
    if expert_map is not None:
        flat = expert_map.long()[flat]
    for e in range(w1.shape[0]):
        sel = flat == e
        if not sel.any():
            continue
        c1 = per_token_matmul(a_q[sel], w1[e], a_s[sel], w1_s[e], hidden.dtype)
        gate, up = torch.chunk(c1, 2, dim=-1)
        act = F.silu(gate) * up
        act_q, act_s = pertoken_quant_torch(act, qdtype)
        out[sel] = per_token_matmul(act_q, w2[e], act_s, w2_s[e], hidden.dtype)
    return (out.view(m, k, -1) * topk_weights.reshape(m, k, 1).to(out.dtype)).sum(dim=1)


# ---------------------------------------------------------------------------
# Seeded synthetic workloads (shapes/distributions of the benchmark configs)
# ---------------------------------------------------------------------------
def make_routing(m: int, num_experts: int, topk: int, seed: int,
                 zipf_alpha: Optional[float] = None):
    """Router logits ~N(0,1) -> softmax -> top-k -> renormalise (fp32 weights,
    int32 ids).  With ``zipf_alpha`` experts are drawn per token without
    replacement from p(e) ~ (rank_e+1)^-alpha over a seed-fixed permutation and
    weighted by the renormalised softmax of those experts' logits."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(m, num_experts, generator=g, dtype=torch.float32)
    if zipf_alpha is None:
        return fused_topk(logits, topk, renormalize=True)
    perm = torch.randperm(num_experts, generator=g)
    p = (torch.arange(num_experts, dtype=torch.float64) + 1.0) ** (-zipf_alpha)
    prob = torch.empty(num_experts, dtype=torch.float64)
    prob[perm] = p / p.sum()
    ids = torch.multinomial(prob.expand(m, -1), topk, replacement=False, generator=g)
    scores = torch.softmax(logits, dim=-1).gather(1, ids)
    weights = scores / scores.sum(dim=-1, keepdim=True)
    return weights.float(), ids.to(torch.int32)


def quantize_weight_block_fp8(w: torch.Tensor, block=(128, 128)):
    """Per-[bn,bk]-block scale = amax/448 (fp32), w_q = (w/scale) -> e4m3."""
    n, k = w.shape[-2:]
    bn, bk = block
    lead = w.shape[:-2]
    wv = w.float().reshape(*lead, n // bn, bn, k // bk, bk)
    amax = wv.abs().amax(dim=(-3, -1), keepdim=True).clamp(min=1e-10)
    s = amax / FP8_MAX
    q = (wv / s).clamp(-FP8_MAX, FP8_MAX).to(FP8).reshape(w.shape)
    return q, s.reshape(*lead, n // bn, k // bk).contiguous()


def quantize_weight_channel_int8(w: torch.Tensor):
    """Per-output-channel scale = amax/127 (fp32), round, clamp."""
    amax = w.float().abs().amax(dim=-1, keepdim=True).clamp(min=1e-10)
    s = amax / INT8_MAX
    q = (w.float() / s).round().clamp(-128, 127).to(torch.int8)
    return q, s.squeeze(-1).contiguous()


# ---------------------------------------------------------------------------
# MXFP8: e4m3 codes with E8M0 exponent bytes per 1 x 32 group
# ---------------------------------------------------------------------------
def mx_quant(value: torch.Tensor):
    """Codes, exponent bytes and dequantised values of the reference's MXFP8 quantiser
    (test/fused_moe/test_fused_moe.py:1904-1909 `native_quant`;
    boltops/fused_moe/triton/mxfp8.py:144-149): byte = clamp(ceil(log2(amax/448)) + 127, 0, 254)
    per 32 elements, q = e4m3(v * 2^(127 - byte))."""
    blocked = value.float().reshape(value.shape[0], -1, 32)
    amax = blocked.abs().amax(-1).clamp_min(torch.finfo(torch.float32).tiny)
    exponent = (torch.ceil(torch.log2(amax / 448.)) + 127).clamp(0, 254)
    q = (blocked * torch.exp2(127 - exponent)[..., None]).to(torch.float8_e4m3fn)
    deq = (q.float() * torch.exp2(exponent - 127)[..., None]).reshape(value.shape)
    return q.reshape(value.shape), exponent.to(torch.uint8), deq


def mx_dequant_weight(w: torch.Tensor, s: torch.Tensor, group: int = 32) -> torch.Tensor:
    """e4m3 weights [E, N, K] with E8M0 bytes [E, N, K/group] -> fp32
    (test/fused_moe/test_fused_moe.py:1893-1894)."""
    return w.float() * torch.exp2(s.float() - 127).repeat_interleave(group, -1)


def mx_gated_activation(g1: torch.Tensor, activation: str = "silu", alpha=None, beta=None,
                        limit=None) -> torch.Tensor:
    """Split [gate | up] activation of the MXFP8 path in fp32
    (boltops/fused_moe/triton/mxfp8.py:137-143; defaults fused_moe.py:1166-1170)."""
    oai = activation == "swigluoai"
    alpha = (1.702 if oai else 1.0) if alpha is None else alpha
    beta = (1.0 if oai else 0.0) if beta is None else beta
    gate, up = g1.float().chunk(2, -1)
    if limit is not None:
        gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
    return gate * torch.sigmoid(alpha * gate) * (up + beta)


def moe_mxfp8(x, w1, w2, s1, s2, topk_weights, topk_ids, *, expert_map=None, activation="silu",
              alpha=None, beta=None, limit=None, no_combine=False):
    """The reference's CPU statement of the native MXFP8 layer
    (test/fused_moe/test_fused_moe.py:1910-1931): activations quantised per 1 x 32 group, GEMM1
    rounded to the input dtype, activation and second quantisation in fp32, GEMM2 and the router
    weights in fp32 until the sum over the routes, one cast at the end."""
    m, k = x.shape
    e = w1.shape[0]
    topk = topk_ids.shape[1]
    b1, b2 = mx_dequant_weight(w1, s1), mx_dequant_weight(w2, s2)
    av = mx_quant(x)[2]
    expected = torch.zeros(m, topk, w2.shape[1], dtype=torch.float32)
    for token in range(m):
        for rank, ge in enumerate(topk_ids[token].tolist()):
            if ge < 0 or ge >= (e if expert_map is None else expert_map.numel()):
                continue
            expert = ge if expert_map is None else int(expert_map[ge])
            if expert < 0:
                continue
            g1 = (av[token:token + 1] @ b1[expert].T).to(x.dtype).float()
            act = mx_gated_activation(g1, activation, alpha, beta, limit)
            a2 = mx_quant(act)[2]
            g2 = (a2 @ b2[expert].T)[0]
            if not no_combine:
                g2 = g2 * topk_weights[token, rank].float()
            expected[token, rank] = g2
    return (expected if no_combine else expected.sum(1)).to(x.dtype)


# ---------------------------------------------------------------------------
# MXFP4 (w4a8): packed e2m1 weights with E8M0 bytes per 32 K elements, e4m3 activations
# ---------------------------------------------------------------------------
def mxfp4_decode(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 codes (low nibble first) with one E8M0 byte per 32 values -> fp32
    (test/fused_moe/test_fused_moe.py:1441-1445 `_decode_mxfp4_reference`)."""
    codes = torch.stack((packed & 15, packed >> 4), -1).flatten(-2).long()
    lut = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6.])
    values = lut[codes & 7] * torch.where(codes & 8 != 0, -1., 1.)
    return values * torch.exp2(scales.float() - 127).repeat_interleave(32, -1)


def mxfp4_quant_g128(x: torch.Tensor):
    """Dynamic 1 x 128 activation quantisation of the MXFP4 recipe: scale = the power of two
    at or above max(amax, 1e-10) / 448 (itself floored at 1e-10), q = e4m3(clamp(x / scale)).
    Returns (codes, fp32 scales [rows, K/128], dequantised values)
    (test/fused_moe/test_fused_moe.py:1424-1438 `_quantize_mxfp4_reference`, group 128;
    kernel: boltops/fused_moe/triton/mxfp4_quant.py:48-54)."""
    groups = x.float().reshape(x.shape[0], -1, 128)
    amax = groups.abs().amax(-1)
    raw = (amax.clamp_min(1.e-10) / 448).clamp_min(1.e-10)
    bits = raw.contiguous().view(torch.int32)
    exponent = ((bits >> 23) & 255) + ((bits & 0x7fffff) != 0).int()
    scale = (exponent << 23).view(torch.float32)
    q = (groups / scale[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    deq = (q.float() * scale[..., None]).reshape(x.shape)
    return q.reshape(x.shape), scale, deq


def _gemm_k32(a: torch.Tensor, w: torch.Tensor, dtype) -> torch.Tensor:
    """fp32 accumulation in K chunks of 32, one output conversion
    (test/fused_moe/test_fused_moe.py:1448-1453 `_mxfp4_reference_gemm`)."""
    result = torch.zeros(a.shape[0], w.shape[0])
    for k in range(0, a.shape[-1], 32):
        result += a[:, k:k + 32] @ w[:, k:k + 32].T
    return result.to(dtype)


def moe_mxfp4(x, w1, w2, s1, s2, topk_weights, topk_ids, *, activation="silu", expert_map=None,
              a1_scale=None, a2_scale=None, b1=None, b2=None, alpha=None, limit=None,
              apply_router_weight_on_input=False, no_combine=False, routed_scaling_factor=1.0):
    """The reference's CPU statement of the MXFP4 layer
    (test/fused_moe/test_fused_moe.py:1506-1563).  Dynamic recipe (a2_scale None): activations
    quantised per 1 x 128 group with power-of-two scales, both GEMMs rounded to the input dtype,
    router weights applied in the fp32 sum over the routes (or to the input when
    apply_router_weight_on_input, top-1 only).  Static recipe (a1_scale / a2_scale one fp32 value
    each): e4m3(x / a1_scale), GEMM1 * a1_scale (+ bias), SwiGLU-OAI with alpha and limit, times the
    router weight when it is applied on the input, e4m3(act / a2_scale), GEMM2 * a2_scale
    (+ bias), times the router weight otherwise; routes summed in fp32."""
    static = a2_scale is not None
    m, hidden = x.shape
    topk = topk_ids.shape[1]
    input_router = apply_router_weight_on_input
    d1, d2 = mxfp4_decode(w1, s1), mxfp4_decode(w2, s2)
    if static:
        alpha = 1.702 if alpha is None else alpha
        a = (x.float() / a1_scale).to(torch.float8_e4m3fn).float()
    else:
        prepared = x * topk_weights.to(x.dtype) if input_router else x
        a = mxfp4_quant_g128(prepared)[2]
    routes = []
    for token in range(m):
        for rank, ge in enumerate(topk_ids[token].tolist()):
            expert = ge if expert_map is None else int(expert_map[ge])
            if expert == -1:
                routes.append(torch.zeros(w2.shape[1], dtype=x.dtype))
                continue
            g1 = _gemm_k32(a[token:token + 1], d1[expert], torch.float32 if static else x.dtype)
            if static:
                g1 = g1 * a1_scale
                if b1 is not None:
                    g1 = g1 + b1[expert]
            gate, up = g1.float().chunk(2, -1)
            if static:
                lim = 7. if limit is None else limit
                gate, up = gate.clamp(max=lim), up.clamp(-lim, lim)
                act = gate * torch.sigmoid(alpha * gate) * (up + 1.)
                if input_router:
                    act = act * topk_weights[token, rank]
            elif activation == "situ":
                act = (1.5 * torch.tanh(gate / 1.5) * torch.sigmoid(gate)
                       * (2.0 * torch.tanh(up / 2.0)))
            elif activation == "swiglustep":
                act = (gate / (1 + torch.exp(-gate))).clamp(max=7.) * up.clamp(-7., 7.)
            else:
                if limit is not None:
                    gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
                act = up * gate / (1 + torch.exp(-gate))
            if not static:
                act = act.bfloat16() if activation == "silu" else act.to(x.dtype)
                qa = mxfp4_quant_g128(act)[2]
            else:
                qa = (act / a2_scale).to(torch.float8_e4m3fn).float()
            g2 = _gemm_k32(qa, d2[expert], torch.float32 if static else x.dtype)[0]
            if static:
                g2 = g2 * a2_scale
                if b2 is not None:
                    g2 = g2 + b2[expert]
                if not no_combine and not input_router:
                    g2 = g2 * topk_weights[token, rank]
            routes.append(g2.to(x.dtype))
    route_output = torch.stack(routes).reshape(m, topk, w2.shape[1])
    if no_combine:
        return route_output
    combined = torch.zeros(m, w2.shape[1])
    for k in range(topk):
        combined += route_output[:, k].float() * (
            1. if input_router or static else topk_weights[:, k, None])
    return (combined * routed_scaling_factor).to(x.dtype)


def rel_l2(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a = actual.double().flatten()
    e = expected.double().flatten()
    den = e.norm().item()
    return (a - e).norm().item() / (den if den > 0 else 1.0)
