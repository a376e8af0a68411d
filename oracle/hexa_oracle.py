"""CPU oracle for HEXA-MoE's expert-specific operators.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch/numpy on the CPU, what the reference computes on its
hot path: the routing/segmentation step, ESMM (forward and input-gradient), ESTMM (per-expert
weight gradient), ESS (per-expert bias-gradient sum) and the MoE layer built from them.  It is
the checker that the CUDA kernels are compared with; nothing in the shipped package imports it.

Parity status ("pinned" means checked against outputs of the reference's own kernels, executed
from the unmodified reference sources with the Triton interpreter; the fixtures and the script
that made them are in tests/golden/):

* routing (`counter`)          pinned  - hexa_moe_triton/hexa_moe/kernels/basics.py:89-118
* ESMM forward / ESMM dX       pinned  - kernels/esmm.py:57-154, kernels/fused.py:142-182
* ESTMM, ESS                   pinned only where every expert holds <= 16 rows per route; beyond
                               that the reference kernels consume chunk 0 twice and never the
                               last chunk (kernels/fused.py:123-134, 199-221), so the oracle
                               follows the published operator definition (figures/formula.jpg,
                               rows 4,5,8,9; dense analogue impls/layers.py:61-72) instead.
* layer forward, l_aux, gate   pinned  - impls/layers.py:212-258, impls/cascaded_moe.py:568-598

Every function cites the reference lines it follows.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

REF_CHUNK = 16  # constant.MAX_TOKEN_CHUNK, kernels/basics.py:11


# --------------------------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------------------------
def counter(routing: torch.Tensor, num_exps: int, chunk: int = REF_CHUNK):
    """One route's segmentation exactly as kernels/basics.py:89-118 returns it.

    routing: int [T] expert id per token (ids outside [0,E) are ignored, basics.py:34,68).
    Returns (num_expanded, exp_start[E+1], tok_ids[num_expanded] with -1 pads, exp_ids[num_expanded/chunk]).
    The reference claims slots with an atomic counter (basics.py:71), so the order inside a
    segment is unspecified on a GPU; sequentially it is ascending token index, which is what a
    stable sort gives and what is produced here.
    """
    r = routing.detach().cpu().numpy().astype(np.int64).reshape(-1)
    valid = (r >= 0) & (r < num_exps)
    counts = np.bincount(r[valid], minlength=num_exps).astype(np.int64)
    padded = (counts + chunk - 1) // chunk * chunk                      # basics.py:55-57
    starts = np.concatenate([[0], np.cumsum(padded)]).astype(np.int64)    # basics.py:99-104
    n_exp = int(starts[-1])
    tok_ids = np.full(n_exp, -1, dtype=np.int32)                          # basics.py:107
    exp_ids = np.full(n_exp // chunk, -1, dtype=np.int32)                 # basics.py:112
    order = np.argsort(np.where(valid, r, num_exps), kind="stable")
    order = order[: int(valid.sum())]
    pos = 0
    for e in range(num_exps):
        c = int(counts[e])
        tok_ids[starts[e]: starts[e] + c] = order[pos: pos + c]
        exp_ids[starts[e] // chunk: starts[e + 1] // chunk] = e           # basics.py:82-87
        pos += c
    return (n_exp, torch.from_numpy(starts.astype(np.int32)), torch.from_numpy(tok_ids),
            torch.from_numpy(exp_ids))


def route(ids: torch.Tensor, num_exps: int, align: int):
    """All k routes of a layer segmented at once (the merged form the CUDA path uses).

    ids: int [T, k].  Routed rows are numbered f = j*T + t (route-major) and stably sorted by
    expert, so the rows of expert e are: route 0's tokens ascending, then route 1's, ...  Each
    per-route sub-list equals what `counter` gives for that route (without pads).
    Every segment is padded to a multiple of `align` rows (the reference pads to 16,
    basics.py:41-58; pad slots hold -1, basics.py:107).

    Returns dict with counts[E], seg_offsets[E+1] (unpadded), pad_offsets[E+1], row_token[n_pad]
    (token id or -1), token_row[T*k] (padded row of routed row (t,j) at index t*k+j, -1 if the
    id is out of range) and tile_expert[n_pad/align].
    """
    T, k = ids.shape
    flat = ids.detach().cpu().numpy().astype(np.int64).T.reshape(-1)       # f = j*T + t
    valid = (flat >= 0) & (flat < num_exps)
    counts = np.bincount(flat[valid], minlength=num_exps).astype(np.int64)
    seg = np.concatenate([[0], np.cumsum(counts)])
    padc = (counts + align - 1) // align * align
    pad = np.concatenate([[0], np.cumsum(padc)])
    n_pad = int(pad[-1])
    order = np.argsort(np.where(valid, flat, num_exps), kind="stable")[: int(valid.sum())]
    row_token = np.full(n_pad, -1, dtype=np.int32)
    token_row = np.full(T * k, -1, dtype=np.int32)
    tile_expert = np.full(n_pad // align, -1, dtype=np.int32)
    for e in range(num_exps):
        c = int(counts[e])
        f = order[seg[e]: seg[e] + c]
        rows = pad[e] + np.arange(c)
        row_token[rows] = (f % T).astype(np.int32)
        token_row[(f % T) * k + (f // T)] = rows.astype(np.int32)
        tile_expert[pad[e] // align: pad[e + 1] // align] = e
    tt = lambda a: torch.from_numpy(np.asarray(a).astype(np.int32))
    # pair tiles for GEMMs that run on two SMs (not in the reference): two consecutive 128-row blocks of one
    # expert; entry = first_block * 2 + (second block belongs to the same expert)
    pairs = []
    if align == 128:
        for e in range(num_exps):
            b0, nb = int(pad[e]) // 128, int(padc[e]) // 128
            pairs += [(b0 + i) * 2 + (1 if i + 1 < nb else 0) for i in range(0, nb, 2)]
    return dict(counts=tt(counts), seg_offsets=tt(seg), pad_offsets=tt(pad), row_token=tt(row_token),
                token_row=tt(token_row), tile_expert=tt(tile_expert), n_pad=n_pad, pair_block=tt(pairs))


# --------------------------------------------------------------------------------------------
# operators, token-order semantics (one route)
# --------------------------------------------------------------------------------------------
def _round(t: torch.Tensor, operand_dtype: Optional[torch.dtype]) -> torch.Tensor:
    """Round operands the way the reference's MMA sees them (kernels/esmm.py:133-134 casts both
    operands to fp16 and accumulates in fp32); None keeps full precision."""
    if operand_dtype is None:
        return t
    return t.to(operand_dtype).to(t.dtype)


def esmm(x, w, b, routing, operand_dtype=None):
    """ESMM forward, kernels/esmm.py:57-154: out[t] = x[t] @ w[e(t)] (+ b[e(t)]); rows whose id is
    out of range stay zero (the output is pre-zeroed, esmm.py:269).  x [T,in], w [E,in,out],
    b [E,out] or None, routing int [T]."""
    x = x.double(); w = w.double()
    T = x.shape[0]; E, _, n_out = w.shape
    out = torch.zeros(T, n_out, dtype=torch.float64)
    xr, wr = _round(x, operand_dtype), _round(w, operand_dtype)
    r = routing.long()
    for e in range(E):
        idx = (r == e).nonzero().flatten()
        if idx.numel():
            y = xr[idx] @ wr[e]
            if b is not None and b.numel():
                y = y + b[e].double()
            out[idx] = y
    return out


def esmm_dgrad(dy, w, routing, operand_dtype=None):
    """ESMM input-gradient, kernels/fused.py:142-182: dx[t] = dy[t] @ w[e(t)]^T with w [E,in,out]."""
    return esmm(dy, w.transpose(1, 2), None, routing, operand_dtype)


def estmm(dy, x, routing, num_exps, operand_dtype=None):
    """ESTMM, the operator definition (formula rows 5 and 9; dense analogue impls/layers.py:61,68):
    dw[e] = sum over tokens of expert e of dy[t]^T (outer) x[t], returned as [E,out,in], the
    orientation kernels/fused.py:183-235 writes (r_estmm)."""
    dy = _round(dy.double(), operand_dtype); x = _round(x.double(), operand_dtype)
    out = torch.zeros(num_exps, dy.shape[1], x.shape[1], dtype=torch.float64)
    r = routing.long()
    for e in range(num_exps):
        idx = (r == e).nonzero().flatten()
        if idx.numel():
            out[e] = dy[idx].T @ x[idx]
    return out


def ess(dy, routing, num_exps):
    """ESS, the operator definition (formula rows 4 and 8; dense analogue impls/layers.py:64,71):
    db[e] = sum over tokens of expert e of dy[t]; [E,out] as kernels/fused.py:111-141 writes."""
    dy = dy.double()
    out = torch.zeros(num_exps, dy.shape[1], dtype=torch.float64)
    r = routing.long()
    valid = (r >= 0) & (r < num_exps)
    out.index_add_(0, r[valid], dy[valid])
    return out


# --------------------------------------------------------------------------------------------
# the MoE layer (single process): impls/layers.py:212-258 forward, :397-474 backward
# --------------------------------------------------------------------------------------------
def act_and_grad(act: Callable, y1: torch.Tensor):
    """act(y1) and its elementwise derivative the way impls/layers.py:264-266 gets it (gradient
    of act(y1).sum())."""
    y = y1.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        h = act(y)
        (g,) = torch.autograd.grad(h.sum(), y)
    return h.detach(), g.detach()


def moe_layer(x, ids, fc1_w, fc2_w, fc1_b, fc2_b, act, dy=None, operand_dtype=None,
              round_hidden: Optional[torch.dtype] = None):
    """Forward (and backward when dy is given) of one MoE layer in float64.

    x [T,d]; ids int [T,k]; fc1_w [E,H,d] and fc2_w [E,H,d_out] in the module's parameter layout
    (impls/cascaded_moe.py:206-211); fc1_b [E,H] / fc2_b [E,d_out] or None.
    Forward, impls/layers.py:240-258: per route y1_j = ESMM(x, fc1_w^T, fc1_b); y = sum_j
    ESMM(act(y1_j), fc2_w, fc2_b)  - an unweighted sum over the k routes, bias added once per route.
    Backward, impls/layers.py:401-447 with ESTMM/ESS by definition:
      db2 = sum_j ESS(dy), dh_j = ESMM(dy, fc2_w^T) * act'(y1_j), dw2 = sum_j act(y1_j)^T dy per expert,
      db1 = sum_j ESS(dh_j), dx = sum_j ESMM(dh_j, fc1_w), dw1 = sum_j dh_j^T x per expert.
    round_hidden: if set, y1/act(y1)/dh are rounded to that dtype where the CUDA path stores them
    in it (used only to build tight expectations for 16-bit runs).
    """
    T, k = ids.shape
    E, H, d = fc1_w.shape
    d_out = fc2_w.shape[2]
    xd = x.double()
    w1 = fc1_w.double().transpose(1, 2)      # [E,d,H], impls/layers.py:112
    w2 = fc2_w.double()                      # [E,H,d_out]
    rh = (lambda t: t.to(round_hidden).double()) if round_hidden is not None else (lambda t: t)
    y = torch.zeros(T, d_out, dtype=torch.float64)
    y1s, hs, gs = [], [], []
    for j in range(k):
        r = ids[:, j]
        y1 = rh(esmm(xd, w1, fc1_b, r, operand_dtype))
        valid = ((r >= 0) & (r < E)).double().unsqueeze(1)
        h, g = act_and_grad(act, y1)
        h = rh(h * valid)                    # unrouted rows never reach fc2 (they are not in any segment)
        y1s.append(y1); hs.append(h); gs.append(g * valid)
        y = y + esmm(h, w2, fc2_b, r, operand_dtype)
    out = dict(y=y, y1=y1s, h=hs)
    if dy is None:
        return out
    dyd = dy.double()
    dx = torch.zeros(T, d, dtype=torch.float64)
    dw1 = torch.zeros(E, H, d, dtype=torch.float64)
    dw2 = torch.zeros(E, H, d_out, dtype=torch.float64)
    db1 = torch.zeros(E, H, dtype=torch.float64)
    db2 = torch.zeros(E, d_out, dtype=torch.float64)
    for j in range(k):
        r = ids[:, j]
        db2 += ess(dyd, r, E)
        dh = rh(esmm_dgrad(dyd, w2, r, operand_dtype) * gs[j])
        dw2 += estmm(dyd, hs[j], r, E, operand_dtype).transpose(1, 2)     # -> [E,H,d_out], layers.py:429
        db1 += ess(dh, r, E)
        dx += esmm_dgrad(dh, w1, r, operand_dtype)
        dw1 += estmm(dh, xd, r, E, operand_dtype)                          # [E,H,d]
    out.update(dx=dx, dw1=dw1, dw2=dw2, db1=db1 if fc1_b is not None else None,
               db2=db2 if fc2_b is not None else None)
    return out


# --------------------------------------------------------------------------------------------
# gate, top-k and auxiliary loss: impls/cascaded_moe.py:568-584, impls/layers.py:480-489,
# impls/losses.py:12-19
# --------------------------------------------------------------------------------------------
def gshard_loss(scores: torch.Tensor, top_ids: torch.Tensor) -> torch.Tensor:
    T, E = scores.shape
    ce = torch.zeros(E, dtype=scores.dtype).index_add_(
        0, top_ids[:, 0].long(), torch.full((T,), E / T, dtype=scores.dtype))
    return (scores.sum(0) * ce).sum() / T


def load_importance_loss(scores_wo_noise: torch.Tensor, topk_logits: torch.Tensor, num_experts: int, gate_noise: float):
    """impls/losses.py:21-43: mean of the squared coefficients of variation of importance (column sums of the clean
    softmax) and load (column sums of Phi((clean score - k-th largest noisy logit) / (gate_noise / E))); unbiased
    variance, 1e-10 added to the squared mean.  Evaluated in the dtype of its inputs (the tests pass float64)."""
    sigma = gate_noise / num_experts
    threshold = topk_logits[:, -1].reshape(-1, 1)
    z = (scores_wo_noise - threshold) / sigma
    load = (0.5 * (1.0 + torch.erf(z / math.sqrt(2.0)))).sum(0)
    importance = scores_wo_noise.sum(0)
    cv2 = lambda v: v.var() / (v.mean() ** 2 + 1e-10)
    return (cv2(importance) + cv2(load)) / 2.0


def gate_topk(x, wg, top_k, noise: Optional[torch.Tensor] = None, gate_noise: float = 0.0):
    """logits = x @ wg^T (gates/top.py:20-22); optional noise * gate_noise / E
    (impls/cascaded_moe.py:571-572); softmax; top-k indices (impls/layers.py:483); gshard loss."""
    logits = x.float() @ wg.float().T
    E = wg.shape[0]
    if noise is not None and gate_noise > 0:
        logits = logits + gate_noise * noise / E
    scores = F.softmax(logits, dim=1)
    ids = torch.topk(scores, min(top_k, E), dim=1).indices
    return ids.to(torch.int32), gshard_loss(scores, ids), scores


def dim_split(hidden_size: int, proportion: Sequence[float]) -> List[int]:
    """Per-rank hidden slice sizes, impls/cascaded_moe.py:341-362 (Triton variant): floor of the
    proportion, then hand out the remainder one unit at a time starting from rank 0."""
    dims = [int(p * hidden_size) for p in proportion]
    i = 0
    while sum(dims) < hidden_size:
        dims[i] += 1
        i = (i + 1) % len(dims)
    return dims


# --------------------------------------------------------------------------------------------
# timed CPU baseline: the same layer as sorted-segment grouped matmuls in fp32 on all host cores
# --------------------------------------------------------------------------------------------
def moe_layer_fast(x, ids, fc1_w, fc2_w, fc1_b, fc2_b, dy):
    """fp32, multi-threaded restatement of moe_layer (GELU activation) used only for timing and
    for large-size property checks: rows are stably sorted by expert and each expert's segment is
    one torch.mm.  Same math as moe_layer up to fp32 rounding."""
    T, k = ids.shape
    E, H, d = fc1_w.shape
    flat = ids.T.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    tok = order % T
    counts = torch.bincount(flat, minlength=E).tolist()
    xs = x.float()[tok]
    dys = dy.float()[tok]
    y1 = torch.empty(xs.shape[0], H); dxs = torch.empty_like(xs); ys = torch.empty_like(dys)
    dw1 = torch.zeros_like(fc1_w, dtype=torch.float32); dw2 = torch.zeros_like(fc2_w, dtype=torch.float32)
    db1 = torch.zeros(E, H); db2 = torch.zeros(E, fc2_w.shape[2])
    s = 0
    w1 = fc1_w.float(); w2 = fc2_w.float()
    for e, c in enumerate(counts):
        if c == 0:
            continue
        sl = slice(s, s + c); s += c
        y1e = xs[sl] @ w1[e].T
        if fc1_b is not None:
            y1e += fc1_b[e].float()
        he = F.gelu(y1e)
        ys[sl] = he @ w2[e]
        if fc2_b is not None:
            ys[sl] += fc2_b[e].float()
        # backward
        db2[e] = dys[sl].sum(0)
        dw2[e] = he.T @ dys[sl]
        dhe = dys[sl] @ w2[e].T
        cdf = 0.5 * (1 + torch.erf(y1e / math.sqrt(2.0)))
        dhe *= cdf + y1e * torch.exp(-0.5 * y1e * y1e) / math.sqrt(2 * math.pi)
        db1[e] = dhe.sum(0)
        dw1[e] = dhe.T @ xs[sl]
        dxs[sl] = dhe @ w1[e]
    y = torch.zeros(T, ys.shape[1]).index_add_(0, tok, ys)
    dx = torch.zeros(T, d).index_add_(0, tok, dxs)
    return dict(y=y, dx=dx, dw1=dw1, dw2=dw2, db1=db1, db2=db2)
