"""Tensor-level wrappers over the C ABI: routing, row movement, ESMM, ESTMM, ESS and the
single-device MoE layer forward/backward assembled from them.

Everything here runs CUDA kernels from libhexa_moe_b200.so on the current stream of the input's
device; no function has a CPU or PyTorch fallback.  Buffers in "sorted-row" layout have
`row_capacity` rows of which the first pad_offsets[E] are meaningful (pad rows hold zeros).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib as L
from ._lib import check, dt, lib, ptr, stream_of


# ---- optional per-call instrumentation (used by bench.py; off by default) --------------------------
# LAUNCHES counts kernels launched through the C ABI.  When PROFILE is a list, every wrapper appends
# (name, start_event, end_event, algorithmic_work, algorithmic_bytes) with CUDA events recorded on the launching stream.
LAUNCHES = 0
PROFILE = None
_KERNELS_PER_CALL = dict(route=3, gather=1, combine=1, esmm=1, estmm=1, ess=2, mask=1, gate=1)


class _Timed:
    __slots__ = ("name", "work", "bytes", "ev")

    def __init__(self, name, work=0.0, nbytes=0.0):
        self.name, self.work, self.bytes, self.ev = name, work, nbytes, None

    def __enter__(self):
        global LAUNCHES
        LAUNCHES += _KERNELS_PER_CALL[self.name.split(":")[0]]
        if PROFILE is not None:
            self.ev = torch.cuda.Event(enable_timing=True)
            self.ev.record()
        return self

    def __exit__(self, *exc):
        if self.ev is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            PROFILE.append((self.name, self.ev, end, self.work, self.bytes))
        return False


@dataclass
class Routing:
    """Device-side result of `route` (all int32 tensors) plus the static sizes."""
    counts: torch.Tensor        # [E]
    seg_offsets: torch.Tensor   # [E+1] exclusive scan of counts
    pad_offsets: torch.Tensor   # [E+1] segment starts, multiples of `align`
    row_token: torch.Tensor     # [row_capacity] token of each sorted row, -1 for pad rows
    token_row: torch.Tensor     # [T*k] sorted row of routed row (t, j) at t*k + j
    tile_expert: torch.Tensor   # [row_capacity/align]
    pair_block: Optional[torch.Tensor]   # pair-tile list for the two-CTA GEMMs (align = 128 only)
    num_tokens: int
    top_k: int
    num_experts: int
    align: int
    row_capacity: int


def route(ids: torch.Tensor, num_experts: int, align: int = L.ROW_TILE, route_major: bool = False) -> Routing:
    """Segment routed rows by expert.  ids: int32 [T, k] (or [k, T] when route_major)."""
    if ids.dtype != torch.int32:
        raise L.HexaError("route: ids must be int32")
    if ids.dim() != 2:
        raise L.HexaError("route: ids must be 2-D")
    if route_major:
        k, T = ids.shape
        st, sk = ids.stride(1), ids.stride(0)
    else:
        T, k = ids.shape
        st, sk = ids.stride(0), ids.stride(1)
    s = stream_of(ids)
    dev = ids.device
    cap = lib().hexa_route_row_capacity(T, k, num_experts, align)
    if cap < 0:
        raise L.HexaError("route: bad sizes")
    i32 = dict(dtype=torch.int32, device=dev)
    pairs = torch.empty(lib().hexa_route_pair_capacity(T, k, num_experts), **i32) if align == L.ROW_TILE else None
    r = Routing(torch.empty(num_experts, **i32), torch.empty(num_experts + 1, **i32), torch.empty(num_experts + 1, **i32),
                torch.empty(max(cap, 1), **i32), torch.empty(max(T * k, 1), **i32), torch.empty(max(cap // align, 1), **i32),
                pairs, T, k, num_experts, align, cap)
    ws_bytes = lib().hexa_route_workspace_bytes(T, k, num_experts)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    with _Timed("route", 12.0 * T * k):
        check(lib().hexa_route(ptr(ids), T, k, st, sk, num_experts, align, ptr(r.counts), ptr(r.seg_offsets), ptr(r.pad_offsets),
                               ptr(r.row_token), ptr(r.token_row), ptr(r.tile_expert), ptr(r.pair_block), ptr(ws), ws.numel(), s),
              "hexa_route")
    return r


def sorted_buffer(rows: int, cols: int, dtype, device) -> torch.Tensor:
    """[rows, cols] buffer whose row pitch is a multiple of 16 bytes (8 elements), as the TMA-fed GEMMs need; for a
    column count that is not (a rank's slice of an unevenly split hidden dimension) it is a view of a wider one."""
    pitch = (cols + 7) // 8 * 8
    if pitch == cols:
        return torch.empty(rows, cols, dtype=dtype, device=device)
    return torch.empty(rows, pitch, dtype=dtype, device=device)[:, :cols]


def _ld(t: torch.Tensor) -> int:
    if t.dim() != 2 or t.stride(1) != 1:
        raise L.HexaError("expected a 2-D tensor with unit inner stride")
    return t.stride(0)


def gather_rows(src: torch.Tensor, r: Routing, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token order -> sorted rows: out[row] = src[row_token[row]] (zeros for pad rows)."""
    cols = src.shape[1]
    if out is None:
        out = sorted_buffer(r.row_capacity, cols, src.dtype, src.device)
    with _Timed("gather", 2.0 * r.num_tokens * r.top_k * cols * src.element_size()):
        check(lib().hexa_gather_rows(ptr(src), _ld(src), ptr(r.row_token), ptr(r.pad_offsets), r.num_experts, r.row_capacity,
                                     cols, ptr(out), _ld(out), dt(src), stream_of(src)), "hexa_gather_rows")
    return out


def combine_rows(src: torch.Tensor, r: Routing, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sorted rows -> token order with the unweighted sum over the k routes."""
    cols = src.shape[1]
    if out is None:
        out = torch.empty(r.num_tokens, cols, dtype=src.dtype, device=src.device)
    with _Timed("combine", (r.top_k + 1.0) * r.num_tokens * cols * src.element_size()):
        check(lib().hexa_combine_rows(ptr(src), _ld(src), ptr(r.token_row), r.num_tokens, r.top_k, cols, ptr(out), _ld(out),
                                      dt(src), stream_of(src)), "hexa_combine_rows")
    return out


def esmm(a: torch.Tensor, b: torch.Tensor, b_layout: int, r: Routing, bias: Optional[torch.Tensor] = None,
         epilogue: int = L.EPI_LINEAR, act: int = L.ACT_NONE, aux: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, engine: int = L.ENGINE_AUTO, n_out: Optional[int] = None,
         k: Optional[int] = None, tag: Optional[str] = None, experts: Optional[tuple] = None,
         sums: Optional[torch.Tensor] = None) -> torch.Tensor:
    """c[row] = a[row] x b[expert(row)] with the fused epilogue.  b: [E, n_out, k] (B_NK) or [E, k, n_out] (B_KN);
    b may be a view with arbitrary expert / row strides (unit inner stride).  experts = (first, end): only the rows of
    those experts are computed (the other rows of `out` are left as they are).  sums: a float32 [E, n_out] tensor that
    receives the per-expert column sums of the output (ESS of `out`) from the same launch."""
    global LAUNCHES
    if r.align % L.ROW_TILE:
        raise L.HexaError("esmm: routing must be aligned to 128 rows")
    if b.dim() != 3 or b.stride(2) != 1:
        raise L.HexaError("esmm: b must be 3-D with unit inner stride")
    if b_layout == L.B_NK:
        nn, kk = b.shape[1], b.shape[2]
    else:
        kk, nn = b.shape[1], b.shape[2]
    n_out = nn if n_out is None else n_out
    k = kk if k is None else k
    if a.dtype != b.dtype:
        raise L.HexaError(f"esmm: a is {a.dtype} but b is {b.dtype}")
    if bias is not None and bias.dtype != torch.float32:
        raise L.HexaError("esmm: bias must be float32")
    if out is None:
        out = sorted_buffer(r.row_capacity, n_out, a.dtype, a.device)
    rows_ = r.num_tokens * r.top_k
    es_ = a.element_size()
    nbytes = es_ * (rows_ * k + r.num_experts * n_out * k + rows_ * n_out * (1 if epilogue == L.EPI_LINEAR else 2))
    e0, e1 = (0, r.num_experts) if experts is None else experts
    share = (e1 - e0) / max(r.num_experts, 1)        # work of a group, taken as its share of the experts
    if sums is not None:
        if experts is not None or sums.dtype != torch.float32 or tuple(sums.shape) != (r.num_experts, n_out) or sums.stride(1) != 1:
            raise L.HexaError("esmm: sums must be float32 [E, n_out] and needs the full expert range")
        ws = torch.empty(max(lib().hexa_ess_workspace_bytes(r.row_capacity, n_out), 4), dtype=torch.uint8, device=a.device)
        with _Timed("esmm:" + (tag or "epilogue%d" % epilogue), 2.0 * rows_ * n_out * k, float(nbytes)):
            check(lib().hexa_esmm_ess(ptr(a), _ld(a), ptr(b), b_layout, b.stride(1), b.stride(0), ptr(bias),
                                      0 if bias is None else _ld(bias), ptr(aux), 0 if aux is None else _ld(aux), ptr(out),
                                      _ld(out), ptr(r.tile_expert), ptr(r.pad_offsets), ptr(r.row_token), ptr(r.pair_block),
                                      r.num_experts, r.row_capacity, n_out, k, dt(a), epilogue, act, engine, ptr(sums),
                                      sums.stride(0), ptr(ws), ws.numel(), stream_of(a)), "hexa_esmm_ess")
        LAUNCHES += 1          # the second pass of ESS over the block sums
        return out
    with _Timed("esmm:" + (tag or "epilogue%d" % epilogue), 2.0 * rows_ * n_out * k * share, float(nbytes) * share):
        check(lib().hexa_esmm_experts(ptr(a), _ld(a), ptr(b), b_layout, b.stride(1), b.stride(0), ptr(bias),
                                      0 if bias is None else _ld(bias), ptr(aux), 0 if aux is None else _ld(aux), ptr(out),
                                      _ld(out), ptr(r.tile_expert), ptr(r.pad_offsets), ptr(r.row_token), ptr(r.pair_block),
                                      r.num_experts, r.row_capacity, n_out, k, dt(a), epilogue, act, engine, e0, e1,
                                      stream_of(a)), "hexa_esmm")
    return out


def estmm(p: torch.Tensor, q: torch.Tensor, r: Routing, out_dtype: Optional[torch.dtype] = None,
          out=None, beta: int = 0, engine: int = L.ENGINE_AUTO, ranks: int = 1, tag: Optional[str] = None):
    """out[e] = p_e^T q_e over expert e's rows: [E, p.cols, q.cols].
    ranks > 1 (p.cols divisible by it): the result is laid out [ranks, E, p.cols/ranks, q.cols], i.e. already
    grouped by the rank that owns each slice of the hidden dimension (what a reduce-scatter consumes).  `out` may
    then also be a list of `ranks` tensors [E, p.cols/ranks, q.cols] in this GPU's memory, one per owner: each slice
    is stored straight into its tensor (hexa_estmm_scatter); the list is returned."""
    if r.align % L.ROW_TILE:
        raise L.HexaError("estmm: routing must be aligned to 128 rows")
    m, n = p.shape[1], q.shape[1]
    if p.dtype != q.dtype:
        raise L.HexaError("estmm: p and q dtypes differ")
    rows_ = r.num_tokens * r.top_k
    if isinstance(out, (list, tuple)):
        if ranks != len(out) or m % ranks or beta:
            raise L.HexaError("estmm: a list of outputs needs ranks == len(out), divisible rows and beta = 0")
        o0 = out[0]
        for t in out:
            if t.shape != o0.shape or t.dtype != o0.dtype or t.stride() != o0.stride() or t.stride(-1) != 1:
                raise L.HexaError("estmm: the per-owner outputs must agree in shape, dtype and strides")
        if tuple(o0.shape) != (r.num_experts, m // ranks, n):
            raise L.HexaError("estmm: per-owner outputs must be [E, rows/ranks, cols]")
        import ctypes as C
        ptrs = (C.c_void_p * ranks)(*[t.data_ptr() for t in out])
        with _Timed("estmm:" + (tag or "dw"), 2.0 * rows_ * m * n,
                    float(p.element_size() * rows_ * (m + n) + o0.element_size() * r.num_experts * m * n)):
            check(lib().hexa_estmm_scatter(ptr(p), _ld(p), ptr(q), _ld(q), ptr(r.pad_offsets), r.num_experts, r.row_capacity, m, n,
                                           ptrs, ranks, o0.stride(1), o0.stride(0), m // ranks, dt(p), dt(o0), stream_of(p)),
                  "hexa_estmm_scatter")
        return out
    if ranks > 1:
        if m % ranks:
            raise L.HexaError("estmm: the row count must be divisible by ranks")
        if out is None:
            out = torch.empty(ranks, r.num_experts, m // ranks, n, dtype=out_dtype or p.dtype, device=p.device)
        ldo, estride, m_split, split_stride = out.stride(2), out.stride(1), m // ranks, out.stride(0)
    else:
        if out is None:
            if beta:
                raise L.HexaError("estmm: beta=1 needs an existing out")
            out = torch.empty(r.num_experts, m, n, dtype=out_dtype or p.dtype, device=p.device)
        ldo, estride, m_split, split_stride = out.stride(1), out.stride(0), 0, 0
    if out.stride(-1) != 1:
        raise L.HexaError("estmm: out must have unit inner stride")
    ws_bytes = lib().hexa_estmm_workspace_bytes(r.num_experts, r.row_capacity, m, n, dt(p)) if engine != L.ENGINE_SIMT else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=p.device) if ws_bytes else None
    with _Timed("estmm:" + (tag or "dw"), 2.0 * rows_ * m * n,
                float(p.element_size() * rows_ * (m + n) + out.element_size() * r.num_experts * m * n)):
        check(lib().hexa_estmm(ptr(p), _ld(p), ptr(q), _ld(q), ptr(r.pad_offsets), r.num_experts, r.row_capacity, m, n, ptr(out),
                               ldo, estride, m_split, split_stride, dt(p), dt(out), beta, engine, ptr(ws), ws_bytes,
                               stream_of(p)), "hexa_estmm")
    return out


def copy_2d(dst: torch.Tensor, dst_pitch: int, src: torch.Tensor, src_pitch: int, width: int, height: int, stream: int = None):
    """Device-to-device copy of `height` blocks of `width` elements (pitches in elements).  Runs on `stream` (a raw
    cudaStream_t) or, by default, on the current stream of dst's device; src or dst may be another GPU's memory."""
    es = src.element_size()
    check(lib().hexa_copy_2d(ptr(dst), dst_pitch * es, ptr(src), src_pitch * es, width * es, height,
                             stream_of(dst) if stream is None else stream), "hexa_copy_2d")


def stream_wait_value(flag: torch.Tensor, value: int, stream: int):
    """`stream` waits until the int32 at flag[0] is >= value."""
    check(lib().hexa_stream_wait_value(ptr(flag), value, stream), "hexa_stream_wait_value")


def mean_slices(local: torch.Tensor, recv: torch.Tensor, n_recv: int, world: int, out: torch.Tensor):
    """out = (local + recv[0] + ... + recv[n_recv-1]) / world with fp32 accumulation; all slices shaped like `local`."""
    check(lib().hexa_mean_slices(ptr(local), ptr(recv), n_recv, local.numel(), world, ptr(out), dt(local), stream_of(out)),
          "hexa_mean_slices")


def ess(src: torch.Tensor, r: Routing, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[e] = sum of expert e's rows of src, float32 [E, cols]."""
    if r.align % L.ROW_TILE:
        raise L.HexaError("ess: routing must be aligned to 128 rows")
    cols = src.shape[1]
    if out is None:
        out = torch.empty(r.num_experts, cols, dtype=torch.float32, device=src.device)
    nbytes = lib().hexa_ess_workspace_bytes(r.row_capacity, cols)
    ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=src.device)
    with _Timed("ess", 1.0 * r.num_tokens * r.top_k * cols * src.element_size()):
        check(lib().hexa_ess(ptr(src), _ld(src), ptr(r.pad_offsets), r.num_experts, r.row_capacity, cols, ptr(out), _ld(out),
                             dt(src), ptr(ws), ws.numel(), stream_of(src)), "hexa_ess")
    return out


def mask_pad_rows(buf: torch.Tensor, r: Routing) -> torch.Tensor:
    with _Timed("mask"):
        check(lib().hexa_mask_pad_rows(ptr(buf), _ld(buf), ptr(r.row_token), ptr(r.pad_offsets), r.num_experts, r.row_capacity,
                                       buf.shape[1], dt(buf), stream_of(buf)), "hexa_mask_pad_rows")
    return buf


# -------------------------------------------------------------------------------------------------
# the step before routing
# -------------------------------------------------------------------------------------------------
def gate_max_experts() -> int:
    return int(lib().hexa_gate_max_experts())


def gate_topk(logits: torch.Tensor, top_k: int):
    """softmax + top-k + GShard loss of float32 logits [T,E] in one kernel.  Returns (ids int32 [k,T] route-major,
    loss float32 scalar tensor, first_count int32 [E], mass float32 [E])."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise L.HexaError("gate_topk: logits must be float32 [T,E] with unit inner stride")
    T, E = logits.shape
    dev = logits.device
    ids = torch.empty(top_k, T, dtype=torch.int32, device=dev)
    mass = torch.empty(E, dtype=torch.float32, device=dev)
    cnt = torch.empty(E, dtype=torch.int32, device=dev)
    loss = torch.empty((), dtype=torch.float32, device=dev)
    ws = torch.empty(int(lib().hexa_gate_workspace_bytes()), dtype=torch.uint8, device=dev)
    with _Timed("gate", 2.0 * T * E * 4):
        check(lib().hexa_gate_topk(ptr(logits), _ld(logits), T, E, top_k, ptr(ids), ptr(mass), ptr(cnt), ptr(loss), ptr(ws),
                                   ws.numel(), stream_of(logits)), "hexa_gate_topk")
    return ids, loss, cnt, mass


def gate_loss_grad(logits: torch.Tensor, first_count: torch.Tensor, dloss: torch.Tensor) -> torch.Tensor:
    """Gradient of gate_topk's loss with respect to the logits, scaled by the device scalar dloss."""
    T, E = logits.shape
    out = torch.empty(T, E, dtype=torch.float32, device=logits.device)
    dloss = dloss.detach().to(torch.float32).reshape(1).contiguous()
    with _Timed("gate", 2.0 * T * E * 4):
        check(lib().hexa_gate_loss_grad(ptr(logits), _ld(logits), T, E, ptr(first_count), ptr(dloss), ptr(out), _ld(out),
                                        stream_of(logits)), "hexa_gate_loss_grad")
    return out


def gate_topk_load_importance(logits: torch.Tensor, logits_w_noise: torch.Tensor, top_k: int, sigma: float):
    """top-k of the noisy logits + the load-importance loss of the clean ones in one kernel.  Returns (ids int32 [k,T]
    route-major, loss float32 scalar tensor, importance float32 [E], load float32 [E])."""
    for t in (logits, logits_w_noise):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise L.HexaError("gate_topk_load_importance: logits must be float32 [T,E] with unit inner stride")
    if logits.shape != logits_w_noise.shape or logits.stride(0) != logits_w_noise.stride(0):
        raise L.HexaError("gate_topk_load_importance: the two logit tensors must have the same shape and row pitch")
    T, E = logits.shape
    dev = logits.device
    ids = torch.empty(top_k, T, dtype=torch.int32, device=dev)
    imp = torch.empty(E, dtype=torch.float32, device=dev)
    load = torch.empty(E, dtype=torch.float32, device=dev)
    loss = torch.empty((), dtype=torch.float32, device=dev)
    ws = torch.empty(int(lib().hexa_gate_workspace_bytes()), dtype=torch.uint8, device=dev)
    with _Timed("gate", 3.0 * T * E * 4):
        check(lib().hexa_gate_topk_load_importance(ptr(logits), ptr(logits_w_noise), _ld(logits), T, E, top_k, float(sigma), ptr(ids),
                                                   ptr(imp), ptr(load), ptr(loss), ptr(ws), ws.numel(), stream_of(logits)),
              "hexa_gate_topk_load_importance")
    return ids, loss, imp, load


def gate_load_importance_grad(logits, logits_w_noise, top_k: int, sigma: float, importance, load, dloss) -> torch.Tensor:
    """Gradient of gate_topk_load_importance's loss with respect to the clean logits, scaled by the device scalar dloss
    (the noisy logits differ from them by a constant, so this is also the whole gradient through the threshold)."""
    T, E = logits.shape
    out = torch.empty(T, E, dtype=torch.float32, device=logits.device)
    dloss = dloss.detach().to(torch.float32).reshape(1).contiguous()
    with _Timed("gate", 3.0 * T * E * 4):
        check(lib().hexa_gate_load_importance_grad(ptr(logits), ptr(logits_w_noise), _ld(logits), T, E, top_k, float(sigma),
                                                   ptr(importance), ptr(load), ptr(dloss), ptr(out), _ld(out), stream_of(logits)),
              "hexa_gate_load_importance_grad")
    return out


# -------------------------------------------------------------------------------------------------
# one MoE layer on one device
# -------------------------------------------------------------------------------------------------
@dataclass
class LayerState:
    """What the backward of a layer needs (all in sorted-row layout)."""
    routing: Routing
    xs: torch.Tensor      # gathered input rows  [cap, d]
    y1: torch.Tensor      # fc1 pre-activation   [cap, H]
    h: torch.Tensor       # act(y1)              [cap, H]
    act_grad: Optional[torch.Tensor] = None   # act'(y1) when the activation is not a fused one
    db1: Optional[torch.Tensor] = None        # ESS of the hidden gradient, when the GEMM that produced it summed it as well


def _f32(t):
    """Bias as the fp32 [E, n] operand of the epilogue; rows padded to whole 16-byte chunks when n is not one."""
    if t is None:
        return None
    t = t.detach()
    n = t.shape[-1]
    if n % 4 == 0:
        return t.to(torch.float32).contiguous()
    out = torch.zeros(*t.shape[:-1], (n + 3) // 4 * 4, dtype=torch.float32, device=t.device)
    out[..., :n] = t
    return out[..., :n]


def moe_forward(x, ids, w1, w2, b1, b2, act_id: int, act_fn=None, route_major=False, engine=L.ENGINE_AUTO,
                need_state=True, before_fc2=None, fc1_groups=None):
    """y[t] = sum_j fc2(act(fc1(x[t]; e_j)); e_j).  x [T,d]; ids int32 [T,k] ([k,T] if route_major);
    w1 [E,H,d]; w2 [E,H,d_out]; b1 [E,H] / b2 [E,d_out] or None.  before_fc2: optional callable run on the host
    between the launches of fc1 and fc2 (the caller may enqueue a stream wait for w2 there).  fc1_groups: optional list of
    (first expert, end expert, callable) - fc1 is then launched once per group, after calling the group's callable
    (the caller enqueues the stream wait for that group's fc1 weights there), so the layer starts before all of w1 is in.
    act_id: an _lib.ACT_* id fused into the fc1 epilogue, or -1 to call `act_fn` (any elementwise
    callable) between the two ESMMs.  Returns (y [T,d_out], LayerState)."""
    E = w1.shape[0]
    r = route(ids, E, L.ROW_TILE, route_major=route_major)
    xs = gather_rows(x, r)
    b1f, b2f = _f32(b1), _f32(b2)
    H = w1.shape[1]
    y1 = sorted_buffer(r.row_capacity, H, x.dtype, x.device)
    g = None
    groups = fc1_groups if fc1_groups else [(0, E, None)]
    if act_id >= 0:
        h = sorted_buffer(r.row_capacity, H, x.dtype, x.device)
        for e0, e1, ready in groups:
            if ready is not None:
                ready()
            esmm(xs, w1, L.B_NK, r, b1f, L.EPI_ACT, act_id, aux=y1, out=h, engine=engine, tag="fc1_forward_act", experts=(e0, e1))
    else:
        for e0, e1, ready in groups:
            if ready is not None:
                ready()
            esmm(xs, w1, L.B_NK, r, b1f, L.EPI_LINEAR, out=y1, engine=engine, tag="fc1_forward", experts=(e0, e1))
        if need_state:
            with torch.enable_grad():
                yy = y1.detach().requires_grad_(True)
                hh = act_fn(yy)
                (g,) = torch.autograd.grad(hh.sum(), yy)
            h = sorted_buffer(r.row_capacity, H, x.dtype, x.device).copy_(hh.detach())
        else:
            h = sorted_buffer(r.row_capacity, H, x.dtype, x.device).copy_(act_fn(y1))
        mask_pad_rows(h, r)
    if before_fc2 is not None:      # e.g. wait for w2 to finish arriving from the other ranks
        before_fc2()
    ys = esmm(h, w2, L.B_KN, r, b2f, L.EPI_LINEAR, engine=engine, tag="fc2_forward")
    y = combine_rows(ys, r)
    return y, (LayerState(r, xs, y1, h, g) if need_state else None)


def _hidden_gradient(st: LayerState, dys, w2, act_id: int, engine, want_db1: bool):
    """dh = dys W2^T * act'(y1) for a fused activation; with want_db1 the same launch leaves ESS(dh) in st.db1."""
    r = st.routing
    st.db1 = None
    if want_db1 and os.environ.get("HEXA_FUSED_ESS", "1") != "0":
        st.db1 = torch.empty(r.num_experts, w2.shape[1], dtype=torch.float32, device=dys.device)
    return esmm(dys, w2, L.B_NK, r, None, L.EPI_DACT, act_id, aux=st.y1, engine=engine, tag="fc2_dgrad_dact", sums=st.db1)


def moe_backward_fc2(st: LayerState, dy, w2, act_id: int, has_b2=True, grad_dtype=None, engine=L.ENGINE_AUTO, ranks=1,
                     dw_out=None, want_db1=False):
    """First half of the layer backward: (dh [cap,H] = dy W2^T * act'(y1), dw2 [E,H,d_out], db2 [E,d_out] | None).
    Split from the fc1 half so a caller can start reducing dw2/db2 across ranks while fc1 runs.  want_db1: the fc1
    half will need the bias gradient ESS(dh); with a fused activation the GEMM that writes dh sums it on the way."""
    r = st.routing
    dys = gather_rows(dy.contiguous(), r)
    db2 = ess(dys, r) if has_b2 else None
    dw2 = estmm(st.h, dys, r, out_dtype=grad_dtype, engine=engine, ranks=ranks, out=dw_out, tag="dw2")
    if act_id >= 0:
        dh = _hidden_gradient(st, dys, w2, act_id, engine, want_db1)
    else:
        dh = esmm(dys, w2, L.B_NK, r, None, L.EPI_LINEAR, engine=engine, tag="fc2_dgrad")
        dh.mul_(st.act_grad)
        mask_pad_rows(dh, r)
    return dh, dw2, db2


def moe_backward_fc1(st: LayerState, dh, w1, has_b1=True, grad_dtype=None, engine=L.ENGINE_AUTO, ranks=1,
                     after_dw=None, dw_out=None):
    """Second half: (dx [T,d], dw1 [E,H,d], db1 [E,H] | None) from dh.  after_dw(dw1, db1), if given, is called on the
    host as soon as both parameter gradients are enqueued, before the input-gradient GEMM: a caller can start
    reducing them across ranks while that GEMM runs."""
    r = st.routing
    db1 = (st.db1 if st.db1 is not None else ess(dh, r)) if has_b1 else None
    st.db1 = None
    dw1 = estmm(dh, st.xs, r, out_dtype=grad_dtype, engine=engine, ranks=ranks, out=dw_out, tag="dw1")
    if after_dw is not None:
        after_dw(dw1, db1)
    dxs = esmm(dh, w1, L.B_KN, r, None, L.EPI_LINEAR, engine=engine, tag="fc1_dgrad")
    dx = combine_rows(dxs, r)
    return dx, dw1, db1


def moe_backward_inputs(st: LayerState, dy, w1, w2, act_id: int, engine=L.ENGINE_AUTO, want_db1=False):
    """The input-gradient half of the layer backward, ahead of the parameter gradients: returns (dx [T,d], kept) where
    `kept` = (dys, dh) is what moe_backward_params needs.  A caller that has to send dx to other ranks can start the
    transfer after this call and let it run beside the two weight-gradient GEMMs."""
    r = st.routing
    dys = gather_rows(dy.contiguous(), r)
    if act_id >= 0:
        dh = _hidden_gradient(st, dys, w2, act_id, engine, want_db1)
    else:
        dh = esmm(dys, w2, L.B_NK, r, None, L.EPI_LINEAR, engine=engine, tag="fc2_dgrad")
        dh.mul_(st.act_grad)
        mask_pad_rows(dh, r)
    dxs = esmm(dh, w1, L.B_KN, r, None, L.EPI_LINEAR, engine=engine, tag="fc1_dgrad")
    return combine_rows(dxs, r), (dys, dh)


def moe_backward_params(st: LayerState, kept, has_b1=True, has_b2=True, grad_dtype=None, engine=L.ENGINE_AUTO, into=None):
    """(dw1 [E,H,d], dw2 [E,H,d_out], db1 [E,H] | None, db2 [E,d_out] | None) from what moe_backward_inputs kept.
    into: the same four from an earlier call over other tokens of the same layer; this call's gradients are added to
    them in place (the weight GEMMs accumulate onto their output) and they are returned."""
    r = st.routing
    dys, dh = kept
    db1_new = (st.db1 if st.db1 is not None else ess(dh, r)) if has_b1 else None
    st.db1 = None
    if into is None:
        dw2 = estmm(st.h, dys, r, out_dtype=grad_dtype, engine=engine, tag="dw2")
        dw1 = estmm(dh, st.xs, r, out_dtype=grad_dtype, engine=engine, tag="dw1")
        return dw1, dw2, db1_new, (ess(dys, r) if has_b2 else None)
    dw1, dw2, db1, db2 = into
    estmm(st.h, dys, r, out=dw2, beta=1, engine=engine, tag="dw2")
    estmm(dh, st.xs, r, out=dw1, beta=1, engine=engine, tag="dw1")
    if has_b1:
        db1 += db1_new
    if has_b2:
        db2 += ess(dys, r)
    return dw1, dw2, db1, db2


def moe_backward(st: LayerState, dy, w1, w2, act_id: int, has_b1=True, has_b2=True, grad_dtype=None,
                 engine=L.ENGINE_AUTO):
    """Gradients of moe_forward.  Returns (dx [T,d], dw1 [E,H,d], dw2 [E,H,d_out], db1 [E,H] | None,
    db2 [E,d_out] | None); bias gradients are float32, weight gradients `grad_dtype` (default: dtype of dy)."""
    dh, dw2, db2 = moe_backward_fc2(st, dy, w2, act_id, has_b2, grad_dtype, engine, want_db1=has_b1)
    dx, dw1, db1 = moe_backward_fc1(st, dh, w1, has_b1, grad_dtype, engine)
    return dx, dw1, dw2, db1, db2


# -------------------------------------------------------------------------------------------------
# the dense FFN as a one-expert layer on the same kernels
# -------------------------------------------------------------------------------------------------
_DENSE_ROUTING = {}


def dense_routing(num_tokens: int, device: torch.device) -> Routing:
    """Routing of `num_tokens` rows to a single expert: sorted row i is token i, the tail up to the next multiple
    of 128 is padding.  Built once per (size, device) by the routing kernel itself and kept."""
    key = (int(num_tokens), device.index if device.index is not None else torch.cuda.current_device())
    r = _DENSE_ROUTING.get(key)
    if r is None:
        if len(_DENSE_ROUTING) >= 64:
            _DENSE_ROUTING.clear()
        r = route(torch.zeros(num_tokens, 1, dtype=torch.int32, device=device), 1, L.ROW_TILE)
        _DENSE_ROUTING[key] = r
    return r


def _dense_rows(t: torch.Tensor, r: Routing) -> torch.Tensor:
    """t [T, c] as the [row_capacity, c] operand of the grouped GEMMs: t itself when T is a multiple of 128."""
    if r.row_capacity == t.shape[0] and t.is_contiguous():
        return t
    return gather_rows(t.contiguous(), r)


def dense_forward(x, w1, w2, b1, b2, act_id: int, need_state=True, engine=L.ENGINE_AUTO):
    """y = act(x w1^T + b1) w2 + b2 with w1 [H,d], w2 [H,d_out] (the layout of the dense FFN parameters): the MoE
    layer with one expert and the identity routing, so the activation, both biases and the pad handling are the
    fused epilogues of the grouped GEMM.  Returns (y [T,d_out], LayerState)."""
    T = x.shape[0]
    r = dense_routing(T, x.device)
    xs = _dense_rows(x, r)
    y1 = sorted_buffer(r.row_capacity, w1.shape[0], x.dtype, x.device)
    h = esmm(xs, w1.unsqueeze(0), L.B_NK, r, None if b1 is None else _f32(b1).unsqueeze(0), L.EPI_ACT, act_id, aux=y1,
             engine=engine)
    ys = esmm(h, w2.unsqueeze(0), L.B_KN, r, None if b2 is None else _f32(b2).unsqueeze(0), L.EPI_LINEAR, engine=engine)
    return ys[:T], (LayerState(r, xs, y1, h, None) if need_state else None)


def dense_backward(st: LayerState, dy, w1, w2, act_id: int, has_b1=True, has_b2=True, grad_dtype=None, engine=L.ENGINE_AUTO):
    """Gradients of dense_forward: (dx [T,d], dw1 [H,d], dw2 [H,d_out], db1 [H] | None, db2 [d_out] | None);
    bias gradients are float32."""
    r = st.routing
    T = r.num_tokens
    dys = _dense_rows(dy, r)
    db2 = ess(dys, r).view(-1) if has_b2 else None
    dw2 = estmm(st.h, dys, r, out_dtype=grad_dtype, engine=engine)[0]
    dh = _hidden_gradient(st, dys, w2.unsqueeze(0), act_id, engine, has_b1)
    db1 = (st.db1 if st.db1 is not None else ess(dh, r)).view(-1) if has_b1 else None
    st.db1 = None
    dw1 = estmm(dh, st.xs, r, out_dtype=grad_dtype, engine=engine)[0]
    dxs = esmm(dh, w1.unsqueeze(0), L.B_KN, r, None, L.EPI_LINEAR, engine=engine)
    return dxs[:T], dw1, dw2, db1, db2
