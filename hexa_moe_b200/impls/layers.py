"""Autograd functions of the FFN / MoE layers and the collectives around them.

Function-level contract of the reference (hexa_moe/impls/layers.py:18-478), kept:

    FusedMoE_Shared_CudaCore.apply(config, x[T,d], fc1_w[E,loc,d], fc2_w[E,loc,d_out],
                                   fc1_b[E,loc] | None, fc2_b[E,d_out] | None) -> y[T,d_out]
    MLP_Implement.apply(config, x[T,d], fc1_w[H,d], fc2_w[H,d_out], fc1_b[H] | None, fc2_b[d_out] | None)

`config.indices_` carries the k routing-id vectors out of band and `config.stage` selects the MoE
layer; backward returns gradients shaped like the inputs and decrements `config.stage`.

Differences from the reference, all deliberate:
  * the expert math runs through `config.backend` (hexa_moe_b200.ops: the sm_100a kernels behind
    the C ABI; there is no CPU path) on the merged, 128-row-aligned segmentation of all k routes,
    with bias, activation and activation derivative fused into the ESMM epilogues and no
    transposed weight copies;
  * ESTMM / ESS follow the operator definition (the reference kernels drop/duplicate 16-row chunks);
  * data-centric expert gradients are reduce-scattered (AVG) along the hidden dimension instead of
    all-reduced at full size and sliced (layers.py:431-474) - the same values, 1/W of the traffic;
  * model-centric token gradients are reduce-scattered over the token dimension; the reference
    sends its local slice to every destination (layers.py:392-396);
  * the dense FFN of 16-bit CUDA tokens runs as a one-expert layer on the same kernels (fused bias,
    activation and activation derivative); other inputs keep the PyTorch-op formulation.
"""
from __future__ import annotations

import os
from typing import Any, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor

from . import losses


# ------------------------------------------------------------------------------------------------
# small collective helpers that work with both NCCL (GPU) and gloo (CPU tests)
# ------------------------------------------------------------------------------------------------
def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _is_nccl(group) -> bool:
    return dist.get_backend(group) == "nccl"


def all_reduce_avg(t: Tensor, group) -> Tensor:
    """In-place mean over ranks (gloo has no AVG)."""
    if _world(group) == 1:
        return t
    if _is_nccl(group):
        dist.all_reduce(t, op=dist.ReduceOp.AVG, group=group)
    else:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        t.div_(_world(group))
    return t


def reduce_scatter_packed_avg(packed: Tensor, group, out: Optional[Tensor] = None) -> Tensor:
    """Mean over ranks of a gradient that is already laid out [W, E, loc, ...]: one reduce_scatter_tensor, no copies."""
    if out is None:
        out = packed.new_empty(tuple(packed.shape[1:]))
    dist.reduce_scatter_tensor(out, packed, op=dist.ReduceOp.AVG, group=group)
    return out


def reduce_scatter_hidden_avg(full: Tensor, split: List[int], rank: int, group) -> Tensor:
    """Mean over ranks of `full` [E, H, ...], returning this rank's hidden slice padded to the widest slice:
    [E, max(split), ...] with zeros behind the first split[rank] hidden units (the shape parameters are stored in).

    NCCL: one reduce_scatter_tensor over the padded slices.  gloo: all-reduce + slice."""
    W = len(split)
    lo, n, bound = sum(split[:rank]), split[rank], max(split)
    E = full.shape[0]
    tail = tuple(full.shape[2:])
    if W == 1:
        return full
    if not _is_nccl(group):
        red = all_reduce_avg(full.contiguous(), group)
        out = full.new_zeros((E, bound) + tail)
        out[:, :n].copy_(red[:, lo: lo + n])
        return out
    even = all(s_ == bound for s_ in split)
    packed = full.new_empty((W, E, bound) + tail)
    off = 0
    for r, nr in enumerate(split):
        packed[r, :, :nr].copy_(full[:, off: off + nr])
        if nr < bound:
            packed[r, :, nr:].zero_()
        off += nr
    out = full.new_empty((E, bound) + tail)
    dist.reduce_scatter_tensor(out, packed, op=dist.ReduceOp.AVG, group=group)
    return out


class _InFlight:
    """A collective that was started with async_op=True.  wait() makes the current stream (NCCL) or the host (gloo) wait
    for it and returns its result; until then the object keeps the buffers of the collective alive."""

    def __init__(self, work, finish, keep=()):
        self.work, self.finish, self.keep = work, finish, keep

    def wait(self) -> Tensor:
        if self.work is not None:
            self.work.wait()
        out = self.finish()
        self.work = self.finish = None
        self.keep = ()
        return out


def all_gather_tokens_start(t: Tensor, sizes: List[int], group) -> _InFlight:
    """Start concatenating every rank's rows ([sizes[r], ...] on rank r) in rank order."""
    W = len(sizes)
    if W == 1:
        return _InFlight(None, lambda: t)
    bound = max(sizes)
    if all(s == bound for s in sizes):
        out = t.new_empty((W * bound,) + tuple(t.shape[1:]))
        src = t.contiguous()
        return _InFlight(dist.all_gather_into_tensor(out, src, group=group, async_op=True), lambda: out, (src,))
    padded = t.new_zeros((bound,) + tuple(t.shape[1:]))
    padded[: t.shape[0]].copy_(t)
    buf = t.new_empty((W, bound) + tuple(t.shape[1:]))
    work = dist.all_gather_into_tensor(buf.view((W * bound,) + tuple(t.shape[1:])), padded, group=group, async_op=True)
    return _InFlight(work, lambda: torch.cat([buf[r, : sizes[r]] for r in range(W)], dim=0), (padded,))


def all_gather_tokens(t: Tensor, sizes: List[int], group) -> Tensor:
    return all_gather_tokens_start(t, sizes, group).wait()


def reduce_scatter_tokens_sum_start(t: Tensor, sizes: List[int], rank: int, group) -> _InFlight:
    """Start the sum over ranks of `t` [sum(sizes), ...]; the result is this rank's token chunk."""
    W = len(sizes)
    if W == 1:
        return _InFlight(None, lambda: t)
    lo = sum(sizes[:rank])
    bound = max(sizes)
    src = t.contiguous()
    if _is_nccl(group) and all(s == bound for s in sizes):
        out = t.new_empty((bound,) + tuple(t.shape[1:]))
        return _InFlight(dist.reduce_scatter_tensor(out, src, op=dist.ReduceOp.SUM, group=group, async_op=True),
                         lambda: out, (src,))
    return _InFlight(dist.all_reduce(src, op=dist.ReduceOp.SUM, group=group, async_op=True),
                     lambda: src[lo: lo + sizes[rank]].contiguous())


def reduce_scatter_tokens_sum(t: Tensor, sizes: List[int], rank: int, group) -> Tensor:
    return reduce_scatter_tokens_sum_start(t, sizes, rank, group).wait()


def token_chunks(sizes: List[int]) -> List[List[int]]:
    """Model-centric mode moves every token to every rank and the partial outputs back; cutting each rank's tokens into
    chunks lets the transfers of one chunk run beside the GEMMs of another.  Returns the per-rank cut points
    [[0, ..., sizes[r]] for r], the same number of chunks on every rank: HEXA_MC_CHUNKS, fewer when a chunk would hold
    less than HEXA_MC_MIN_CHUNK_TOKENS (default 2048) tokens of the smallest rank.  The default is one chunk: then only
    the reduce-scatter of the input gradients overlaps (with the two weight-gradient GEMMs of its layer), which was the
    fastest setting at 2 GPUs and within 1 % of two chunks at 8; more chunks hide more of the transfers but their
    GEMMs are shorter, padded per chunk and kept off the SMs reserved for NCCL.  HEXA_MC_CHUNKS=0: one chunk and
    every collective waited for where it is issued (the reference's order, layers.py:131-211, 317-396)."""
    want = max(1, int(os.environ.get("HEXA_MC_CHUNKS", "1")))
    least = max(1, int(os.environ.get("HEXA_MC_MIN_CHUNK_TOKENS", "2048")))
    C = max(1, min(want, min(sizes) // least)) if len(sizes) > 1 else 1
    return [[s * c // C for c in range(C + 1)] for s in sizes]


def _reserve_comm_sms(on: bool, t: Tensor, group):
    """While NCCL kernels are meant to run beside the persistent GEMMs, keep the GEMMs off HEXA_COMM_SMS SMs
    (default 16): their tile schedule is static, so a CTA that has to wait for an SM held by NCCL delays its launch."""
    if not (t.is_cuda and _world(group) > 1 and _is_nccl(group)):
        return
    from .. import _lib
    n = 0
    reserve = int(os.environ.get("HEXA_COMM_SMS", "16"))
    if on and reserve > 0:
        n = max(2, torch.cuda.get_device_properties(t.device).multi_processor_count - reserve)
    _lib.lib().hexa_set_sm_limit(n)


def gather_token_counts(n: int, device, group) -> List[int]:
    """Token count of every rank (the reference uses all_gather_object, layers.py:132)."""
    W = _world(group)
    if W == 1:
        return [n]
    mine = torch.tensor([n], dtype=torch.int64, device=device)
    out = torch.empty(W, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(out, mine, group=group)
    return [int(v) for v in out.tolist()]


# ------------------------------------------------------------------------------------------------
# routing glue
# ------------------------------------------------------------------------------------------------
def simplified_extract_critical(scores, top_k, loss_fn=losses.gshard_loss):
    """top-k expert ids as a list of k vectors, plus the auxiliary loss (reference layers.py:480-489)."""
    num_global_experts = int(scores.size(1))
    top_k = min(top_k, num_global_experts)
    topk_indices = torch.topk(scores, top_k, dim=1).indices
    indices_s = [col.view(-1) for col in topk_indices.chunk(top_k, dim=1)]
    l_loss = loss_fn(scores, topk_indices) if loss_fn is not None else None
    return indices_s, l_loss


def _stack_ids(indices_: List[Tensor], device) -> Tensor:
    """k int vectors [T] -> one int32 [k, T] tensor (route-major, what the routing kernel reads)."""
    return torch.stack([i.reshape(-1).to(device=device, dtype=torch.int32) for i in indices_], dim=0).contiguous()


def x_is_cuda(t: Tensor) -> bool:
    return t.is_cuda


def _cast(w: Optional[Tensor], dtype) -> Optional[Tensor]:
    if w is None:
        return None
    return w if w.dtype == dtype else w.to(dtype)


# ------------------------------------------------------------------------------------------------
# dense FFN (the layers either side of every MoE layer)
# ------------------------------------------------------------------------------------------------
def _dense_on_kernels(cfg, x: Tensor) -> bool:
    """16-bit CUDA tokens with an activation the GEMM epilogue knows run as a one-expert layer on the grouped-GEMM
    kernels (fused bias + activation, fused activation derivative); anything else is plain PyTorch."""
    if os.environ.get("HEXA_DENSE_KERNELS", "1") == "0":        # A/B switch: keep the dense FFN on PyTorch ops
        return False
    return (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and getattr(cfg, "act_id", -1) >= 0
            and getattr(cfg, "backend", None) is not None and hasattr(cfg.backend, "dense_forward")
            and x.shape[0] > 0 and x.shape[1] % 8 == 0
            and x.shape[1] >= int(os.environ.get("HEXA_DENSE_MIN_DIM", "256")))


class MLP_Implement(torch.autograd.Function):
    """y = act(x fc1_w^T + b1) fc2_w + b2 with fc1_w [H,d], fc2_w [H,d_out]; weight and bias gradients are
    averaged over the data-parallel ranks inside backward (reference layers.py:18-88)."""

    @staticmethod
    def forward(ctx: Any, config: Any, tokens_input: Tensor, fc1_w, fc2_w, fc1_bias, fc2_bias):
        ctx.config = config
        assert tokens_input.shape[1] == fc1_w.shape[1] and fc1_w.shape[0] == fc2_w.shape[0]
        if getattr(config, "dense_reducer", None) is not None:
            config.dense_reducer.drop_stale()
        ctx.params = (fc1_w, fc2_w, fc1_bias, fc2_bias)
        dtype = tokens_input.dtype
        ctx.has_b1, ctx.has_b2 = fc1_bias is not None, fc2_bias is not None
        ctx.fused = _dense_on_kernels(config, tokens_input) and fc1_w.shape[0] % 8 == 0 and fc2_w.shape[1] % 8 == 0
        if ctx.fused:
            x = tokens_input.contiguous()
            w1, w2 = _cast(fc1_w.detach(), dtype), _cast(fc2_w.detach(), dtype)
            y, st = config.backend.dense_forward(x, w1, w2, None if fc1_bias is None else fc1_bias.detach(),
                                                 None if fc2_bias is None else fc2_bias.detach(), config.act_id,
                                                 need_state=any(ctx.needs_input_grad))
            ctx.state, ctx.w = st, (w1, w2)
            ctx.param_dtypes = (fc1_w.dtype, fc2_w.dtype, None if fc1_bias is None else fc1_bias.dtype,
                                None if fc2_bias is None else fc2_bias.dtype)
            return y
        hid = tokens_input @ fc1_w.to(dtype).t()
        if fc1_bias is not None:
            hid = hid + fc1_bias.to(dtype)
        ctx.save_for_backward(tokens_input, hid, fc1_w, fc2_w)
        y = config.activation_fn(hid) @ fc2_w.to(dtype)
        if fc2_bias is not None:
            y = y + fc2_bias.to(dtype)
        return y

    @staticmethod
    def backward(ctx: Any, dy: Tensor):
        cfg = ctx.config
        if ctx.fused:
            (w1, w2), st = ctx.w, ctx.state
            ctx.state = ctx.w = None
            dx, dw1, dw2, db1, db2 = cfg.backend.dense_backward(st, dy.contiguous(), w1, w2, cfg.act_id,
                                                                has_b1=ctx.has_b1, has_b2=ctx.has_b2)
            pd = ctx.param_dtypes
            dw1, dw2 = dw1.to(pd[0]), dw2.to(pd[1])
            db1 = None if db1 is None else db1.to(pd[2])
            db2 = None if db2 is None else db2.to(pd[3])
        else:
            x, hid, fc1_w, fc2_w = ctx.saved_tensors
            with torch.enable_grad():
                hh = hid.detach().requires_grad_(True)
                act = cfg.activation_fn(hh)
                (dact,) = torch.autograd.grad(act.sum(), hh)
            act = act.detach()
            dtype = dy.dtype
            d_act = dy @ fc2_w.to(dtype).t()
            dw2 = (act.t() @ dy).to(fc2_w.dtype)
            db2 = dy.sum(0).to(fc2_w.dtype) if ctx.has_b2 else None
            d_hid = d_act * dact
            dx = d_hid @ fc1_w.to(dtype)
            dw1 = (d_hid.t() @ x).to(fc1_w.dtype)
            db1 = d_hid.sum(0).to(fc1_w.dtype) if ctx.has_b1 else None
        reducer = getattr(cfg, "dense_reducer", None)
        if _world(cfg.group) > 1 and reducer is not None and os.environ.get("HEXA_DEFER_GRADS", "1") != "0":
            # bucketed, on a side stream, delivered to .grad when the backward pass ends (see DenseGradReducer)
            reducer.add(list(zip(ctx.params, (dw1, dw2, db1, db2))))
            return None, dx, None, None, None, None
        for g in (dw2, db2, dw1, db1):
            if g is not None:
                all_reduce_avg(g, cfg.group)
        return None, dx, dw1, dw2, db1, db2


# ------------------------------------------------------------------------------------------------
# the MoE layer
# ------------------------------------------------------------------------------------------------
class FusedMoE_Shared_CudaCore(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, config: Any, tokens_input: Tensor, fc1_w, fc2_w, fc1_bias, fc2_bias):
        cfg = config
        ctx.config = cfg
        stage = cfg.stage
        ctx.stage = stage
        x = tokens_input.contiguous()
        assert x.shape[1] == fc1_w.shape[2], "token width does not match fc1_w"
        T = x.shape[0]
        dtype = x.dtype
        W, rank = cfg.world_size, cfg.local_rank
        ids = _stack_ids(cfg.indices_, x.device)                              # [k, T]
        ctx.has_b1, ctx.has_b2 = fc1_bias is not None, fc2_bias is not None
        ctx.param_dtypes = (fc1_w.dtype, fc2_w.dtype,
                            None if fc1_bias is None else fc1_bias.dtype, None if fc2_bias is None else fc2_bias.dtype)
        need_state = any(ctx.needs_input_grad)

        if cfg.data_centric:
            if W > 1:
                # full expert weights of this layer from the pipeline-shared cache; start fetching the next layer's
                # fc1 can start as soon as its weights are in; fc2's may still be arriving
                w1, w2, b1 = cfg.cache.get(stage, wait=("b1",))
                cfg.cache.prefetch(stage + 1)                     # overlaps this layer's kernels
                cfg.cache.limit_compute_sms(cfg.cache.uses_sms() and stage + 1 < cfg.cache.o.total_depth_moe)
                fc1_groups = cfg.cache.ready_groups(stage, "w1")  # the first layer's w1 arrives in groups of experts
                if fc1_groups is None or w1.dtype != dtype:
                    cfg.cache.wait(stage, "w1")
                    fc1_groups = None
                before_fc2 = lambda: cfg.cache.wait(stage, "w2")
            else:
                w1, w2, b1 = fc1_w, fc2_w, fc1_bias
                before_fc2 = fc1_groups = None
            if w1.dtype != dtype or w2.dtype != dtype:            # a cast reads both tensors now
                if before_fc2 is not None:
                    before_fc2()
                    before_fc2 = None
                w1, w2 = _cast(w1.detach(), dtype), _cast(w2.detach(), dtype)
            y, st = cfg.backend.moe_forward(x, ids, w1.detach(), w2.detach(), None if b1 is None else b1.detach(),
                                            None if fc2_bias is None else fc2_bias.detach(), cfg.act_id,
                                            act_fn=cfg.activation_fn, route_major=True, need_state=need_state,
                                            before_fc2=before_fc2, **({"fc1_groups": fc1_groups} if fc1_groups else {}))
            if W > 1:
                cfg.cache.release(stage)
                cfg.cache.limit_compute_sms(False)
            ctx.sizes = None
            ctx.local_w = (w1, w2) if W == 1 else None
        else:
            # model-centric: every rank sees all tokens and owns a slice of the hidden dimension
            # (the token chunks are gathered up front; the partial outputs of chunk c travel while chunk c+1 computes)
            sizes = gather_token_counts(T, x.device, cfg.group)
            cuts = token_chunks(sizes)
            C = len(cuts[0]) - 1
            chunk_sizes = [[cuts[r][c + 1] - cuts[r][c] for r in range(W)] for c in range(C)]
            mine = cuts[rank]
            ids_t = ids.t().contiguous()                                                    # [T, k]
            arriving = [(all_gather_tokens_start(x[mine[c]: mine[c + 1]], chunk_sizes[c], cfg.group),
                         all_gather_tokens_start(ids_t[mine[c]: mine[c + 1]], chunk_sizes[c], cfg.group)) for c in range(C)]
            loc = cfg.local_dim_list_all[rank][stage]
            w1 = _cast(fc1_w.detach()[:, :loc], dtype)
            w2 = _cast(fc2_w.detach()[:, :loc], dtype)
            b1 = None if fc1_bias is None else fc1_bias.detach()[:, :loc]
            b2 = fc2_bias.detach() if (fc2_bias is not None and rank == 0) else None       # bias enters the sum once
            _reserve_comm_sms(C > 1, x, cfg.group)
            st, leaving = [], []
            for c in range(C):
                x_all = arriving[c][0].wait()
                ids_all = arriving[c][1].wait().t().contiguous()                            # [k, tokens of the chunk]
                y_all, st_c = cfg.backend.moe_forward(x_all, ids_all, w1, w2, b1, b2, cfg.act_id, act_fn=cfg.activation_fn,
                                                      route_major=True, need_state=need_state)
                leaving.append(reduce_scatter_tokens_sum_start(y_all, chunk_sizes[c], rank, cfg.group))
                st.append(st_c)
            _reserve_comm_sms(False, x, cfg.group)
            parts = [p.wait() for p in leaving]
            y = parts[0] if C == 1 else torch.cat(parts, dim=0)
            ctx.sizes = (chunk_sizes, mine)
            ctx.local_w = (w1, w2)
        ctx.state = st
        return y.reshape(T, -1)

    @staticmethod
    def backward(ctx: Any, j_tokens_output: Tensor):
        cfg = ctx.config
        stage = ctx.stage
        st = ctx.state
        W, rank = cfg.world_size, cfg.local_rank
        dy = j_tokens_output.contiguous()
        dtype = dy.dtype
        w1_dt, w2_dt, b1_dt, b2_dt = ctx.param_dtypes
        be = cfg.backend

        if cfg.data_centric:
            if W > 1:
                w1, w2, _ = cfg.cache.get(stage, order=("w2", "w1"), wait=("w2", "w1"))
                cfg.cache.prefetch(stage - 1, order=("w2", "w1"))
                w1, w2 = _cast(w1.detach(), dtype), _cast(w2.detach(), dtype)
            else:
                w1, w2 = ctx.local_w
            split = [cfg.local_dim_list_all[r][stage] for r in range(W)]
            # with equal slices on NCCL the weight gradients are produced directly in the [W, E, loc, d] layout the
            # reduce-scatter reads (no packing pass)
            packed = W > 1 and x_is_cuda(dy) and _is_nccl(cfg.group) and all(s_ == split[0] for s_ in split)
            kw = dict(ranks=W) if packed else {}
            kw2 = dict(kw, dw_out=cfg.cache.grad_buffer("fc2", stage)) if packed else {}
            dh, dw2, db2 = be.moe_backward_fc2(st, dy, w2, cfg.act_id, has_b2=ctx.has_b2, grad_dtype=w2_dt, want_db1=ctx.has_b1, **kw2)
            # By default the reduced gradients are added to the parameters' .grad by a callback at the end of the
            # backward pass (nothing waits for the transfer); HEXA_DEFER_GRADS=0 returns them through autograd instead
            # (hooks, torch.autograd.grad and wrappers that inspect the returned gradients then see them).
            defer = os.environ.get("HEXA_DEFER_GRADS", "1") != "0"
            red = {}
            if W > 1:   # reductions run on the side stream
                red["fc2"] = cfg.cache.reduce_deferred(stage, "fc2", dw2, None if db2 is None else db2.to(b2_dt), split, rank,
                                                       packed, defer=defer)
                cfg.cache.limit_compute_sms(cfg.cache.reduce_uses_sms())
            if packed:
                kw["dw_out"] = cfg.cache.grad_buffer("fc1", stage)
            if W > 1:   # fc1's gradients start their reduction before the input-gradient GEMM is even launched
                def _after(g, b):
                    red["fc1"] = cfg.cache.reduce_deferred(stage, "fc1", g, None if b is None else b.to(b1_dt), split, rank,
                                                           packed, defer=defer)
                kw["after_dw"] = _after
            dx, dw1, db1 = be.moe_backward_fc1(st, dh, w1, has_b1=ctx.has_b1, grad_dtype=w1_dt, **kw)
            if W > 1:
                cfg.cache.release(stage)
                if defer:
                    dw1 = dw2 = db1 = db2 = None
                else:
                    (dw2, db2), (dw1, db1) = red["fc2"], red["fc1"]
        else:
            # per chunk: input gradients first, their reduce-scatter then runs beside the two weight-gradient GEMMs
            chunk_sizes, mine = ctx.sizes
            C = len(chunk_sizes)
            w1, w2 = ctx.local_w
            arriving = [all_gather_tokens_start(dy[mine[c]: mine[c + 1]], chunk_sizes[c], cfg.group) for c in range(C)]
            grads, leaving = None, []
            _reserve_comm_sms(C > 1, dy, cfg.group)
            for c in range(C):
                dx_all, kept = be.moe_backward_inputs(st[c], arriving[c].wait(), w1, w2, cfg.act_id, want_db1=ctx.has_b1)
                leaving.append(reduce_scatter_tokens_sum_start(dx_all, chunk_sizes[c], rank, cfg.group))
                if os.environ.get("HEXA_MC_CHUNKS") == "0":
                    done = leaving[-1].wait()
                    leaving[-1] = _InFlight(None, lambda done=done: done)
                else:
                    _reserve_comm_sms(W > 1, dy, cfg.group)
                grads = be.moe_backward_params(st[c], kept, has_b1=ctx.has_b1, has_b2=ctx.has_b2, grad_dtype=w1_dt, into=grads)
                st[c] = None
            _reserve_comm_sms(False, dy, cfg.group)
            dw1, dw2, db1, db2 = grads
            if dw2.dtype != w2_dt:
                dw2 = dw2.to(w2_dt)
            parts = [p.wait() for p in leaving]
            dx = parts[0] if C == 1 else torch.cat(parts, dim=0)
        ctx.state = None
        cfg.stage = stage - 1
        if db1 is not None:
            db1 = db1.to(b1_dt)
        if db2 is not None:
            db2 = db2.to(b2_dt)
        return None, dx, dw1, dw2, db1, db2
