"""The pipeline-shared cache of the data-centric mode.

Each rank stores a slice of every expert's hidden dimension (`[E, loc_r, d]`, padded to the largest
slice).  Before MoE layer s computes, the full `[E, H, d]` weights are assembled here; the gather
for the next layer is issued while the current one computes, and in backward the gather of layer
s-1 overlaps the backward of layer s.  One pair of buffers (two slots, sized for the largest
layer) serves every layer of the network, which is why all FFN/MoE layers live in one module.

Reference: hexa_moe/impls/cascaded_moe.py:244-256 (pools), :388-411 (cache_gather),
hexa_moe/impls/layers.py:109-124 and :288-315 (consumers).  Differences: slices are gathered with
one all_gather_into_tensor per tensor straight from the padded parameter storage into a staging
buffer and unpacked once into `[E, H, d]` (the reference zero-fills the pool, builds W temporary
slices, gathers a list, then cat + permute-copies); two slots let the next gather run while the
current weights are still in use; on CUDA everything is enqueued on a side stream and ordered
with events, so no host thread ever blocks.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import layers as _layers


class _Pending:
    """Result of reduce_async: the reduced slices, valid after wait()."""

    def __init__(self, event, tensors):
        self._event, self._tensors = event, tensors

    def wait(self):
        if self._event is not None:
            torch.cuda.current_stream().wait_event(self._event)
        return self._tensors


class PipelineSharedCache:
    def __init__(self, owner):
        self.o = owner            # the MoE_Cascaded module (parameters, split tables, group)
        self.slots = None         # two dicts: w1, w2, b1 flat storage + bookkeeping
        self.stage_buf = None
        self.side: Optional[torch.cuda.Stream] = None

    # -- storage ---------------------------------------------------------------------------------
    def _ensure(self, device, dtype):
        o = self.o
        if self.slots is not None and self.slots[0]["w1"].device == device and self.slots[0]["w1"].dtype == dtype:
            return
        E = o.num_global_experts
        n1 = E * o.hidden_size_bound * o.input_dim_bound
        n2 = E * o.hidden_size_bound * o.output_dim_bound
        W = o.world_size
        s1 = W * E * max(o.local_dim_bound_list) * o.input_dim_bound
        s2 = W * E * max(o.local_dim_bound_list) * o.output_dim_bound
        mk = lambda n: torch.empty(n, device=device, dtype=dtype)
        self.slots = [dict(w1=mk(n1), w2=mk(n2), b1=mk(E * o.hidden_size_bound) if o.has_fc1_bias else None,
                           stage=-1, ready=None, free=None) for _ in range(2)]
        self.stage_buf = dict(w1=mk(s1), w2=mk(s2), b1=mk(W * E * max(o.local_dim_bound_list)) if o.has_fc1_bias else None)
        self.side = torch.cuda.Stream(device=device) if device.type == "cuda" else None

    def invalidate(self):
        """Forget cached weights (call when parameters may have changed, i.e. at the first MoE layer of a step)."""
        if self.slots is not None:
            for s in self.slots:
                s["stage"] = -1

    # -- gather ----------------------------------------------------------------------------------
    def _views(self, slot, stage):
        o = self.o
        E, H = o.num_global_experts, o.hidden_size_list_moe[stage]
        d_in, d_out = o.input_dim_list_moe[stage], o.output_dim_list_moe[stage]
        w1 = slot["w1"][: E * H * d_in].view(E, H, d_in)
        w2 = slot["w2"][: E * H * d_out].view(E, H, d_out)
        b1 = slot["b1"][: E * H].view(E, H) if slot["b1"] is not None else None
        return w1, w2, b1

    def _gather_into(self, slot, stage):
        o = self.o
        W, E = o.world_size, o.num_global_experts
        bound = o.local_dim_bound_list[stage]
        split = [o.local_dim_list_all[r][stage] for r in range(W)]
        w1, w2, b1 = self._views(slot, stage)
        jobs = [(o.batched_fc1_w[stage].data, self.stage_buf["w1"], w1), (o.batched_fc2_w[stage].data, self.stage_buf["w2"], w2)]
        if o.has_fc1_bias:
            jobs.append((o.batched_fc1_bias[stage].data, self.stage_buf["b1"], b1))
        for local, staging, full in jobs:
            tail = tuple(local.shape[2:])
            n = W * E * bound * (tail[0] if tail else 1)
            st = staging[:n].view((W, E, bound) + tail)
            dist.all_gather_into_tensor(st.view((W * E, bound) + tail), local.contiguous(), group=o.group)
            off = 0
            for r, nloc in enumerate(split):                      # unpack: one strided copy per rank
                full[:, off: off + nloc].copy_(st[r, :, :nloc])
                off += nloc

    def prefetch(self, stage: int):
        """Start assembling layer `stage` (no-op when out of range or already present)."""
        o = self.o
        if stage < 0 or stage >= o.total_depth_moe or o.world_size == 1:
            return
        p = o.batched_fc1_w[stage]
        self._ensure(p.device, p.dtype)
        slot = self.slots[stage % 2]
        if slot["stage"] == stage:
            return
        if self.side is None:                                    # CPU / gloo: synchronous
            self._gather_into(slot, stage)
        else:
            cur = torch.cuda.current_stream()
            if slot["free"] is not None:
                self.side.wait_event(slot["free"])               # the slot's previous reader has finished
            if stage == 0 or slot["free"] is None:
                self.side.wait_stream(cur)                       # parameters may have just been updated
            with torch.cuda.stream(self.side):
                self._gather_into(slot, stage)
                ev = torch.cuda.Event()
                ev.record(self.side)
            slot["ready"] = ev
        slot["stage"] = stage

    def get(self, stage: int):
        """Full (w1 [E,H,d_in], w2 [E,H,d_out], b1 [E,H] | None) of layer `stage`; orders the current stream after the gather."""
        self.prefetch(stage)
        slot = self.slots[stage % 2]
        if slot["ready"] is not None:
            torch.cuda.current_stream().wait_event(slot["ready"])
        return self._views(slot, stage)

    def release(self, stage: int):
        """The current stream is done reading layer `stage` (everything enqueued so far)."""
        if self.side is None or self.slots is None:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.slots[stage % 2]["free"] = ev

    # -- gradient reduction ----------------------------------------------------------------------
    def reduce_async(self, dw2, db2, split: List[int], rank: int) -> _Pending:
        """Reduce-scatter(AVG) dw2 along the hidden dimension and all-reduce(AVG) db2 on the side stream,
        so the transfer overlaps the fc1 half of the backward."""
        o = self.o
        if self.side is None:
            out = _layers.reduce_scatter_hidden_avg(dw2, split, rank, o.group)
            if db2 is not None:
                _layers.all_reduce_avg(db2, o.group)
            return _Pending(None, (out, db2))
        cur = torch.cuda.current_stream()
        self.side.wait_stream(cur)
        with torch.cuda.stream(self.side):
            out = _layers.reduce_scatter_hidden_avg(dw2, split, rank, o.group)
            if db2 is not None:
                _layers.all_reduce_avg(db2, o.group)
            ev = torch.cuda.Event()
            ev.record(self.side)
        for t in (dw2, db2, out):
            if t is not None:
                t.record_stream(self.side)
        return _Pending(ev, (out, db2))
