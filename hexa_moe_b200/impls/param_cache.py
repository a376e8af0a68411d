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

import os
import threading
import time
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

from .._lib import HexaError
from . import layers as _layers


class BarrierWatchdog:
    """Host-side deadline for stream waits that only another rank can release.

    The SM-free barrier between ranks is a `cuStreamWaitValue32` on a word that a peer writes: if that peer has
    raised, exited or taken another branch, the wait never ends, every stream ordered after it stalls, and the host
    blocks for good at its next synchronisation.  Every barrier therefore registers here a `done()` probe (an event
    recorded right behind the wait).  A daemon thread polls the oldest probes; one that stays unfinished for
    `timeout_s` after it was enqueued trips the watchdog: `release()` is called once (it writes the awaited values
    from a second stream, so the stalled streams drain - with meaningless data), `failed` names the barrier, and the
    owner raises `HexaError` at its next call instead of hanging.  No kernel spins and nothing faults.
    """

    def __init__(self, timeout_s: float, release: Callable[[], None], poll_s: float = 0.05, clock=time.monotonic,
                 on_thread_start: Optional[Callable[[], None]] = None):
        self.timeout_s, self.release, self.poll_s, self.clock = float(timeout_s), release, poll_s, clock
        self.on_thread_start = on_thread_start
        self.failed: Optional[str] = None
        self._items = []                 # (done, tag, enqueue time), oldest first
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()

    def watch(self, done: Callable[[], bool], tag: str):
        with self._lock:
            self._items.append((done, tag, self.clock()))
            if self._thread is None and self.failed is None:
                self._stop.clear()
                self._thread = threading.Thread(target=self._run, name="hexa-barrier-watchdog", daemon=True)
                self._thread.start()

    def poll_once(self) -> bool:
        """One pass of the watchdog (also what the thread runs).  Returns True when the deadline was hit."""
        with self._lock:
            while self._items and self._items[0][0]():
                self._items.pop(0)
            if not self._items or self.failed is not None:
                return self.failed is not None
            _done, tag, t0 = self._items[0]
            if self.clock() - t0 <= self.timeout_s:
                return False
            self.failed = tag
            self._items = []
        try:
            self.release()
        except Exception as exc:  # noqa: BLE001  (the failure is reported either way)
            self.failed = f"{tag} (and releasing the stalled streams failed: {exc})"
        return True

    def _run(self):
        if self.on_thread_start is not None:
            try:
                self.on_thread_start()
            except Exception:  # noqa: BLE001
                pass
        while not self._stop.wait(self.poll_s):
            if self.poll_once():
                return
            with self._lock:
                if not self._items:          # nothing outstanding: let the thread end, the next watch() restarts it
                    self._thread = None
                    return

    def pending(self) -> int:
        with self._lock:
            return len(self._items)

    def stop(self):
        self._stop.set()
        t = self._thread
        if t is not None and t is not threading.current_thread():
            t.join(timeout=2.0)
        self._thread = None


class DenseGradReducer:
    """Mean over the data-parallel ranks of the dense FFN layers' parameter gradients, bucketed and off the compute
    stream.

    The reference starts four asynchronous all-reduces per dense layer and waits for them before the layer's
    backward returns (hexa_moe/impls/layers.py:62-88).  Here backward only copies the layer's gradients into a flat
    bucket per dtype; a full bucket (HEXA_DENSE_BUCKET_MB, default 16) is all-reduced on a side stream while the rest
    of the backward pass computes, and an autograd-engine callback at the end of the pass launches what is left,
    waits, and hands every parameter a view of the reduced bucket as (or added to) its .grad.  One collective per
    bucket instead of four per layer: a network like Swin-MoE-B has 14 dense layers of 2-8 MB of gradients each."""

    def __init__(self, group):
        self.group = group
        self.side: Optional[torch.cuda.Stream] = None
        self.bucket_bytes = int(float(os.environ.get("HEXA_DENSE_BUCKET_MB", "16")) * (1 << 20))
        self._open = {}          # dtype -> [flat buffer, elements filled, [(param, offset, numel)]]
        self._done = []          # (event | None, flat buffer, entries) of buckets already launched
        self._queued = False

    def add(self, pairs):
        """pairs: [(parameter, gradient)] of one layer (gradients on the current stream)."""
        for prm, g in pairs:
            if g is None:
                continue
            st = self._open.get(g.dtype)
            n = g.numel()
            if st is not None and st[1] + n > st[0].numel():
                self._launch(g.dtype)
                st = None
            if st is None:
                cap = max(self.bucket_bytes // g.element_size(), n)
                st = self._open[g.dtype] = [torch.empty(cap, dtype=g.dtype, device=g.device), 0, []]
            st[0][st[1]: st[1] + n].copy_(g.reshape(-1))
            st[2].append((prm, st[1], n))
            st[1] += n
            if st[1] >= st[0].numel():
                self._launch(g.dtype)
        if not self._queued:
            self._queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._flush)

    def drop_stale(self):
        """Called from a dense layer's forward: gradients still queued here outside a backward pass were left by a
        backward pass that raised before its end-of-pass callback ran; they belong to no step, and the callback flag
        they left set would keep every later pass from queueing its own."""
        if self._queued and not PipelineSharedCache._in_backward():
            self._open, self._done, self._queued = {}, [], False

    def _launch(self, dtype):
        flat, fill, entries = self._open.pop(dtype)
        if fill == 0:
            return
        used = flat[:fill]
        if used.is_cuda:
            if self.side is None:
                self.side = torch.cuda.Stream(device=used.device)
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                _layers.all_reduce_avg(used, self.group)
                ev = torch.cuda.Event()
                ev.record(self.side)
        else:
            _layers.all_reduce_avg(used, self.group)
            ev = None
        self._done.append((ev, flat, entries))

    def _flush(self):
        self._queued = False
        try:
            for dtype in list(self._open):
                self._launch(dtype)
            done, self._done = self._done, []
            for ev, flat, entries in done:
                if ev is not None:
                    torch.cuda.current_stream().wait_event(ev)
                    flat.record_stream(torch.cuda.current_stream())
                for prm, off, n in entries:
                    g = flat[off: off + n].view(prm.shape)
                    if prm.grad is None:
                        prm.grad = g
                    else:
                        prm.grad.add_(g)
        finally:
            self._open, self._done = {}, []


class PipelineSharedCache:
    def __init__(self, owner):
        self.o = owner            # the MoE_Cascaded module (parameters, split tables, group)
        self.slots = None         # two dicts: w1, w2, b1 flat storage + bookkeeping
        self.stage_buf = None
        self._peers = None
        self._p2p = False
        self.side: Optional[torch.cuda.Stream] = None
        self._pending = []
        self._callback_queued = False
        self._red = None          # peer-copy reduce-scatter state (buffers, flags), built on first use
        self._watchdog: Optional[BarrierWatchdog] = None
        self.timeline = None      # a list while a caller wants spans recorded: (site, stream name, start event, end event)

    # -- instrumentation and health --------------------------------------------------------------
    def _span(self, site: str, stream_name: str, stream):
        """Context manager recording a pair of timing events around what the body enqueues on `stream`."""
        cache = self

        class _S:
            def __enter__(self_):
                self_.a = None
                if cache.timeline is not None:
                    self_.a = torch.cuda.Event(enable_timing=True)
                    self_.a.record(stream)
                return self_

            def __exit__(self_, *exc):
                if self_.a is not None and cache.timeline is not None:
                    b = torch.cuda.Event(enable_timing=True)
                    b.record(stream)
                    cache.timeline.append((site, stream_name, self_.a, b))
                return False
        return _S()

    def _compute_wait(self, ev, site: str):
        """Order the current (compute) stream after `ev`; with a timeline, record how long that held it."""
        if ev is None:
            return
        cur = torch.cuda.current_stream()
        with self._span(site, "compute", cur):
            cur.wait_event(ev)

    def check_health(self):
        """Raise if a barrier between ranks ran into its host-side deadline (a peer is gone or out of step)."""
        wd = self._watchdog
        if wd is not None and wd.failed is not None:
            raise HexaError(f"pipeline-shared cache: {wd.failed} was not reached by every rank within "
                            f"{wd.timeout_s:.0f} s (HEXA_BARRIER_TIMEOUT_S); the stalled streams were released, their "
                            "data is meaningless; a peer has failed or left")

    # -- storage ---------------------------------------------------------------------------------
    def _ensure(self, device, dtype):
        o = self.o
        if self.slots is not None and self.slots[0]["w1"].device == device and self.slots[0]["w1"].dtype == dtype:
            return
        E = o.num_global_experts
        n1 = E * o.hidden_size_bound * o.input_dim_bound
        n2 = E * o.hidden_size_bound * o.output_dim_bound
        mk = lambda n: torch.empty(n, device=device, dtype=dtype)
        self.slots = [dict(w1=mk(n1), w2=mk(n2), b1=mk(E * o.hidden_size_bound) if o.has_fc1_bias else None,
                           stage=-1, ready={}, free=None) for _ in range(2)]
        self.stage_buf = None      # staging for the NCCL path, allocated on first use
        self.side = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self._peers = None
        self._peer_ptrs = None
        self._p2p = device.type == "cuda" and os.environ.get("HEXA_P2P_GATHER", "1") != "0"

    def invalidate(self):
        """Forget cached weights (call when parameters may have changed, i.e. at the first MoE layer of a step)."""
        if self.slots is not None:
            for s in self.slots:
                s["stage"] = -1
        # reductions queued by a backward pass that never finished (it raised) belong to no step any more
        if self._callback_queued and not self._in_backward():
            self._pending, self._callback_queued = [], False

    @staticmethod
    def _in_backward() -> bool:
        try:
            return bool(torch._C._current_graph_task_id() != -1)
        except Exception:  # noqa: BLE001
            return False

    # -- gather ----------------------------------------------------------------------------------
    def _views(self, slot, stage):
        o = self.o
        E, H = o.num_global_experts, o.hidden_size_list_moe[stage]
        d_in, d_out = o.input_dim_list_moe[stage], o.output_dim_list_moe[stage]
        w1 = slot["w1"][: E * H * d_in].view(E, H, d_in)
        w2 = slot["w2"][: E * H * d_out].view(E, H, d_out)
        b1 = slot["b1"][: E * H].view(E, H) if slot["b1"] is not None else None
        return dict(w1=w1, w2=w2, b1=b1)

    def _local(self, stage):
        o = self.o
        return dict(w1=o.batched_fc1_w[stage].data, w2=o.batched_fc2_w[stage].data,
                    b1=o.batched_fc1_bias[stage].data if o.has_fc1_bias else None)

    def _peer_setup(self):
        """Map every rank's parameter slices into this process (CUDA IPC over NVLink peer memory) so that a gather
        is a handful of copy-engine transfers straight into the [E, H, d] slot: no SMs, no staging, no unpack pass.
        Returns False (and the cache falls back to NCCL all-gathers) if the mapping cannot be made."""
        o = self.o
        ptrs = tuple(t.data_ptr() for st in range(o.total_depth_moe) for t in self._local(st).values() if t is not None)
        if self._peers is not None and self._peer_ptrs == ptrs:
            return True
        try:
            from torch.multiprocessing.reductions import rebuild_cuda_tensor, reduce_tensor
            mine = [{k: (None if t is None else reduce_tensor(t)[1]) for k, t in self._local(st).items()}
                    for st in range(o.total_depth_moe)]
            everyone = [None] * o.world_size
            dist.all_gather_object(everyone, mine, group=o.group)
            peers = []
            for r, handles in enumerate(everyone):
                if r == o.local_rank:
                    peers.append([self._local(st) for st in range(o.total_depth_moe)])
                else:
                    peers.append([{k: (None if a is None else rebuild_cuda_tensor(*a)) for k, a in h.items()} for h in handles])
            # one framework copy from every peer device turns on direct peer access for this process; without it
            # the driver stages cross-device copies through host memory (26 GB/s instead of ~770 GB/s)
            probe = torch.empty(1, device=self.side.device, dtype=peers[o.local_rank][0]["w1"].dtype)
            for r in range(o.world_size):
                if r != o.local_rank:
                    probe.copy_(peers[r][0]["w1"].view(-1)[:1])
            ok = torch.tensor([1], device=self.side.device)
        except Exception:  # noqa: BLE001  (no IPC between these processes: different nodes, masked devices, ...)
            peers, ok = None, torch.tensor([0], device=self.side.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=o.group)       # all ranks take the same path
        if int(ok.item()) == 0:
            self._p2p = False
            self._peers = None
            return False
        self._peers, self._peer_ptrs = peers, ptrs
        if not getattr(self, "_atexit_registered", False):
            import atexit
            atexit.register(self.close)      # mappings of other ranks' memory must go before interpreter teardown
            self._atexit_registered = True
        return True

    def _gather_peer(self, slot, stage, order):
        """Copy-engine gather: for every tensor and every rank, E blocks of loc_r * d elements from the owner's
        parameter storage into this rank's slot."""
        from .. import ops as _ops
        o = self.o
        W, E = o.world_size, o.num_global_experts
        split = [o.local_dim_list_all[r][stage] for r in range(W)]
        views = self._views(slot, stage)
        if stage == 0 or self._sync_needed:
            # every rank's parameters are final (its optimizer has run) before anyone reads them
            with self._span("gather.params_final_barrier", "side", self.side):
                if self._red not in (None, False):
                    self._peer_barrier("parameters-final barrier before the gather of layer %d" % stage)
                else:
                    dist.all_reduce(self._flag, group=o.group)
            self._sync_needed = False
        slot.setdefault("groups", {}).pop("w1", None)
        for kind in order:
            full = views[kind]
            if full is None:
                continue
            inner = full.shape[2] if full.dim() == 3 else 1
            # The first layer's fc1 weights are the one gather of a step that nothing overlaps (it can only start when
            # the parameters are final): they arrive in groups of experts, each with its own event, and the layer
            # launches fc1 per group, so it starts after the first group instead of after the whole tensor.
            n_groups = int(os.environ.get("HEXA_GATHER_GROUPS", "4")) if (kind == "w1" and stage == 0) else 1
            n_groups = max(1, min(n_groups, E))
            bounds = [E * g // n_groups for g in range(n_groups + 1)]
            group_events = []
            for g in range(n_groups):
                e0, e1 = bounds[g], bounds[g + 1]
                with self._span("gather.copy_" + kind, "side", self.side):
                    for r in range(W):
                        rr = (o.local_rank + 1 + r) % W         # start with the neighbour: spreads the load over the links
                        src = self._peers[rr][stage][kind]
                        nloc = split[rr]
                        lo = sum(split[:rr])
                        _ops.copy_2d(full[e0:e1, lo: lo + nloc], full.stride(0), src[e0:e1], src.stride(0), nloc * inner, e1 - e0)
                ev = torch.cuda.Event()
                ev.record(self.side)
                group_events.append((e0, e1, ev))
            if n_groups > 1:
                slot["groups"][kind] = group_events
            slot["ready"][kind] = group_events[-1][2]

    def _gather_nccl(self, slot, stage, order):
        o = self.o
        W, E = o.world_size, o.num_global_experts
        bound = o.local_dim_bound_list[stage]
        split = [o.local_dim_list_all[r][stage] for r in range(W)]
        views, local = self._views(slot, stage), self._local(stage)
        if self.stage_buf is None:
            n = W * E * max(o.local_dim_bound_list) * max(o.input_dim_bound, o.output_dim_bound)
            self.stage_buf = torch.empty(n, device=local["w1"].device, dtype=local["w1"].dtype)
        for kind in order:
            full = views[kind]
            if full is None:
                continue
            tail = tuple(local[kind].shape[2:])
            inner = tail[0] if tail else 1
            st = self.stage_buf[: W * E * bound * inner].view((W, E, bound) + tail)
            dist.all_gather_into_tensor(st.view((W * E, bound) + tail), local[kind].contiguous(), group=o.group)
            off = 0
            for r, nloc in enumerate(split):                      # unpack: E blocks of nloc*inner elements per rank
                if st.is_cuda:                                    # block copy (cudaMemcpy2DAsync): no SMs spent on it
                    from .. import ops as _ops
                    _ops.copy_2d(full[:, off: off + nloc], full.stride(0), st[r], st.stride(1), nloc * inner, E)
                else:
                    full[:, off: off + nloc].copy_(st[r, :, :nloc])
                off += nloc
            if self.side is not None:
                ev = torch.cuda.Event()
                ev.record(self.side)
                slot["ready"][kind] = ev

    def prefetch(self, stage: int, order=("b1", "w1", "w2")):
        """Start assembling layer `stage` (no-op when out of range or already present).  `order`: which tensors,
        first needed first (forward: fc1's bias - tiny, so that nothing waits for it behind the weights - then fc1, then fc2;
        backward: ("w2", "w1"))."""
        o = self.o
        if stage < 0 or stage >= o.total_depth_moe or o.world_size == 1:
            return
        self.check_health()
        p = o.batched_fc1_w[stage]
        self._ensure(p.device, p.dtype)
        slot = self.slots[stage % 2]
        if slot["stage"] == stage and all(k in slot["ready"] or self.side is None for k in order if self._views(slot, stage)[k] is not None):
            return
        if slot["stage"] != stage:
            slot["ready"] = {}
        todo = tuple(k for k in order if k not in slot["ready"])
        if self.side is None:                                    # CPU / gloo: synchronous
            self._gather_nccl(slot, stage, todo)
            for k in todo:
                slot["ready"][k] = None
        else:
            use_peer = self._p2p and self._peer_setup()
            if not hasattr(self, "_flag"):
                self._flag = torch.zeros(1, device=self.side.device)
                self._sync_needed = True
            cur = torch.cuda.current_stream()
            if slot["free"] is not None:
                self.side.wait_event(slot["free"])               # the slot's previous reader has finished
            if stage == 0 or slot["free"] is None:
                self.side.wait_stream(cur)                       # parameters may have just been updated
            with torch.cuda.stream(self.side):
                if use_peer:
                    self._gather_peer(slot, stage, todo)
                else:
                    self._gather_nccl(slot, stage, todo)
        slot["stage"] = stage

    def wait(self, stage: int, kind: str):
        """Order the current stream after the arrival of one tensor ("w1", "w2" or "b1") of layer `stage`."""
        slot = self.slots[stage % 2]
        self._compute_wait(slot["ready"].get(kind), "wait." + kind)

    def ready_groups(self, stage: int, kind: str = "w1"):
        """[(first expert, end expert, wait)] when tensor `kind` of layer `stage` arrives in expert groups (wait() orders
        the current stream after a group's arrival), else None: the tensor has a single arrival event (see wait())."""
        slot = self.slots[stage % 2]
        groups = slot.get("groups", {}).get(kind)
        if not groups or slot["stage"] != stage:
            return None
        return [(e0, e1, (lambda ev=ev: self._compute_wait(ev, "wait." + kind))) for e0, e1, ev in groups]

    def get(self, stage: int, order=("b1", "w1", "w2"), wait=("w1", "b1", "w2")):
        """Full (w1 [E,H,d_in], w2 [E,H,d_out], b1 [E,H] | None) of layer `stage`.  Starts the gather if needed and
        orders the current stream after the tensors named in `wait`; call wait() for the others before using them."""
        self.prefetch(stage, order)
        v = self._views(self.slots[stage % 2], stage)
        for k in wait:
            if v[k] is not None:
                self.wait(stage, k)
        return v["w1"], v["w2"], v["b1"]

    def release(self, stage: int):
        """The current stream is done reading layer `stage` (everything enqueued so far)."""
        if self.side is None or self.slots is None:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.slots[stage % 2]["free"] = ev

    # -- reduce-scatter over peer memory (copy engines + stream memory operations, no NCCL kernels) ----------
    def _reducer_setup(self):
        """Persistent, IPC-shared buffers for the weight gradients in reduce-scatter layout ([W, E, loc, d], two per
        kind so consecutive layers alternate), a receive area, and one int32 flag per peer for an SM-free barrier."""
        if self._red is not None:
            return self._red is not False
        o = self.o
        ok = False
        try:
            if not (self._p2p and self._peer_setup()) or os.environ.get("HEXA_P2P_REDUCE", "1") == "0":
                raise RuntimeError("peer access unavailable")
            from torch.multiprocessing.reductions import rebuild_cuda_tensor, reduce_tensor
            dev, dtype = self.side.device, o.batched_fc1_w[0].dtype
            W, E = o.world_size, o.num_global_experts
            n1 = max(W * E * o.local_dim_bound_list[i] * o.input_dim_list_moe[i] for i in range(o.total_depth_moe))
            n2 = max(W * E * o.local_dim_bound_list[i] * o.output_dim_list_moe[i] for i in range(o.total_depth_moe))
            red = dict(
                grad=dict(fc1=[torch.empty(n1, device=dev, dtype=dtype) for _ in range(2)],
                          fc2=[torch.empty(n2, device=dev, dtype=dtype) for _ in range(2)]),
                recv=None, recv_elems=max(n1, n2) // W * max(W - 1, 1),     # staging of the copy-engine variant, on demand
                flags=torch.zeros(W, device=dev, dtype=torch.int32),
                seq_table=torch.arange(1, (1 << 16) + 1, device=dev, dtype=torch.int32), seq=0, seq_base=0, old_tables=[],
                free={("fc1", 0): None, ("fc1", 1): None, ("fc2", 0): None, ("fc2", 1): None})
            mine = dict(fc1=[reduce_tensor(t)[1] for t in red["grad"]["fc1"]], fc2=[reduce_tensor(t)[1] for t in red["grad"]["fc2"]],
                        flags=reduce_tensor(red["flags"])[1])
            everyone = [None] * W
            dist.all_gather_object(everyone, mine, group=o.group)
            red["peer_grad"], red["peer_flags"] = [], []
            for r, h in enumerate(everyone):
                if r == o.local_rank:
                    red["peer_grad"].append(red["grad"]); red["peer_flags"].append(red["flags"])
                else:
                    red["peer_grad"].append(dict(fc1=[rebuild_cuda_tensor(*a) for a in h["fc1"]],
                                                 fc2=[rebuild_cuda_tensor(*a) for a in h["fc2"]]))
                    red["peer_flags"].append(rebuild_cuda_tensor(*h["flags"]))
            ok = True
        except Exception:  # noqa: BLE001
            red = False
        flag = torch.tensor([1 if ok else 0], device=self.side.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=o.group)       # all ranks take the same path
        self._red = red if int(flag.item()) == 1 else False
        return self._red is not False

    def _peer_barrier(self, what: str = "barrier between ranks"):
        """Every rank's side stream has reached this point before any rank's side stream continues.  Each rank copies
        the next sequence number into its slot of every peer's flag array (4-byte peer copies) and then makes its
        stream wait until all of its own slots have reached that number.  The wait has no limit on the device; the
        host-side watchdog gives it one (see BarrierWatchdog)."""
        from .. import ops as _ops
        self.check_health()
        red, o = self._red, self.o
        red["seq"] += 1
        seq = red["seq"]
        if seq - red["seq_base"] > red["seq_table"].numel():       # next block of sequence numbers
            red["old_tables"] = [red["seq_table"]]                 # copies already enqueued may still read it
            red["seq_base"] = seq - 1
            red["seq_table"] = torch.arange(seq, seq + (1 << 16), device=red["flags"].device, dtype=torch.int32)
        val = red["seq_table"][seq - red["seq_base"] - 1: seq - red["seq_base"]]
        stream = self.side.cuda_stream
        for r in range(o.world_size):
            if r != o.local_rank:
                _ops.copy_2d(red["peer_flags"][r][o.local_rank: o.local_rank + 1], 1, val, 1, 1, 1, stream=stream)
        for r in range(o.world_size):
            if r != o.local_rank:
                _ops.stream_wait_value(red["flags"][r: r + 1], seq, stream)
        ev = torch.cuda.Event()
        ev.record(self.side)
        self._watch_barrier(ev, "%s (sequence %d)" % (what, seq))

    def _watch_barrier(self, ev, tag: str):
        if self._watchdog is None:
            timeout = float(os.environ.get("HEXA_BARRIER_TIMEOUT_S", "300"))
            dev = self.side.device
            self._watchdog = BarrierWatchdog(timeout, self._release_barriers,
                                             on_thread_start=lambda: torch.cuda.set_device(dev))
        self._watchdog.watch(ev.query, tag)

    def _release_barriers(self):
        """Watchdog action: write the newest awaited sequence number into this rank's own flag words from a second
        stream, so that every stream wait enqueued so far completes and the stalled streams drain."""
        from .. import ops as _ops
        red, o = self._red, self.o
        if red in (None, False):
            return
        seq = red["seq"]
        val = red["seq_table"][seq - red["seq_base"] - 1: seq - red["seq_base"]]
        with torch.cuda.device(self.side.device):
            rescue = torch.cuda.Stream(device=self.side.device)
            for r in range(o.world_size):
                if r != o.local_rank:
                    _ops.copy_2d(red["flags"][r: r + 1], 1, val, 1, 1, 1, stream=rescue.cuda_stream)

    def grad_buffer(self, which: str, stage: int):
        """Where ESTMM should write this layer's weight gradient so that the peer-copy reduce-scatter can read it:
        a [W, E, loc, d] view of a persistent shared buffer, or None when that path is not in use.  Orders the
        current stream after the last remote reader of the buffer's previous contents."""
        if self.side is None or not self._reducer_setup():
            return None
        o = self.o
        W, E, loc = o.world_size, o.num_global_experts, o.local_dim_list[stage]
        d = o.input_dim_list_moe[stage] if which == "fc1" else o.output_dim_list_moe[stage]
        self._compute_wait(self._red["free"][(which, stage % 2)], "wait.grad_buffer_free")
        return self._red["grad"][which][stage % 2][: W * E * loc * d].view(W, E, loc, d)

    def _reduce_peer(self, which: str, stage: int, out):
        """Side stream: out[E, loc, d] = mean over ranks of their packed gradient's slice for this rank."""
        from .. import ops as _ops
        red, o = self._red, self.o
        W, rank = o.world_size, o.local_rank
        n = out.numel()
        par = stage % 2
        with self._span("reduce.grads_complete_barrier", "side", self.side):
            self._peer_barrier("gradients-complete barrier of %s, layer %d" % (which, stage))
        if red["recv"] is None:      # allocated on the side stream, the only stream that uses it
            red["recv"] = torch.empty(red["recv_elems"], device=out.device, dtype=out.dtype)
        recv = red["recv"][: (W - 1) * n].view(W - 1, n)
        i = 0
        with self._span("reduce.copy", "side", self.side):
            for k in range(1, W):
                r = (rank + k) % W
                src = red["peer_grad"][r][which][par][rank * n: (rank + 1) * n]
                _ops.copy_2d(recv[i], n, src, n, n, 1, stream=self.side.cuda_stream)
                i += 1
        local = red["grad"][which][par][rank * n: (rank + 1) * n]
        with self._span("reduce.mean_kernel", "side", self.side):
            _ops.mean_slices(local, recv, W - 1, W, out.view(-1))
        with self._span("reduce.readers_done_barrier", "side", self.side):
            self._peer_barrier("readers-done barrier of %s, layer %d" % (which, stage))
        ev = torch.cuda.Event()
        ev.record(self.side)
        red["free"][(which, par)] = ev

    # -- gradient reduction ----------------------------------------------------------------------
    def reduce_deferred(self, stage: int, which: str, dw, db, split: List[int], rank: int, packed: bool = False,
                        defer: bool = True):
        """Average one layer's expert gradients over the ranks without stalling the compute stream.

        dw [E, H, d*] (and db: [E, H] for "fc1", [E, d_out] for "fc2") are reduce-scattered along the hidden
        dimension (fc2's bias: all-reduced) on the side stream.  With `defer` (the default) the reduced slices are
        not returned through autograd: they are accumulated into the parameters' .grad by a callback that the
        autograd engine runs when the whole backward pass has finished, so the transfer overlaps everything that is
        still to run.  With defer=False the current stream waits for the reduction and the reduced (dw, db) are
        returned, shaped like this rank's parameter slices, for the caller to hand to autograd."""
        o = self.o
        self.check_health()
        if which == "fc1":
            targets = [(o.batched_fc1_w[stage], dw, True), (o.batched_fc1_bias[stage] if o.has_fc1_bias else None, db, True)]
        else:
            targets = [(o.batched_fc2_w[stage], dw, True), (o.batched_fc2_bias[stage] if o.has_fc2_bias else None, db, False)]
        targets = [t for t in targets if t[0] is not None and t[1] is not None]

        peer_out = None
        if packed and self._red not in (None, False) and dw is not None and dw.dim() == 4:
            # allocated on the compute stream: it becomes the parameter's .grad
            peer_out = dw.new_empty(tuple(dw.shape[1:]))

        def run():
            outs = []
            for prm, g, sharded in targets:
                if sharded and peer_out is not None and g is dw:
                    self._reduce_peer(which, stage, peer_out)
                    outs.append((prm, peer_out))
                elif sharded and packed and g.dim() == prm.dim() + 1:     # already [W, E, loc, d]
                    outs.append((prm, _layers.reduce_scatter_packed_avg(g, o.group)))
                elif sharded:
                    outs.append((prm, _layers.reduce_scatter_hidden_avg(g, split, rank, o.group)))
                else:
                    outs.append((prm, _layers.all_reduce_avg(g, o.group)))
            return outs

        if self.side is None:
            ev, outs, keep = None, run(), None
        else:
            cur = torch.cuda.current_stream()
            self.side.wait_stream(cur)
            with torch.cuda.stream(self.side):
                outs = run()
                ev = torch.cuda.Event()
                ev.record(self.side)
            # the inputs stay referenced until the flush (after the compute stream has waited for `ev`), so their
            # memory cannot be handed out again while the side stream still reads it
            keep = [g for _, g, _ in targets]
        if not defer:
            self._compute_wait(ev, "wait.reduction_inline")
            for _, g in outs:
                if g.is_cuda:
                    g.record_stream(torch.cuda.current_stream())
            loc = split[rank]
            red = {id(prm): (g[:, :loc] if sharded else g) for (prm, g), (_, _, sharded) in zip(outs, targets)}
            w_prm = o.batched_fc1_w[stage] if which == "fc1" else o.batched_fc2_w[stage]
            b_prm = (o.batched_fc1_bias[stage] if o.has_fc1_bias else None) if which == "fc1" else \
                    (o.batched_fc2_bias[stage] if o.has_fc2_bias else None)
            return red.get(id(w_prm)), (red.get(id(b_prm)) if b_prm is not None else None)
        self._pending.append((ev, outs, keep))
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._flush_grads)
        return None, None

    def _flush_grads(self):
        """End of a backward pass: wait for the reductions and add their results to the parameters' .grad."""
        pending, self._pending = self._pending, []
        self._callback_queued = False
        try:
            self.check_health()
            for ev, outs, _keep in pending:
                self._compute_wait(ev, "wait.reductions_at_end_of_backward")
                for prm, g in outs:
                    if g.shape != prm.shape:        # a slice narrower than the stored (padded) parameter
                        full = torch.zeros_like(prm)
                        full[:, : g.shape[1]].copy_(g)
                        g = full
                    if prm.grad is None:
                        prm.grad = g
                    else:
                        prm.grad.add_(g)
        finally:
            self.limit_compute_sms(False)

    def uses_sms(self) -> bool:
        """True when gathers run as NCCL kernels (the peer-copy path leaves every SM to the GEMMs)."""
        return not (self._p2p and self._peers is not None)

    def reduce_uses_sms(self) -> bool:
        """True when the large gradient reductions run as NCCL kernels."""
        return self._red in (None, False)

    def close(self):
        """Drop the mappings of other ranks' memory (call on every rank before the process group is destroyed)."""
        wd, self._watchdog = self._watchdog, None
        failed = wd is not None and wd.failed is not None
        if wd is not None:
            if not failed and self.side is not None and wd.pending():
                # outstanding barriers get the same deadline here as anywhere else: never block on them for good
                t0 = time.monotonic()
                while wd.pending() and wd.failed is None and time.monotonic() - t0 < wd.timeout_s + 1.0:
                    wd.poll_once()
                    time.sleep(0.01)
                failed = wd.failed is not None
            wd.stop()
        if self.side is not None and not failed:
            torch.cuda.synchronize()
        self._pending = []
        self._callback_queued = False
        self._peers = None
        self._peer_ptrs = None
        self._red = None
        if self.side is not None:
            import gc
            gc.collect()
            torch.cuda.ipc_collect()      # give the mapped segments back before their owners exit

    def limit_compute_sms(self, on: bool):
        """While a collective may be running, keep the persistent GEMM kernels off `HEXA_COMM_SMS` SMs (default 16)
        so that NCCL's CTAs and the GEMM's static tile schedule do not wait for each other."""
        if self.side is None:
            return
        from .. import _lib
        n = 0
        if on:
            reserve = int(os.environ.get("HEXA_COMM_SMS", "16"))
            n = max(2, torch.cuda.get_device_properties(self.side.device).multi_processor_count - reserve) if reserve > 0 else 0
        _lib.lib().hexa_set_sm_limit(n)
