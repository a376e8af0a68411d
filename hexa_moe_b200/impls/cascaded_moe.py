"""MoE_Cascaded / MoE_Buffer: the drop-in module that owns every FFN and MoE layer of a network.

Public surface of the reference kept unchanged (hexa_moe/impls/cascaded_moe.py:38-80, 82-621):
constructor arguments and defaults, `forward(depth_idx, input, gate_index=0, top_k=None,
a2a_ffn_overlap_degree=None, reserve_dims=1) -> (y, l_aux)`, `cuda_cache()`, `cache_gather(d)`,
`load_ckpt`, `save_ckpt`, the attributes a model reads (`sharded_count`, `num_global_experts`, ...)
and the parameter names/shapes (`batched_fc1_w.{i} [E, loc_bound, d_in]`, `batched_fc2_w.{i}
[E, loc_bound, d_out]`, `batched_fc1_bias.{i} [E, loc_bound]`, `batched_fc2_bias.{i} [E, d_out]`,
`mlp_fc1_w.{j} [H, d]`, `mlp_fc2_w.{j} [H, d_out]`, `mlp_fc1_b.{j}`, `mlp_fc2_b.{j}`,
`gates.{i}.*`), so state dicts load either way.

Documented differences:
  * expert parameters are passed to the autograd function live, so they receive gradients (the
    reference passes `.data`, cascaded_moe.py:606-611, and silently trains only fc2's bias);
  * tokens keep the module's compute dtype (parameter dtype, or the autocast dtype); the gate runs
    in fp32 when `fp32_gate`.  The reference re-runs routing under a forced fp16 autocast on CUDA
    (:586-589); bf16 is supported here and does not exist there;
  * a `cosine_top` gate stays a cosine gate for every MoE layer (the reference's gate dict is
    mutated to 'top' after the first layer, :299-317);
  * a process group is optional: without torch.distributed the module runs as world size 1.
"""
from __future__ import annotations

import logging
import os
import re
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import Tensor
from torch.nn import ModuleList, Parameter, ParameterList

from .. import _lib as L
from . import losses
from .activations import classify
from .gating import GATES, fused_topk_gshard, fused_topk_load_importance
from .layers import FusedMoE_Shared_CudaCore, MLP_Implement, simplified_extract_critical
from .param_cache import DenseGradReducer, PipelineSharedCache


class AttrDict(dict):
    """dict with attribute access (the reference carries layer state in an EasyDict)."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k)

    def __setattr__(self, k, v):
        self[k] = v


def _plist(shapes: List[Optional[tuple]]):
    return ParameterList([None if s is None else Parameter(torch.empty(*s)) for s in shapes])


def split_hidden(hidden_size: int, proportion: List[float]) -> List[int]:
    """Hidden units per rank: floor(p * H), remainder handed out one at a time from rank 0
    (the Triton variant's rule, cascaded_moe.py:346-352)."""
    dims = [int(p * hidden_size) for p in proportion]
    i = 0
    while sum(dims) < hidden_size:
        dims[i] += 1
        i = (i + 1) % len(dims)
    return dims


class MoE_Buffer(torch.nn.Module):
    """CPU-resident, unsharded copy of the expert parameters used to save / load checkpoints."""

    def __init__(self, model_dim_list_moe: list, num_global_experts: int, total_depth_moe: int, mlp_ratio=4.,
                 output_dim_list_moe=None, mlp_fc1_bias=True, mlp_fc2_bias=True):
        super().__init__()
        self.total_depth_moe = total_depth_moe
        self.input_dim_list_moe = model_dim_list_moe
        self.hidden_size_list_moe = [int(mlp_ratio * d) for d in model_dim_list_moe]
        self.num_global_experts = num_global_experts
        self.output_dim_list_moe = output_dim_list_moe or model_dim_list_moe
        self.has_fc1_bias, self.has_fc2_bias = mlp_fc1_bias, mlp_fc2_bias
        E, n = num_global_experts, total_depth_moe
        H, di, do = self.hidden_size_list_moe, self.input_dim_list_moe, self.output_dim_list_moe
        self.batched_fc1_w = _plist([(E, H[i], di[i]) for i in range(n)])
        self.batched_fc2_w = _plist([(E, H[i], do[i]) for i in range(n)])
        self.batched_fc1_bias = _plist([(E, H[i]) if mlp_fc1_bias else None for i in range(n)])
        self.batched_fc2_bias = _plist([(E, do[i]) if mlp_fc2_bias else None for i in range(n)])


class MoE_Cascaded(torch.nn.Module):
    def __init__(self, gate_type, model_dim_list: list, moe_idx_list: list, num_global_experts: int, total_depth: int,
                 data_centric: True, mlp_ratio=4., mlp_proportion=None, output_dim_list=None, mlp_fc1_bias=True,
                 mlp_fc2_bias=True, activation_fn=None, activation_fn_with_self=None, result_func=None, group=None,
                 seeds=None, a2a_ffn_overlap_degree=1, batch_prioritized_routing=False, normalize_gate=True,
                 is_gshard_loss=True, parallel_type='adaptive:1', use_2dh=False):
        super().__init__()
        self._dist = dist.is_available() and dist.is_initialized()
        self.group = (group or dist.group.WORLD) if self._dist else None
        self.world_size = dist.get_world_size(self.group) if self._dist else 1
        self.local_rank = dist.get_rank(self.group) if self._dist else 0
        self.result_func = result_func
        self.skip_moe = int(os.environ.get('SKIP_MOE', '0')) != 0
        self.batch_prioritized_routing = batch_prioritized_routing or int(os.environ.get('BATCH_PRIO', 0)) != 0
        self.normalize_gate = normalize_gate
        self.is_gshard_loss = is_gshard_loss
        self.a2a_ffn_overlap_degree = a2a_ffn_overlap_degree
        self.use_2dh = use_2dh
        if seeds is not None and seeds[1] is not None:
            torch.manual_seed(seeds[1])

        # ---- which depths are MoE and which are dense ----
        self.moe_idx_list = moe_idx_list
        self.mlp_idx_list = [i for i in range(total_depth) if i not in moe_idx_list]
        out_dims = output_dim_list or model_dim_list
        self.total_depth_moe, self.total_depth_mlp = len(self.moe_idx_list), len(self.mlp_idx_list)
        self.input_dim_list_moe = [model_dim_list[i] for i in self.moe_idx_list]
        self.output_dim_list_moe = [out_dims[i] for i in self.moe_idx_list]
        self.hidden_size_list_moe = [int(d * mlp_ratio) for d in self.input_dim_list_moe]
        self.input_dim_list_mlp = [model_dim_list[i] for i in self.mlp_idx_list]
        self.output_dim_list_mlp = [out_dims[i] for i in self.mlp_idx_list]
        self.hidden_size_list_mlp = [int(d * mlp_ratio) for d in self.input_dim_list_mlp]
        self.has_fc1_bias, self.has_fc2_bias = mlp_fc1_bias, mlp_fc2_bias
        self.num_global_experts = num_global_experts
        self.is_cuda = None
        self.kernel_pool = dict()

        # ---- Tutel leftovers the reference parses and consumers may read ----
        self.sharded_count = self.world_size // num_global_experts if num_global_experts < self.world_size else 1
        self.auto_parallel, self.adaptive_degree, self.use_model_parallel = False, self.sharded_count, True
        self.valid_rs = [0] + [i for i in range(1, self.sharded_count + 1) if self.sharded_count % i == 0]
        if parallel_type.startswith('adaptive:'):
            self.adaptive_degree = min(max(int(parallel_type[parallel_type.index(':') + 1:]), 0), self.sharded_count)
            if self.adaptive_degree not in self.valid_rs:
                raise Exception("Unexpected value of adaptive_degree: %d, expecting a candidate within %s." %
                                (self.adaptive_degree, self.valid_rs))
        elif self.sharded_count == 1:
            pass
        elif parallel_type in ('data', 'model'):
            self.adaptive_degree = 1 if parallel_type == 'data' else self.sharded_count
        elif parallel_type == 'auto':
            self.adaptive_degree = 1
        else:
            raise Exception('Unrecognized parallel type specified: %s' % parallel_type)

        # ---- hidden-dimension sharding ----
        if mlp_proportion is None:
            self.mlp_proportion = [1.0 / self.world_size] * self.world_size
        else:
            assert len(mlp_proportion) == self.world_size and abs(sum(mlp_proportion) - 1) < 0.001, "incorrect mlp_proportion"
            self.mlp_proportion = mlp_proportion
        self.local_dim_list_all, self.ids_list_global, self.local_dim_bound_list = self.dim_split(self.hidden_size_list_moe)
        self.local_dim_list = self.local_dim_list_all[self.local_rank]
        self.input_dim_bound = max(self.input_dim_list_moe, default=0)
        self.hidden_size_bound = max(self.hidden_size_list_moe, default=0)
        self.output_dim_bound = max(self.output_dim_list_moe, default=0)
        self.local_dim_bound = max(self.local_dim_list, default=0)

        # ---- parameters ----
        E, nm, nd = num_global_experts, self.total_depth_moe, self.total_depth_mlp
        lb = self.local_dim_bound_list
        self.batched_fc1_w = _plist([(E, lb[i], self.input_dim_list_moe[i]) for i in range(nm)])
        self.batched_fc2_w = _plist([(E, lb[i], self.output_dim_list_moe[i]) for i in range(nm)])
        self.batched_fc1_bias = _plist([(E, lb[i]) if mlp_fc1_bias else None for i in range(nm)])
        self.batched_fc2_bias = _plist([(E, self.output_dim_list_moe[i]) if mlp_fc2_bias else None for i in range(nm)])
        self.mlp_fc1_w = _plist([(self.hidden_size_list_mlp[i], self.input_dim_list_mlp[i]) for i in range(nd)])
        self.mlp_fc2_w = _plist([(self.hidden_size_list_mlp[i], self.output_dim_list_mlp[i]) for i in range(nd)])
        self.mlp_fc1_b = _plist([(self.hidden_size_list_mlp[i],) if mlp_fc1_bias else None for i in range(nd)])
        self.mlp_fc2_b = _plist([(self.output_dim_list_mlp[i],) if mlp_fc2_bias else None for i in range(nd)])

        # ---- activation ----
        if activation_fn_with_self is not None:
            assert activation_fn is None, "Option `activation_fn_with_self` has been specified, please keep exactly one of them."
            activation_fn = lambda x: activation_fn_with_self(x, self)
        if activation_fn is None:
            activation_fn = lambda x: F.relu(x)

        # ---- state shared with the autograd functions ----
        from .. import ops as _ops
        cfg = AttrDict()
        cfg.activation_fn = activation_fn
        cfg.act_id = classify(activation_fn)          # fused epilogue id, or -1: call activation_fn between the ESMMs
        cfg.backend = _ops                            # the CUDA kernels; there is no other execution path
        cfg.stage = 0
        cfg.indices_ = None
        cfg.world_size, cfg.local_rank, cfg.group = self.world_size, self.local_rank, self.group
        cfg.has_fc1_bias, cfg.has_fc2_bias = mlp_fc1_bias, mlp_fc2_bias
        cfg.input_dim_list_moe, cfg.output_dim_list_moe = self.input_dim_list_moe, self.output_dim_list_moe
        cfg.hidden_size_list_moe = self.hidden_size_list_moe
        cfg.local_dim_list, cfg.local_dim_list_all = self.local_dim_list, self.local_dim_list_all
        cfg.ids_list_global = self.ids_list_global
        cfg.num_global_experts = int(num_global_experts)
        cfg.data_centric = bool(data_centric)
        cfg.cache = PipelineSharedCache(self) if data_centric else None
        cfg.dense_reducer = DenseGradReducer(self.group) if self.world_size > 1 else None
        self.dispatch_params = cfg

        self._init_moe()

        # ---- gates: one per (MoE depth, gate spec) ----
        if isinstance(gate_type, str):
            assert re.match(r'^Top[0-9]+Gate$', gate_type), "Unrecognized gate_type: %s" % gate_type
            top_k = int(gate_type[3:-4])
            logging.warning(f"gate_type value `{gate_type}` has been deprecated, please use gate_type = "
                            f"{{'type': 'top', 'k': {top_k}}} instead.")
            gate_type = {'type': 'top', 'k': top_k}
        if not isinstance(gate_type, list):
            gate_type = [gate_type]
        self.gate_len = len(gate_type)
        gates = []
        for j in range(nm):
            for gi, spec in enumerate(gate_type):
                opts = dict(spec)
                kind = opts.pop('type')
                assert re.match(r'[a-zA-Z0-9\_]+', kind), "Gate type must only include digits, letters and underline characters."
                if kind not in GATES:
                    raise Exception("Unrecognized gate_type: %s" % kind)
                if seeds is not None and seeds[0] is not None:
                    torch.manual_seed(seeds[0] + gi)
                gate = GATES[kind](model_dim=self.input_dim_list_moe[j], num_global_experts=num_global_experts, **opts)
                if not hasattr(gate, 'gate_noise'):
                    gate.gate_noise = opts.get('gate_noise', 0.0)
                gates.append(gate)
        self.gates = ModuleList(gates)
        if seeds is not None and len(seeds) > 2 and seeds[2] is not None:
            torch.manual_seed(seeds[2])

    # ------------------------------------------------------------------------------------------
    def _init_moe(self):
        """Truncated normal (std 0.005) weights, zero biases (reference cascaded_moe.py:324-339)."""
        tn = torch.nn.init.trunc_normal_
        for i in range(self.total_depth_moe):
            tn(self.batched_fc1_w[i].data, std=0.005)
            tn(self.batched_fc2_w[i].data, std=0.005)
            if self.has_fc1_bias:
                self.batched_fc1_bias[i].data.zero_()
            if self.has_fc2_bias:
                self.batched_fc2_bias[i].data.zero_()
        for i in range(self.total_depth_mlp):
            tn(self.mlp_fc1_w[i].data, std=0.005)
            tn(self.mlp_fc2_w[i].data, std=0.005)
            if self.has_fc1_bias:
                self.mlp_fc1_b[i].data.zero_()
            if self.has_fc2_bias:
                self.mlp_fc2_b[i].data.zero_()

    def dim_split(self, hidden_size_list):
        """Per rank and per MoE layer: slice width, the hidden indices of the slice, and the widest slice."""
        W = self.world_size
        dims_global = [[] for _ in range(W)]
        ids_global = [[] for _ in range(W)]
        bounds = []
        for H in hidden_size_list:
            dims = split_hidden(H, self.mlp_proportion)
            start = 0
            for r in range(W):
                dims_global[r].append(dims[r])
                ids_global[r].append(list(range(start, start + dims[r])))
                start += dims[r]
            bounds.append(max(dims))
        return dims_global, ids_global, bounds

    # ---- cache API kept for callers of the reference ------------------------------------------------
    def cuda_cache(self):
        """The reference moves its CPU-allocated pools to the GPU here; the cache of this module
        allocates on the parameters' device on first use, so this only validates placement."""
        return self

    def cache_gather(self, depth_idx=0):
        """Start assembling the full expert weights of MoE layer `depth_idx` (asynchronous on CUDA)."""
        if self.dispatch_params.data_centric and self.world_size > 1:
            self.dispatch_params.cache.prefetch(depth_idx)

    # ---- checkpoint helpers --------------------------------------------------------------------------
    def _slice(self, depth):
        lo = sum(self.local_dim_list_all[r][depth] for r in range(self.local_rank))
        return lo, lo + self.local_dim_list[depth]

    def load_ckpt(self, load_moe: MoE_Buffer, src_rank=0):
        """Fill the local slices from an unsharded MoE_Buffer held on `src_rank` (reference :465-525)."""
        for i in range(self.total_depth_moe):
            tensors = [load_moe.batched_fc1_w[i].data, load_moe.batched_fc2_w[i].data]
            if self.has_fc1_bias:
                tensors.append(load_moe.batched_fc1_bias[i].data)
            if self.has_fc2_bias:
                tensors.append(load_moe.batched_fc2_bias[i].data)
            dev = self.batched_fc1_w[i].device
            full = [t.to(dev) if self.local_rank == src_rank else torch.empty_like(t, device=dev) for t in tensors]
            if self.world_size > 1:
                for t in full:
                    dist.broadcast(t, src=src_rank, group=self.group)
            lo, hi = self._slice(i)
            n = hi - lo
            self.batched_fc1_w[i].data[:, :n].copy_(full[0][:, lo:hi])
            self.batched_fc2_w[i].data[:, :n].copy_(full[1][:, lo:hi])
            j = 2
            if self.has_fc1_bias:
                self.batched_fc1_bias[i].data[:, :n].copy_(full[j][:, lo:hi]); j += 1
            if self.has_fc2_bias:
                self.batched_fc2_bias[i].data.copy_(full[j])
        if self.dispatch_params.cache is not None:
            self.dispatch_params.cache.invalidate()

    def save_ckpt(self, dst_moe: MoE_Buffer, dst_rank=0):
        """Assemble the unsharded parameters into `dst_moe` on `dst_rank` (reference :413-463)."""
        W = self.world_size
        for i in range(self.total_depth_moe):
            pairs = [(self.batched_fc1_w[i].data, dst_moe.batched_fc1_w[i]), (self.batched_fc2_w[i].data, dst_moe.batched_fc2_w[i])]
            if self.has_fc1_bias:
                pairs.append((self.batched_fc1_bias[i].data, dst_moe.batched_fc1_bias[i]))
            for local, dst in pairs:
                if W > 1:
                    buf = local.new_empty((W,) + tuple(local.shape))
                    dist.all_gather_into_tensor(buf.view((W * local.shape[0],) + tuple(local.shape[1:])), local.contiguous(),
                                                group=self.group)
                else:
                    buf = local.unsqueeze(0)
                if self.local_rank == dst_rank:
                    off = 0
                    for r in range(W):
                        n = self.local_dim_list_all[r][i]
                        dst.data[:, off: off + n] = buf[r, :, :n].cpu()
                        off += n
            if self.has_fc2_bias and self.local_rank == dst_rank:
                dst_moe.batched_fc2_bias[i].data = self.batched_fc2_bias[i].data.cpu()

    # ---- forward ----------------------------------------------------------------------------------------
    def _route(self, gate, x, top_k):
        logits = gate(x)
        if self.training and gate.gate_noise > 0:
            logits_w_noise = logits + gate.gate_noise * torch.randn_like(logits) / self.num_global_experts
        else:
            logits_w_noise = logits
        if self.is_gshard_loss:
            fused = fused_topk_gshard(logits_w_noise, top_k, getattr(self.dispatch_params, "backend", None))
            if fused is not None:
                return fused
        elif logits_w_noise is not logits:
            fused = fused_topk_load_importance(logits, logits_w_noise, top_k, gate.gate_noise,
                                               getattr(self.dispatch_params, "backend", None))
            if fused is not None:
                return fused
        scores = F.softmax(logits_w_noise, dim=1)
        if self.is_gshard_loss:
            loss_fn = losses.gshard_loss
        else:
            loss_fn = lambda gates, ids: losses.load_importance_loss(
                F.softmax(logits, dim=1), logits_w_noise.gather(index=ids, dim=1), self.num_global_experts, gate.gate_noise)
        return simplified_extract_critical(scores, top_k=top_k, loss_fn=loss_fn)

    def forward(self, depth_idx: int, input: Tensor, gate_index=0, top_k=None, a2a_ffn_overlap_degree=None, reserve_dims=1):
        cfg = self.dispatch_params
        is_moe = depth_idx in self.moe_idx_list
        i_moe = self.moe_idx_list.index(depth_idx) if is_moe else -1
        i_mlp = -1 if is_moe else self.mlp_idx_list.index(depth_idx)

        if i_moe == 0 and cfg.data_centric and self.world_size > 1:
            cfg.cache.invalidate()            # parameters may have changed since the previous step
            cfg.cache.prefetch(0)
        if self.skip_moe:
            return (self.result_func(input) if self.result_func is not None else input), None

        original_shape, original_dtype = input.shape, input.dtype
        assert len(original_shape) >= 2, "Input data must be at least 2D tensor: (s)amples, .., (m)odel_dim"
        x = input.reshape(-1, original_shape[-reserve_dims:].numel())
        if torch.is_autocast_enabled():
            x = x.to(torch.get_autocast_gpu_dtype() if x.is_cuda else torch.get_autocast_cpu_dtype())
        else:
            for p in self.parameters():
                x = x.to(p.dtype)
                break

        if not is_moe:
            y = MLP_Implement.apply(cfg, x, self.mlp_fc1_w[i_mlp], self.mlp_fc2_w[i_mlp], self.mlp_fc1_b[i_mlp],
                                    self.mlp_fc2_b[i_mlp]).to(x.dtype)
            y = y.view(list(original_shape[:-reserve_dims]) + list(y.shape[-reserve_dims:])).to(original_dtype)
            return (self.result_func(y) if self.result_func is not None else y), 0

        gate = self.gates[i_moe * self.gate_len + gate_index]
        if a2a_ffn_overlap_degree is not None:
            self.a2a_ffn_overlap_degree = a2a_ffn_overlap_degree
        indices_, l_aux = self._route(gate, x, top_k or gate.top_k)
        assert x.is_contiguous(), "Input tensor for encode/decode should be in contiguous memory format."
        cfg.indices_ = [i.to(torch.int32).view(-1) for i in indices_]
        cfg.stage = i_moe

        loc = self.local_dim_list[i_moe]
        w1 = self.batched_fc1_w[i_moe][:, :loc]
        w2 = self.batched_fc2_w[i_moe][:, :loc]
        b1 = self.batched_fc1_bias[i_moe][:, :loc] if self.has_fc1_bias else None
        b2 = self.batched_fc2_bias[i_moe] if self.has_fc2_bias else None
        y = FusedMoE_Shared_CudaCore.apply(cfg, x, w1, w2, b1, b2).to(x.dtype)
        y = y.view(list(original_shape[:-reserve_dims]) + list(y.shape[-reserve_dims:])).to(original_dtype)
        return (self.result_func(y) if self.result_func is not None else y), l_aux
