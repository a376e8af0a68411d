"""Router networks of the MoE layers, and the fused softmax / top-k / GShard-loss step that follows them.

Two gate types, selected by gate_type['type'] exactly as in the reference ('top' and
'cosine_top', hexa_moe/gates/top.py:6-25 and hexa_moe/gates/cosine_top.py:7-37).  Parameter
names are kept (`wg.weight`; `temperature`, `cosine_projector.*`, `sim_matrix`) so that state
dicts are interchangeable.  Both accept only `capacity_factor` and `gate_noise` as extra options.

The projections themselves are library GEMMs (a d x E product is not kernel work); what follows the logits
(softmax, top-k, the int32 route-major ids, the GShard loss and its gradient) is two kernels of this library.
"""
import math
import os

import torch
import torch.nn.functional as F


def _check_options(options):
    for opt in options:
        if opt not in ("capacity_factor", "gate_noise"):
            raise Exception("Unrecognized argument provided to Gating module: %s" % opt)


def _split_terms(t, dtype, n):
    """t (fp32) as n tensors of `dtype` whose sum reproduces t: each term is the rounding of what the previous ones
    left over.  Three bf16 terms carry 24 mantissa bits, i.e. all of an fp32 value."""
    terms, rest = [], t
    for _ in range(n):
        p = rest.to(dtype)
        terms.append(p)
        rest = rest - p.float()
    return terms


class _SplitPrecisionLinear(torch.autograd.Function):
    """logits = x W^T for bf16 tokens x [T,d] and an fp32 gate weight W [E,d], with fp32-GEMM accuracy but on the
    tensor cores and without materialising an fp32 copy of the tokens.

    x is exact in bf16 and W = hi + mid + lo exactly, so one bf16 GEMM against the stacked terms [3E,d] with fp32
    accumulation yields three partial logits whose sum differs from an fp32 GEMM only by summation order.  Backward
    does the same for the fp32 logit gradient: dW = sum of three (term^T x) products, and the token gradient, which
    leaves in bf16 anyway, keeps the leading cross terms (hi*hi + lo*hi + hi*mid)."""

    @staticmethod
    def forward(ctx, x, w):
        E = w.shape[0]
        w_terms = torch.cat(_split_terms(w.detach(), x.dtype, 3), dim=0)            # [3E, d]
        part = torch.mm(x, w_terms.t(), out_dtype=torch.float32)                    # [T, 3E]
        ctx.save_for_backward(x, w_terms)
        return (part[:, :E] + part[:, E:2 * E]) + part[:, 2 * E:]

    @staticmethod
    def backward(ctx, dlogits):
        x, w_terms = ctx.saved_tensors
        E = w_terms.shape[0] // 3
        dx = dw = None
        g_terms = _split_terms(dlogits.float(), x.dtype, 3)
        if ctx.needs_input_grad[1]:
            part = torch.mm(torch.cat(g_terms, dim=1).t(), x, out_dtype=torch.float32)   # [3E, d]
            dw = (part[:E] + part[E:2 * E]) + part[2 * E:]
        if ctx.needs_input_grad[0]:
            g = torch.cat([g_terms[0], g_terms[1], g_terms[0]], dim=1)              # [T, 3E]
            w = torch.cat([w_terms[:E], w_terms[:E], w_terms[E:2 * E]], dim=0)      # [3E, d]
            dx = torch.mm(g, w)
        return dx, dw


class LinearTopKGate(torch.nn.Module):
    """Bias-free linear projection to expert logits; optionally kept and evaluated in fp32."""

    def __init__(self, model_dim, num_global_experts, k=1, fp32_gate=False, **options):
        super().__init__()
        _check_options(options)
        self.wg = torch.nn.Linear(model_dim, num_global_experts, bias=False,
                                  dtype=torch.float32 if fp32_gate else None)
        self.top_k = min(num_global_experts, int(k))
        self.fp32_gate = fp32_gate

    def forward(self, x):
        wg = self.wg.float() if self.fp32_gate else self.wg
        if (self.fp32_gate and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2
                and os.environ.get("HEXA_SPLIT_GATE", "1") != "0"):
            return _SplitPrecisionLinear.apply(x, wg.weight)
        return wg(x.to(dtype=wg.weight.dtype))


class CosineTopKGate(torch.nn.Module):
    """Cosine similarity between projected tokens and expert embeddings, scaled by a learned,
    clamped temperature (clamp at log(100))."""

    def __init__(self, model_dim, num_global_experts, k=1, fp32_gate=False, proj_dim=256, init_t=0.5, **options):
        super().__init__()
        _check_options(options)
        self.top_k = min(num_global_experts, int(k))
        self.fp32_gate = fp32_gate
        self.temperature = torch.nn.Parameter(torch.log(torch.full([1], 1.0 / init_t)), requires_grad=True)
        self.cosine_projector = torch.nn.Linear(model_dim, proj_dim)
        self.sim_matrix = torch.nn.Parameter(torch.randn(size=(proj_dim, num_global_experts)), requires_grad=True)
        self.clamp_max = math.log(1.0 / 0.01)
        torch.nn.init.normal_(self.sim_matrix, 0, 0.01)

    def forward(self, x):
        proj, sim = self.cosine_projector, self.sim_matrix
        if self.fp32_gate:
            x, proj, sim = x.float(), proj.float(), sim.float()
        logits = torch.matmul(F.normalize(proj(x), dim=1), F.normalize(sim, dim=0))
        return logits * torch.clamp(self.temperature, max=self.clamp_max).exp()


class _TopKWithGShardLoss(torch.autograd.Function):
    """(ids int32 [k,T], l_aux) from float32 logits [T,E]: softmax, top-k and the GShard loss in one kernel, and the
    loss gradient in another (softmax recomputed, no [T,E] scores kept).  Same values as
    F.softmax -> torch.topk -> gshard_loss (reference cascaded_moe.py:568-598, losses.py:12-19) up to the summation
    order of the loss; ties between equal scores go to the lowest expert id."""

    @staticmethod
    def forward(ctx, logits, top_k, backend):
        ids, loss, first_count, _ = backend.gate_topk(logits, top_k)
        ctx.backend = backend
        ctx.save_for_backward(logits, first_count)
        ctx.mark_non_differentiable(ids)
        return ids, loss

    @staticmethod
    def backward(ctx, _d_ids, d_loss):
        if d_loss is None:
            return None, None, None
        logits, first_count = ctx.saved_tensors
        return ctx.backend.gate_loss_grad(logits, first_count, d_loss), None, None


def fused_topk_gshard(logits, top_k, backend):
    """The fused path when it applies (float32 CUDA logits, expert count within the kernel's limit), else None."""
    if (backend is None or not hasattr(backend, "gate_topk") or not logits.is_cuda or logits.dtype != torch.float32
            or logits.dim() != 2 or os.environ.get("HEXA_FUSED_GATE", "1") == "0"):
        return None
    E = logits.shape[1]
    if E > backend.gate_max_experts() or logits.shape[0] == 0:
        return None
    ids, l_aux = _TopKWithGShardLoss.apply(logits.contiguous(), min(int(top_k), E), backend)
    return list(ids.unbind(0)), l_aux


class _TopKWithLoadImportanceLoss(torch.autograd.Function):
    """(ids int32 [k,T], l_aux) from the clean and the noisy float32 logits [T,E]: top-k of the noisy logits and the
    load-importance loss of the clean ones in one kernel, its gradient in another.  Same values as the reference chain
    F.softmax(noisy) -> torch.topk, load_importance_loss(F.softmax(clean), noisy.gather(ids), E, gate_noise)
    (cascaded_moe.py:568-598, losses.py:21-43) up to summation order."""

    @staticmethod
    def forward(ctx, logits, logits_w_noise, top_k, sigma, backend):
        ids, loss, importance, load = backend.gate_topk_load_importance(logits, logits_w_noise, top_k, sigma)
        ctx.backend, ctx.top_k, ctx.sigma = backend, top_k, sigma
        ctx.save_for_backward(logits, logits_w_noise, importance, load)
        ctx.mark_non_differentiable(ids)
        return ids, loss

    @staticmethod
    def backward(ctx, _d_ids, d_loss):
        if d_loss is None:
            return None, None, None, None, None
        logits, noisy, importance, load = ctx.saved_tensors
        g = ctx.backend.gate_load_importance_grad(logits, noisy, ctx.top_k, ctx.sigma, importance, load, d_loss)
        # the loss depends on the clean logits through softmax and on the noisy ones through the threshold; the noisy
        # logits are the clean ones plus a constant, so the kernel returns the sum and the noisy input gets none
        return g, None, None, None, None


def fused_topk_load_importance(logits, logits_w_noise, top_k, gate_noise, backend):
    """The fused path of the load-importance loss when it applies (float32 CUDA logits, noise > 0, expert count within
    the kernel's limit), else None."""
    if (backend is None or not hasattr(backend, "gate_topk_load_importance") or not logits.is_cuda
            or logits.dtype != torch.float32 or logits_w_noise.dtype != torch.float32 or logits.dim() != 2
            or logits_w_noise is logits or gate_noise <= 0 or os.environ.get("HEXA_FUSED_GATE", "1") == "0"):
        return None
    E = logits.shape[1]
    if E > backend.gate_max_experts() or logits.shape[0] == 0:
        return None
    ids, l_aux = _TopKWithLoadImportanceLoss.apply(logits.contiguous(), logits_w_noise.detach().contiguous(), min(int(top_k), E),
                                                   float(gate_noise) / E, backend)
    return list(ids.unbind(0)), l_aux


GATES = {"top": LinearTopKGate, "cosine_top": CosineTopKGate}
