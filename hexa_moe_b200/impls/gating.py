"""Router networks of the MoE layers (plain PyTorch: a d x E projection is not kernel work).

Two gate types, selected by gate_type['type'] exactly as in the reference ('top' and
'cosine_top', hexa_moe/gates/top.py:6-25 and hexa_moe/gates/cosine_top.py:7-37).  Parameter
names are kept (`wg.weight`; `temperature`, `cosine_projector.*`, `sim_matrix`) so that state
dicts are interchangeable.  Both accept only `capacity_factor` and `gate_noise` as extra options.
"""
import math

import torch
import torch.nn.functional as F


def _check_options(options):
    for opt in options:
        if opt not in ("capacity_factor", "gate_noise"):
            raise Exception("Unrecognized argument provided to Gating module: %s" % opt)


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


GATES = {"top": LinearTopKGate, "cosine_top": CosineTopKGate}
