"""Auxiliary routing losses (plain PyTorch; O(T*E) elementwise work, not on the kernel path).

Same definitions as the reference's hexa_moe/impls/losses.py:12-43.
"""
import torch
from torch.distributions.normal import Normal


def gshard_loss(scores_w_noise, top_ids):
    """E/T-weighted count of first-choice experts dotted with the summed scores (losses.py:12-19)."""
    num_samples, num_experts = scores_w_noise.shape
    ce = torch.zeros(num_experts, device=scores_w_noise.device, dtype=scores_w_noise.dtype)
    ce.index_add_(0, top_ids[:, 0], torch.full((num_samples,), num_experts / num_samples,
                                               device=scores_w_noise.device, dtype=scores_w_noise.dtype))
    me = scores_w_noise.sum(dim=0)
    return (me * ce).sum() / num_samples


def load_importance_loss(scores_wo_noise, topk_logits, num_global_experts, gate_noise):
    """Mean of the squared coefficients of variation of importance and load (losses.py:21-43)."""
    assert gate_noise > 0, "`gate_noise` must be > 0 for normalization in load_importance_loss()."

    def cv2(v):
        v = v.float()
        return v.var() / (v.mean() ** 2 + 1e-10)

    dev = scores_wo_noise.device
    normal = Normal(torch.tensor([0.0], device=dev), torch.tensor([gate_noise / num_global_experts], device=dev))
    threshold = topk_logits[:, -1].view(-1, 1).float()
    load = normal.cdf(scores_wo_noise.float() - threshold).sum(0)
    importance = scores_wo_noise.float().sum(0)
    return (cv2(importance) + cv2(load)) / 2.0
