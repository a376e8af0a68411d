"""The Swin-MoE-like harness end to end on CPU at a tiny size, with the CPU oracle standing in for the kernels:
shapes through patch embedding / windows / patch merging, the shared MoE_Cascaded serving every depth, and gradients
reaching every parameter."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def test_tiny_harness_forward_backward_on_cpu():
    import oracle_backend
    from swin_moe_harness import SwinMoEHarness
    torch.manual_seed(0)
    m = SwinMoEHarness(img_size=96, patch=4, dims=(16, 32, 64, 128), depths=(2, 2, 4, 2), heads=(2, 2, 4, 4), window=3,
                       num_experts=4, top_k=1, num_classes=10)
    m.cascaded_moe.dispatch_params.backend = oracle_backend        # test double for the CUDA kernels
    assert m.total_depth == 10 and m.moe_idx == [5, 7, 9]
    assert m.moe_tokens_per_image() == [36, 36, 9]
    with torch.no_grad():
        for n, p in m.cascaded_moe.named_parameters():
            if "batched" in n and "bias" not in n:
                p.normal_(0, 0.1)
    x = torch.randn(2, 3, 96, 96)
    logits, l_aux = m(x)
    assert logits.shape == (2, 10) and torch.isfinite(logits).all()
    (F_loss := torch.nn.functional.cross_entropy(logits, torch.tensor([1, 2])) + 0.01 * l_aux).backward()
    missing = [n for n, p in m.named_parameters() if p.grad is None]
    assert not missing, missing
    assert all(torch.isfinite(p.grad).all() for p in m.parameters())
