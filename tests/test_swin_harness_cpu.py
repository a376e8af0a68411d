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


def _attention_by_hand(att, x, hw):
    """Window attention spelled out (roll, partition, per-pair bias from the MLP, -100 mask, softmax) - the
    formulation of the reference's blocks (models/swin_transformer_moe_cascaded.py:135-236, 338-354, 386-401)."""
    import math
    from swin_moe_harness import shifted_window_mask
    B, _, C = x.shape
    heads, w = att.heads, min(att.window, hw)
    sh = att.shift if (att.shift and w < hw) else 0
    xi = x.view(B, hw, hw, C)
    if sh:
        xi = torch.roll(xi, (-sh, -sh), (1, 2))
    nw, n = hw // w, w * w
    win = xi.view(B, nw, w, nw, w, C).permute(0, 1, 3, 2, 4, 5).reshape(B * nw * nw, n, C)
    q, k, v = att.qkv(win).reshape(-1, n, 3, heads, C // heads).permute(2, 0, 3, 1, 4)
    a = (q * (C // heads) ** -0.5) @ k.transpose(-2, -1)
    bias = torch.zeros(heads, n, n)
    for i in range(n):
        for j in range(n):
            c = torch.tensor([i // w - j // w, i % w - j % w], dtype=torch.float32) / max(w - 1, 1) * 8
            bias[:, i, j] = att.cpb_mlp(torch.sign(c) * torch.log2(c.abs() + 1) / math.log2(8)).detach()
    a = a + bias
    if sh:
        a = (a.view(B, nw * nw, heads, n, n) + shifted_window_mask(hw, w, sh)[None, :, None]).view(-1, heads, n, n)
    o = att.proj((a.softmax(-1) @ v).transpose(1, 2).reshape(-1, n, C))
    o = o.view(B, nw, nw, w, w, C).permute(0, 1, 3, 2, 4, 5).reshape(B, hw, hw, C)
    if sh:
        o = torch.roll(o, (sh, sh), (1, 2))
    return o.reshape(B, hw * hw, C)


def test_window_attention_has_relative_position_bias_and_shift_mask():
    from swin_moe_harness import WindowAttention, shifted_window_mask
    torch.manual_seed(1)
    for hw, w, shift, heads, dim in [(12, 3, 1, 2, 16), (6, 3, 0, 4, 32), (8, 4, 2, 2, 8), (3, 3, 1, 1, 8)]:
        att = WindowAttention(dim, heads, w, shift)
        x = torch.randn(2, hw * hw, dim)
        with torch.no_grad():
            assert float((att(x, hw) - _attention_by_hand(att, x, hw)).abs().max()) < 1e-5
    m = shifted_window_mask(8, 4, 2)
    assert m.shape == (4, 16, 16) and float(m[0].abs().max()) == 0 and float(m[3].min()) == -100.0
    # the bias depends on the offset only and reaches the MLP's parameters
    att = WindowAttention(8, 2, 3, 0)
    att(torch.randn(1, 9, 8), 3).sum().backward()
    assert att.cpb_mlp[0].weight.grad is not None and float(att.cpb_mlp[2].weight.grad.abs().max()) > 0
