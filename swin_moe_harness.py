"""Synthetic Swin-MoE-like network around MoE_Cascaded, for running the data-centric mode in the setting it was
designed for: attention blocks between the MoE layers give the pipeline-shared cache something to overlap with.

Shape of the reference's Swin-MoE-B example (Swin-Transformer-MoE/configs/swinmoe/
swin_moe_base_patch4_window12_192_*.yaml and models/swin_transformer_moe_cascaded.py:650-879): 4x4 patch embedding,
stage dims 128/256/512/1024 with depths 2/2/18/2 and heads 4/8/16/32, window 12, patch merging between stages,
every block's FFN served by ONE shared MoE_Cascaded (dense FFN in even blocks, MoE in every other block of stages 3
and 4: 32 experts, top-1, mlp_ratio 4, no fc1 bias).  Window attention follows the reference's blocks
(models/swin_transformer_moe_cascaded.py:135-236, 256-407): scaled dot products plus a continuous relative position
bias (a two-layer MLP over log-spaced relative coordinates, one value per head) and, in the shifted blocks, the
mask that keeps tokens from different image regions of a rolled window apart.  It is built from stock PyTorch ops
(one scaled_dot_product_attention call per block with an additive mask); drop-path, dropout and the window-process
kernels of the reference are left out: this is a timing and parity harness, not a model to train.
"""
from __future__ import annotations

import math
from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F

from hexa_moe import moe as hmoe


def shifted_window_mask(hw: int, w: int, shift: int) -> torch.Tensor:
    """Additive mask [windows, w*w, w*w] for windows cut from an hw x hw map rolled by `shift`: 0 between tokens that
    come from the same region of the unrolled image, -100 otherwise (the value the reference adds, ...:338-354)."""
    region = torch.zeros(hw, hw)
    edges = (0, hw - w, hw - shift, hw)
    for i in range(3):
        for j in range(3):
            region[edges[i]: edges[i + 1], edges[j]: edges[j + 1]] = 3 * i + j
    nw = hw // w
    per_window = region.view(nw, w, nw, w).permute(0, 2, 1, 3).reshape(nw * nw, w * w)
    return (per_window.unsqueeze(1) != per_window.unsqueeze(2)).float() * -100.0


def _attention(q, k, v, mask):
    """scaled_dot_product_attention with an additive mask.  On CUDA the fused backends that take a bias are preferred in
    the order given by SWIN_SDPA_BACKENDS (default "cudnn,efficient,math"); whichever accepts the shapes runs."""
    if not q.is_cuda:
        return F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    import os
    from torch.nn.attention import SDPBackend, sdpa_kernel
    names = {"cudnn": SDPBackend.CUDNN_ATTENTION, "efficient": SDPBackend.EFFICIENT_ATTENTION, "math": SDPBackend.MATH,
             "flash": SDPBackend.FLASH_ATTENTION}
    order = [names[n] for n in os.environ.get("SWIN_SDPA_BACKENDS", "cudnn,efficient,math").split(",") if n in names]
    try:
        with sdpa_kernel(order, set_priority=True):
            return F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    except TypeError:        # an older sdpa_kernel without set_priority
        with sdpa_kernel(order):
            return F.scaled_dot_product_attention(q, k, v, attn_mask=mask)


class WindowAttention(nn.Module):
    def __init__(self, dim: int, heads: int, window: int, shift: int):
        super().__init__()
        self.heads, self.window, self.shift = heads, window, shift
        self.qkv = nn.Linear(dim, 3 * dim)
        self.proj = nn.Linear(dim, dim)
        # continuous relative position bias: MLP(2 -> 512 -> heads) over the (2w-1)^2 possible offsets
        self.cpb_mlp = nn.Sequential(nn.Linear(2, 512), nn.ReLU(inplace=True), nn.Linear(512, heads, bias=False))
        self._tables = {}      # window size actually used -> (offset coordinates, offset index of every token pair)
        self._masks = {}       # (hw, w) -> additive shift mask

    def _bias_tables(self, w: int, device):
        key = (w, device)
        if key not in self._tables:
            off = torch.arange(-(w - 1), w, dtype=torch.float32)
            grid = torch.stack(torch.meshgrid(off, off, indexing="ij"), dim=-1) / max(w - 1, 1) * 8.0     # [2w-1, 2w-1, 2]
            coords = torch.sign(grid) * torch.log2(grid.abs() + 1.0) / math.log2(8.0)
            pos = torch.stack(torch.meshgrid(torch.arange(w), torch.arange(w), indexing="ij"), dim=0).flatten(1)   # [2, w*w]
            rel = pos[:, :, None] - pos[:, None, :] + (w - 1)                                              # [2, N, N]
            index = rel[0] * (2 * w - 1) + rel[1]
            self._tables[key] = (coords.view(-1, 2).to(device), index.to(device))
        return self._tables[key]

    def additive_mask(self, hw: int, w: int, dtype, device) -> torch.Tensor:
        """[1, windows * heads, N, N] (windows = 1 without a shift): relative position bias + shift mask."""
        coords, index = self._bias_tables(w, device)
        table = self.cpb_mlp(coords.to(self.cpb_mlp[0].weight.dtype))                  # [(2w-1)^2, heads]
        bias = table[index.view(-1)].view(w * w, w * w, self.heads).permute(2, 0, 1)   # [heads, N, N]
        if self.shift and w < hw:
            key = (hw, w, device)
            if key not in self._masks:
                self._masks[key] = shifted_window_mask(hw, w, self.shift).to(device)
            m = self._masks[key].to(bias.dtype)                                         # [windows, N, N]
            bias = bias.unsqueeze(0) + m.unsqueeze(1)                                   # [windows, heads, N, N]
            bias = bias.reshape(1, -1, w * w, w * w)
        else:
            bias = bias.unsqueeze(0)
        return bias.to(dtype)

    def forward(self, x: torch.Tensor, hw: int) -> torch.Tensor:
        B, N, C = x.shape
        w = min(self.window, hw)
        shifted = bool(self.shift) and w < hw
        x = x.view(B, hw, hw, C)
        if shifted:
            x = torch.roll(x, shifts=(-self.shift, -self.shift), dims=(1, 2))
        nw = hw // w
        n, hd = w * w, C // self.heads
        x = x.view(B, nw, w, nw, w, C).permute(0, 1, 3, 2, 4, 5).reshape(B, nw * nw, n, C)
        # [3, B, windows, heads, n, hd]; the windows of an image become extra heads so that one mask of
        # [1, windows * heads, n, n] (or [1, heads, n, n] without a shift) broadcasts over the batch
        qkv = self.qkv(x).view(B, nw * nw, n, 3, self.heads, hd).permute(3, 0, 1, 4, 2, 5)
        mask = self.additive_mask(hw, w, x.dtype, x.device)
        if shifted:
            q, k, v = (t.reshape(B, nw * nw * self.heads, n, hd) for t in qkv)
        else:
            q, k, v = (t.reshape(B * nw * nw, self.heads, n, hd) for t in qkv)
        o = _attention(q, k, v, mask)
        o = o.view(B, nw * nw, self.heads, n, hd).transpose(2, 3).reshape(B, nw, nw, w, w, C)
        o = self.proj(o).permute(0, 1, 3, 2, 4, 5).reshape(B, hw, hw, C)
        if shifted:
            o = torch.roll(o, shifts=(self.shift, self.shift), dims=(1, 2))
        return o.reshape(B, N, C)


class Block(nn.Module):
    """Attention half of a Swin block; returns (norm2(x), shortcut) like the reference's blocks (…:403-407) so that
    the caller can run the FFN / MoE of this depth through the shared MoE_Cascaded."""

    def __init__(self, dim, heads, window, shift):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.attn = WindowAttention(dim, heads, window, shift)

    def forward(self, x, hw):
        x = x + self.attn(self.norm1(x), hw)
        return self.norm2(x), x


class PatchMerging(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.norm = nn.LayerNorm(4 * dim)
        self.reduction = nn.Linear(4 * dim, 2 * dim, bias=False)

    def forward(self, x, hw):
        B, N, C = x.shape
        x = x.view(B, hw // 2, 2, hw // 2, 2, C).permute(0, 1, 3, 2, 4, 5).reshape(B, (hw // 2) ** 2, 4 * C)
        return self.reduction(self.norm(x))


class SwinMoEHarness(nn.Module):
    def __init__(self, img_size=192, patch=4, dims=(128, 256, 512, 1024), depths=(2, 2, 18, 2), heads=(4, 8, 16, 32),
                 window=12, num_experts=32, top_k=1, moe_stages=(2, 3), num_classes=1000, data_centric=True,
                 mlp_proportion=None):
        super().__init__()
        self.hw0 = img_size // patch
        self.patch_embed = nn.Conv2d(3, dims[0], kernel_size=patch, stride=patch)
        self.embed_norm = nn.LayerNorm(dims[0])
        blocks, merges, dim_list, moe_idx, self.stage_of = [], [], [], [], []
        depth = 0
        for s, (d, n, h) in enumerate(zip(dims, depths, heads)):
            for i in range(n):
                blocks.append(Block(d, h, window, shift=(window // 2 if i % 2 else 0)))
                dim_list.append(d)
                self.stage_of.append(s)
                if s in moe_stages and i % 2 == 1:       # every other block of the MoE stages
                    moe_idx.append(depth)
                depth += 1
            merges.append(PatchMerging(d) if s + 1 < len(dims) else nn.Identity())
        self.blocks, self.merges = nn.ModuleList(blocks), nn.ModuleList(merges)
        self.depths, self.total_depth, self.moe_idx = list(depths), depth, moe_idx
        self.cascaded_moe = hmoe.MoE_Cascaded(
            gate_type={'type': 'top', 'k': top_k, 'fp32_gate': True}, model_dim_list=dim_list, moe_idx_list=moe_idx,
            mlp_ratio=4, mlp_proportion=mlp_proportion, num_global_experts=num_experts, total_depth=depth,
            data_centric=data_centric, mlp_fc1_bias=False, mlp_fc2_bias=True, activation_fn=lambda t: F.gelu(t))
        self.norm = nn.LayerNorm(dims[-1])
        self.head = nn.Linear(dims[-1], num_classes)

    def moe_tokens_per_image(self) -> List[int]:
        """Tokens per image entering each MoE layer."""
        out = []
        for d in self.moe_idx:
            hw = self.hw0 // (2 ** self.stage_of[d])
            out.append(hw * hw)
        return out

    def forward(self, images: torch.Tensor):
        x = self.patch_embed(images).flatten(2).transpose(1, 2)
        x = self.embed_norm(x)
        hw, depth, l_aux = self.hw0, 0, 0.0
        for s, n in enumerate(self.depths):
            for _ in range(n):
                y, shortcut = self.blocks[depth](x, hw)
                y, aux = self.cascaded_moe(depth, y)
                x = shortcut + y
                if aux is not None:
                    l_aux = l_aux + aux
                depth += 1
            if not isinstance(self.merges[s], nn.Identity):
                x = self.merges[s](x, hw)
                hw //= 2
        x = self.norm(x).mean(dim=1)
        return self.head(x), l_aux
