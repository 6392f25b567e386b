"""ViT-B/16: 12 blocks, width 768, 12 heads, MLP 3072, 197 tokens at 224x224
(the shape of the reference's Model/ViT/ViT.py:89-133 instantiated as ViT-B/16)."""
from __future__ import annotations

import torch
import torch.fx
import torch.nn.functional as F
from torch import nn

from ..modules.attention import split_heads

torch.fx.wrap("split_heads")      # a leaf for torch.fx: the Controller's trace keeps the call, not its branches


class Attention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(dim, dim * 3)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x):
        B, T, D = x.shape
        # the reference's view / permute / index (Model/ViT/ViT.py:39-42) as three strided views,
        # with a one-pass backward (modules/attention.py)
        q, k, v = split_heads(self.qkv(x), self.heads)
        out = F.scaled_dot_product_attention(q, k, v)
        return self.proj(out.transpose(1, 2).reshape(B, T, D))


class Block(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_dim: int):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.attn = Attention(dim, heads)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.fc1 = nn.Linear(dim, mlp_dim)
        self.gelu = nn.GELU(approximate="tanh")
        self.fc2 = nn.Linear(mlp_dim, dim)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.fc2(self.gelu(self.fc1(self.norm2(x))))


class VisionTransformer(nn.Module):
    def __init__(self, image: int = 224, patch: int = 16, dim: int = 768, depth: int = 12, heads: int = 12,
                 mlp_dim: int = 3072, num_classes: int = 1000):
        super().__init__()
        self.patch_embed = nn.Conv2d(3, dim, patch, stride=patch, bias=False)
        tokens = (image // patch) ** 2 + 1
        self.cls_token = nn.Parameter(torch.zeros(1, 1, dim))
        self.pos_embed = nn.Parameter(torch.randn(1, tokens, dim) * 0.02)
        self.blocks = nn.Sequential(*[Block(dim, heads, mlp_dim) for _ in range(depth)])
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.head = nn.Linear(dim, num_classes)

    def forward(self, x):
        x = self.patch_embed(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1) + self.pos_embed.to(x.dtype)
        return self.head(self.norm(self.blocks(x))[:, 0])


def vit_b16(num_classes: int = 1000) -> VisionTransformer:
    return VisionTransformer(num_classes=num_classes)
