"""Benchmark workloads: model definitions that only serve as sources of parameter shapes
and gradients for the optimizer step (random init, synthetic N(0,1) inputs).

The reference builds its ViT and Swin models through timm (models/vit.py:15-20,
models/swin.py:4-15); timm is not a dependency here, so ViT-Base/32 is written out from
its architecture: 224x224x3 input, patch 32, 12 layers, width 768, 12 heads, MLP 3072,
1000 classes (88 224 232 parameters).
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class _Block(nn.Module):
    def __init__(self, dim, heads, mlp):
        super().__init__()
        self.heads = heads
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.qkv = nn.Linear(dim, 3 * dim)
        self.proj = nn.Linear(dim, dim)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.fc1 = nn.Linear(dim, mlp)
        self.fc2 = nn.Linear(mlp, dim)

    def forward(self, x):
        B, T, C = x.shape
        qkv = self.qkv(self.norm1(x)).reshape(B, T, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, C))
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class VisionTransformer(nn.Module):
    def __init__(self, img=224, patch=32, dim=768, depth=12, heads=12, mlp=3072, classes=1000):
        super().__init__()
        self.patch_embed = nn.Conv2d(3, dim, patch, patch)
        tokens = (img // patch) ** 2 + 1
        self.cls_token = nn.Parameter(torch.zeros(1, 1, dim))
        self.pos_embed = nn.Parameter(torch.randn(1, tokens, dim) * 0.02)
        self.blocks = nn.ModuleList(_Block(dim, heads, mlp) for _ in range(depth))
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.head = nn.Linear(dim, classes)

    def forward(self, x):
        x = self.patch_embed(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1), x], dim=1) + self.pos_embed
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.norm(x)[:, 0])


def vit_base_patch32_224(classes=1000):
    return VisionTransformer(classes=classes)


def vit_tiny_for_tests(classes=10):
    """Same structure at a size a CPU steps in a second (orders 64..192)."""
    return VisionTransformer(img=32, patch=8, dim=64, depth=2, heads=4, mlp=192, classes=classes)


def preconditioner_census(shapes, prec_maxorder=1200):
    """{order: count} of the preconditioner matrices the optimizers create for `shapes`."""
    from optimizers._base import preconditioner_orders
    census = {}
    for s in shapes:
        for n in preconditioner_orders(tuple(s), prec_maxorder):
            census[n] = census.get(n, 0) + 1
    return dict(sorted(census.items()))


def synthetic_gradients(model, batch, img, classes, device, autocast_bf16=True, seed=0):
    """One cross-entropy backward pass on N(0,1) images with uniform labels; leaves .grad set."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(batch, 3, img, img, generator=g).to(device)
    y = torch.randint(0, classes, (batch,), generator=g).to(device)
    model.zero_grad(set_to_none=True)
    with torch.autocast(device_type=torch.device(device).type, dtype=torch.bfloat16, enabled=autocast_bf16):
        loss = F.cross_entropy(model(x).float(), y)
    loss.backward()
    return float(loss.detach())
