"""Benchmark workloads: model definitions that only serve as sources of parameter shapes
and gradients for the optimizer step (random init, synthetic N(0,1) inputs).

The reference builds its ViT and Swin models through timm (models/vit.py:15-20,
models/swin.py:4-15); timm is not a dependency here, so they are written out from their
architectures:
  ViT-Base/32   224x224x3 input, patch 32, 12 layers, width 768, 12 heads, MLP 3072,
                1000 classes (88 224 232 parameters);
  Swin-Tiny     for 32x32 inputs: patch 2, window 4, width 96, depths 2/2/6/2, heads
                3/6/12/24, 100 classes, patch merging between stages;
  ResNet-34     CIFAR variant (3x3 stem, no max-pool, stages of 3/4/6/3 basic blocks at
                64/128/256/512 channels, 100 classes) - the parameter shapes of the
                reference's models/resnet.py:110-113.
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


class _BasicBlock(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(cout)
        self.shortcut = None
        if stride != 1 or cin != cout:
            self.shortcut = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        y = self.bn2(self.conv2(F.relu(self.bn1(self.conv1(x)))))
        return F.relu(y + (x if self.shortcut is None else self.shortcut(x)))


class ResNetCifar(nn.Module):
    def __init__(self, depths=(3, 4, 6, 3), widths=(64, 128, 256, 512), classes=100):
        super().__init__()
        self.conv1 = nn.Conv2d(3, widths[0], 3, 1, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(widths[0])
        stages, cin = [], widths[0]
        for i, (d, w) in enumerate(zip(depths, widths)):
            for j in range(d):
                stages.append(_BasicBlock(cin, w, 2 if (j == 0 and i > 0) else 1))
                cin = w
        self.stages = nn.Sequential(*stages)
        self.linear = nn.Linear(cin, classes)

    def forward(self, x):
        x = self.stages(F.relu(self.bn1(self.conv1(x))))
        return self.linear(F.adaptive_avg_pool2d(x, 1).flatten(1))


def resnet34_cifar(classes=100):
    return ResNetCifar(classes=classes)


class _WindowAttention(nn.Module):
    def __init__(self, dim, heads, window):
        super().__init__()
        self.heads, self.window = heads, window
        self.relative_position_bias_table = nn.Parameter(torch.zeros((2 * window - 1) ** 2, heads))
        nn.init.trunc_normal_(self.relative_position_bias_table, std=0.02)
        ys, xs = torch.meshgrid(torch.arange(window), torch.arange(window), indexing="ij")
        pos = torch.stack([ys.flatten(), xs.flatten()])                     # (2, w*w)
        rel = pos[:, :, None] - pos[:, None, :] + (window - 1)              # (2, w*w, w*w), values 0..2w-2
        self.register_buffer("rel_index", rel[0] * (2 * window - 1) + rel[1], persistent=False)
        self.qkv = nn.Linear(dim, 3 * dim)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x, mask):
        B, T, C = x.shape                                                   # B = batch * windows
        qkv = self.qkv(x).reshape(B, T, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        bias = self.relative_position_bias_table[self.rel_index.reshape(-1)].reshape(T, T, self.heads).permute(2, 0, 1)
        bias = bias.unsqueeze(0)
        if mask is not None:                                                # (windows, T, T)
            nw = mask.shape[0]
            bias = (bias + mask.unsqueeze(1)).repeat(B // nw, 1, 1, 1)
        a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2], attn_mask=bias.to(qkv.dtype))
        return self.proj(a.transpose(1, 2).reshape(B, T, C))


class _SwinBlock(nn.Module):
    def __init__(self, dim, heads, res, window, shift):
        super().__init__()
        if res <= window:                                                   # one window covers the map: no shift
            window, shift = res, 0
        self.res, self.window, self.shift = res, window, shift
        self.norm1 = nn.LayerNorm(dim)
        self.attn = _WindowAttention(dim, heads, window)
        self.norm2 = nn.LayerNorm(dim)
        self.fc1 = nn.Linear(dim, 4 * dim)
        self.fc2 = nn.Linear(4 * dim, dim)
        mask = None
        if shift:
            img = torch.zeros(res, res)
            cnt = 0
            for hs in (slice(0, -window), slice(-window, -shift), slice(-shift, None)):
                for ws in (slice(0, -window), slice(-window, -shift), slice(-shift, None)):
                    img[hs, ws] = cnt
                    cnt += 1
            win = img.reshape(res // window, window, res // window, window).permute(0, 2, 1, 3).reshape(-1, window * window)
            diff = win[:, None, :] - win[:, :, None]
            mask = torch.zeros_like(diff).masked_fill(diff != 0, -100.0)
        self.register_buffer("mask", mask, persistent=False)

    def forward(self, x):
        B, L, C = x.shape
        r, w = self.res, self.window
        y = self.norm1(x).reshape(B, r, r, C)
        if self.shift:
            y = torch.roll(y, (-self.shift, -self.shift), (1, 2))
        y = y.reshape(B, r // w, w, r // w, w, C).permute(0, 1, 3, 2, 4, 5).reshape(-1, w * w, C)
        y = self.attn(y, self.mask)
        y = y.reshape(B, r // w, r // w, w, w, C).permute(0, 1, 3, 2, 4, 5).reshape(B, r, r, C)
        if self.shift:
            y = torch.roll(y, (self.shift, self.shift), (1, 2))
        x = x + y.reshape(B, L, C)
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class _PatchMerging(nn.Module):
    def __init__(self, dim, res):
        super().__init__()
        self.res = res
        self.norm = nn.LayerNorm(4 * dim)
        self.reduction = nn.Linear(4 * dim, 2 * dim, bias=False)

    def forward(self, x):
        B, L, C = x.shape
        r = self.res
        x = x.reshape(B, r // 2, 2, r // 2, 2, C).permute(0, 1, 3, 4, 2, 5).reshape(B, (r // 2) ** 2, 4 * C)
        return self.reduction(self.norm(x))


class SwinTransformer(nn.Module):
    def __init__(self, img=32, patch=2, dim=96, depths=(2, 2, 6, 2), heads=(3, 6, 12, 24), window=4, classes=100):
        super().__init__()
        self.patch_embed = nn.Conv2d(3, dim, patch, patch)
        self.patch_norm = nn.LayerNorm(dim)
        res = img // patch
        layers = []
        for i, (d, h) in enumerate(zip(depths, heads)):
            if i > 0:
                layers.append(_PatchMerging(dim, res))
                dim, res = 2 * dim, res // 2
            for j in range(d):
                layers.append(_SwinBlock(dim, h, res, window, 0 if j % 2 == 0 else window // 2))
        self.layers = nn.Sequential(*layers)
        self.norm = nn.LayerNorm(dim)
        self.head = nn.Linear(dim, classes)

    def forward(self, x):
        x = self.patch_norm(self.patch_embed(x).flatten(2).transpose(1, 2))
        return self.head(self.norm(self.layers(x)).mean(dim=1))


def swin_tiny_32(classes=100):
    return SwinTransformer(classes=classes)


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
