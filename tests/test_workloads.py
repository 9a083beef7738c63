"""Parameter-shape sources of the benchmark configurations: the model definitions reproduce the
preconditioner censuses that the reference's blocking rule (optimizers/shampoo2.py:43-65) gives
for ResNet-34 (models/resnet.py:110-113), Swin-Tiny for 32 x 32 inputs (models/swin.py:4-15) and
ViT-Base/32 (models/vit.py:15-20)."""
import torch

import workloads


def census(model):
    return workloads.preconditioner_census([tuple(p.shape) for p in model.parameters()])


def test_resnet34_census():
    c = census(workloads.resnet34_cifar())
    assert c == {27: 1, 64: 8, 100: 1, 128: 10, 256: 25, 512: 24, 576: 7, 1008: 5, 1104: 12, 1152: 8, 1200: 27}
    assert sum(c.values()) == 128 and sum(k for n, k in c.items() if n * n >= 4096) == 127
    assert abs(sum(n ** 3 * k for n, k in c.items()) / 8.5e10 - 1) < 0.01


def test_swin_tiny_census():
    m = workloads.swin_tiny_32()
    c = census(m)
    low = {n: k for n, k in c.items() if n * n >= 4096}
    assert low == {96: 11, 100: 1, 192: 11, 288: 2, 336: 13, 384: 48, 576: 2, 672: 4, 768: 28, 1104: 2, 1152: 6, 1200: 23}
    assert sum(low.values()) == 151 and sum(c.values()) == 176 and sum(c.values()) - sum(low.values()) == 25
    assert abs(sum(p.numel() for p in m.parameters()) / 27.58e6 - 1) < 1e-3
    assert abs(sum(n ** 3 * k for n, k in c.items()) / 6.9e10 - 1) < 0.01


def test_vit_base_census():
    m = workloads.vit_base_patch32_224()
    assert sum(p.numel() for p in m.parameters()) == 88224232
    assert census(m) == {50: 1, 672: 25, 768: 125, 1000: 1, 1104: 12, 1200: 62}


def test_small_models_run_forward_and_backward():
    for m, img in ((workloads.resnet34_cifar(), 32), (workloads.swin_tiny_32(), 32)):
        loss = workloads.synthetic_gradients(m, 4, img, 100, "cpu", autocast_bf16=False)
        assert loss == loss and all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())
