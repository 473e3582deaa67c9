"""Seeded synthetic inputs shared by the oracle tests, the GPU parity tests, the
golden-vector generator and the bench (stand-ins for ImageNet-shaped activations).

All tensors are drawn on the CPU in float32 with torch.manual_seed(seed), always in
the order weight, input, kernel-space offsets, image-space offsets, upstream
gradient, and only then cast or moved, so that every consumer sees the same values.
"""
import math

import torch


def out_size(i, k, s, p, d):
    return (i + 2 * p - (d * (k - 1) + 1)) // s + 1


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def make_case(n, c, h, w, scope=(4, 4), k=3, stride=1, pad=1, dil=1, groups=1, rot_std=0.5, off_std=None,
              seed=0, weight_init="kaiming"):
    """Inputs of one local-DK (off_std None) or DK+DCN call."""
    k2, s2, p2, d2 = _pair(k), _pair(stride), _pair(pad), _pair(dil)
    ho, wo = out_size(h, k2[0], s2[0], p2[0], d2[0]), out_size(w, k2[1], s2[1], p2[1], d2[1])
    gen = torch.Generator().manual_seed(seed)
    taps = k2[0] * k2[1]
    if weight_init == "kaiming":
        weight = torch.randn(c, 1, *scope, generator=gen) * math.sqrt(2.0 / (scope[0] * scope[1]))
    else:
        bound = 1.0 / math.sqrt(taps)
        weight = (torch.rand(c, 1, *scope, generator=gen) * 2 - 1) * bound
    x = torch.randn(n, c, h, w, generator=gen)
    rot = torch.randn(n, groups * taps * 2, ho, wo, generator=gen) * rot_std
    case = dict(weight=weight, input=x, rotation=rot,
                args=dict(kernel_size=k2, stride=s2, padding=p2, dilation=d2, rotation_groups=groups))
    if off_std is not None:
        case["offset"] = torch.randn(n, taps * 2, ho, wo, generator=gen) * off_std
    case["grad_output"] = torch.randn(n, c, ho, wo, generator=gen)
    return case


def make_nd_case(c, shape, b, seed=0, lo=-1.5, hi_pad=1.5, snap=0.3):
    """nd_linear_sample inputs: coordinates spread past both ends of every axis, a
    fraction `snap` of them snapped onto integers (the kinks)."""
    gen = torch.Generator().manual_seed(seed)
    data = torch.randn(c, *shape, generator=gen)
    d = len(shape)
    span = torch.tensor([s + hi_pad - lo for s in shape], dtype=torch.float32)
    coord = torch.rand(b, d, generator=gen) * span + lo
    pick = torch.rand(b, d, generator=gen) < snap
    coord = torch.where(pick, torch.round(coord), coord)
    grad_output = torch.randn(b, c, generator=gen)
    return dict(data=data, coord=coord, grad_output=grad_output)


def global_dk_coord(raw, weight_shape, kernel_size=1):
    """Coordinates as GlobalDeformKernel2d forms them (modules/deform_kernel.py:64-83):
    raw FC output + scope-centred tap positions, clamped to [0, weight_shape[0]-1]."""
    start_h = (weight_shape[0] - (kernel_size - 1) - 1) / 2.0
    start_w = (weight_shape[1] - (kernel_size - 1) - 1) / 2.0
    bias = []
    for hh in range(kernel_size):
        for ww in range(kernel_size):
            bias += [start_h + hh, start_w + ww]
            for i in range(len(weight_shape) - 2):
                bias += [(weight_shape[i + 2] - 1) / 2.0]
    coord = raw + torch.tensor(bias, dtype=raw.dtype).unsqueeze(0)
    coord = torch.clamp(coord, 0, weight_shape[0] - 1)
    return coord.view(raw.shape[0] * kernel_size * kernel_size, len(weight_shape))


# BASELINE.json configs 1-4 at full size (config 3 is the ten-layer sweep).
def cfg1():
    return make_case(2, 64, 28, 28, (4, 4), 3, 1, 1, rot_std=0.5, seed=0)


def cfg2(seed=0):
    gen = torch.Generator().manual_seed(seed)
    weight = torch.randn(256, 1, 2, 2, generator=gen) * math.sqrt(2.0 / 4)
    x = torch.randn(32, 256, 14, 14, generator=gen)
    raw = torch.rand(32, 2, generator=gen) * 2 - 1
    coord = global_dk_coord(raw, (2, 2), 1)
    grad_output = torch.randn(32, 256, generator=gen)
    return dict(data=weight.view(256, 2, 2), coord=coord, grad_output=grad_output, input=x, raw=raw, weight=weight)


CFG3_LAYERS = [(96, 112), (144, 56), (192, 28), (384, 14), (960, 7)]


def cfg3(c, hw, stride, n=128, seed=0):
    return make_case(n, c, hw, hw, (4, 4), 3, stride, 1, rot_std=1.0, seed=seed)


def cfg4(n=64, c=256, hw=56, seed=0):
    return make_case(n, c, hw, hw, (4, 4), 3, 1, 1, rot_std=0.5, off_std=2.0, seed=seed)


def rel_err(a, b):
    """max|a-b| / max|b| -- the tolerance definition used everywhere."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    den = b.abs().max().item()
    num = (a - b).abs().max().item()
    return num / den if den > 0 else num
