"""Second, independent CPU oracle: the three operators composed from stock PyTorch
ops, differentiable by autograd -- TEST INFRASTRUCTURE ONLY.

It shares no code with oracle/dk_oracle.c: values come from unfold + gather, and
every gradient comes from autograd instead of a hand-written adjoint.  The two
oracles must agree in float64 to ~1e-12 before either is trusted
(tests/test_oracle.py).  It is also the timed "pure-PyTorch composition" CPU
baseline, because the reference has no CPU implementation
(functions/filter_sample_depthwise.py:43-44 raises NotImplementedError).

Conventions (all from the reference; FS.cu = csrc/filter_sample_depthwise_cuda_kernel.cu,
ND.cu = csrc/nd_linear_sample_cuda_kernel.cu):
  * floor-based pieces, so that at an integer coordinate the derivative is the
    right-hand one (FS.cu:137-158), never relu(1-|t|) hats;
  * a bank sample is valid iff -1 < u < sH and -1 < v < sW (FS.cu:59); corners that
    fall outside the bank read zero (FS.cu:71-78);
  * an image sample is used iff -1 < p_h < H and -1 < p_w < W (FS.cu:500);
  * taps of the local operator that lie in the padding contribute nothing to any
    output or gradient (FS.cu:359, 1345): unfold's zero padding gives exactly that;
  * channel c reads kernel-space offsets of group c % G (FS.cu:307).
"""
import itertools

import torch
import torch.nn.functional as F


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _out(in_size, k, s, p, d):
    return (in_size + 2 * p - (d * (k - 1) + 1)) // s + 1


def _bilinear_gather(table, hpos, wpos, size_h, size_w, outer_valid):
    """Zero-extended, floor-based bilinear read.

    table: [A, B, size_h*size_w]; hpos, wpos: [A, B, M] positions; returns [A, B, M].
    outer_valid: bool [A, B, M] mask applied on top (no gradient flows through it).
    """
    h0 = torch.floor(hpos).detach()
    w0 = torch.floor(wpos).detach()
    lh = hpos - h0
    lw = wpos - w0
    hh = 1 - lh
    hw = 1 - lw
    h0 = h0.long()
    w0 = w0.long()
    out = torch.zeros_like(hpos)
    for dh, dw, coef in ((0, 0, hh * hw), (0, 1, hh * lw), (1, 0, lh * hw), (1, 1, lh * lw)):
        hi = h0 + dh
        wi = w0 + dw
        ok = (hi >= 0) & (hi <= size_h - 1) & (wi >= 0) & (wi <= size_w - 1) & outer_valid
        idx = (hi.clamp(0, size_h - 1) * size_w + wi.clamp(0, size_w - 1))
        val = torch.gather(table, 2, idx)
        out = out + torch.where(ok, coef * val, torch.zeros_like(val))
    return out


def _bank_kernel(weight, rotation, k, groups, n, c, p):
    """Per-location resampled kernels [N, C, kH*kW, P] (FS.cu:51-83 and 338-341)."""
    s_h, s_w = weight.shape[-2:]
    taps = k[0] * k[1]
    rot = rotation.reshape(n, groups, taps, 2, p)
    fh = torch.arange(k[0], dtype=rot.dtype).repeat_interleave(k[1]).view(1, 1, taps, 1)
    fw = torch.arange(k[1], dtype=rot.dtype).repeat(k[0]).view(1, 1, taps, 1)
    u = fh + rot[:, :, :, 0] + (s_h - k[0]) / 2.0
    v = fw + rot[:, :, :, 1] + (s_w - k[1]) / 2.0
    gidx = torch.arange(c) % groups
    u = u[:, gidx].reshape(n, c, taps * p)
    v = v[:, gidx].reshape(n, c, taps * p)
    valid = (u > -1) & (v > -1) & (u < s_h) & (v < s_w)
    table = weight.reshape(1, c, s_h * s_w).expand(n, c, s_h * s_w)
    return _bilinear_gather(table, u, v, s_h, s_w, valid).view(n, c, taps, p)


def sample_depthwise(input, rotation, weight, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1),
                     dilation=(1, 1), rotation_groups=1):
    """Local deformable kernel (FS.cu:297-385) from unfold + gather."""
    k, s, pd, d = _pair(kernel_size), _pair(stride), _pair(padding), _pair(dilation)
    n, c, h, w = input.shape
    ho, wo = _out(h, k[0], s[0], pd[0], d[0]), _out(w, k[1], s[1], pd[1], d[1])
    p = ho * wo
    taps = k[0] * k[1]
    cols = F.unfold(input, k, dilation=d, padding=pd, stride=s).view(n, c, taps, p)
    kern = _bank_kernel(weight, rotation, k, rotation_groups, n, c, p)
    return (cols * kern).sum(2).view(n, c, ho, wo)


def deform_sample_depthwise(input, offset, rotation, weight, kernel_size=(3, 3), stride=(1, 1),
                            padding=(1, 1), dilation=(1, 1), rotation_groups=1):
    """Deformable kernel + deformable convolution (FS.cu:461-527)."""
    k, s, pd, d = _pair(kernel_size), _pair(stride), _pair(padding), _pair(dilation)
    n, c, h, w = input.shape
    ho, wo = _out(h, k[0], s[0], pd[0], d[0]), _out(w, k[1], s[1], pd[1], d[1])
    p = ho * wo
    taps = k[0] * k[1]
    dt = input.dtype
    oh = torch.arange(ho, dtype=dt).view(ho, 1).expand(ho, wo).reshape(1, 1, p)
    ow = torch.arange(wo, dtype=dt).view(1, wo).expand(ho, wo).reshape(1, 1, p)
    fh = torch.arange(k[0], dtype=dt).repeat_interleave(k[1]).view(1, taps, 1)
    fw = torch.arange(k[1], dtype=dt).repeat(k[0]).view(1, taps, 1)
    off = offset.reshape(n, taps, 2, p)
    ph = (oh * s[0] - pd[0] + fh * d[0]) + off[:, :, 0]
    pw = (ow * s[1] - pd[1] + fw * d[1]) + off[:, :, 1]
    used = (ph > -1) & (pw > -1) & (ph < h) & (pw < w)          # [N, taps, P]
    ph = ph.reshape(n, 1, taps * p).expand(n, c, taps * p)
    pw = pw.reshape(n, 1, taps * p).expand(n, c, taps * p)
    used = used.reshape(n, 1, taps * p).expand(n, c, taps * p)
    cols = _bilinear_gather(input.reshape(n, c, h * w), ph, pw, h, w, used).view(n, c, taps, p)
    kern = _bank_kernel(weight, rotation, k, rotation_groups, n, c, p)
    return (cols * kern).sum(2).view(n, c, ho, wo)


def nd_linear_sample(data, coord):
    """N-d multilinear sample (ND.cu:45-88): data [C, s1..sD], coord [B, D] -> [B, C]."""
    c = data.shape[0]
    shape = data.shape[1:]
    dims = len(shape)
    b = coord.shape[0]
    flat = data.reshape(c, -1)
    valid = torch.ones(b, dtype=torch.bool)
    for d_ in range(dims):
        valid &= ~((coord[:, d_] <= -1) | (coord[:, d_] >= shape[d_]))
    low = torch.floor(coord).detach()
    frac = coord - low
    low = low.long()
    out = coord.new_zeros(b, c)
    for corner in itertools.product((0, 1), repeat=dims):
        ok = valid.clone()
        weight = torch.ones(b, dtype=coord.dtype)
        idx = torch.zeros(b, dtype=torch.long)
        for d_ in range(dims):
            pos = low[:, d_] + corner[d_]
            if corner[d_] == 0:
                ok &= pos >= 0
                weight = weight * (1 - frac[:, d_])
            else:
                ok &= pos <= shape[d_] - 1
                weight = weight * frac[:, d_]
            idx = idx * shape[d_] + pos.clamp(0, shape[d_] - 1)
        vals = flat[:, idx].t()                                   # [B, C]
        out = out + torch.where(ok.view(b, 1), weight.view(b, 1) * vals, torch.zeros_like(vals))
    return out


def grads(fn, inputs, grad_output):
    """Run fn on leaf copies of `inputs` and return (output, [grad per input])."""
    leaves = [t.detach().clone().requires_grad_(True) for t in inputs]
    out = fn(*leaves)
    gs = torch.autograd.grad(out, leaves, grad_output, allow_unused=True)
    return out.detach(), [g if g is not None else torch.zeros_like(t) for g, t in zip(gs, leaves)]
