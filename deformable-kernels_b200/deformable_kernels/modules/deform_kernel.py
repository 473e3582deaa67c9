"""User-facing layers that produce the offsets and call the operators.

Same class names, constructor arguments and sub-module / parameter names as the
reference's modules/deform_kernel.py (``GlobalDeformKernel2d`` :28-132,
``LocalDeformKernel2d`` = ``DeformKernel2d`` :135-225, ``DeformKernelConv2d`` :228-281), so
state dicts are interchangeable: ``weight``, ``fc.*``; ``rotation_conv.*``,
``inner_conv.weight``; ``offset_conv.*``, ``inner_conv.weight``.
"""
import torch
from torch import nn

from ..ops.deform_kernel.functions import clip_offsets, global_dk_scale, nd_linear_sample, plane_scale
from ..ops.deform_kernel.modules import SampleDepthwise, DeformableSampleDepthwise

__all__ = ['GlobalDeformKernel2d', 'LocalDeformKernel2d', 'DeformKernel2d', 'DeformKernelConv2d']


def _tap_positions(weight_shape, kernel_size, weight_dilate=1):
    """Scope-centred coordinates of the kernel taps: the additive bias of the coordinate
    head (reference :64-74)."""
    start_h = (weight_shape[0] - (kernel_size - 1) * weight_dilate - 1) / 2.0
    start_w = (weight_shape[1] - (kernel_size - 1) * weight_dilate - 1) / 2.0
    out = []
    for h in range(kernel_size):
        for w in range(kernel_size):
            out += [start_h + h * weight_dilate, start_w + w * weight_dilate]
            for i in range(len(weight_shape) - 2):
                out += [(weight_shape[i + 2] - 1) / 2.0]
    return out


class GlobalDeformKernel2d(nn.Module):
    """One resampled kernel per sample: global-average-pool -> FC -> coordinates -> N-d
    linear sample of the weight bank -> per-sample grouped convolution."""

    def __init__(self, weight_shape, in_planes, out_planes, kernel_size=1, stride=1, padding=0, dilation=1, groups=1,
                 bias=False):
        super().__init__()
        assert not bias
        assert len(weight_shape) >= 2
        self.kernel_size = kernel_size
        self.weight_shape = tuple(weight_shape)
        self.weight_dilate = 1
        self.stride = stride
        self.padding = padding
        self.dilation = dilation
        self.out_planes = out_planes
        self.in_planes = in_planes
        self.group = groups
        self.weight = nn.Parameter(torch.empty(out_planes, in_planes // groups, *self.weight_shape))
        self.fc = nn.Linear(in_planes, kernel_size * kernel_size * len(self.weight_shape))
        self.fc.zero_init = True
        self.fc_bias = _tap_positions(self.weight_shape, kernel_size, self.weight_dilate)
        # the reference leaves `weight` uninitialised (torch.Tensor(...), :54); give it a defined start
        nn.init.kaiming_normal_(self.weight.view(out_planes, -1, *self.weight_shape[-2:]))
        self.register_buffer('_tap_bias', torch.tensor(self.fc_bias, dtype=torch.float32), persistent=False)

    def dynamic_weight(self, x, weight):
        n, c, h, w = x.shape
        k2 = self.kernel_size * self.kernel_size
        avg_x = x.float().view(n, c, -1).mean(2)
        coord = self.fc(avg_x) * self.weight_dilate + self._tap_bias.unsqueeze(0)
        coord = torch.clamp(coord, 0, self.weight_shape[0] - 1)
        bank = weight.float().reshape(self.out_planes * self.in_planes // self.group, *self.weight_shape)
        coord = coord.view(n * k2, len(self.weight_shape))
        sample = nd_linear_sample(bank, coord).view(n, k2, self.out_planes * self.in_planes // self.group)
        return sample.transpose(1, 2).reshape(n * self.out_planes, self.in_planes // self.group, self.kernel_size,
                                              self.kernel_size)

    def _is_plane_scale(self):
        return (self.kernel_size == 1 and self.stride in (1, (1, 1)) and self.padding in (0, (0, 0)) and
                self.group == self.in_planes == self.out_planes)

    def _fused_head_ok(self, x):
        return (x.is_cuda and self._is_plane_scale() and self.weight_dilate == 1 and len(self.weight_shape) <= 8 and
                x.dtype in (torch.float16, torch.float32) and self.weight.dtype == torch.float32 and
                self.fc.weight.dtype == torch.float32 and self.fc.bias is not None and not torch.is_autocast_enabled())

    def forward(self, x):
        n, c, h, w = x.shape
        if self._fused_head_ok(x):
            # pool, coordinate head, bank sampling and the per-plane scale in one call each way
            return global_dk_scale(x, self.weight.view(c, *self.weight_shape), self.fc.weight, self.fc.bias, self._tap_bias)
        weight = self.dynamic_weight(x, self.weight).to(x.dtype)
        if self._is_plane_scale() and x.is_cuda:
            # 1x1 depthwise: the per-sample grouped convolution is a per-plane scale
            return plane_scale(x, weight.view(n, c))
        out = nn.functional.conv2d(x.reshape(1, n * c, h, w), weight, stride=self.stride, padding=self.padding,
                                   dilation=self.dilation, groups=n * self.group)
        return out.view(n, self.out_planes, out.shape[2], out.shape[3])

    def extra_repr(self):
        s = ('{in_planes}, {out_planes}, weight_shape={weight_shape}, kernel_size={kernel_size}, stride={stride}, '
             'weight_dilate={weight_dilate}')
        if self.padding != 0:
            s += ', padding={padding}'
        if self.dilation != 1:
            s += ', dilation={dilation}'
        if self.group != 1:
            s += ', group={group}'
        return s.format(**self.__dict__)


class LocalDeformKernel2d(nn.Module):
    """Kernel-space offsets from a dense conv, then the local deformable kernel."""

    def __init__(self, weight_shape, in_planes, out_planes, kernel_size=1, stride=1, padding=0, dilation=1, groups=1,
                 rotation_groups=1, bias=False, rotation_clip=None):
        super().__init__()
        assert not bias
        assert len(weight_shape) >= 2
        self.kernel_size = kernel_size
        self.weight_shape = tuple(weight_shape)
        self.weight_dilate = 1
        self.stride = stride
        self.padding = padding
        self.dilation = dilation
        self.out_planes = out_planes
        self.in_planes = in_planes
        self.rotation_groups = rotation_groups
        self.group = groups
        self.rotation_conv = nn.Conv2d(in_planes, rotation_groups * kernel_size * kernel_size * 2, kernel_size, stride,
                                       padding, dilation, bias=True)
        self.rotation_conv.zero_init = True
        self.rotation_clip = rotation_clip
        self.inner_conv = SampleDepthwise(self.weight_shape, in_planes, out_planes, kernel_size=kernel_size,
                                          stride=stride, padding=padding, dilation=dilation, groups=groups,
                                          rotation_groups=rotation_groups, bias=bias)

    def _clip_rotation(self, rotation):
        if isinstance(self.rotation_clip, tuple):
            return rotation.clamp(*self.rotation_clip)
        if self.rotation_clip == 'scope':
            bias = rotation.new_tensor(_tap_positions(self.weight_shape, self.kernel_size, self.weight_dilate)) \
                .repeat(self.rotation_groups)[None, :, None, None]
            coord = (rotation * self.weight_dilate + bias).clamp(0, self.weight_shape[0] - 1)
            return (coord - bias) / self.weight_dilate
        raise NotImplementedError(
            'Expect rotation_clip to be tuple or "scope", but get {}'.format(self.rotation_clip))

    def _fused_clip(self, rotation):
        """Clip and scale in one pass on CUDA; None when the configuration is not one the fused op covers."""
        if not rotation.is_cuda or rotation.dtype not in (torch.float16, torch.float32, torch.float64):
            return None
        if isinstance(self.rotation_clip, tuple) and len(self.rotation_clip) == 2:
            return clip_offsets(rotation, None, self.rotation_clip[0], self.rotation_clip[1], 1.0, self.weight_dilate)
        if self.rotation_clip == 'scope':
            bias = rotation.new_tensor(_tap_positions(self.weight_shape, self.kernel_size, self.weight_dilate),
                                       dtype=torch.float32).repeat(self.rotation_groups)
            return clip_offsets(rotation, bias, 0.0, self.weight_shape[0] - 1, self.weight_dilate, self.weight_dilate)
        return None

    def forward(self, x):
        rotation = self.rotation_conv(x)
        fused = self._fused_clip(rotation) if self.rotation_clip is not None else None
        if fused is not None:
            return self.inner_conv(x, fused)
        if self.rotation_clip is not None:
            rotation = self._clip_rotation(rotation)
        if self.weight_dilate != 1:
            rotation = rotation * self.weight_dilate
        return self.inner_conv(x, rotation)


DeformKernel2d = LocalDeformKernel2d


class DeformKernelConv2d(nn.Module):
    """Image-space (DCN) offsets from a dense conv, then DK + DCN with zero kernel-space offsets."""

    def __init__(self, weight_shape, in_planes, out_planes, kernel_size=1, stride=1, padding=0, dilation=1, groups=1,
                 bias=False, offset_clip=None):
        super().__init__()
        assert not bias
        self.kernel_size = kernel_size
        self.stride = stride
        self.padding = padding
        self.dilation = dilation
        self.out_planes = out_planes
        self.in_planes = in_planes
        self.group = groups
        self.offset_conv = nn.Conv2d(in_planes, kernel_size * kernel_size * 2, kernel_size, stride, padding, dilation,
                                     bias=True)
        self.offset_conv.zero_init = True
        self.offset_clip = offset_clip
        self.inner_conv = DeformableSampleDepthwise(tuple(weight_shape), in_planes, out_planes, kernel_size=kernel_size,
                                                    stride=stride, padding=padding, dilation=dilation, groups=groups,
                                                    bias=bias)

    def forward(self, x):
        offset = self.offset_conv(x)
        clip = self.offset_clip
        if (clip is not None and offset.is_cuda and isinstance(clip, dict) and set(clip) <= {'min', 'max'} and
                isinstance(self.dilation, (int, float))):
            # clamp and dilation scaling in one pass
            offset = clip_offsets(offset, None, clip.get('min', float('-inf')), clip.get('max', float('inf')), 1.0,
                                  float(self.dilation))
            return self.inner_conv(x, offset, None)
        if clip is not None:
            offset = offset.clamp(**clip)
        if self.dilation != 1:
            offset = offset * self.dilation
        return self.inner_conv(x, offset, None)
