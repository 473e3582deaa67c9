"""nn.Module wrappers that own the weight bank.

Same class names, constructor arguments, parameter names (``weight`` [C,1,sH,sW], optional
``bias`` [C]) and initialisation as the reference's modules/filter_sample_depthwise.py:27-206,
so that checkpoints and the reference's higher-level layers work unchanged.
"""
import math

import torch
import torch.nn as nn
from torch.nn.modules.utils import _pair

from ..functions.filter_sample_depthwise import sample_depthwise, deform_sample_depthwise

__all__ = ['SampleDepthwise', 'DeformableSampleDepthwise']


class _BankConv(nn.Module):
    def __init__(self, scope_size, in_channels, out_channels, kernel_size=3, stride=1, padding=1, dilation=1,
                 groups=1, rotation_groups=1, bias=False):
        super().__init__()
        # depthwise only, as in the reference (:41-43)
        assert in_channels == out_channels and groups == in_channels
        assert in_channels % rotation_groups == 0 and out_channels % rotation_groups == 0
        self.in_channels = in_channels
        self.scope_size = tuple(scope_size)
        self.kernel_size = _pair(kernel_size)
        self.stride = _pair(stride)
        self.padding = _pair(padding)
        self.dilation = _pair(dilation)
        self.rotation_groups = rotation_groups
        self.weight = nn.Parameter(torch.empty(in_channels, 1, *self.scope_size))
        self.bias = nn.Parameter(torch.empty(in_channels)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        # U(-1/sqrt(kH*kW), +1/sqrt(kH*kW)), zero bias (:59-66)
        stdv = 1.0 / math.sqrt(self.kernel_size[0] * self.kernel_size[1])
        with torch.no_grad():
            self.weight.uniform_(-stdv, stdv)
            if self.bias is not None:
                self.bias.zero_()

    def _output_size(self, input):
        size = (input.size(0), self.weight.size(0))
        for d in range(input.dim() - 2):
            kernel = self.dilation[d] * (self.kernel_size[d] - 1) + 1
            size += ((input.size(d + 2) + 2 * self.padding[d] - kernel) // self.stride[d] + 1,)
        if not all(s > 0 for s in size):
            raise ValueError("convolution input is too small (output would be {})".format('x'.join(map(str, size))))
        return size

    def _zero_offsets(self, input, groups):
        size = self._output_size(input)
        return input.new_zeros(input.size(0), groups * self.kernel_size[0] * self.kernel_size[1] * 2, size[2], size[3])

    def _add_bias(self, out):
        if self.bias is not None:
            out = out + self.bias.view(1, self.in_channels, 1, 1).to(out.dtype)
        return out

    def extra_repr(self):
        s = 'scope_size={scope_size}, in_channels={in_channels}, kernel_size={kernel_size}, stride={stride}'
        if self.padding != (0,) * len(self.padding):
            s += ', padding={padding}'
        if self.dilation != (1,) * len(self.dilation):
            s += ', dilation={dilation}'
        if self.rotation_groups != 1:
            s += ', rotation_groups={rotation_groups}'
        if self.bias is None:
            s += ', bias=False'
        return s.format(**self.__dict__)


class SampleDepthwise(_BankConv):
    """Local deformable kernel: forward(input, rotation=None); zero offsets when omitted (:68-76)."""

    def forward(self, input, rotation=None):
        if rotation is None:
            rotation = self._zero_offsets(input, self.rotation_groups)
        out = sample_depthwise(input, rotation, self.weight, self.kernel_size, self.stride, self.padding,
                               self.dilation, self.rotation_groups)
        return self._add_bias(out)


class DeformableSampleDepthwise(_BankConv):
    """DK + DCN: forward(input, offset=None, rotation=None); zero offsets when omitted (:155-170)."""

    def forward(self, input, offset=None, rotation=None):
        if offset is None:
            offset = self._zero_offsets(input, 1)
        out = deform_sample_depthwise(input, offset, rotation, self.weight, self.kernel_size, self.stride,
                                      self.padding, self.dilation, self.rotation_groups)
        return self._add_bias(out)
