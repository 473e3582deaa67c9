"""Depthwise deformable convolution = DK + DCN with scope == kernel size
(reference: modules/deform_conv.py:15-42)."""
from .deform_kernel import DeformKernelConv2d

__all__ = ['DeformConv2d']


class DeformConv2d(DeformKernelConv2d):
    def __init__(self, in_planes, out_planes, kernel_size=1, stride=1, padding=0, dilation=1, groups=1, bias=False,
                 offset_clip=None):
        super().__init__((kernel_size, kernel_size), in_planes, out_planes, kernel_size, stride, padding, dilation,
                         groups, bias, offset_clip)
