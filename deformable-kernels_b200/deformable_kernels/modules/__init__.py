from .deform_conv import DeformConv2d
from .deform_kernel import (
    GlobalDeformKernel2d,
    LocalDeformKernel2d,
    DeformKernel2d,
    DeformKernelConv2d,
)

__all__ = [
    'DeformConv2d',
    'GlobalDeformKernel2d',
    'LocalDeformKernel2d',
    'DeformKernel2d',
    'DeformKernelConv2d',
]
