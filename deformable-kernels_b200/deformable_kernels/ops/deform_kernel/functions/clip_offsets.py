"""Clipping and scaling of produced offsets in one pass (reference modules/deform_kernel.py:185-218 `_clip_rotation`,
:165-170 `rotation * weight_dilate`, :273-276 offset clamp and `* dilation`):

    v = offsets * dilate + bias[channel];  output = (clamp(v, lo, hi) - bias[channel]) / dilate * post_scale
"""
import torch
from torch.autograd import Function

from .... import _cabi as C

__all__ = ['clip_offsets']


class ClipOffsetsFunction(Function):
    @staticmethod
    def forward(ctx, offsets, bias, lo, hi, dilate, post_scale):
        C.require_cuda(offsets, bias)
        if offsets.dim() != 4:
            raise ValueError("expected offsets [N, C, H, W]")
        if bias is not None:
            if bias.dtype != torch.float32 or bias.numel() != offsets.size(1):
                raise ValueError("bias must be float32 with one entry per offset channel")
            bias = bias.contiguous()
        offsets = offsets.contiguous()
        ctx.save_for_backward(offsets, bias)
        ctx.args = (float(lo), float(hi), float(dilate), float(post_scale))
        output = torch.empty_like(offsets)
        n, c, h, w = offsets.shape
        with C.device_of(offsets):
            C.check(C.lib.dk_offset_clip_forward(C.ptr(offsets), C.ptr(bias), C.ptr(output), n, c, h * w, *ctx.args,
                                                 C.dtype_code(offsets), C.stream_ptr(offsets.device)), "clip_offsets forward")
        return output

    @staticmethod
    def backward(ctx, grad_output):
        offsets, bias = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        grad = torch.empty_like(offsets)
        n, c, h, w = offsets.shape
        with C.device_of(offsets):
            C.check(C.lib.dk_offset_clip_backward(C.ptr(grad_output), C.ptr(offsets), C.ptr(bias), C.ptr(grad), n, c, h * w,
                                                  *ctx.args, C.dtype_code(offsets), C.stream_ptr(offsets.device)),
                    "clip_offsets backward")
        return grad, None, None, None, None, None


def clip_offsets(offsets, bias=None, lo=float('-inf'), hi=float('inf'), dilate=1.0, post_scale=1.0):
    return ClipOffsetsFunction.apply(offsets, bias, lo, hi, dilate, post_scale)
