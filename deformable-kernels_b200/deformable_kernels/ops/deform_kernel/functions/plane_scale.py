"""Per-(sample, channel) scaling y[n,c] = x[n,c] * k[n,c]: the global deformable kernel's per-sample grouped
convolution (reference modules/deform_kernel.py:105-118) in the 1x1 depthwise case, as one streaming pass with a
fused backward (grad-input and the per-plane reduction grad-k in the same kernel)."""
import torch
from torch.autograd import Function

from .... import _cabi as C

__all__ = ['plane_scale']


class PlaneScaleFunction(Function):
    @staticmethod
    def forward(ctx, input, scale):
        C.require_cuda(input, scale)
        C.same_dtype(input, scale)
        C.same_device(input, scale)
        if input.dim() != 4 or tuple(scale.shape) != tuple(input.shape[:2]):
            raise ValueError("expected input [N,C,H,W] and scale [N,C]")
        input, scale = input.contiguous(), scale.contiguous()
        ctx.save_for_backward(input, scale)
        output = torch.empty_like(input)
        n, c, h, w = input.shape
        with C.device_of(input):
            C.check(C.lib.dk_plane_scale_forward(C.ptr(input), C.ptr(scale), C.ptr(output), n * c, h * w,
                                                 C.dtype_code(input), C.stream_ptr(input.device)), "plane_scale forward")
        return output

    @staticmethod
    def backward(ctx, grad_output):
        input, scale = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        n, c, h, w = input.shape
        grad_input = torch.empty_like(input) if ctx.needs_input_grad[0] else None
        grad_scale = torch.empty_like(scale) if ctx.needs_input_grad[1] else None
        with C.device_of(input):
            C.check(C.lib.dk_plane_scale_backward(C.ptr(grad_output), C.ptr(input), C.ptr(scale), C.ptr(grad_input),
                                                  C.ptr(grad_scale), n * c, h * w, C.dtype_code(input),
                                                  C.stream_ptr(input.device)), "plane_scale backward")
        return grad_input, grad_scale


plane_scale = PlaneScaleFunction.apply
