"""Autograd function of the N-d multilinear sampler used by the global deformable kernel.

Same name and signature as the reference's functions/nd_linear_sample.py:18-65:
``nd_linear_sample(input[C, s1..sD], coord[B, D]) -> [B, C]``.  The coordinate gradient
is reduced over channels inside the kernel (the reference materialises [B, D, C] and
sums in Python, :49-55) and no ``shape`` tensor is built on the host per call (:22, :36).
"""
import ctypes

import torch
from torch.autograd import Function

from .... import _cabi as C

__all__ = ['nd_linear_sample']


class NdLinearSampleFunction(Function):
    @staticmethod
    def forward(ctx, input, coord):
        C.require_cuda(input, coord)
        C.same_dtype(input, coord)
        C.same_device(input, coord)
        if input.dim() < 2 or coord.dim() != 2 or coord.size(1) != input.dim() - 1:
            raise ValueError("expected input [C, s1..sD] and coord [B, D]")
        input, coord = input.contiguous(), coord.contiguous()
        ctx.save_for_backward(input, coord)
        dims = input.dim() - 1
        shape = (ctypes.c_int * dims)(*input.shape[1:])
        output = input.new_empty(coord.size(0), input.size(0))
        with C.device_of(input):
            C.check(C.lib.dk_nd_linear_sample_forward(C.ptr(input), C.ptr(coord), C.ptr(output), coord.size(0),
                                                      input.size(0), dims, shape, C.dtype_code(input),
                                                      C.stream_ptr(input.device)), "nd_linear_sample forward")
        return output

    @staticmethod
    def backward(ctx, grad_output):
        input, coord = ctx.saved_tensors
        C.require_cuda(grad_output)
        grad_output = grad_output.contiguous()
        dims = input.dim() - 1
        shape = (ctypes.c_int * dims)(*input.shape[1:])
        grad_input = grad_coord = None
        code = C.dtype_code(input)
        with C.device_of(input):
            if ctx.needs_input_grad[0]:
                grad_input = torch.empty_like(input)
                C.check(C.lib.dk_nd_linear_sample_backward_data(
                    C.ptr(grad_output), C.ptr(coord), C.ptr(grad_input), coord.size(0), input.size(0), dims, shape,
                    code, C.stream_ptr(input.device)), "nd_linear_sample backward (data)")
            if ctx.needs_input_grad[1]:
                grad_coord = torch.empty_like(coord)
                C.check(C.lib.dk_nd_linear_sample_backward_coord_sum(
                    C.ptr(grad_output), C.ptr(input), C.ptr(coord), C.ptr(grad_coord), coord.size(0), input.size(0),
                    dims, shape, code, C.stream_ptr(input.device)), "nd_linear_sample backward (coord)")
        return grad_input, grad_coord


nd_linear_sample = NdLinearSampleFunction.apply
