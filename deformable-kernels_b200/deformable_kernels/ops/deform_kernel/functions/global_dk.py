"""GlobalDeformKernel2d with a 1x1 depthwise kernel as one forward and one backward call
(reference modules/deform_kernel.py:76-118: global average pool -> linear coordinate head ->
clamp -> N-d linear sample of the bank -> per-sample grouped convolution, here a per-plane
scale).  The coordinate head runs in fp32 whatever the dtype of the feature map."""
import ctypes

import torch
from torch.autograd import Function

from .... import _cabi as C

__all__ = ['global_dk_scale']


class GlobalDKScaleFunction(Function):
    @staticmethod
    def forward(ctx, input, bank, fc_weight, fc_bias, tap_bias):
        C.require_cuda(input, bank, fc_weight, fc_bias, tap_bias)
        for t in (bank, fc_weight, fc_bias, tap_bias):
            if t.dtype != torch.float32:
                raise TypeError("the coordinate head's tensors must be float32")
        if input.dim() != 4 or bank.size(0) != input.size(1):
            raise ValueError("expected input [N,C,H,W] and bank [C, shape...]")
        dims = bank.dim() - 1
        if tuple(fc_weight.shape) != (dims, input.size(1)) or fc_bias.numel() != dims or tap_bias.numel() != dims:
            raise ValueError("expected fc_weight [dims, C], fc_bias [dims], tap_bias [dims]")
        input, bank = input.contiguous(), bank.contiguous()
        fc_weight, fc_bias, tap_bias = fc_weight.contiguous(), fc_bias.contiguous(), tap_bias.contiguous()
        n, c, h, w = input.shape
        output = torch.empty_like(input)
        f32 = dict(dtype=torch.float32, device=input.device)
        pooled, scale = torch.empty(n, c, **f32), torch.empty(n, c, **f32)
        raw, coord = torch.empty(n, dims, **f32), torch.empty(n, dims, **f32)
        shape = (ctypes.c_int * dims)(*bank.shape[1:])
        with C.device_of(input):
            C.check(C.lib.dk_global_dk_forward(
                C.ptr(input), C.ptr(bank), C.ptr(fc_weight), C.ptr(fc_bias), C.ptr(tap_bias), C.ptr(output), C.ptr(pooled),
                C.ptr(raw), C.ptr(coord), C.ptr(scale), n, c, h * w, dims, shape, C.dtype_code(input),
                C.stream_ptr(input.device)), "global_dk_scale forward")
        ctx.save_for_backward(input, bank, fc_weight, pooled, raw, coord, scale)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        input, bank, fc_weight, pooled, raw, coord, scale = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        n, c, h, w = input.shape
        dims = bank.dim() - 1
        need = ctx.needs_input_grad
        grad_input = torch.empty_like(input) if need[0] else None
        grad_bank = torch.empty_like(bank) if need[1] else None
        grad_fc_weight = torch.empty_like(fc_weight) if need[2] else None
        grad_fc_bias = torch.empty(dims, dtype=torch.float32, device=input.device) if need[3] else None
        shape = (ctypes.c_int * dims)(*bank.shape[1:])
        with C.device_of(input):
            nbytes = C.lib.dk_global_dk_backward_workspace_bytes(n, c, dims)
            ws = C.workspace(nbytes, input.device)
            C.check(C.lib.dk_global_dk_backward(
                C.ptr(grad_output), C.ptr(input), C.ptr(bank), C.ptr(fc_weight), C.ptr(pooled), C.ptr(raw), C.ptr(coord),
                C.ptr(scale), C.ptr(grad_input), C.ptr(grad_bank), C.ptr(grad_fc_weight), C.ptr(grad_fc_bias), n, c, h * w,
                dims, shape, C.dtype_code(input), C.ptr(ws), nbytes, C.stream_ptr(input.device)), "global_dk_scale backward")
        return grad_input, grad_bank, grad_fc_weight, grad_fc_bias, None


global_dk_scale = GlobalDKScaleFunction.apply
