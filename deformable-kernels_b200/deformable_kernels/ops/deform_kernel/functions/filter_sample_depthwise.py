"""Autograd functions of the local deformable kernel and of DK + DCN.

Same names, argument order and defaults as the reference's
functions/filter_sample_depthwise.py:18-211 (``sample_depthwise``,
``deform_sample_depthwise``); what differs underneath:
  * one fused C-ABI call computes every requested gradient (the reference issues three
    or four launches and zero-fills each buffer first, :63-85 and :151-189);
  * ``backward`` returns one gradient per forward argument (the reference returns one
    too few, :87 and :191, which current PyTorch rejects);
  * work is enqueued on the current stream of the input's device.
CPU tensors raise NotImplementedError exactly as in the reference (:43-44).
"""
import torch
from torch.autograd import Function
from torch.nn.modules.utils import _pair

from .... import _cabi as C

__all__ = ['sample_depthwise', 'deform_sample_depthwise']


def _output_size(input, kernel_size, stride, padding, dilation):
    output_size = (input.size(0), input.size(1))
    for d in range(input.dim() - 2):
        kernel = dilation[d] * (kernel_size[d] - 1) + 1
        output_size += ((input.size(d + 2) + 2 * padding[d] - kernel) // stride[d] + 1,)
    if not all(s > 0 for s in output_size):
        raise ValueError("convolution input is too small (output would be {})".format(
            'x'.join(map(str, output_size))))
    return output_size


def _check_shapes(input, rotation, weight, out_size, kernel_size, groups, offset=None):
    if input.dim() != 4 or weight.dim() != 4 or weight.size(0) != input.size(1) or weight.size(1) != 1:
        raise ValueError("expected input [N,C,H,W] and a depthwise weight bank [C,1,sH,sW]")
    if input.size(1) % groups != 0:
        raise ValueError("channels must be divisible by rotation_groups")
    taps2 = kernel_size[0] * kernel_size[1] * 2
    want = (input.size(0), groups * taps2, out_size[2], out_size[3])
    if rotation is not None and tuple(rotation.shape) != want:
        raise ValueError("rotation must have shape {}, got {}".format(want, tuple(rotation.shape)))
    if offset is not None:
        want = (input.size(0), taps2, out_size[2], out_size[3])
        if tuple(offset.shape) != want:
            raise ValueError("offset must have shape {}, got {}".format(want, tuple(offset.shape)))


class SampleDepthwiseFunction(Function):
    @staticmethod
    def forward(ctx, input, rotation, weight, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1), dilation=(1, 1),
                rotation_groups=1):
        C.require_cuda(input, rotation, weight)
        C.same_dtype(input, rotation, weight)
        C.same_device(input, rotation, weight)
        kernel_size, stride, padding, dilation = _pair(kernel_size), _pair(stride), _pair(padding), _pair(dilation)
        out_size = _output_size(input, kernel_size, stride, padding, dilation)
        _check_shapes(input, rotation, weight, out_size, kernel_size, rotation_groups)
        input, rotation, weight = input.contiguous(), rotation.contiguous(), weight.contiguous()
        ctx.geom = C.geom(input.shape, kernel_size, stride, padding, dilation, weight.shape[2:], rotation_groups)
        ctx.save_for_backward(input, rotation, weight)
        output = input.new_empty(out_size)
        with C.device_of(input):
            C.check(C.lib.dk_sample_depthwise_forward(C.ptr(input), C.ptr(rotation), C.ptr(weight), C.ptr(output),
                                                      ctx.geom, C.dtype_code(input), C.stream_ptr(input.device)),
                    "sample_depthwise forward")
        return output

    @staticmethod
    def backward(ctx, grad_output):
        input, rotation, weight = ctx.saved_tensors
        C.require_cuda(grad_output)
        grad_output = grad_output.contiguous()
        if grad_output.dtype != input.dtype:
            grad_output = grad_output.to(input.dtype)
        need = ctx.needs_input_grad
        grad_input = torch.empty_like(input) if need[0] else None
        grad_rotation = torch.empty_like(rotation) if need[1] else None
        grad_weight = torch.empty_like(weight) if need[2] else None
        code = C.dtype_code(input)
        with C.device_of(input):
            nbytes = C.lib.dk_sample_depthwise_backward_workspace_bytes(ctx.geom, code)
            ws = C.workspace(nbytes, input.device)
            C.check(C.lib.dk_sample_depthwise_backward(
                C.ptr(grad_output), C.ptr(input), C.ptr(rotation), C.ptr(weight), C.ptr(grad_input),
                C.ptr(grad_rotation), C.ptr(grad_weight), ctx.geom, code, C.ptr(ws), nbytes,
                C.stream_ptr(input.device)), "sample_depthwise backward")
        return (grad_input, grad_rotation, grad_weight) + (None,) * 5


class DeformableSampleDepthwiseFunction(Function):
    @staticmethod
    def forward(ctx, input, offset, rotation, weight, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1),
                dilation=(1, 1), rotation_groups=1):
        C.require_cuda(input, offset, rotation, weight)
        C.same_dtype(input, offset, rotation, weight)
        C.same_device(input, offset, rotation, weight)
        kernel_size, stride, padding, dilation = _pair(kernel_size), _pair(stride), _pair(padding), _pair(dilation)
        out_size = _output_size(input, kernel_size, stride, padding, dilation)
        taps2 = kernel_size[0] * kernel_size[1] * 2
        rot_shape = (input.size(0), rotation_groups * taps2, out_size[2], out_size[3])
        output = input.new_empty(out_size)
        ctx.geom = C.geom(input.shape, kernel_size, stride, padding, dilation, weight.shape[2:], rotation_groups)
        if rotation is None:
            # zero kernel-space offsets: the library builds the (pixel-independent) kernel once where it can
            _check_shapes(input, None, weight, out_size, kernel_size, rotation_groups, offset)
            input, offset, weight = input.contiguous(), offset.contiguous(), weight.contiguous()
            with C.device_of(input):
                status = C.lib.dk_deform_sample_depthwise_forward(
                    C.ptr(input), C.ptr(offset), None, C.ptr(weight), C.ptr(output), ctx.geom, C.dtype_code(input),
                    C.stream_ptr(input.device))
            if status == 0:
                ctx.save_for_backward(input, offset, None, weight)
                return output
            if status != C.UNSUPPORTED:
                C.check(status, "deform_sample_depthwise forward")
            rotation = input.new_zeros(rot_shape)
        _check_shapes(input, rotation, weight, out_size, kernel_size, rotation_groups, offset)
        input, offset, rotation, weight = (input.contiguous(), offset.contiguous(), rotation.contiguous(),
                                           weight.contiguous())
        ctx.save_for_backward(input, offset, rotation, weight)
        with C.device_of(input):
            C.check(C.lib.dk_deform_sample_depthwise_forward(
                C.ptr(input), C.ptr(offset), C.ptr(rotation), C.ptr(weight), C.ptr(output), ctx.geom,
                C.dtype_code(input), C.stream_ptr(input.device)), "deform_sample_depthwise forward")
        return output

    @staticmethod
    def backward(ctx, grad_output):
        input, offset, rotation, weight = ctx.saved_tensors
        C.require_cuda(grad_output)
        grad_output = grad_output.contiguous()
        if grad_output.dtype != input.dtype:
            grad_output = grad_output.to(input.dtype)
        need = ctx.needs_input_grad
        grad_input = torch.empty_like(input) if need[0] else None
        grad_offset = torch.empty_like(offset) if need[1] else None
        grad_weight = torch.empty_like(weight) if need[3] else None
        code = C.dtype_code(input)
        if rotation is None:
            with C.device_of(input):
                nbytes = C.lib.dk_deform_sample_depthwise_backward_workspace_bytes(ctx.geom, code)
                ws = C.workspace(nbytes, input.device)
                status = C.lib.dk_deform_sample_depthwise_backward(
                    C.ptr(grad_output), C.ptr(input), C.ptr(offset), None, C.ptr(weight), C.ptr(grad_input),
                    C.ptr(grad_offset), None, C.ptr(grad_weight), ctx.geom, code, C.ptr(ws), nbytes,
                    C.stream_ptr(input.device))
            if status == 0:
                return (grad_input, grad_offset, None, grad_weight) + (None,) * 5
            if status != C.UNSUPPORTED:
                C.check(status, "deform_sample_depthwise backward")
            g = ctx.geom
            rotation = input.new_zeros((input.size(0), g.rotation_groups * g.kernel_h * g.kernel_w * 2) +
                                       tuple(grad_output.shape[2:]))
        grad_rotation = torch.empty_like(rotation) if need[2] else None
        with C.device_of(input):
            nbytes = C.lib.dk_deform_sample_depthwise_backward_workspace_bytes(ctx.geom, code)
            ws = C.workspace(nbytes, input.device)
            C.check(C.lib.dk_deform_sample_depthwise_backward(
                C.ptr(grad_output), C.ptr(input), C.ptr(offset), C.ptr(rotation), C.ptr(weight), C.ptr(grad_input),
                C.ptr(grad_offset), C.ptr(grad_rotation), C.ptr(grad_weight), ctx.geom, code, C.ptr(ws), nbytes,
                C.stream_ptr(input.device)), "deform_sample_depthwise backward")
        return (grad_input, grad_offset, grad_rotation, grad_weight) + (None,) * 5


def _common_dtype(input, *others):
    """Offsets produced under autocast and fp32 parameters may differ in dtype from the
    activations; the kernels want one dtype per call, so follow the input's."""
    return [t if t.dtype == input.dtype else t.to(input.dtype) for t in others]


def sample_depthwise(input, rotation, weight, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1), dilation=(1, 1),
                     rotation_groups=1):
    rotation, weight = _common_dtype(input, rotation, weight)
    return SampleDepthwiseFunction.apply(input, rotation, weight, kernel_size, stride, padding, dilation,
                                         rotation_groups)


def deform_sample_depthwise(input, offset, rotation, weight, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1),
                            dilation=(1, 1), rotation_groups=1):
    if rotation is None:
        offset, weight = _common_dtype(input, offset, weight)
    else:
        offset, rotation, weight = _common_dtype(input, offset, rotation, weight)
    return DeformableSampleDepthwiseFunction.apply(input, offset, rotation, weight, kernel_size, stride, padding,
                                                   dilation, rotation_groups)
