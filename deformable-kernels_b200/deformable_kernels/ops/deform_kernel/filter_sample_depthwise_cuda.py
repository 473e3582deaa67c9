"""Stand-in for the reference's pybind11 module of the same name: the nine functions of
csrc/filter_sample_depthwise_cuda.cpp:540-569 with their argument order, running on
libdk_b200.so.  With this module importable as ``..filter_sample_depthwise_cuda`` the
reference's own functions/filter_sample_depthwise.py runs unchanged.

Differences a caller can rely on: launches go to the current stream of the tensors'
device, errors raise instead of printing, and gradient buffers need not be zeroed.
"""
import torch

from ... import _cabi as C


def _geom(input, kH, kW, dH, dW, padH, padW, dilH, dilW, scopeH, scopeW, groupS):
    return C.geom(input.shape, (kH, kW), (dH, dW), (padH, padW), (dilH, dilW), (scopeH, scopeW), groupS)


def _prep(*ts):
    C.require_cuda(*ts)
    C.same_dtype(*ts)
    return [t.contiguous() for t in ts]


def _out(out):
    if not out.is_contiguous():
        raise ValueError("output tensor must be contiguous")
    return out


def sample_depthwise_forward_cuda(input, rotation, filter, output, *ints):
    input, rotation, filter = _prep(input, rotation, filter)
    g = _geom(input, *ints)
    with C.device_of(input):
        C.check(C.lib.dk_sample_depthwise_forward(C.ptr(input), C.ptr(rotation), C.ptr(filter), C.ptr(_out(output)), g,
                                                  C.dtype_code(input), C.stream_ptr(input.device)),
                "sample_depthwise_forward")
    return 1


def sample_depthwise_backward_data_cuda(gradOutput, input, rotation, filter, gradInput, *ints):
    gradOutput, rotation, filter = _prep(gradOutput, rotation, filter)
    g = _geom(input, *ints)
    with C.device_of(input):
        C.check(C.lib.dk_sample_depthwise_backward_data(C.ptr(gradOutput), C.ptr(rotation), C.ptr(filter),
                                                        C.ptr(_out(gradInput)), g, C.dtype_code(gradOutput),
                                                        C.stream_ptr(input.device)), "sample_depthwise_backward_data")
    return 1


def sample_depthwise_backward_filter_cuda(gradOutput, input, rotation, filter, gradFilter, *ints):
    gradOutput, input, rotation = _prep(gradOutput, input, rotation)
    g = _geom(input, *ints)
    code = C.dtype_code(input)
    with C.device_of(input):
        nbytes = C.lib.dk_sample_depthwise_backward_filter_workspace_bytes(g, code)
        ws = C.workspace(nbytes, input.device)
        C.check(C.lib.dk_sample_depthwise_backward_filter(C.ptr(gradOutput), C.ptr(input), C.ptr(rotation),
                                                          C.ptr(_out(gradFilter)), g, code, C.ptr(ws), nbytes,
                                                          C.stream_ptr(input.device)), "sample_depthwise_backward_filter")
    return 1


def sample_depthwise_backward_rotation_cuda(gradOutput, input, rotation, filter, gradRotation, *ints):
    gradOutput, input, rotation, filter = _prep(gradOutput, input, rotation, filter)
    g = _geom(input, *ints)
    code = C.dtype_code(input)
    with C.device_of(input):
        nbytes = C.lib.dk_sample_depthwise_backward_rotation_workspace_bytes(g, code)
        ws = C.workspace(nbytes, input.device)
        C.check(C.lib.dk_sample_depthwise_backward_rotation(C.ptr(gradOutput), C.ptr(input), C.ptr(rotation),
                                                            C.ptr(filter), C.ptr(_out(gradRotation)), g, code,
                                                            C.ptr(ws), nbytes, C.stream_ptr(input.device)),
                "sample_depthwise_backward_rotation")
    return 1


def deformable_sample_depthwise_forward_cuda(input, offset, rotation, filter, output, *ints):
    input, offset, rotation, filter = _prep(input, offset, rotation, filter)
    g = _geom(input, *ints)
    with C.device_of(input):
        C.check(C.lib.dk_deform_sample_depthwise_forward(C.ptr(input), C.ptr(offset), C.ptr(rotation), C.ptr(filter),
                                                         C.ptr(_out(output)), g, C.dtype_code(input),
                                                         C.stream_ptr(input.device)), "deform_sample_depthwise_forward")
    return 1


def deformable_sample_depthwise_backward_data_cuda(gradOutput, input, offset, rotation, filter, gradInput, *ints):
    gradOutput, offset, rotation, filter = _prep(gradOutput, offset, rotation, filter)
    g = _geom(input, *ints)
    code = C.dtype_code(gradOutput)
    with C.device_of(input):
        nbytes = C.lib.dk_deform_sample_depthwise_backward_data_workspace_bytes(g, code)
        ws = C.workspace(nbytes, input.device)
        C.check(C.lib.dk_deform_sample_depthwise_backward_data(C.ptr(gradOutput), C.ptr(offset), C.ptr(rotation),
                                                               C.ptr(filter), C.ptr(_out(gradInput)), g, code,
                                                               C.ptr(ws), nbytes, C.stream_ptr(input.device)),
                "deform_sample_depthwise_backward_data")
    return 1


def deformable_sample_depthwise_backward_filter_cuda(gradOutput, input, offset, rotation, filter, gradFilter, *ints):
    gradOutput, input, offset, rotation = _prep(gradOutput, input, offset, rotation)
    g = _geom(input, *ints)
    code = C.dtype_code(input)
    with C.device_of(input):
        nbytes = C.lib.dk_deform_sample_depthwise_backward_filter_workspace_bytes(g, code)
        ws = C.workspace(nbytes, input.device)
        C.check(C.lib.dk_deform_sample_depthwise_backward_filter(C.ptr(gradOutput), C.ptr(input), C.ptr(offset),
                                                                 C.ptr(rotation), C.ptr(_out(gradFilter)), g, code,
                                                                 C.ptr(ws), nbytes, C.stream_ptr(input.device)),
                "deform_sample_depthwise_backward_filter")
    return 1


def deformable_sample_depthwise_backward_offset_cuda(gradOutput, input, offset, rotation, filter, gradOffset, *ints):
    gradOutput, input, offset, rotation, filter = _prep(gradOutput, input, offset, rotation, filter)
    g = _geom(input, *ints)
    with C.device_of(input):
        C.check(C.lib.dk_deform_sample_depthwise_backward_offset(C.ptr(gradOutput), C.ptr(input), C.ptr(offset),
                                                                 C.ptr(rotation), C.ptr(filter), C.ptr(_out(gradOffset)),
                                                                 g, C.dtype_code(input), C.stream_ptr(input.device)),
                "deform_sample_depthwise_backward_offset")
    return 1


def deformable_sample_depthwise_backward_rotation_cuda(gradOutput, input, offset, rotation, filter, gradRotation,
                                                       *ints):
    gradOutput, input, offset, rotation, filter = _prep(gradOutput, input, offset, rotation, filter)
    g = _geom(input, *ints)
    with C.device_of(input):
        C.check(C.lib.dk_deform_sample_depthwise_backward_rotation(C.ptr(gradOutput), C.ptr(input), C.ptr(offset),
                                                                   C.ptr(rotation), C.ptr(filter),
                                                                   C.ptr(_out(gradRotation)), g, C.dtype_code(input),
                                                                   C.stream_ptr(input.device)),
                "deform_sample_depthwise_backward_rotation")
    return 1
