"""Stand-in for the reference's pybind11 module ``nd_linear_sample_cuda``: the three
functions of csrc/nd_linear_sample_cuda.cpp:67-74 with their argument order, running on
libdk_b200.so.  The ``shape`` tensor the reference passes is accepted and ignored: the
extent is read from ``data`` itself."""
import ctypes

import torch

from ... import _cabi as C


def _shape(data):
    dims = data.dim() - 1
    return dims, (ctypes.c_int * dims)(*data.shape[1:])


def nd_linear_sample_forward_cuda(data, shape, coord, output):
    C.require_cuda(data, coord, output)
    C.same_dtype(data, coord, output)
    data, coord = data.contiguous(), coord.contiguous()
    dims, sh = _shape(data)
    with C.device_of(data):
        C.check(C.lib.dk_nd_linear_sample_forward(C.ptr(data), C.ptr(coord), C.ptr(output), coord.size(0), data.size(0),
                                                  dims, sh, C.dtype_code(data), C.stream_ptr(data.device)),
                "nd_linear_sample_forward")
    return 1


def nd_linear_sample_backward_data_cuda(out_grad, data, shape, coord, in_grad):
    C.require_cuda(out_grad, coord, in_grad)
    C.same_dtype(out_grad, coord, in_grad)
    out_grad, coord = out_grad.contiguous(), coord.contiguous()
    dims, sh = _shape(data)
    with C.device_of(data):
        C.check(C.lib.dk_nd_linear_sample_backward_data(C.ptr(out_grad), C.ptr(coord), C.ptr(in_grad), coord.size(0),
                                                        data.size(0), dims, sh, C.dtype_code(out_grad),
                                                        C.stream_ptr(data.device)), "nd_linear_sample_backward_data")
    return 1


def nd_linear_sample_backward_coord_cuda(out_grad, data, shape, coord, coord_grad_c):
    C.require_cuda(out_grad, data, coord, coord_grad_c)
    C.same_dtype(out_grad, data, coord, coord_grad_c)
    out_grad, data, coord = out_grad.contiguous(), data.contiguous(), coord.contiguous()
    dims, sh = _shape(data)
    with C.device_of(data):
        C.check(C.lib.dk_nd_linear_sample_backward_coord(C.ptr(out_grad), C.ptr(data), C.ptr(coord), C.ptr(coord_grad_c),
                                                         coord.size(0), data.size(0), dims, sh, C.dtype_code(data),
                                                         C.stream_ptr(data.device)), "nd_linear_sample_backward_coord")
    return 1
