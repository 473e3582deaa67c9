"""Python face of the CPU oracle (oracle/dk_oracle.c) -- TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and bench.py's CPU-baseline legs may import this
module.  The product package never does: it has no CPU path at all.

Every function takes CPU torch tensors (float32 or float64, all of one dtype) and
returns new CPU tensors of that dtype.  Half-precision cases are checked against
the float32 oracle evaluated on the half-rounded inputs (the reference itself runs
in fp32 under Apex: functions/filter_sample_depthwise.py:209-211).

Parity pin: tests/golden/ holds outputs of the reference's own CUDA build run on a
B200 (see oracle/build_ref.py and tests/golden/make_golden.py); tests/test_oracle.py
checks this oracle against them.
"""
import ctypes
import os
import subprocess

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "libdk_oracle.so")
_SRC = [os.path.join(HERE, f) for f in ("dk_oracle.c", "dk_oracle_impl.inc", "dk_oracle.h")]


class Geom(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "batch", "channel", "in_h", "in_w",
        "k_h", "k_w", "stride_h", "stride_w", "pad_h", "pad_w", "dil_h", "dil_w",
        "out_h", "out_w", "scope_h", "scope_w", "groups")]


def build(force=False):
    """Compile the oracle with gcc + OpenMP (a second or two)."""
    if not force and os.path.exists(LIB_PATH) and all(
            os.path.getmtime(LIB_PATH) >= os.path.getmtime(s) for s in _SRC):
        return LIB_PATH
    os.makedirs(os.path.dirname(LIB_PATH), exist_ok=True)
    subprocess.check_call(["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", _SRC[0], "-o", LIB_PATH, "-lm"])
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.dk_oracle_max_threads.restype = ctypes.c_int
    return _lib


def max_threads():
    return lib().dk_oracle_max_threads()


def set_threads(n):
    lib().dk_oracle_set_threads(int(n))


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def out_size(in_size, k, s, p, d):
    """functions/filter_sample_depthwise.py:90-97."""
    return (in_size + 2 * p - (d * (k - 1) + 1)) // s + 1


def geom(input, weight, kernel_size, stride, padding, dilation, groups):
    k, s, p, d = _pair(kernel_size), _pair(stride), _pair(padding), _pair(dilation)
    n, c, h, w = input.shape
    g = Geom(n, c, h, w, k[0], k[1], s[0], s[1], p[0], p[1], d[0], d[1],
             out_size(h, k[0], s[0], p[0], d[0]), out_size(w, k[1], s[1], p[1], d[1]),
             weight.shape[-2], weight.shape[-1], groups)
    return g


def _suffix(t):
    if t.dtype == torch.float32:
        return "_f32"
    if t.dtype == torch.float64:
        return "_f64"
    raise TypeError("oracle runs in float32 or float64, got %s" % t.dtype)


def _c(t):
    assert t.device.type == "cpu"
    return t.detach().contiguous()


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call(name, ref, *args):
    fn = getattr(lib(), name + _suffix(ref))
    fn.restype = None
    fn(*args)


# ---------------------------------------------------------------- local DK

def sample_depthwise_forward(input, rotation, weight, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1),
                             dilation=(1, 1), rotation_groups=1):
    input, rotation, weight = _c(input), _c(rotation), _c(weight)
    g = geom(input, weight, kernel_size, stride, padding, dilation, rotation_groups)
    out = input.new_empty(g.batch, g.channel, g.out_h, g.out_w)
    _call("dk_oracle_sample_depthwise_forward", input, _p(input), _p(rotation), _p(weight), _p(out), ctypes.byref(g))
    return out


def sample_depthwise_backward(grad_output, input, rotation, weight, kernel_size=(3, 3), stride=(1, 1),
                              padding=(1, 1), dilation=(1, 1), rotation_groups=1):
    """Returns (grad_input, grad_rotation, grad_weight)."""
    dy, input, rotation, weight = _c(grad_output), _c(input), _c(rotation), _c(weight)
    g = geom(input, weight, kernel_size, stride, padding, dilation, rotation_groups)
    dx = torch.empty_like(input)
    drot = torch.empty_like(rotation)
    dw = torch.empty_like(weight)
    _call("dk_oracle_sample_depthwise_backward_data", input, _p(dy), _p(rotation), _p(weight), _p(dx), ctypes.byref(g))
    _call("dk_oracle_sample_depthwise_backward_rotation", input, _p(dy), _p(input), _p(rotation), _p(weight),
          _p(drot), ctypes.byref(g))
    _call("dk_oracle_sample_depthwise_backward_filter", input, _p(dy), _p(input), _p(rotation), _p(dw),
          ctypes.byref(g))
    return dx, drot, dw


# ---------------------------------------------------------------- DK + DCN

def deform_sample_depthwise_forward(input, offset, rotation, weight, kernel_size=(3, 3), stride=(1, 1),
                                    padding=(1, 1), dilation=(1, 1), rotation_groups=1):
    input, offset, rotation, weight = _c(input), _c(offset), _c(rotation), _c(weight)
    g = geom(input, weight, kernel_size, stride, padding, dilation, rotation_groups)
    out = input.new_empty(g.batch, g.channel, g.out_h, g.out_w)
    _call("dk_oracle_deform_sample_depthwise_forward", input, _p(input), _p(offset), _p(rotation), _p(weight),
          _p(out), ctypes.byref(g))
    return out


def deform_sample_depthwise_backward(grad_output, input, offset, rotation, weight, kernel_size=(3, 3),
                                     stride=(1, 1), padding=(1, 1), dilation=(1, 1), rotation_groups=1):
    """Returns (grad_input, grad_offset, grad_rotation, grad_weight)."""
    dy, input, offset, rotation, weight = _c(grad_output), _c(input), _c(offset), _c(rotation), _c(weight)
    g = geom(input, weight, kernel_size, stride, padding, dilation, rotation_groups)
    dx = torch.empty_like(input)
    doff = torch.empty_like(offset)
    drot = torch.empty_like(rotation)
    dw = torch.empty_like(weight)
    gp = ctypes.byref(g)
    _call("dk_oracle_deform_sample_depthwise_backward_data", input, _p(dy), _p(offset), _p(rotation), _p(weight),
          _p(dx), gp)
    _call("dk_oracle_deform_sample_depthwise_backward_offset", input, _p(dy), _p(input), _p(offset), _p(rotation),
          _p(weight), _p(doff), gp)
    _call("dk_oracle_deform_sample_depthwise_backward_rotation", input, _p(dy), _p(input), _p(offset), _p(rotation),
          _p(weight), _p(drot), gp)
    _call("dk_oracle_deform_sample_depthwise_backward_filter", input, _p(dy), _p(input), _p(offset), _p(rotation),
          _p(dw), gp)
    return dx, doff, drot, dw


# ---------------------------------------------------------------- N-d linear sample

def _nd_args(data, coord):
    data, coord = _c(data), _c(coord)
    shape = torch.tensor(data.shape[1:], dtype=data.dtype)  # functions/nd_linear_sample.py:22
    batch, dims = coord.shape
    assert dims == data.dim() - 1
    prod = int(np.prod(data.shape[1:]))
    return data, coord, shape, batch, data.shape[0], dims, prod


def nd_linear_sample_forward(data, coord):
    data, coord, shape, b, c, d, prod = _nd_args(data, coord)
    out = data.new_empty(b, c)
    _call("dk_oracle_nd_linear_sample_forward", data, _p(data), _p(shape), _p(coord), _p(out), b, c, d, prod)
    return out


def nd_linear_sample_backward(grad_output, data, coord):
    """Returns (grad_data, grad_coord); grad_coord is the channel sum of the per-channel
    coordinate gradient, functions/nd_linear_sample.py:49-55."""
    dy = _c(grad_output)
    data, coord, shape, b, c, d, prod = _nd_args(data, coord)
    ddata = torch.empty_like(data)
    dcoord_c = coord.new_empty(b, d, c)
    _call("dk_oracle_nd_linear_sample_backward_data", data, _p(dy), _p(shape), _p(coord), _p(ddata), b, c, d, prod)
    _call("dk_oracle_nd_linear_sample_backward_coord", data, _p(dy), _p(data), _p(shape), _p(coord), _p(dcoord_c),
          b, c, d, prod)
    return ddata, dcoord_c.sum(2)


def nd_linear_sample_backward_coord_per_channel(grad_output, data, coord):
    dy = _c(grad_output)
    data, coord, shape, b, c, d, prod = _nd_args(data, coord)
    dcoord_c = coord.new_empty(b, d, c)
    _call("dk_oracle_nd_linear_sample_backward_coord", data, _p(dy), _p(data), _p(shape), _p(coord), _p(dcoord_c),
          b, c, d, prod)
    return dcoord_c
