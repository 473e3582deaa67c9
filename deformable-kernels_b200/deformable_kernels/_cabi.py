"""ctypes binding of libdk_b200.so (declared in include/dk_b200.h).

There is no CPU path and no fallback: if the library has not been built, importing
this module raises, and every operator raises NotImplementedError for CPU tensors
just as the reference does (functions/filter_sample_depthwise.py:43-44).
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("DK_B200_LIB", os.path.join(os.path.dirname(_HERE), "lib", "libdk_b200.so"))

DK_F32, DK_F16, DK_F64 = 0, 1, 2
_DTYPES = {torch.float32: DK_F32, torch.float16: DK_F16, torch.float64: DK_F64}


class Geom(ctypes.Structure):
    """struct dk_geom."""
    _fields_ = [(n, ctypes.c_int) for n in (
        "batch", "channels", "in_h", "in_w", "kernel_h", "kernel_w", "stride_h", "stride_w",
        "pad_h", "pad_w", "dil_h", "dil_w", "scope_h", "scope_w", "rotation_groups")]


if not os.path.exists(LIB_PATH):
    raise ImportError(
        "libdk_b200.so not found at %s: build it with `python deformable-kernels_b200/build.py` "
        "(there is no CPU fallback)" % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

_vp, _sz, _int = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
_gp = ctypes.POINTER(Geom)
_ip = ctypes.POINTER(ctypes.c_int)

_PROTOS = {
    "dk_sample_depthwise_forward": (_int, [_vp, _vp, _vp, _vp, _gp, _int, _vp]),
    "dk_sample_depthwise_backward_data": (_int, [_vp, _vp, _vp, _vp, _gp, _int, _vp]),
    "dk_sample_depthwise_backward_filter_workspace_bytes": (_sz, [_gp, _int]),
    "dk_sample_depthwise_backward_filter": (_int, [_vp, _vp, _vp, _vp, _gp, _int, _vp, _sz, _vp]),
    "dk_sample_depthwise_backward_filter_noalloc_max_bytes": (_sz, []),
    "dk_sample_depthwise_backward_filter_noalloc_bytes": (_sz, [_gp, _int]),
    "dk_sample_depthwise_backward_filter_noalloc": (_int, [_vp, _vp, _vp, _vp, _gp, _int, _vp]),
    "dk_sample_depthwise_backward_rotation_workspace_bytes": (_sz, [_gp, _int]),
    "dk_sample_depthwise_backward_rotation": (_int, [_vp, _vp, _vp, _vp, _vp, _gp, _int, _vp, _sz, _vp]),
    "dk_sample_depthwise_backward_workspace_bytes": (_sz, [_gp, _int]),
    "dk_sample_depthwise_backward": (_int, [_vp] * 7 + [_gp, _int, _vp, _sz, _vp]),
    "dk_sample_depthwise_backward_one_pass": (_int, [_vp] * 7 + [_gp, _int, _vp, _sz, _vp]),
    "dk_deform_sample_depthwise_forward": (_int, [_vp] * 5 + [_gp, _int, _vp]),
    "dk_deform_sample_depthwise_backward_data_workspace_bytes": (_sz, [_gp, _int]),
    "dk_deform_sample_depthwise_backward_data": (_int, [_vp] * 5 + [_gp, _int, _vp, _sz, _vp]),
    "dk_deform_sample_depthwise_backward_filter_workspace_bytes": (_sz, [_gp, _int]),
    "dk_deform_sample_depthwise_backward_filter": (_int, [_vp] * 5 + [_gp, _int, _vp, _sz, _vp]),
    "dk_deform_sample_depthwise_backward_offset": (_int, [_vp] * 6 + [_gp, _int, _vp]),
    "dk_deform_sample_depthwise_backward_rotation": (_int, [_vp] * 6 + [_gp, _int, _vp]),
    "dk_deform_sample_depthwise_backward_workspace_bytes": (_sz, [_gp, _int]),
    "dk_deform_sample_depthwise_backward": (_int, [_vp] * 9 + [_gp, _int, _vp, _sz, _vp]),
    "dk_nd_linear_sample_forward": (_int, [_vp, _vp, _vp, _int, _int, _int, _ip, _int, _vp]),
    "dk_nd_linear_sample_backward_data": (_int, [_vp, _vp, _vp, _int, _int, _int, _ip, _int, _vp]),
    "dk_nd_linear_sample_backward_coord": (_int, [_vp, _vp, _vp, _vp, _int, _int, _int, _ip, _int, _vp]),
    "dk_nd_linear_sample_backward_coord_sum": (_int, [_vp, _vp, _vp, _vp, _int, _int, _int, _ip, _int, _vp]),
    "dk_plane_scale_forward": (_int, [_vp, _vp, _vp, ctypes.c_longlong, _int, _int, _vp]),
    "dk_plane_scale_backward": (_int, [_vp, _vp, _vp, _vp, _vp, ctypes.c_longlong, _int, _int, _vp]),
    "dk_global_dk_forward": (_int, [_vp] * 10 + [_int, _int, _int, _int, _ip, _int, _vp]),
    "dk_global_dk_backward_workspace_bytes": (ctypes.c_size_t, [_int, _int, _int]),
    "dk_global_dk_backward": (_int, [_vp] * 12 + [_int, _int, _int, _int, _ip, _int, _vp, ctypes.c_size_t, _vp]),
    "dk_offset_clip_forward": (_int, [_vp, _vp, _vp, _int, _int, _int] + [ctypes.c_double] * 4 + [_int, _vp]),
    "dk_offset_clip_backward": (_int, [_vp, _vp, _vp, _vp, _int, _int, _int] + [ctypes.c_double] * 4 + [_int, _vp]),
    "dk_output_size": (_int, [_gp, _ip, _ip]),
    "dk_status_string": (ctypes.c_char_p, [_int]),
    "dk_last_cuda_error": (_int, []),
    "dk_version": (ctypes.c_char_p, []),
    "dk_local_plan_query": (_int, [_gp, _int, _int, ctypes.POINTER(ctypes.c_longlong)]),
    "dk_ring_error_status": (_int, []),
}
for _name, (_res, _args) in _PROTOS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTS = tuple(_PROTOS)


UNSUPPORTED = 2  # DK_ERR_UNSUPPORTED


class DkError(RuntimeError):
    pass


def check(status, what):
    if status != 0:
        msg = lib.dk_status_string(status).decode()
        if status == 4:
            msg += " (cudaError %d)" % lib.dk_last_cuda_error()
        raise DkError("%s: %s" % (what, msg))


def dtype_code(t):
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError("deformable kernels support float16, float32 and float64 tensors, got %s" % t.dtype)


def geom(input_shape, kernel_size, stride, padding, dilation, scope, groups):
    n, c, h, w = input_shape
    return Geom(n, c, h, w, kernel_size[0], kernel_size[1], stride[0], stride[1], padding[0], padding[1],
                dilation[0], dilation[1], scope[0], scope[1], groups)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device):
    """cudaStream_t of torch's current stream on `device` (the raw-handle query is several times cheaper than
    building a Stream object, which matters for the small latency-bound calls)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(device.index if device.index is not None else torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class device_of:
    """Device guard that does nothing when the tensor already lives on the current device."""
    __slots__ = ("idx", "prev")

    def __init__(self, tensor):
        self.idx = tensor.device.index

    def __enter__(self):
        self.prev = torch.cuda.current_device()
        if self.idx is not None and self.idx != self.prev:
            torch.cuda.set_device(self.idx)
        else:
            self.prev = None

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def require_cuda(*tensors):
    """CPU tensors are refused the way the reference refuses them."""
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NotImplementedError("deformable kernels run on CUDA tensors only")


def same_dtype(first, *rest):
    for t in rest:
        if t is not None and t.dtype != first.dtype:
            raise TypeError("all tensors of one call must share a dtype (%s vs %s)" % (first.dtype, t.dtype))


def same_device(first, *rest):
    """The library launches on the first tensor's device with raw pointers: every tensor of a call must live there."""
    for t in rest:
        if t is not None and t.device != first.device:
            raise RuntimeError("all tensors of one call must be on the same device (%s vs %s)" % (first.device, t.device))


def workspace(nbytes, device):
    if nbytes == 0:
        return None
    return torch.empty(nbytes, dtype=torch.uint8, device=device)
