"""The entry point that allocates nothing: dk_sample_depthwise_backward_filter_noalloc.

It exists for callers that are not allowed to request device memory when they call the library
(a plugin inside a runtime that plans all memory up front, a fixed-memory control loop, a host
language whose FFI has no CUDA allocator) and therefore cannot provide the workspace that
dk_sample_depthwise_backward_filter needs; the partial sums go to an 8 MiB array built into the
library instead, and the call shrinks its block count where the usual partial sums would not fit.
The tests call it through the C ABI twice in a row (the array is shared and keeps the previous
call's contents) and check the results against the workspace-taking entry point and against the
CPU oracle.  Named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

from dk_cases import make_case, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_pair(C, case, dtype):
    x, r, dy = (case[k].to(dtype).to(DEV).contiguous() for k in ("input", "rotation", "grad_output"))
    a = case["args"]
    g = C.geom(x.shape, a["kernel_size"], a["stride"], a["padding"], a["dilation"], case["weight"].shape[2:],
               a["rotation_groups"])
    code = C.dtype_code(x)
    stream = C.stream_ptr(x.device)
    want = torch.empty_like(case["weight"], dtype=dtype, device=DEV)
    nbytes = C.lib.dk_sample_depthwise_backward_filter_workspace_bytes(g, code)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    C.check(C.lib.dk_sample_depthwise_backward_filter(C.ptr(dy), C.ptr(x), C.ptr(r), C.ptr(want), g, code, C.ptr(ws), nbytes,
                                                      stream), "reference entry point")
    got = torch.full_like(want, float("nan"))
    C.check(C.lib.dk_sample_depthwise_backward_filter_noalloc(C.ptr(dy), C.ptr(x), C.ptr(r), C.ptr(got), g, code, stream),
            "no-alloc entry point")
    torch.cuda.synchronize()
    return got, want


def _oracle_bank_gradient(case, dtype):
    """fp32 oracle on the tensors rounded to `dtype`, as the parity tests do for fp16."""
    from oracle import dk_oracle as O
    odt = torch.float32 if dtype == torch.float16 else torch.float64
    x, r, w, dy = (case[k].to(dtype).to(odt) for k in ("input", "rotation", "weight", "grad_output"))
    return O.sample_depthwise_backward(dy, x, r, w, **case["args"])[2]


def test_noalloc_bank_gradient_matches_workspace_entry_point_twice_in_a_row():
    from deformable_kernels import _cabi as C
    assert C.lib.dk_sample_depthwise_backward_filter_noalloc_max_bytes() == 8 << 20
    first = make_case(4, 96, 28, 28, rot_std=1.0, seed=41)               # fp16 tensor-core path
    second = make_case(3, 40, 17, 13, stride=2, rot_std=1.0, seed=42)    # different shape right after: stale partials must not leak
    for case, dtype, tol in ((first, torch.float16, 2e-3), (second, torch.float32, 1e-5), (first, torch.float16, 2e-3)):
        got, want = _run_pair(C, case, dtype)
        assert torch.isfinite(got).all()
        assert rel_err(got, want) < tol
        oracle = _oracle_bank_gradient(case, dtype)
        assert rel_err(got, oracle.to(dtype)) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-3), (torch.float32, 1e-5)])
def test_noalloc_covers_the_widest_sweep_layer_at_full_batch(dtype, tol):
    """C = 960 on 7 x 7 planes at batch 128: the usual partial sums of the general kernel (8.97 MB) exceed the
    8 MiB array, so the fp32 call runs with fewer pixel blocks; fp16 takes the tensor-core kernel, which needs less."""
    from deformable_kernels import _cabi as C
    case = make_case(128, 960, 7, 7, rot_std=1.0, seed=43)
    a = case["args"]
    g = C.geom(case["input"].shape, a["kernel_size"], a["stride"], a["padding"], a["dilation"], (4, 4), 1)
    used = C.lib.dk_sample_depthwise_backward_filter_noalloc_bytes(g, C.dtype_code(case["input"].to(dtype)))
    assert 0 < used <= (8 << 20)
    got, want = _run_pair(C, case, dtype)
    assert rel_err(got, want) < tol
    assert rel_err(got, _oracle_bank_gradient(case, dtype).to(dtype)) < tol


def test_noalloc_refuses_shapes_beyond_its_fixed_scratch():
    from deformable_kernels import _cabi as C
    # 200 x 200 bank cells for each of 64 channels: one block's partial sums (10 MB) cannot fit 8 MiB; refused
    # before anything is launched
    g = C.geom((64, 64, 600, 600), (3, 3), (1, 1), (1, 1), (1, 1), (200, 200), 1)
    assert C.lib.dk_sample_depthwise_backward_filter_noalloc_bytes(g, C.DK_F32) == 0
    one = ctypes.c_void_p(256)
    assert C.lib.dk_sample_depthwise_backward_filter_noalloc(one, one, one, one, g, C.DK_F32, ctypes.c_void_p(0)) == 3
