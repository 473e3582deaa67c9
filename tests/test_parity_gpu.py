"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle,
against the committed golden vectors (outputs of the reference's own CUDA kernels), and,
at full size, against the reference extension itself when its build travelled with the
repository (oracle/_ref/) plus size-independent properties.

Tolerances (max|a-b| / max|b| per tensor): 1e-5 for fp32, 2e-3 for fp16 (fp16 results are
compared with the fp32 oracle evaluated on the fp16-rounded inputs), 1e-11 for fp64.
"""
import glob
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import dk_cases
from dk_cases import make_case, make_nd_case, rel_err

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = {torch.float64: 1e-11, torch.float32: 1e-5, torch.float16: 2e-3}
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from deformable_kernels.ops.deform_kernel import functions
    return functions


@pytest.fixture(scope="module")
def oracle():
    from oracle import dk_oracle
    return dk_oracle


def _ref_modules():
    from oracle import build_ref
    try:
        return (build_ref.load_module("filter_sample_depthwise_cuda"), build_ref.load_module("nd_linear_sample_cuda"))
    except (FileNotFoundError, ImportError, OSError):
        return None


def snap(t, frac=0.25, seed=1):
    gen = torch.Generator().manual_seed(seed)
    pick = torch.rand(t.shape, generator=gen) < frac
    return torch.where(pick, torch.round(t * 2) / 2, t)


def mine_local(ops, case, dtype):
    x, r, w, dy = (case[k].to(dtype).to(DEV) for k in ("input", "rotation", "weight", "grad_output"))
    x.requires_grad_(True), r.requires_grad_(True), w.requires_grad_(True)
    y = ops.sample_depthwise(x, r, w, **case["args"])
    dx, dr, dw = torch.autograd.grad(y, [x, r, w], dy)
    return dict(output=y.detach(), grad_input=dx, grad_rotation=dr, grad_weight=dw)


def mine_deform(ops, case, dtype):
    x, o, r, w, dy = (case[k].to(dtype).to(DEV) for k in ("input", "offset", "rotation", "weight", "grad_output"))
    for t in (x, o, r, w):
        t.requires_grad_(True)
    y = ops.deform_sample_depthwise(x, o, r, w, **case["args"])
    dx, do, dr, dw = torch.autograd.grad(y, [x, o, r, w], dy)
    return dict(output=y.detach(), grad_input=dx, grad_offset=do, grad_rotation=dr, grad_weight=dw)


def mine_nd(ops, case, dtype):
    data, coord, dy = (case[k].to(dtype).to(DEV) for k in ("data", "coord", "grad_output"))
    data.requires_grad_(True), coord.requires_grad_(True)
    y = ops.nd_linear_sample(data, coord)
    dd, dc = torch.autograd.grad(y, [data, coord], dy)
    return dict(output=y.detach(), grad_data=dd, grad_coord=dc)


def oracle_inputs(case, dtype):
    """What the oracle computes on: fp64 copies for fp64/fp32 runs (the truth both are judged
    against), fp32 copies of the fp16-rounded inputs for fp16 runs."""
    odt = torch.float32 if dtype == torch.float16 else torch.float64
    return {k: (v.to(dtype).to(odt) if torch.is_tensor(v) else v) for k, v in case.items()}


def oracle_local(O, case, dtype):
    c = oracle_inputs(case, dtype)
    y = O.sample_depthwise_forward(c["input"], c["rotation"], c["weight"], **c["args"])
    dx, dr, dw = O.sample_depthwise_backward(c["grad_output"], c["input"], c["rotation"], c["weight"], **c["args"])
    return dict(output=y, grad_input=dx, grad_rotation=dr, grad_weight=dw)


def oracle_deform(O, case, dtype):
    c = oracle_inputs(case, dtype)
    y = O.deform_sample_depthwise_forward(c["input"], c["offset"], c["rotation"], c["weight"], **c["args"])
    dx, do, dr, dw = O.deform_sample_depthwise_backward(c["grad_output"], c["input"], c["offset"], c["rotation"],
                                                        c["weight"], **c["args"])
    return dict(output=y, grad_input=dx, grad_offset=do, grad_rotation=dr, grad_weight=dw)


def oracle_nd(O, case, dtype):
    c = oracle_inputs(case, dtype)
    y = O.nd_linear_sample_forward(c["data"], c["coord"])
    dd, dc = O.nd_linear_sample_backward(c["grad_output"], c["data"], c["coord"])
    return dict(output=y, grad_data=dd, grad_coord=dc)


def compare(got, want, dtype, what=""):
    for k, v in want.items():
        if dtype == torch.float16:
            v = v.to(torch.float16)
        err = rel_err(got[k], v)
        assert err < TOL[dtype], "%s %s: rel err %.3e (tol %.0e)" % (what, k, err, TOL[dtype])


SMALL = [
    dict(n=2, c=6, h=9, w=7, scope=(4, 4), k=3, stride=1, pad=1, dil=1, groups=1, rot_std=1.0),
    dict(n=2, c=6, h=9, w=8, scope=(4, 4), k=3, stride=2, pad=1, dil=1, groups=2, rot_std=1.0),
    dict(n=1, c=4, h=11, w=10, scope=(3, 5), k=3, stride=1, pad=2, dil=2, groups=4, rot_std=1.5),
    dict(n=2, c=4, h=8, w=8, scope=(2, 2), k=1, stride=1, pad=0, dil=1, groups=1, rot_std=0.7),
    dict(n=1, c=3, h=12, w=9, scope=(6, 4), k=5, stride=2, pad=2, dil=1, groups=3, rot_std=1.0),
    dict(n=1, c=2, h=10, w=10, scope=(4, 4), k=(3, 1), stride=(1, 2), pad=(1, 0), dil=1, groups=1, rot_std=1.0),
    dict(n=3, c=40, h=17, w=13, scope=(4, 4), k=3, stride=1, pad=1, dil=1, groups=1, rot_std=1.0),   # > one channel chunk
    dict(n=2, c=70, h=7, w=7, scope=(4, 4), k=3, stride=2, pad=1, dil=1, groups=1, rot_std=2.5),     # many invalid samples
    dict(n=1, c=33, h=6, w=5, scope=(4, 4), k=3, stride=1, pad=1, dil=1, groups=33, rot_std=1.0),    # one group per channel
]


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.float16])
@pytest.mark.parametrize("cfg", SMALL)
def test_local_dk_matches_oracle(ops, oracle, cfg, dtype):
    case = make_case(seed=31, **cfg)
    case["rotation"] = snap(case["rotation"])
    compare(mine_local(ops, case, dtype), oracle_local(oracle, case, dtype), dtype, "local")


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.float16])
@pytest.mark.parametrize("cfg", SMALL)
def test_deform_dk_matches_oracle(ops, oracle, cfg, dtype):
    case = make_case(seed=32, off_std=2.0, **cfg)
    case["rotation"] = snap(case["rotation"])
    case["offset"] = snap(case["offset"], seed=2)
    compare(mine_deform(ops, case, dtype), oracle_deform(oracle, case, dtype), dtype, "deform")


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(2, 2), (4, 4), (3, 5), (5,), (2, 3, 4), (2, 2, 2, 3)])
def test_nd_linear_matches_oracle(ops, oracle, shape, dtype):
    case = make_nd_case(70, shape, 50, seed=33)
    compare(mine_nd(ops, case, dtype), oracle_nd(oracle, case, dtype), dtype, "nd")


FAST = [   # shapes inside the fp16 tensor-core fast path (3x3, pad 1, dil 1, one group, C % 16 == 0, <= 16 cells)
    dict(n=2, c=16, h=12, w=20, scope=(4, 4), k=3, stride=1, pad=1, rot_std=1.0),      # partial 8-pixel blocks
    dict(n=3, c=32, h=7, w=7, scope=(4, 4), k=3, stride=1, pad=1, rot_std=1.0),        # odd width: scalar loader
    dict(n=2, c=48, h=14, w=14, scope=(4, 4), k=3, stride=2, pad=1, rot_std=1.0),      # odd output width
    dict(n=1, c=144, h=28, w=28, scope=(4, 4), k=3, stride=1, pad=1, rot_std=1.5),     # two channel groups, 16-byte loader
    dict(n=2, c=16, h=56, w=56, scope=(4, 4), k=3, stride=2, pad=1, rot_std=1.0),
    dict(n=1, c=32, h=9, w=16, scope=(2, 2), k=3, stride=1, pad=1, rot_std=0.6),       # 4 cells, zero-padded to 16
    dict(n=1, c=16, h=10, w=12, scope=(3, 5), k=3, stride=1, pad=1, rot_std=1.2),      # 15 cells, non-square scope
    dict(n=2, c=16, h=5, w=6, scope=(4, 4), k=3, stride=2, pad=1, rot_std=3.0),        # most samples outside the bank
    dict(n=1, c=16, h=1, w=1, scope=(4, 4), k=3, stride=1, pad=1, rot_std=1.0),        # a single pixel
    dict(n=3, c=32, h=2, w=9, scope=(1, 1), k=3, stride=2, pad=1, rot_std=0.8),        # one bank cell, 1 x 5 output
    dict(n=2, c=16, h=1, w=17, scope=(2, 8), k=3, stride=1, pad=1, rot_std=1.5),       # 16 cells in a flat scope, one row
    dict(n=1, c=16, h=33, w=2, scope=(4, 4), k=3, stride=2, pad=1, rot_std=1.0),       # one output column
]


@pytest.mark.parametrize("cfg", FAST)
def test_local_dk_fp16_fast_path_matches_oracle(ops, oracle, cfg):
    case = make_case(seed=36, **cfg)
    case["rotation"] = snap(case["rotation"])
    compare(mine_local(ops, case, torch.float16), oracle_local(oracle, case, torch.float16), torch.float16, "fast")


@pytest.mark.parametrize("cfg", FAST)
def test_deform_dk_fp16_fast_shapes_match_oracle(ops, oracle, cfg):
    case = make_case(seed=38, off_std=2.0, **cfg)
    case["rotation"] = snap(case["rotation"])
    case["offset"] = snap(case["offset"], seed=3)
    compare(mine_deform(ops, case, torch.float16), oracle_deform(oracle, case, torch.float16), torch.float16, "deform-fast")


# DK + DCN shapes with enough (sample, 16-channel group) pairs for the whole-sample grad-input kernel
DCN_BATCHED = [
    dict(n=6, c=256, h=14, w=14, scope=(4, 4), k=3, stride=1, pad=1, rot_std=0.7),
    dict(n=12, c=128, h=9, w=7, scope=(4, 4), k=3, stride=1, pad=1, rot_std=0.7),      # odd sizes: scalar loads and stores
    dict(n=8, c=192, h=20, w=16, scope=(4, 4), k=3, stride=2, pad=1, rot_std=1.0),
    dict(n=24, c=64, h=12, w=12, scope=(3, 5), k=3, stride=1, pad=1, rot_std=1.0),     # 15 cells
]


@pytest.mark.parametrize("cfg", DCN_BATCHED)
def test_deform_dk_fp16_batched_shapes_match_oracle(ops, oracle, cfg):
    case = make_case(seed=39, off_std=2.0, **cfg)
    case["rotation"] = snap(case["rotation"])
    case["offset"] = snap(case["offset"], seed=3)
    compare(mine_deform(ops, case, torch.float16), oracle_deform(oracle, case, torch.float16), torch.float16, "deform-batched")


@pytest.mark.parametrize("cfg", [DCN_BATCHED[0], DCN_BATCHED[2], FAST[3]])
def test_deform_dk_without_kernel_offsets_matches_zero_offsets(ops, oracle, cfg):
    """rotation=None (what DeformKernelConv2d and DeformConv2d pass) against the oracle with a tensor of zeros: fp16
    takes the path that builds the pixel-independent kernel once, fp32 falls back to zeros inside the binding."""
    case = make_case(seed=42, off_std=2.0, **cfg)
    case["rotation"] = torch.zeros_like(case["rotation"])
    for dtype in (torch.float16, torch.float32):
        x, o, w, dy = (case[k].to(dtype).to(DEV) for k in ("input", "offset", "weight", "grad_output"))
        for t in (x, o, w):
            t.requires_grad_(True)
        y = ops.deform_sample_depthwise(x, o, None, w, **case["args"])
        dx, do, dw = torch.autograd.grad(y, [x, o, w], dy)
        want = oracle_deform(oracle, case, dtype)
        got = dict(output=y.detach(), grad_input=dx, grad_offset=do, grad_weight=dw)
        want.pop("grad_rotation")
        compare(got, want, dtype, "deform-no-rotation")


def _random_fast_shapes(count, seed):
    """Seeded random geometries inside the fp16 tensor-core fast path (3x3, pad 1, C % 16 == 0, <= 16 cells)."""
    import random
    rng = random.Random(seed)
    out = []
    for _ in range(count):
        scope = rng.choice([(4, 4), (4, 4), (3, 3), (2, 2), (3, 5), (4, 2), (1, 4)])
        out.append(dict(n=rng.randint(1, 5), c=rng.choice([16, 32, 48, 64, 80, 96, 144]), h=rng.randint(3, 36),
                        w=rng.randint(3, 36), scope=scope, k=3, stride=rng.choice([1, 1, 2]), pad=1,
                        rot_std=rng.choice([0.5, 1.0, 2.5])))
    return out


@pytest.mark.parametrize("cfg", _random_fast_shapes(16, 101))
def test_local_dk_fp16_random_shapes_match_oracle(ops, oracle, cfg):
    case = make_case(seed=43, **cfg)
    case["rotation"] = snap(case["rotation"])
    compare(mine_local(ops, case, torch.float16), oracle_local(oracle, case, torch.float16), torch.float16, "random-local")


@pytest.mark.parametrize("cfg", _random_fast_shapes(12, 202))
def test_deform_dk_fp16_random_shapes_match_oracle(ops, oracle, cfg):
    cfg = dict(cfg, n=cfg["n"] * 6)   # enough (sample, channel group) pairs for the whole-sample grad-input kernel on most
    case = make_case(seed=44, off_std=2.0, **cfg)
    case["rotation"] = snap(case["rotation"])
    case["offset"] = snap(case["offset"], seed=5)
    compare(mine_deform(ops, case, torch.float16), oracle_deform(oracle, case, torch.float16), torch.float16, "random-deform")


@pytest.mark.parametrize("n,c,hw,stride,with_rot", [(3, 64, 28, 1, True), (2, 32, 56, 1, True), (4, 48, 14, 2, True),
                                                     (40, 64, 28, 1, False), (150, 32, 14, 1, True)])   # without kernel-space offsets the C ABI wants a batch the
                                                     # whole-sample grad-input kernel takes
def test_deform_bank_gradient_rides_along_with_the_offset_gradients(oracle, n, c, hw, stride, with_rot):
    """fp16 DK + DCN, fused backward through the C ABI: when both offset gradients (or, without kernel-space offsets, the
    image-space one) are wanted together with the bank gradient, the bank gradient comes out of the same pass.  It must
    agree with the stand-alone bank-gradient entry point and with the oracle, twice in a row (partial sums do not leak)."""
    from deformable_kernels import _cabi as C
    case = make_case(n, c, hw, hw, stride=stride, rot_std=0.8, off_std=1.5, seed=700 + c + hw)
    x, o, r, w, dy = (case[k].half().to(DEV) for k in ("input", "offset", "rotation", "weight", "grad_output"))
    if not with_rot:
        case["rotation"] = torch.zeros_like(case["rotation"])
        r = torch.zeros_like(r)
    g = C.geom(x.shape, (3, 3), (stride, stride), (1, 1), (1, 1), (4, 4), 1)
    nb = C.lib.dk_deform_sample_depthwise_backward_workspace_bytes(g, C.DK_F16)
    ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=DEV)
    gx, go, gr, gw = torch.empty_like(x), torch.empty_like(o), torch.empty_like(r), torch.full_like(w, float("nan"))
    for _ in range(2):
        C.check(C.lib.dk_deform_sample_depthwise_backward(
            C.ptr(dy), C.ptr(x), C.ptr(o), C.ptr(r) if with_rot else None, C.ptr(w), C.ptr(gx), C.ptr(go),
            C.ptr(gr) if with_rot else None, C.ptr(gw), g, C.DK_F16, C.ptr(ws), nb, C.stream_ptr(x.device)), "fused backward")
    gw2 = torch.empty_like(w)
    nbf = C.lib.dk_deform_sample_depthwise_backward_filter_workspace_bytes(g, C.DK_F16)
    wsf = torch.empty(max(nbf, 1), dtype=torch.uint8, device=DEV)
    C.check(C.lib.dk_deform_sample_depthwise_backward_filter(C.ptr(dy), C.ptr(x), C.ptr(o), C.ptr(r), C.ptr(gw2), g, C.DK_F16,
                                                             C.ptr(wsf), nbf, C.stream_ptr(x.device)), "bank gradient")
    torch.cuda.synchronize()
    assert rel_err(gw, gw2) < 2e-3
    want = oracle_deform(oracle, case, torch.float16)
    got = dict(grad_input=gx, grad_offset=go, grad_weight=gw)
    if with_rot:
        got["grad_rotation"] = gr
    compare(got, {k: want[k] for k in got}, torch.float16, "fused DK+DCN backward")


def test_deform_grad_input_fixed_point_accumulation(ops, oracle):
    """The fp16 grad-input kernel sums in fixed point.  Bit-reproducible; an outlier in dy coarsens only its own
    (sample, channel) plane and the result still holds the tolerance on every plane taken by itself; offsets that
    send every sample of an image to one pixel (the worst case for the accumulator's headroom) do not overflow."""
    cfg = dict(n=6, c=256, h=14, w=14, scope=(4, 4), k=3, stride=1, pad=1, rot_std=0.7)
    case = make_case(seed=40, off_std=2.0, **cfg)
    case["grad_output"][1, 5, 3, 4] *= 1024.0
    case["grad_output"][4, 200, 9, 9] *= -300.0
    # sample 2: every tap of every pixel lands next to input pixel (6, 7)
    ho = wo = 14
    oh = torch.arange(ho).view(ho, 1).expand(ho, wo).float()
    ow = torch.arange(wo).view(1, wo).expand(ho, wo).float()
    for t in range(9):
        case["offset"][2, 2 * t] = 6.3 - (oh - 1 + t // 3)
        case["offset"][2, 2 * t + 1] = 7.6 - (ow - 1 + t % 3)
    got = mine_deform(ops, case, torch.float16)
    again = mine_deform(ops, case, torch.float16)
    assert torch.equal(got["grad_input"], again["grad_input"])
    want = oracle_deform(oracle, case, torch.float16)
    compare(got, want, torch.float16, "deform-fixed-point")
    g, w = got["grad_input"].float().cpu(), want["grad_input"].to(torch.float16).float()
    err = (g - w).abs()
    plane_max = w.abs().amax(dim=(2, 3), keepdim=True).clamp_min(1e-6)
    keep = [0, 1, 3, 4, 5]
    worst = float((err / plane_max)[keep].max())
    assert worst < TOL[torch.float16], "per-plane rel err %.3e" % worst
    # sample 2: 1764 terms per pixel, sums that cancel to almost nothing on some channels; judged against the sample
    worst2 = float(err[2].max() / w[2].abs().max())
    assert worst2 < TOL[torch.float16], "concentrated sample rel err %.3e" % worst2

@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
def test_plane_scale_is_the_per_sample_grouped_1x1_conv(ops, dtype):
    gen = torch.Generator().manual_seed(37)
    x = torch.randn(5, 12, 7, 9, generator=gen).to(dtype).to(DEV).requires_grad_(True)
    k = torch.randn(5, 12, generator=gen).to(dtype).to(DEV).requires_grad_(True)
    dy = torch.randn(5, 12, 7, 9, generator=gen).to(dtype).to(DEV)
    y = ops.plane_scale(x, k)
    gx, gk = torch.autograd.grad(y, [x, k], dy)
    xr, kr = x.detach().double().requires_grad_(True), k.detach().double().requires_grad_(True)
    ref = F.conv2d(xr.view(1, 60, 7, 9), kr.view(60, 1, 1, 1), groups=60).view(5, 12, 7, 9)   # reference formulation
    rx, rk = torch.autograd.grad(ref, [xr, kr], dy.double())
    tol = TOL[dtype]
    assert rel_err(y, ref.to(dtype)) < tol and rel_err(gx, rx.to(dtype)) < tol and rel_err(gk, rk.to(dtype)) < tol


def test_empty_and_degenerate_inputs(ops):
    from deformable_kernels._cabi import DkError
    x = torch.randn(1, 4, 2, 2, device=DEV)
    w = torch.randn(4, 1, 4, 4, device=DEV)
    with pytest.raises(ValueError):      # convolution input is too small
        ops.sample_depthwise(x, torch.zeros(1, 18, 1, 1, device=DEV), w, (5, 5), (1, 1), (0, 0), (1, 1), 1)
    with pytest.raises(ValueError):      # offsets of the wrong shape
        ops.sample_depthwise(x, torch.zeros(1, 18, 3, 3, device=DEV), w)
    with pytest.raises(TypeError):       # mixed dtypes at the Function level
        from deformable_kernels.ops.deform_kernel.functions.filter_sample_depthwise import SampleDepthwiseFunction
        SampleDepthwiseFunction.apply(x, torch.zeros(1, 18, 2, 2, device=DEV).half(), w)
    assert issubclass(DkError, RuntimeError)
    # all samples outside the bank -> exact zeros in value and every gradient
    r = torch.full((1, 18, 2, 2), 50.0, device=DEV)
    x.requires_grad_(True), r.requires_grad_(True), w.requires_grad_(True)
    y = ops.sample_depthwise(x, r, w)
    assert torch.count_nonzero(y) == 0
    gx, gr, gw = torch.autograd.grad(y, [x, r, w], torch.ones_like(y))
    assert torch.count_nonzero(gx) == 0 and torch.count_nonzero(gr) == 0 and torch.count_nonzero(gw) == 0
    # NaN offsets sample nothing (comparisons are false in the reference too)
    r2 = torch.full((1, 18, 2, 2), float("nan"), device=DEV)
    assert torch.count_nonzero(ops.sample_depthwise(x.detach(), r2, w.detach())) == 0


@pytest.mark.parametrize("c,hw,stride", [(32, 56, 1), (32, 56, 2), (96, 14, 1), (192, 14, 2), (32, 28, 1), (16, 7, 1)])
@pytest.mark.parametrize("fill", [50.0, float("nan")])
def test_fp16_fast_paths_with_offsets_that_sample_nothing(ops, c, hw, stride, fill):
    """Every kernel-space offset far outside the bank, or NaN (comparisons are false in the reference too): the tensor-core
    paths (row-ring kernels, the one-pass band kernel, the separate band kernels) return exact zeros in the value and in
    every gradient, never NaN."""
    gen = torch.Generator().manual_seed(13)
    x = torch.randn(3, c, hw, hw, generator=gen).half().to(DEV).requires_grad_(True)
    w = (torch.randn(c, 1, 4, 4, generator=gen) * 0.3).half().to(DEV).requires_grad_(True)
    ho = (hw - 1) // stride + 1
    r = torch.full((3, 18, ho, ho), fill, device=DEV, dtype=torch.float16).requires_grad_(True)
    y = ops.sample_depthwise(x, r, w, (3, 3), (stride, stride), (1, 1), (1, 1), 1)
    assert torch.count_nonzero(y) == 0
    gx, gr, gw = torch.autograd.grad(y, [x, r, w], torch.randn(y.shape, generator=gen).half().to(DEV))
    for t in (gx, gr, gw):
        assert torch.isfinite(t).all() and torch.count_nonzero(t) == 0


def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "*.npz")))


@pytest.mark.parametrize("path", _golden_files() or [None])
def test_kernels_match_reference_cuda_golden(ops, path):
    if path is None:
        pytest.skip("no golden vectors committed yet")
    z = np.load(path)
    kind = str(z["kind"])
    t = {k: torch.from_numpy(z[k]) for k in z.files if k not in ("kind", "args")}
    dtype = t["grad_output"].dtype
    tol = 1e-11 if dtype == torch.float64 else 2e-5
    if kind == "nd":
        got = mine_nd(ops, t, dtype)
    else:
        a = [int(v) for v in z["args"]]
        t["args"] = dict(kernel_size=(a[0], a[1]), stride=(a[2], a[3]), padding=(a[4], a[5]), dilation=(a[6], a[7]),
                         rotation_groups=a[8])
        got = mine_local(ops, t, dtype) if kind == "local" else mine_deform(ops, t, dtype)
    for k, v in got.items():
        err = rel_err(v, t["ref_" + k])
        assert err < tol, "%s %s: %.3e" % (os.path.basename(path), k, err)


def test_reference_named_entry_points_agree_with_fused_calls(ops):
    """The nine + three functions named like the reference's pybind11 functions, called the
    way the reference's own autograd code calls them, give the fused path's results."""
    from deformable_kernels.ops.deform_kernel import filter_sample_depthwise_cuda as fs
    from deformable_kernels.ops.deform_kernel import nd_linear_sample_cuda as nd
    case = make_case(2, 40, 12, 11, stride=2, groups=2, rot_std=1.0, off_std=2.0, seed=34)
    for dtype in (torch.float32, torch.float16):
        fused = mine_deform(ops, case, dtype)
        x, o, r, w, dy = (case[k].to(dtype).to(DEV) for k in ("input", "offset", "rotation", "weight", "grad_output"))
        tail = (3, 3, 2, 2, 1, 1, 1, 1, 4, 4, 2)
        y = torch.empty_like(dy)
        fs.deformable_sample_depthwise_forward_cuda(x, o, r, w, y, *tail)
        dx, do, dr, dw = torch.zeros_like(x), torch.zeros_like(o), torch.zeros_like(r), torch.zeros_like(w)
        fs.deformable_sample_depthwise_backward_data_cuda(dy, x, o, r, w, dx, *tail)
        fs.deformable_sample_depthwise_backward_offset_cuda(dy, x, o, r, w, do, *tail)
        fs.deformable_sample_depthwise_backward_rotation_cuda(dy, x, o, r, w, dr, *tail)
        fs.deformable_sample_depthwise_backward_filter_cuda(dy, x, o, r, w, dw, *tail)
        for a, b in ((y, "output"), (dx, "grad_input"), (do, "grad_offset"), (dr, "grad_rotation"), (dw, "grad_weight")):
            assert rel_err(a, fused[b]) < (1e-6 if dtype == torch.float32 else 1e-3), b
        fusedl = mine_local(ops, case, dtype)
        y = torch.empty_like(dy)
        fs.sample_depthwise_forward_cuda(x, r, w, y, *tail)
        dx, dr, dw = torch.zeros_like(x), torch.zeros_like(r), torch.zeros_like(w)
        fs.sample_depthwise_backward_data_cuda(dy, x, r, w, dx, *tail)
        fs.sample_depthwise_backward_rotation_cuda(dy, x, r, w, dr, *tail)
        fs.sample_depthwise_backward_filter_cuda(dy, x, r, w, dw, *tail)
        for a, b in ((y, "output"), (dx, "grad_input"), (dr, "grad_rotation"), (dw, "grad_weight")):
            assert rel_err(a, fusedl[b]) < (1e-6 if dtype == torch.float32 else 1e-3), b
    ndc = make_nd_case(20, (4, 4), 30, seed=35)
    fused = mine_nd(ops, ndc, torch.float32)
    data, coord, dy = (ndc[k].to(DEV) for k in ("data", "coord", "grad_output"))
    shape = torch.tensor(data.shape[1:], dtype=data.dtype, device=DEV)
    y = data.new_empty(30, 20)
    nd.nd_linear_sample_forward_cuda(data, shape, coord, y)
    dd = data.new_empty(*data.size())
    nd.nd_linear_sample_backward_data_cuda(dy, data, shape, coord, dd)
    dcc = coord.new_empty(30, 2, 20)
    nd.nd_linear_sample_backward_coord_cuda(dy, data, shape, coord, dcc)
    assert rel_err(y, fused["output"]) < 1e-6
    assert rel_err(dd, fused["grad_data"]) < 1e-6
    assert rel_err(dcc.sum(2), fused["grad_coord"]) < 1e-5


# ------------------------------------------------------------------ BASELINE configs

def test_cfg1_full_size_matches_oracle(ops, oracle):
    case = dk_cases.cfg1()
    for dtype in (torch.float32, torch.float64):
        compare(mine_local(ops, case, dtype), oracle_local(oracle, case, dtype), dtype, "cfg1")


def test_cfg2_full_size_matches_oracle_and_module_runs(ops, oracle):
    case = dk_cases.cfg2()
    compare(mine_nd(ops, case, torch.float32), oracle_nd(oracle, case, torch.float32), torch.float32, "cfg2")
    from deformable_kernels.modules import GlobalDeformKernel2d
    torch.manual_seed(0)
    m = GlobalDeformKernel2d((2, 2), 256, 256, kernel_size=1, groups=256).to(DEV)
    with torch.no_grad():
        m.weight.copy_(case["weight"].to(DEV))
        m.fc.weight.normal_(0, 0.05)
    x = case["input"].to(DEV).requires_grad_(True)
    y = m(x)
    y.sum().backward()
    # per-sample 1x1 depthwise kernel: y = x * k[n, c]
    with torch.no_grad():
        avg = x.view(32, 256, -1).mean(2)
        coord = torch.clamp(m.fc(avg) + 0.5, 0, 1).cpu()
        k = oracle.nd_linear_sample_forward(case["data"], coord).to(DEV)
    assert rel_err(y, x.detach() * k.view(32, 256, 1, 1)) < 1e-5
    assert m.weight.grad is not None and m.fc.weight.grad is not None and x.grad is not None


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape,c,n,hw,fc_std", [((2, 2), 256, 32, 14, 0.05), ((3, 3), 40, 5, 9, 0.6), ((2, 3, 2), 24, 7, 6, 0.4)])
def test_fused_global_dk_matches_its_composition(dtype, shape, c, n, hw, fc_std):
    """GlobalDeformKernel2d (1x1 depthwise) through the two fused calls against the same module evaluated as the
    reference composes it (pool, nn.Linear, clamp, nd_linear_sample, per-plane scale), values and all four gradients.
    fc_std is large enough in two of the cases for part of the coordinates to sit on the clamp."""
    from deformable_kernels.modules import GlobalDeformKernel2d
    torch.manual_seed(5)
    m = GlobalDeformKernel2d(shape, c, c, kernel_size=1, groups=c).to(DEV)
    with torch.no_grad():
        m.fc.weight.normal_(0, fc_std)
        m.fc.bias.normal_(0, 0.2)
    x = torch.randn(n, c, hw, hw, device=DEV).to(dtype)
    dy = torch.randn(n, c, hw, hw, device=DEV).to(dtype)
    params = [m.weight, m.fc.weight, m.fc.bias]

    def run(fused):
        xi = x.clone().requires_grad_(True)
        if not fused:
            m._fused_head_ok = lambda _x: False
        try:
            y = m(xi)
        finally:
            if not fused:
                del m._fused_head_ok
        return [y.detach()] + list(torch.autograd.grad(y, [xi] + params, dy))

    assert m._fused_head_ok(x)
    got, want = run(True), run(False)
    tol = 2e-5 if dtype == torch.float32 else 4e-3   # fp16: the composition rounds the scale to fp16 before use
    for name, a, b in zip(("y", "dx", "dbank", "dfc_weight", "dfc_bias"), got, want):
        assert rel_err(a, b) < tol, "%s: %.3e" % (name, rel_err(a, b))


def test_operators_capture_into_cuda_graphs():
    """The operators enqueue on the current stream, never synchronise and take their scratch from the caller, so their
    forward and backward capture into CUDA graphs (torch.cuda.make_graphed_callables) and replay to the same result."""
    import warnings
    from deformable_kernels.modules import GlobalDeformKernel2d
    from deformable_kernels.ops.deform_kernel.modules import DeformableSampleDepthwise, SampleDepthwise
    gen = torch.Generator(device=DEV).manual_seed(6)

    def rnd(*shape, std=1.0, dtype=torch.float32):
        return (torch.randn(*shape, device=DEV, generator=gen) * std).to(dtype).requires_grad_(True)

    cases = [
        (SampleDepthwise((4, 4), 32, 32, 3, 1, 1, groups=32).to(DEV), [rnd(2, 32, 20, 20), rnd(2, 18, 20, 20, std=0.7)]),
        (SampleDepthwise((4, 4), 64, 64, 3, 1, 1, groups=64).to(DEV).half(),
         [rnd(4, 64, 28, 28, dtype=torch.float16), rnd(4, 18, 28, 28, std=0.7, dtype=torch.float16)]),
        (DeformableSampleDepthwise((4, 4), 64, 64, 3, 1, 1, groups=64).to(DEV).half(),
         [rnd(24, 64, 14, 14, dtype=torch.float16), rnd(24, 18, 14, 14, std=2.0, dtype=torch.float16),
          rnd(24, 18, 14, 14, std=0.7, dtype=torch.float16)]),
        (GlobalDeformKernel2d((2, 2), 64, 64, kernel_size=1, groups=64).to(DEV), [rnd(4, 64, 14, 14)]),
    ]
    for layer, ins in cases:
        with torch.no_grad():
            for p in layer.parameters():
                if p.abs().max() == 0:
                    p.normal_(0, 0.1)
        params = list(layer.parameters())
        # graph first: an eager backward on the default stream beforehand would tie the parameters' gradient
        # accumulation to that stream, which PyTorch then cannot capture
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            graphed = torch.cuda.make_graphed_callables(layer, tuple(t.detach().clone().requires_grad_(True) for t in ins))
            dy = None
            for _ in range(2):
                yg = graphed(*ins)
                dy = torch.randn_like(yg) if dy is None else dy
                got = [yg.detach().clone()] + [g.clone() for g in torch.autograd.grad(yg, ins + params, dy)]
            y = layer(*ins)
            want = [y.detach()] + list(torch.autograd.grad(y, ins + params, dy))
        for a_, b_ in zip(got, want):
            assert rel_err(a_, b_) < (1e-5 if a_.dtype == torch.float32 else 1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
def test_clip_offsets_matches_the_elementwise_composition(ops, dtype):
    """(clamp(r * d + b, lo, hi) - b) / d * post in one pass, against the five PyTorch passes of
    LocalDeformKernel2d._clip_rotation, and the plain clamp * dilation of DeformKernelConv2d."""
    gen = torch.Generator().manual_seed(41)
    r = (torch.randn(3, 18, 9, 11, generator=gen) * 2).to(dtype).to(DEV)
    dy = torch.randn(3, 18, 9, 11, generator=gen).to(dtype).to(DEV)
    bias = (torch.rand(18, generator=gen) * 3).to(DEV)
    for b, lo, hi, d, post in ((bias, 0.0, 3.0, 1.0, 1.0), (bias, 0.0, 3.0, 2.0, 2.0), (None, -1.5, 0.75, 1.0, 3.0)):
        a = r.clone().requires_grad_(True)
        y = ops.clip_offsets(a, b, lo, hi, d, post)
        ga, = torch.autograd.grad(y, a, dy)
        # fp16: the composition evaluated in fp32 on the fp16 inputs (in fp16 it rounds r * d + b before clamping
        # and so decides a few boundary elements differently)
        wide = torch.float32 if dtype == torch.float16 else dtype
        c = r.to(wide).requires_grad_(True)
        bb = 0 if b is None else b.to(wide)[None, :, None, None]
        want = ((c * d + bb).clamp(lo, hi) - bb) / d * post
        gc, = torch.autograd.grad(want, c, dy.to(wide))
        want, gc = want.to(dtype), gc.to(dtype)
        tol = {torch.float64: 1e-12, torch.float32: 1e-6, torch.float16: 2e-3}[dtype]
        assert rel_err(y, want) < tol and rel_err(ga, gc) < tol


def test_layers_with_offset_clipping_match_the_composition():
    from deformable_kernels.modules import DeformKernel2d, DeformKernelConv2d
    torch.manual_seed(7)
    x = torch.randn(2, 16, 12, 12, device=DEV)
    for clip in ('scope', (-0.4, 0.6)):
        m = DeformKernel2d((4, 4), 16, 16, 3, 1, 1, groups=16, rotation_clip=clip).to(DEV)
        with torch.no_grad():
            m.rotation_conv.weight.normal_(0, 0.3)
        got = m(x)
        m._fused_clip = lambda rot: None
        want = m(x)
        assert rel_err(got, want) < 1e-5
    m = DeformKernelConv2d((4, 4), 16, 16, 3, 1, 1, groups=16, offset_clip=dict(min=-1.0, max=1.5)).to(DEV)
    with torch.no_grad():
        m.offset_conv.weight.normal_(0, 0.5)
    got = m(x)
    want = m.inner_conv(x, m.offset_conv(x).clamp(min=-1.0, max=1.5), None)
    assert rel_err(got, want) < 1e-5


@pytest.mark.parametrize("c,hw,stride,n", [(96, 112, 1, 2), (144, 56, 2, 3), (960, 7, 1, 8), (384, 14, 2, 4)])
def test_cfg3_reduced_batch_fp16_matches_oracle(ops, oracle, c, hw, stride, n):
    case = dk_cases.cfg3(c, hw, stride, n=n)
    compare(mine_local(ops, case, torch.float16), oracle_local(oracle, case, torch.float16), torch.float16, "cfg3")


def test_cfg4_reduced_fp16_matches_oracle(ops, oracle):
    case = dk_cases.cfg4(n=2, c=64, hw=56)
    compare(mine_deform(ops, case, torch.float16), oracle_deform(oracle, case, torch.float16), torch.float16, "cfg4")


def _ref_local(fs, case, dtype):
    x, r, w, dy = (case[k].to(dtype).to(DEV) for k in ("input", "rotation", "weight", "grad_output"))
    a = case["args"]
    tail = (*a["kernel_size"], *a["stride"], *a["padding"], *a["dilation"], w.size(2), w.size(3), a["rotation_groups"])
    y = torch.empty_like(dy)
    fs.sample_depthwise_forward_cuda(x, r, w, y, *tail)
    dx, dr, dw = torch.zeros_like(x), torch.zeros_like(r), torch.zeros_like(w)
    fs.sample_depthwise_backward_data_cuda(dy, x, r, w, dx, *tail)
    fs.sample_depthwise_backward_rotation_cuda(dy, x, r, w, dr, *tail)
    fs.sample_depthwise_backward_filter_cuda(dy, x, r, w, dw, *tail)
    torch.cuda.synchronize()
    return dict(output=y, grad_input=dx, grad_rotation=dr, grad_weight=dw)


def _ref_deform(fs, case, dtype):
    x, o, r, w, dy = (case[k].to(dtype).to(DEV) for k in ("input", "offset", "rotation", "weight", "grad_output"))
    a = case["args"]
    tail = (*a["kernel_size"], *a["stride"], *a["padding"], *a["dilation"], w.size(2), w.size(3), a["rotation_groups"])
    y = torch.empty_like(dy)
    fs.deformable_sample_depthwise_forward_cuda(x, o, r, w, y, *tail)
    dx, do, dr, dw = torch.zeros_like(x), torch.zeros_like(o), torch.zeros_like(r), torch.zeros_like(w)
    fs.deformable_sample_depthwise_backward_data_cuda(dy, x, o, r, w, dx, *tail)
    fs.deformable_sample_depthwise_backward_offset_cuda(dy, x, o, r, w, do, *tail)
    fs.deformable_sample_depthwise_backward_rotation_cuda(dy, x, o, r, w, dr, *tail)
    fs.deformable_sample_depthwise_backward_filter_cuda(dy, x, o, r, w, dw, *tail)
    torch.cuda.synchronize()
    return dict(output=y, grad_input=dx, grad_offset=do, grad_rotation=dr, grad_weight=dw)


def _half_inputs_as_float(case):
    return {k: (v.half().float() if torch.is_tensor(v) else v) for k, v in case.items()}


@pytest.mark.parametrize("c,hw,stride", [(c, hw, s) for (c, hw) in dk_cases.CFG3_LAYERS for s in (1, 2)])
def test_cfg3_full_size_fp16_against_live_reference(ops, c, hw, stride):
    """Full batch (128).  The reference runs in fp32 on the fp16-rounded inputs, which is what
    it does under Apex (functions/filter_sample_depthwise.py:209-211)."""
    mods = _ref_modules()
    if mods is None:
        pytest.skip("reference build (oracle/_ref) not present")
    case = dk_cases.cfg3(c, hw, stride, n=128)
    got = mine_local(ops, case, torch.float16)
    want = _ref_local(mods[0], _half_inputs_as_float(case), torch.float32)
    compare(got, want, torch.float16, "cfg3-full")


@pytest.mark.parametrize("c,hw,stride,n", [(96, 112, 1, 3), (48, 112, 2, 5), (144, 56, 1, 4), (32, 56, 2, 7)])
def test_one_pass_backward_matches_oracle(oracle, c, hw, stride, n):
    """dk_sample_depthwise_backward_one_pass (all three gradients from one stream of rows) through the C ABI; batch sizes
    that make the blocks' row ranges start and end inside samples."""
    from deformable_kernels import _cabi as C
    case = make_case(n, c, hw, hw, stride=stride, rot_std=1.0, seed=90 + n)
    x, r, w, dy = (case[k].half().to(DEV) for k in ("input", "rotation", "weight", "grad_output"))
    g = C.geom(x.shape, (3, 3), (stride, stride), (1, 1), (1, 1), (4, 4), 1)
    nb = C.lib.dk_sample_depthwise_backward_workspace_bytes(g, C.DK_F16)
    ws = torch.empty(nb, dtype=torch.uint8, device=DEV)
    gx, gr, gw = torch.empty_like(x), torch.empty_like(r), torch.empty_like(w)
    C.check(C.lib.dk_sample_depthwise_backward_one_pass(C.ptr(dy), C.ptr(x), C.ptr(r), C.ptr(w), C.ptr(gx), C.ptr(gr), C.ptr(gw), g,
                                                        C.DK_F16, C.ptr(ws), nb, C.stream_ptr(x.device)), "one-pass backward")
    torch.cuda.synchronize()
    assert C.lib.dk_ring_error_status() == 0
    want = oracle_local(oracle, case, torch.float16)
    compare(dict(grad_input=gx, grad_rotation=gr, grad_weight=gw),
            {k: want[k] for k in ("grad_input", "grad_rotation", "grad_weight")}, torch.float16, "one pass")


@pytest.mark.parametrize("n,c,h,w,stride", [(1, 16, 1, 56, 1), (1, 16, 2, 56, 2), (2, 48, 7, 112, 2), (3, 32, 5, 112, 1),
                                            (1, 144, 3, 56, 1), (200, 16, 2, 56, 1), (1, 160, 9, 56, 2),
                                            (5, 192, 28, 28, 1), (3, 48, 5, 28, 1), (2, 64, 9, 28, 2), (150, 16, 1, 28, 1),
                                            (2, 208, 28, 28, 2)])
def test_row_ring_kernels_on_short_and_non_square_planes(ops, oracle, n, c, h, w, stride):
    """Rows of 112 / 56 / 28 elements go to the row-ring kernels whatever the plane's height (28-wide rows are not a
    multiple of 16 bytes: the producer copies them in 8-byte pieces instead of by TMA; at stride 2 only their grad-input
    runs there): planes of one to nine rows (fewer rows than ring slots, blocks that own a single row or none), odd
    heights at stride 2, more samples than blocks, and more channels than one block keeps bank gradients for."""
    from deformable_kernels import _cabi as C
    case = make_case(n, c, h, w, stride=stride, rot_std=1.0, seed=500 + h)
    compare(mine_local(ops, case, torch.float16), oracle_local(oracle, case, torch.float16), torch.float16, "short planes")
    assert C.lib.dk_ring_error_status() == 0


@pytest.mark.parametrize("n,c,h,w,stride", [(3, 32, 9, 11, 1), (2, 48, 14, 14, 2), (5, 192, 12, 16, 1), (4, 96, 7, 7, 1),
                                            (6, 96, 7, 7, 2), (3, 160, 13, 20, 2), (130, 384, 14, 14, 1), (2, 16, 1, 1, 1)])
def test_offsets_and_bank_gradients_in_one_band_pass(oracle, n, c, h, w, stride):
    """The fused backward on planes the row-ring kernels do not take: grad-offsets and grad-bank come from ONE pass over the
    products dy * x (band form: channel groups of up to 96, partial sums per group and per block).  Odd and tiny planes,
    pixels beyond the row inside the last item, several channel groups, more units than blocks."""
    from deformable_kernels import _cabi as C
    case = make_case(n, c, h, w, stride=stride, rot_std=1.0, seed=300 + c + h)
    x, r, wt, dy = (case[k].half().to(DEV) for k in ("input", "rotation", "weight", "grad_output"))
    g = C.geom(x.shape, (3, 3), (stride, stride), (1, 1), (1, 1), (4, 4), 1)
    nb = C.lib.dk_sample_depthwise_backward_workspace_bytes(g, C.DK_F16)
    ws = torch.empty(max(nb, 1), dtype=torch.uint8, device=DEV)
    gr, gw = torch.full_like(r, float("nan")), torch.full_like(wt, float("nan"))
    for _ in range(2):  # twice: the partial sums of the first call must not leak into the second
        C.check(C.lib.dk_sample_depthwise_backward(C.ptr(dy), C.ptr(x), C.ptr(r), C.ptr(wt), None, C.ptr(gr), C.ptr(gw), g,
                                                   C.DK_F16, C.ptr(ws), nb, C.stream_ptr(x.device)), "fused backward")
    torch.cuda.synchronize()
    want = oracle_local(oracle, case, torch.float16)
    compare(dict(grad_rotation=gr, grad_weight=gw), {k: want[k] for k in ("grad_rotation", "grad_weight")}, torch.float16,
            "band pass")
    # and the separate entry points agree
    gr2, gw2 = torch.empty_like(r), torch.empty_like(wt)
    C.check(C.lib.dk_sample_depthwise_backward_rotation(C.ptr(dy), C.ptr(x), C.ptr(r), C.ptr(wt), C.ptr(gr2), g, C.DK_F16,
                                                        C.ptr(ws), nb, C.stream_ptr(x.device)), "grad-offsets")
    C.check(C.lib.dk_sample_depthwise_backward_filter(C.ptr(dy), C.ptr(x), C.ptr(r), C.ptr(gw2), g, C.DK_F16, C.ptr(ws), nb,
                                                      C.stream_ptr(x.device)), "grad-bank")
    torch.cuda.synchronize()
    assert rel_err(gr, gr2) < 2e-3 and rel_err(gw, gw2) < 2e-3


@pytest.mark.parametrize("shift", [10, 11])
@pytest.mark.parametrize("c,hw,stride", [(96, 56, 1), (32, 112, 2), (64, 28, 1)])
def test_local_dk_fp16_with_loss_scaled_gradients(ops, oracle, c, hw, stride, shift):
    """Upstream gradients scaled by 2^10 and 2^11, as a GradScaler hands them over.  The grad-offsets and grad-bank kernels
    form dy * x in fp16 (tensor-core operands), so |dy * x| must stay below 65504: with |dy| up to ~4.5 * 2^11 and |x| up
    to ~5 this still holds, and the results keep the 2e-3 tolerance; the limit is stated in include/dk_b200.h.  The scaled
    gradient is kept sparse (2 % of its entries) so that the fp16 OUTPUTS, sums of many such products, stay representable:
    what is under test is the intermediate product, not the range of the result type."""
    case = make_case(2, c, hw, hw, stride=stride, rot_std=1.0, seed=60 + shift)
    keep = torch.rand(case["grad_output"].shape, generator=torch.Generator().manual_seed(shift)) < 0.02
    case["grad_output"] = case["grad_output"] * keep * float(2 ** shift)
    assert 1e4 < float((case["grad_output"].abs().max() * case["input"].abs().max())) < 65504
    got = mine_local(ops, case, torch.float16)
    assert all(torch.isfinite(v).all() for v in got.values())
    compare(got, oracle_local(oracle, case, torch.float16), torch.float16, "scaled dy")


@pytest.mark.parametrize("hw,stride", [(56, 1), (56, 2), (112, 1)])
def test_infinite_input_next_to_the_padding_stays_local(ops, oracle, hw, stride):
    """An infinite input element on the plane's border.  On the row-ring kernels (rows of 112 / 56 elements) the padding
    is real zeros delivered by the TMA unit and multiplied by a finite kernel value, so, as in the reference (which skips
    padded taps), only outputs whose window contains the element itself are affected: wherever the oracle is finite the
    kernels are finite and agree."""
    case = make_case(2, 16, hw, hw, stride=stride, rot_std=0.7, seed=70)
    case["input"][0, 3, 5, hw - 1] = float("inf")     # last column: the next row's column -1 is its neighbour in memory
    case["input"][1, 7, 0, 0] = float("-inf")
    h = {k: (v.half() if torch.is_tensor(v) else v) for k, v in case.items()}
    x, r, w = (h[k].to(DEV) for k in ("input", "rotation", "weight"))
    y = ops.sample_depthwise(x, r, w, **case["args"]).float().cpu()
    want = oracle.sample_depthwise_forward(h["input"].float(), h["rotation"].float(), h["weight"].float(), **case["args"])
    ok = torch.isfinite(want)
    assert int((~ok).sum()) > 0 and int((~ok).sum()) <= 2 * 9
    assert torch.isfinite(y[ok]).all()
    assert float((y[ok] - want[ok].half().float()).abs().max() / want[ok].abs().max()) < 2e-3


def test_cfg4_full_size_fp16_against_live_reference(ops):
    mods = _ref_modules()
    if mods is None:
        pytest.skip("reference build (oracle/_ref) not present")
    case = dk_cases.cfg4()
    got = mine_deform(ops, case, torch.float16)
    want = _ref_deform(mods[0], _half_inputs_as_float(case), torch.float32)
    compare(got, want, torch.float16, "cfg4-full")


def test_cfg1_cfg2_fp32_against_live_reference(ops):
    mods = _ref_modules()
    if mods is None:
        pytest.skip("reference build (oracle/_ref) not present")
    case = dk_cases.cfg1()
    got = mine_local(ops, case, torch.float32)
    want = _ref_local(mods[0], case, torch.float32)
    for k in want:
        assert rel_err(got[k], want[k]) < 2e-5, k     # both sides carry fp32 rounding
    c2 = dk_cases.cfg2()
    data, coord, dy = (c2[k].to(DEV) for k in ("data", "coord", "grad_output"))
    shape = torch.tensor(data.shape[1:], dtype=data.dtype, device=DEV)
    y = data.new_empty(32, 256)
    mods[1].nd_linear_sample_forward_cuda(data, shape, coord, y)
    dd = data.new_empty(*data.size())
    mods[1].nd_linear_sample_backward_data_cuda(dy, data, shape, coord, dd)
    dcc = coord.new_empty(32, 2, 256)
    mods[1].nd_linear_sample_backward_coord_cuda(dy, data, shape, coord, dcc)
    got = mine_nd(ops, c2, torch.float32)
    assert rel_err(got["output"], y) < 1e-6
    assert rel_err(got["grad_data"], dd) < 1e-5
    assert rel_err(got["grad_coord"], dcc.sum(2)) < 1e-5


# ------------------------------------------------------------------ full-size properties (no oracle)

def test_full_size_properties_largest_layer_fp32(ops):
    """C=96, 112x112, batch 32, fp32: zero offsets reduce to a stock depthwise convolution with the
    2x2-averaged bank; the operator is linear in x and in W, so <dy, y> = <dx, x> = <dW, W>; the
    offset gradient agrees with a central difference along a random direction."""
    n, c, hw = 32, 96, 112
    case = dk_cases.cfg3(c, hw, 1, n=n)
    x, r, w, dy = (case[k].to(DEV) for k in ("input", "rotation", "weight", "grad_output"))
    y0 = ops.sample_depthwise(x, torch.zeros_like(r), w)
    ref = F.conv2d(x, F.avg_pool2d(w, 2, stride=1), padding=1, groups=c)
    assert rel_err(y0, ref) < 1e-5
    x.requires_grad_(True), r.requires_grad_(True), w.requires_grad_(True)
    y = ops.sample_depthwise(x, r, w)
    dx, dr, dw = torch.autograd.grad(y, [x, r, w], dy)
    # the three inner products cancel heavily, so the mismatch is judged against the sum of magnitudes
    lhs = (dy.double() * y.detach().double()).sum()
    gx = dx.double() * x.detach().double()
    gw = dw.double() * w.detach().double()
    assert abs(float(gx.sum() - lhs)) < 1e-6 * float(gx.abs().sum())
    assert abs(float(gw.sum() - lhs)) < 1e-6 * float(gw.abs().sum())
    v = torch.randn(r.shape, device=DEV, generator=torch.Generator(device=DEV).manual_seed(12))
    eps = 1e-3
    with torch.no_grad():
        yp = ops.sample_depthwise(x, r + eps * v, w).double()
        ym = ops.sample_depthwise(x, r - eps * v, w).double()
        fd = ((yp - ym) * dy.double()).sum() / (2 * eps)
    an = dr.double() * v.double()
    # the directional derivative is a heavily cancelling sum too (and the central difference steps over kinks)
    assert abs(float(fd - an.sum())) < 5e-3 * float(an.abs().sum())
