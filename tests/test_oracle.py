"""CPU tests of the oracle itself (no GPU): the C restatement against the independent
PyTorch composition in float64, against known-answer reductions to stock ops, and
against the golden vectors produced by the reference's own CUDA build on a B200."""
import glob
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import dk_cases
from dk_cases import make_case, make_nd_case, rel_err
from oracle import dk_oracle as O
from oracle import torch_composition as TC

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

LOCAL_CASES = [
    dict(n=2, c=6, h=9, w=7, scope=(4, 4), k=3, stride=1, pad=1, dil=1, groups=1, rot_std=1.0),
    dict(n=2, c=6, h=9, w=7, scope=(4, 4), k=3, stride=2, pad=1, dil=1, groups=2, rot_std=1.0),
    dict(n=1, c=4, h=11, w=10, scope=(3, 5), k=3, stride=1, pad=2, dil=2, groups=4, rot_std=1.5),
    dict(n=2, c=4, h=8, w=8, scope=(2, 2), k=1, stride=1, pad=0, dil=1, groups=1, rot_std=0.7),
    dict(n=1, c=3, h=12, w=9, scope=(6, 4), k=5, stride=2, pad=2, dil=1, groups=3, rot_std=1.0),
    dict(n=1, c=2, h=10, w=10, scope=(4, 4), k=(3, 1), stride=(1, 2), pad=(1, 0), dil=1, groups=1, rot_std=1.0),
]


def _dbl(case):
    out = {}
    for key, v in case.items():
        out[key] = v.double() if torch.is_tensor(v) else v
    return out


def _snap(t, frac=0.25, seed=1):
    """Put a share of the offsets on exact halves/integers so that bank coordinates hit
    the integer kinks (u = f + r + 0.5 for scope 4 / kernel 3)."""
    gen = torch.Generator().manual_seed(seed)
    pick = torch.rand(t.shape, generator=gen) < frac
    return torch.where(pick, torch.round(t * 2) / 2, t)


@pytest.mark.parametrize("cfg", LOCAL_CASES)
def test_local_dk_restatement_equals_composition_fp64(cfg):
    case = _dbl(make_case(seed=3, **cfg))
    case["rotation"] = _snap(case["rotation"])
    x, r, w, dy, a = case["input"], case["rotation"], case["weight"], case["grad_output"], case["args"]
    y = O.sample_depthwise_forward(x, r, w, **a)
    dx, dr, dw = O.sample_depthwise_backward(dy, x, r, w, **a)
    y2, (dx2, dr2, dw2) = TC.grads(lambda x_, r_, w_: TC.sample_depthwise(x_, r_, w_, **a), [x, r, w], dy)
    assert rel_err(y, y2) < 1e-12
    assert rel_err(dx, dx2) < 1e-12
    assert rel_err(dr, dr2) < 1e-12
    assert rel_err(dw, dw2) < 1e-12


@pytest.mark.parametrize("cfg", LOCAL_CASES)
def test_deform_dk_restatement_equals_composition_fp64(cfg):
    case = _dbl(make_case(seed=5, off_std=2.0, **cfg))
    case["rotation"] = _snap(case["rotation"])
    case["offset"] = _snap(case["offset"], seed=2)
    x, o, r, w, dy, a = (case["input"], case["offset"], case["rotation"], case["weight"], case["grad_output"],
                         case["args"])
    y = O.deform_sample_depthwise_forward(x, o, r, w, **a)
    dx, do, dr, dw = O.deform_sample_depthwise_backward(dy, x, o, r, w, **a)
    y2, (dx2, do2, dr2, dw2) = TC.grads(
        lambda x_, o_, r_, w_: TC.deform_sample_depthwise(x_, o_, r_, w_, **a), [x, o, r, w], dy)
    assert rel_err(y, y2) < 1e-12
    assert rel_err(dx, dx2) < 1e-12
    assert rel_err(do, do2) < 1e-12
    assert rel_err(dr, dr2) < 1e-12
    assert rel_err(dw, dw2) < 1e-12


@pytest.mark.parametrize("shape", [(2, 2), (4, 4), (3, 5), (5,), (2, 3, 4), (2, 2, 2, 3)])
def test_nd_linear_restatement_equals_composition_fp64(shape):
    case = make_nd_case(7, shape, 40, seed=11)
    data, coord, dy = case["data"].double(), case["coord"].double(), case["grad_output"].double()
    y = O.nd_linear_sample_forward(data, coord)
    dd, dc = O.nd_linear_sample_backward(dy, data, coord)
    y2, (dd2, dc2) = TC.grads(TC.nd_linear_sample, [data, coord], dy)
    assert rel_err(y, y2) < 1e-12
    assert rel_err(dd, dd2) < 1e-12
    assert rel_err(dc, dc2) < 1e-12


# ------------------------------------------------------------------ known answers

def test_zero_offsets_scope_equals_kernel_is_depthwise_conv():
    case = _dbl(make_case(2, 5, 10, 9, scope=(3, 3), k=3, stride=2, pad=1, seed=2))
    x, w, dy, a = case["input"], case["weight"], case["grad_output"], case["args"]
    r = torch.zeros_like(case["rotation"])
    y = O.sample_depthwise_forward(x, r, w, **a)
    xx = x.clone().requires_grad_(True)
    ww = w.clone().requires_grad_(True)
    ref = F.conv2d(xx, ww, stride=2, padding=1, groups=5)
    assert rel_err(y, ref) < 1e-13
    gx, gw = torch.autograd.grad(ref, [xx, ww], dy)
    dx, _, dw = O.sample_depthwise_backward(dy, x, r, w, **a)
    assert rel_err(dx, gx) < 1e-13
    assert rel_err(dw, gw) < 1e-13


def test_zero_offsets_scope4_kernel3_is_conv_with_averaged_bank():
    # every bank coordinate is f + 0.5, so the sampled 3x3 kernel is the 2x2 average pool of the bank
    case = _dbl(make_case(2, 4, 8, 8, scope=(4, 4), k=3, stride=1, pad=1, seed=4))
    x, w, a = case["input"], case["weight"], case["args"]
    r = torch.zeros_like(case["rotation"])
    y = O.sample_depthwise_forward(x, r, w, **a)
    ref = F.conv2d(x, F.avg_pool2d(w, 2, stride=1), padding=1, groups=4)
    assert rel_err(y, ref) < 1e-13


def test_deform_scope_equals_kernel_is_torchvision_deform_conv():
    tv = pytest.importorskip("torchvision.ops")
    case = _dbl(make_case(2, 4, 9, 8, scope=(3, 3), k=3, stride=2, pad=1, off_std=2.0, seed=6))
    x, o, w, dy, a = case["input"], case["offset"], case["weight"], case["grad_output"], case["args"]
    r = torch.zeros_like(case["rotation"])
    y = O.deform_sample_depthwise_forward(x, o, r, w, **a)
    xx, oo, ww = (t.clone().requires_grad_(True) for t in (x, o, w))
    ref = tv.deform_conv2d(xx, oo, ww, stride=2, padding=1)
    assert rel_err(y, ref) < 1e-13
    gx, go, gw = torch.autograd.grad(ref, [xx, oo, ww], dy)
    dx, do, _, dw = O.deform_sample_depthwise_backward(dy, x, o, r, w, **a)
    assert rel_err(dx, gx) < 1e-13
    assert rel_err(do, go) < 1e-12
    assert rel_err(dw, gw) < 1e-13


def test_nd_linear_integer_coordinates_are_lookups_and_outside_is_zero():
    gen = torch.Generator().manual_seed(0)
    data = torch.randn(5, 3, 4, generator=gen, dtype=torch.float64)
    coord = torch.tensor([[0., 0.], [2., 3.], [1., 2.], [-1., 1.], [3., 0.], [1., 4.], [-0.5, 0.], [2.5, 3.5]],
                         dtype=torch.float64)
    y = O.nd_linear_sample_forward(data, coord)
    assert torch.equal(y[0], data[:, 0, 0])
    assert torch.equal(y[1], data[:, 2, 3])
    assert torch.equal(y[2], data[:, 1, 2])
    assert torch.equal(y[3], torch.zeros(5, dtype=torch.float64))      # x <= -1
    assert torch.equal(y[4], torch.zeros(5, dtype=torch.float64))      # x >= s
    assert torch.equal(y[5], torch.zeros(5, dtype=torch.float64))
    assert torch.allclose(y[6], 0.5 * data[:, 0, 0])                  # low corner missing
    assert torch.allclose(y[7], 0.25 * data[:, 2, 3])                 # three corners missing
    dy = torch.ones(8, 5, dtype=torch.float64)
    dd, dc = O.nd_linear_sample_backward(dy, data, coord)
    assert torch.equal(dc[3], torch.zeros(2, dtype=torch.float64))
    assert torch.equal(dc[4], torch.zeros(2, dtype=torch.float64))
    # at the upper edge the derivative goes into the zero extension: -data[last]
    assert torch.allclose(dc[1], torch.stack([-data[:, 2, 3].sum(), -data[:, 2, 3].sum()]))


def test_nd_linear_2d_is_grid_sample_loosely():
    case = make_nd_case(6, (4, 5), 30, seed=9, lo=0.0, hi_pad=-1.0, snap=0.0)
    data, coord = case["data"].double(), case["coord"].double()
    y = O.nd_linear_sample_forward(data, coord)
    gx = coord[:, 1] / (5 - 1) * 2 - 1
    gy = coord[:, 0] / (4 - 1) * 2 - 1
    grid = torch.stack([gx, gy], -1).view(1, 1, -1, 2)
    ref = F.grid_sample(data.unsqueeze(0), grid, mode="bilinear", padding_mode="zeros", align_corners=True)
    assert rel_err(y, ref[0, :, 0].t()) < 1e-6


def test_rotation_groups_use_channel_mod_groups():
    case = _dbl(make_case(1, 4, 6, 6, groups=2, rot_std=1.0, seed=8))
    x, r, w, a = case["input"], case["rotation"], case["weight"], case["args"]
    y = O.sample_depthwise_forward(x, r, w, **a)
    a1 = dict(a, rotation_groups=1)
    for c in range(4):
        g = c % 2
        yc = O.sample_depthwise_forward(x[:, c:c + 1], r[:, g * 18:(g + 1) * 18], w[c:c + 1], **a1)
        assert torch.equal(y[:, c:c + 1], yc)


def test_gradcheck_on_composition_away_from_kinks():
    case = _dbl(make_case(1, 2, 5, 5, rot_std=0.3, off_std=0.7, seed=12))
    x, o, r, w, a = case["input"], case["offset"], case["rotation"], case["weight"], case["args"]
    o = o + 0.013
    r = r + 0.007
    ins = [t.clone().requires_grad_(True) for t in (x, o, r, w)]
    assert torch.autograd.gradcheck(lambda *t: TC.deform_sample_depthwise(*t, **a), ins, eps=1e-6, atol=1e-5)


def test_oracle_f32_tracks_f64():
    case = make_case(2, 8, 12, 12, rot_std=1.0, off_std=2.0, seed=13)
    x, o, r, w, dy, a = (case["input"], case["offset"], case["rotation"], case["weight"], case["grad_output"],
                         case["args"])
    y32 = O.deform_sample_depthwise_forward(x, o, r, w, **a)
    y64 = O.deform_sample_depthwise_forward(x.double(), o.double(), r.double(), w.double(), **a)
    assert rel_err(y32, y64) < 1e-6
    g32 = O.deform_sample_depthwise_backward(dy, x, o, r, w, **a)
    g64 = O.deform_sample_depthwise_backward(dy.double(), x.double(), o.double(), r.double(), w.double(), **a)
    for p, q in zip(g32, g64):
        assert rel_err(p, q) < 1e-5


# ------------------------------------------------------------------ golden vectors

def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "*.npz")))


@pytest.mark.parametrize("path", _golden_files() or [None])
def test_oracle_matches_reference_cuda_golden(path):
    """The golden files hold inputs and the outputs the reference's own CUDA kernels
    produced for them on a B200 (tests/golden/make_golden.py)."""
    if path is None:
        pytest.skip("no golden vectors committed yet")
    z = np.load(path)
    kind = str(z["kind"])
    t = {k: torch.from_numpy(z[k]) for k in z.files if k not in ("kind", "args")}
    tol = 1e-12 if t[next(iter(t))].dtype == torch.float64 else 2e-5
    if kind == "nd":
        y = O.nd_linear_sample_forward(t["data"], t["coord"])
        dd, dc = O.nd_linear_sample_backward(t["grad_output"], t["data"], t["coord"])
        assert rel_err(y, t["ref_output"]) < tol
        assert rel_err(dd, t["ref_grad_data"]) < tol
        assert rel_err(dc, t["ref_grad_coord"]) < tol
        return
    a = [int(v) for v in z["args"]]
    args = dict(kernel_size=(a[0], a[1]), stride=(a[2], a[3]), padding=(a[4], a[5]), dilation=(a[6], a[7]),
                rotation_groups=a[8])
    if kind == "local":
        y = O.sample_depthwise_forward(t["input"], t["rotation"], t["weight"], **args)
        dx, dr, dw = O.sample_depthwise_backward(t["grad_output"], t["input"], t["rotation"], t["weight"], **args)
        got = dict(ref_output=y, ref_grad_input=dx, ref_grad_rotation=dr, ref_grad_weight=dw)
    else:
        y = O.deform_sample_depthwise_forward(t["input"], t["offset"], t["rotation"], t["weight"], **args)
        dx, do, dr, dw = O.deform_sample_depthwise_backward(t["grad_output"], t["input"], t["offset"],
                                                            t["rotation"], t["weight"], **args)
        got = dict(ref_output=y, ref_grad_input=dx, ref_grad_offset=do, ref_grad_rotation=dr, ref_grad_weight=dw)
    for name, val in got.items():
        assert rel_err(val, t[name]) < tol, name
