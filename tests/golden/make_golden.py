#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own CUDA
kernels (the unmodified extension built by oracle/build_ref.py into oracle/_ref/) on a GPU.

    python tests/golden/make_golden.py [out_dir]        # needs a CUDA device

Each .npz holds the seeded inputs of one small case (tests/dk_cases.py) and the
reference's forward output and gradients for them, called the way the reference's
autograd functions call the extension (functions/filter_sample_depthwise.py:39-85,
127-189; functions/nd_linear_sample.py:22-55): outputs from new_empty, gradient
buffers from zeros_like.  float32 and float64 runs are stored; the CPU oracle is
checked against them in tests/test_oracle.py and the CUDA kernels in
tests/test_parity_gpu.py.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import build_ref  # noqa: E402
import dk_cases  # noqa: E402

CASES = {
    "local_s1": dict(n=2, c=6, h=9, w=7, scope=(4, 4), k=3, stride=1, pad=1, dil=1, groups=1, rot_std=1.0),
    "local_s2_g2": dict(n=2, c=6, h=9, w=8, scope=(4, 4), k=3, stride=2, pad=1, dil=1, groups=2, rot_std=1.0),
    "local_dil2_scope35": dict(n=1, c=4, h=11, w=10, scope=(3, 5), k=3, stride=1, pad=2, dil=2, groups=4, rot_std=1.5),
    "local_k1_scope2": dict(n=2, c=4, h=8, w=8, scope=(2, 2), k=1, stride=1, pad=0, dil=1, groups=1, rot_std=0.7),
    "local_k5": dict(n=1, c=3, h=12, w=9, scope=(6, 4), k=5, stride=2, pad=2, dil=1, groups=3, rot_std=1.0),
}
ND_CASES = {"nd_2x2": (2, 2), "nd_4x4": (4, 4), "nd_3d": (2, 3, 4), "nd_1d": (5,)}


def snap(t, frac=0.25, seed=1):
    gen = torch.Generator().manual_seed(seed)
    pick = torch.rand(t.shape, generator=gen) < frac
    return torch.where(pick, torch.round(t * 2) / 2, t)


def ints(a):
    return (a["kernel_size"][0], a["kernel_size"][1], a["stride"][0], a["stride"][1], a["padding"][0], a["padding"][1],
            a["dilation"][0], a["dilation"][1])


def run_local(fs, case, dtype, dev):
    x, r, w, dy = (case[k].to(dtype).to(dev) for k in ("input", "rotation", "weight", "grad_output"))
    a = case["args"]
    tail = ints(a) + (w.size(2), w.size(3), a["rotation_groups"])
    y = torch.empty_like(dy)
    fs.sample_depthwise_forward_cuda(x, r, w, y, *tail)
    dx, dr, dw = torch.zeros_like(x), torch.zeros_like(r), torch.zeros_like(w)
    fs.sample_depthwise_backward_data_cuda(dy, x, r, w, dx, *tail)
    fs.sample_depthwise_backward_rotation_cuda(dy, x, r, w, dr, *tail)
    fs.sample_depthwise_backward_filter_cuda(dy, x, r, w, dw, *tail)
    torch.cuda.synchronize()
    return dict(ref_output=y, ref_grad_input=dx, ref_grad_rotation=dr, ref_grad_weight=dw)


def run_deform(fs, case, dtype, dev):
    x, o, r, w, dy = (case[k].to(dtype).to(dev) for k in ("input", "offset", "rotation", "weight", "grad_output"))
    a = case["args"]
    tail = ints(a) + (w.size(2), w.size(3), a["rotation_groups"])
    y = torch.empty_like(dy)
    fs.deformable_sample_depthwise_forward_cuda(x, o, r, w, y, *tail)
    dx, do, dr, dw = torch.zeros_like(x), torch.zeros_like(o), torch.zeros_like(r), torch.zeros_like(w)
    fs.deformable_sample_depthwise_backward_data_cuda(dy, x, o, r, w, dx, *tail)
    fs.deformable_sample_depthwise_backward_offset_cuda(dy, x, o, r, w, do, *tail)
    fs.deformable_sample_depthwise_backward_rotation_cuda(dy, x, o, r, w, dr, *tail)
    fs.deformable_sample_depthwise_backward_filter_cuda(dy, x, o, r, w, dw, *tail)
    torch.cuda.synchronize()
    return dict(ref_output=y, ref_grad_input=dx, ref_grad_offset=do, ref_grad_rotation=dr, ref_grad_weight=dw)


def run_nd(nd, case, dtype, dev):
    data, coord, dy = (case[k].to(dtype).to(dev) for k in ("data", "coord", "grad_output"))
    shape = torch.tensor(data.shape[1:], dtype=dtype, device=dev)
    y = data.new_empty(coord.size(0), data.size(0))
    nd.nd_linear_sample_forward_cuda(data, shape, coord, y)
    dd = data.new_empty(*data.size())
    nd.nd_linear_sample_backward_data_cuda(dy, data, shape, coord, dd)
    dcc = coord.new_empty(coord.size(0), coord.size(1), data.size(0))
    nd.nd_linear_sample_backward_coord_cuda(dy, data, shape, coord, dcc)
    torch.cuda.synchronize()
    return dict(ref_output=y, ref_grad_data=dd, ref_grad_coord=dcc.sum(2))


def save(path, kind, case, outs, dtype, args=None):
    arrs = {k: v.to(dtype).numpy() for k, v in case.items() if torch.is_tensor(v)}
    arrs.update({k: v.cpu().numpy() for k, v in outs.items()})
    arrs["kind"] = np.array(kind)
    if args is not None:
        arrs["args"] = np.array(ints(args) + (args["rotation_groups"],), dtype=np.int64)
    np.savez_compressed(path, **arrs)


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda:0")
    fs = build_ref.load_module("filter_sample_depthwise_cuda")
    nd = build_ref.load_module("nd_linear_sample_cuda")
    for name, cfg in CASES.items():
        for tag, dtype in (("f32", torch.float32), ("f64", torch.float64)):
            case = dk_cases.make_case(seed=21, **cfg)
            case["rotation"] = snap(case["rotation"])
            save(os.path.join(out_dir, "%s_%s.npz" % (name, tag)), "local", case, run_local(fs, case, dtype, dev), dtype,
                 case["args"])
            case = dk_cases.make_case(seed=22, off_std=2.0, **cfg)
            case["rotation"] = snap(case["rotation"])
            case["offset"] = snap(case["offset"], seed=2)
            save(os.path.join(out_dir, "deform_%s_%s.npz" % (name[6:], tag)), "deform", case,
                 run_deform(fs, case, dtype, dev), dtype, case["args"])
    for name, shape in ND_CASES.items():
        for tag, dtype in (("f32", torch.float32), ("f64", torch.float64)):
            case = dk_cases.make_nd_case(7, shape, 24, seed=23)
            save(os.path.join(out_dir, "%s_%s.npz" % (name, tag)), "nd", case, run_nd(nd, case, dtype, dev), dtype)
    print("wrote golden vectors to", out_dir)


if __name__ == "__main__":
    main()
