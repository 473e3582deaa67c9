"""CPU-side checks of the C-ABI library: it loads, it exports every symbol that
include/dk_b200.h declares, and its host-side argument validation answers without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cabi():
    from deformable_kernels import _cabi
    return _cabi


def _declared():
    text = open(os.path.join(ROOT, "include", "dk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(cabi):
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(cabi.lib, n), n
    assert set(cabi.EXPORTS) == set(names)


def test_version_and_status_strings(cabi):
    assert b"sm_100a" in cabi.lib.dk_version()
    assert cabi.lib.dk_status_string(0) == b"ok"
    for s in range(1, 5):
        assert cabi.lib.dk_status_string(s) not in (b"ok", b"unknown status")


def test_output_size_matches_reference_formula(cabi):
    g = cabi.geom((2, 8, 28, 30), (3, 3), (2, 1), (1, 1), (1, 2), (4, 4), 1)
    h, w = ctypes.c_int(), ctypes.c_int()
    assert cabi.lib.dk_output_size(g, ctypes.byref(h), ctypes.byref(w)) == 0
    assert h.value == (28 + 2 - 3) // 2 + 1
    assert w.value == (30 + 2 - (2 * 2 + 1)) // 1 + 1
    bad = cabi.geom((2, 8, 2, 2), (5, 5), (1, 1), (0, 0), (1, 1), (4, 4), 1)   # input too small
    assert cabi.lib.dk_output_size(bad, ctypes.byref(h), ctypes.byref(w)) == 1


def test_bad_arguments_are_refused_before_any_launch(cabi):
    g = cabi.geom((1, 4, 8, 8), (3, 3), (1, 1), (1, 1), (1, 1), (4, 4), 1)
    null = ctypes.c_void_p(0)
    assert cabi.lib.dk_sample_depthwise_forward(null, null, null, null, g, 0, null) == 1
    g3 = cabi.geom((1, 4, 8, 8), (3, 3), (1, 1), (1, 1), (1, 1), (4, 4), 3)          # 4 % 3 != 0
    one = ctypes.c_void_p(16)
    assert cabi.lib.dk_sample_depthwise_forward(one, one, one, one, g3, 0, null) == 1
    assert cabi.lib.dk_sample_depthwise_forward(one, one, one, one, g, 7, null) == 1    # unknown dtype
    shape = (ctypes.c_int * 9)(*([2] * 9))
    assert cabi.lib.dk_nd_linear_sample_forward(one, one, one, 1, 1, 9, shape, 0, null) == 2  # > 8 dims


def test_workspace_queries(cabi):
    g = cabi.geom((4, 64, 28, 28), (3, 3), (1, 1), (1, 1), (1, 1), (4, 4), 1)
    n32 = cabi.lib.dk_sample_depthwise_backward_filter_workspace_bytes(g, cabi.DK_F32)
    assert n32 > 0 and n32 % 256 == 0 and n32 % (64 * 16 * 4) == 0
    assert cabi.lib.dk_deform_sample_depthwise_backward_data_workspace_bytes(g, cabi.DK_F32) == 0
    assert cabi.lib.dk_deform_sample_depthwise_backward_data_workspace_bytes(g, cabi.DK_F16) >= 4 * 64 * 28 * 28 * 4


def test_noalloc_entry_point_fits_every_sweep_layer(cabi):
    """Host-only sizing of dk_sample_depthwise_backward_filter_noalloc: each of the ten MobileNetV2 sweep layers at
    batch 128, in fp16 and fp32, is accepted and uses at most the 8 MiB array; the two 7 x 7 layers, whose usual
    general-kernel partial sums (8.97 / 9.03 MB) exceed it, run with fewer pixel blocks in fp32 and with the tensor-core
    kernel's smaller partial sums in fp16.  fp64 is accepted too (its partial sums are twice as large, the block count shrinks)."""
    cap = cabi.lib.dk_sample_depthwise_backward_filter_noalloc_max_bytes()
    assert cap == 8 << 20
    for c, hw in [(96, 112), (144, 56), (192, 28), (384, 14), (960, 7)]:
        for s in (1, 2):
            g = cabi.geom((128, c, hw, hw), (3, 3), (s, s), (1, 1), (1, 1), (4, 4), 1)
            for dt in (cabi.DK_F16, cabi.DK_F32, cabi.DK_F64):
                used = cabi.lib.dk_sample_depthwise_backward_filter_noalloc_bytes(g, dt)
                assert 0 < used <= cap, (c, hw, s, dt, used)
                assert used % (c * 16 * 4) == 0, (c, hw, s, dt, used)
            usual = cabi.lib.dk_sample_depthwise_backward_filter_workspace_bytes(g, cabi.DK_F32)
            if (c, hw) == (960, 7):
                assert usual > cap   # the case the shrinking plan exists for
                assert cabi.lib.dk_sample_depthwise_backward_filter_noalloc_bytes(g, cabi.DK_F16) < (2 << 20)
    # one block's partial sums beyond the array: refused
    g = cabi.geom((64, 64, 600, 600), (3, 3), (1, 1), (1, 1), (1, 1), (200, 200), 1)
    assert cabi.lib.dk_sample_depthwise_backward_filter_noalloc_bytes(g, cabi.DK_F32) == 0


def test_block_shapes_of_the_fp16_fast_path_are_launchable(cabi):
    """Planner invariants over many geometries (host only): every block shape the tensor-core kernels would launch covers
    the plane and all channels, fits shared memory and the kernels' launch bounds, and the workspace query covers the
    partial sums the plan needs."""
    import random
    rng = random.Random(7)
    layers = [(96, 112), (144, 56), (192, 28), (384, 14), (960, 7)]
    cases = [(128, c, hw, hw, s, (4, 4)) for c, hw in layers for s in (1, 2)]
    for _ in range(300):
        cases.append((rng.choice([1, 2, 3, 8, 33, 128, 257]), 16 * rng.randint(1, 64), rng.randint(1, 130), rng.randint(1, 130),
                      rng.choice([1, 2]), rng.choice([(4, 4), (3, 3), (2, 2), (4, 3), (1, 1), (3, 5)])))
    out = (ctypes.c_longlong * 8)()
    max_warps = {0: 14, 1: 14, 2: 16, 3: 14}
    seen = 0
    for n, c, h, w, s, scope in cases:
        g = cabi.geom((n, c, h, w), (3, 3), (s, s), (1, 1), (1, 1), scope, 1)
        ho, wo = (h + 2 - 3) // s + 1, (w + 2 - 3) // s + 1
        for p in range(4):
            rc = cabi.lib.dk_local_plan_query(g, cabi.DK_F16, p, out)
            assert rc in (0, 2), (n, c, h, w, s, scope, p, rc)
            if rc:
                continue
            seen += 1
            bh, cg, groups, warps, bands, smem, blocks, ws = list(out)
            rows = h if p == 1 else ho
            tag = (n, c, h, w, s, scope, p, list(out))
            assert 1 <= bh <= rows and bands * bh >= rows and (bands - 1) * bh < rows, tag
            assert cg % 16 == 0 and cg * groups >= c and cg * (groups - 1) < c, tag
            assert 1 <= warps <= max_warps[p], tag
            assert 0 < smem <= 227 * 1024, tag
            assert 0 < blocks < 2 ** 31 and groups <= 65535, tag
            if p == 2:
                assert ws == (groups * n * 18 * ho * wo * 4 if groups > 1 else 0), tag
                assert cabi.lib.dk_sample_depthwise_backward_rotation_workspace_bytes(g, cabi.DK_F16) >= ws, tag
            if p == 3:
                assert ws == blocks // groups * c * 16 * 4, tag
                assert cabi.lib.dk_sample_depthwise_backward_filter_workspace_bytes(g, cabi.DK_F16) >= ws, tag
    assert seen > 600
    # the highest shared-memory byte a lane of the forward kernel can read, recomputed from the reported block shape
    # (band layout of csrc/dk_mma_common.cuh: rows of the group's channels back to back, 8 halves of slack in front, 16
    # behind; a lane reads six halves from source column ow * S - 2 of the three rows of its item), stays inside the
    # block's shared memory for every reported shape
    def band_pitch(rb, wp):
        need = rb * wp + 8 + 16
        pitch = ((need + 7) & ~15) + 8
        return pitch + 16 if pitch < need else pitch
    checked = 0
    for n, c, h, w, s, scope in cases:
        g = cabi.geom((n, c, h, w), (3, 3), (s, s), (1, 1), (1, 1), scope, 1)
        if cabi.lib.dk_local_plan_query(g, cabi.DK_F16, 0, out):
            continue
        bh, cg, groups, warps, bands, smem, blocks, ws = list(out)
        ho, wo = (h + 2 - 3) // s + 1, (w + 2 - 3) // s + 1
        wp, rb = w + (w & 1), (bh - 1) * s + 3
        pitch = band_pitch(rb, wp)
        nb = (wo + 7) // 8
        worst = 0
        for band in (0, bands - 1):
            row_lo = band * bh * s - 1
            for mode in (2, 1, 0):                      # 16-byte, 4-byte and 2-byte copies lay the rows out differently
                if mode == 2 and ((h * w) % 8 or w % 2):
                    continue
                if mode == 1 and w % 2:
                    continue
                org = ((row_lo * w) & ~7) if mode == 2 else row_lo * wp
                last_row = min(band * bh + bh, ho) - 1  # last destination row of the band that exists
                top = 8 + (last_row * s - 1 + 2) * wp + ((nb * 8 - 2) * s - 2) + 6 - org   # one past the last half read
                worst = max(worst, (cg - 1) * pitch + top)
        assert worst * 2 <= smem, (n, c, h, w, s, scope, list(out), worst * 2)
        assert worst <= cg * pitch + 8, (n, c, h, w, s, scope, list(out), worst, cg * pitch)   # within the bands (+ next region's slack)
        checked += 1
    assert checked > 150
    # outside the fast path: other dtypes, kernels other than 3x3
    g = cabi.geom((4, 64, 28, 28), (3, 3), (1, 1), (1, 1), (1, 1), (4, 4), 1)
    assert cabi.lib.dk_local_plan_query(g, cabi.DK_F32, 0, out) == 2
    g5 = cabi.geom((4, 64, 28, 28), (5, 5), (1, 1), (2, 2), (1, 1), (4, 4), 1)
    assert cabi.lib.dk_local_plan_query(g5, cabi.DK_F16, 0, out) == 2
    assert cabi.lib.dk_local_plan_query(g, cabi.DK_F16, 9, out) == 1
    assert cabi.lib.dk_local_plan_query(g, cabi.DK_F16, 0, None) == 1


def test_row_ring_plans_fit_the_kernels_layouts(cabi):
    """Planner of the producer / consumer row-ring kernels (host only; without a device the library plans for the one
    target: 227 KB of shared memory, 148 SMs).  For the MobileNetV2 sweep layers and a spread of other shapes: the reported
    ring depths, warps and channel split are launchable, and the highest shared-memory byte the kernel's own layout reaches
    (recomputed here region by region: rings, bank copies, per-warp scratch, barriers, fill counters) stays inside the
    dynamic shared memory the launch asks for."""
    BUDGET = 227 * 1024
    def inner(w):                      # halves per channel row of a ring slot (RowLayout)
        return (w + 8 + 7) // 16 * 16 + 8
    def rot_slot(w):                   # halves per slot of the offsets ring (RotLayout)
        return 18 * (8 + (w + 7) // 8 * 8 + 8)
    BANK, GW_SCRATCH, BWD_SCRATCH = 24, 3 * 36 * 8 * 4 + 24 * 8, 3 * 16 * 8 * 4 + 24 * 8
    def up(v, a):
        return (v + a - 1) // a * a
    def top_conv(w, wr, cg, r, rr):                         # ring_conv_kernel
        bars = up((r * cg * inner(w) + 16 + rr * rot_slot(wr) + cg * BANK) * 2, 8)
        return bars + (2 * r + 2 * rr) * 8 + 2 * 4
    def top_convT2(wo, cg, r):                              # ring_convT2_kernel
        bars = up((r * cg * inner(wo) + 64 + r * rot_slot(wo) + cg * BANK) * 2, 8)
        return bars + 4 * r * 8 + 2 * 4
    def top_gw(w, wo, cg, r, rr, ncw):                      # ring_gw_kernel
        rings = (r * cg * inner(w) + 64 + rr * cg * inner(wo) + 64 + rr * rot_slot(wo)) * 2
        after = up(max(rings, ncw * cg * 16 * 4), 16)
        bars = up(after + 16 * (cg + 8) * 2 + ncw * GW_SCRATCH, 8)
        return bars + (2 * r + 4 * rr) * 8 + 3 * 4
    def top_bwd(w, wo, cg, rx, rd, ncw):                    # ring_bwd_kernel
        rings = (rx * cg * inner(w) + 64 + rd * cg * inner(wo) + 64 + rd * rot_slot(wo)) * 2
        after = up(max(rings, ncw * cg * 16 * 4), 16)
        bars = up(after + (cg * BANK + 16 * (cg + 8)) * 2 + ncw * BWD_SCRATCH, 8)
        return bars + (2 * rx + 4 * rd) * 8 + 3 * 4
    sweep = [(96, 112), (144, 56), (192, 28), (384, 14), (960, 7)]
    cases = [(128, c, hw, hw, s) for c, hw in sweep for s in (1, 2)]
    cases += [(n, c, h, w, s) for w in (112, 56, 28) for s in (1, 2) for n, c, h in
              ((1, 16, 1), (3, 48, 5), (2, 160, 9), (7, 208, 28), (64, 256, 56), (2, 1024, 3), (300, 32, 2))]
    out = (ctypes.c_longlong * 8)()
    plans = {}
    for n, c, h, w, s in cases:
        g = cabi.geom((n, c, h, w), (3, 3), (s, s), (1, 1), (1, 1), (4, 4), 1)
        wo = (w - 1) // s + 1
        for p in (4, 5, 6, 7):
            rc = cabi.lib.dk_local_plan_query(g, cabi.DK_F16, p, out)
            assert rc in (0, 2), (n, c, h, w, s, p, rc)
            if rc:
                continue
            r, rr, warps, np_, cg, groups, smem, blocks = list(out)
            tag = (n, c, h, w, s, p, list(out))
            plans[(n, c, h, w, s, p)] = list(out)
            assert cg % 16 == 0 and cg * groups == c and groups <= 65535, tag
            assert 1 <= np_ <= 4 and warps - np_ >= 1 and warps <= 24, tag
            assert (np_ > 1) == ((w if p in (4, 6) or s == 1 else wo) % 8 != 0 and p != 6), tag   # several producers only for rows TMA cannot fetch
            assert r >= 4 and rr >= 2 and 0 < smem <= BUDGET and 0 < blocks <= 148, tag
            ncw = warps - np_
            if p == 4 or (p == 5 and s == 1):
                top = top_conv(w, w if p == 5 else wo, cg, r, rr)
            elif p == 5:
                top = top_convT2(wo, cg, r)
            elif p == 6:
                top = top_gw(w, wo, cg, r, rr, ncw)
                assert cg <= 144, tag
            else:
                top = top_bwd(w, wo, cg, r, rr, ncw)
                assert cg <= 144 and groups == 1, tag
            assert top <= smem, tag + (top,)
    # which sweep layers run here: rows of 112 and 56 every pass, rows of 28 at stride 1, and the grad-input of 28 at stride 2
    for c, hw in sweep:
        for s in (1, 2):
            got = sorted(p for p in (4, 5, 6) if (128, c, hw, hw, s, p) in plans)
            want = [4, 5, 6] if hw in (112, 56) or (hw == 28 and s == 1) else ([5] if hw == 28 else [])
            assert got == want, (c, hw, s, got)
    # the stride-2 passes need five source rows for two destination rows: no four-slot source ring on the sweep layers
    for key in ((128, 96, 112, 112, 2, 6), (128, 144, 56, 56, 2, 6), (128, 144, 56, 56, 2, 7), (128, 96, 112, 112, 2, 4)):
        assert plans[key][0] >= 5, (key, plans[key])
    g = cabi.geom((4, 64, 28, 28), (3, 3), (1, 1), (1, 1), (1, 1), (3, 3), 1)
    assert cabi.lib.dk_local_plan_query(g, cabi.DK_F16, 4, out) == 2          # scope other than 4 x 4: band kernels


def test_ring_slot_arithmetic_for_any_depth():
    """The row rings address fill k as slot k mod n, phase k / n, with k / n taken as the high word of k * ceil(2^32 / n)
    (csrc/dk_ring.cuh, `Ring::turn`): exact for every depth the planners can choose and every fill number a block can
    reach (rows per block are far below 2^22), including the largest k with k * n < 2^32."""
    for n in range(2, 33):
        magic = (2 ** 32 + n - 1) // n
        assert magic < 2 ** 32
        ks = list(range(0, 4096)) + [2 ** 22 - 1, 2 ** 22, 2 ** 22 + 1, 2 ** 32 // n - 1]
        ks += [m * n + d for m in (1, 7, 1000, 99999) for d in (-1, 0, 1)]
        for k in ks:
            turn = (k * magic) >> 32
            assert turn == k // n and k - turn * n == k % n, (n, k)


def test_cpu_tensors_raise_like_the_reference():
    import torch
    from deformable_kernels.ops.deform_kernel.functions import sample_depthwise, nd_linear_sample
    with pytest.raises(NotImplementedError):
        sample_depthwise(torch.randn(1, 2, 5, 5), torch.zeros(1, 18, 5, 5), torch.randn(2, 1, 4, 4))
    with pytest.raises(NotImplementedError):
        nd_linear_sample(torch.randn(3, 2, 2), torch.rand(4, 2))


def test_modules_keep_reference_names_and_shapes():
    import torch
    from deformable_kernels.modules import (DeformConv2d, DeformKernel2d, DeformKernelConv2d, GlobalDeformKernel2d,
                                            LocalDeformKernel2d)
    assert DeformKernel2d is LocalDeformKernel2d
    m = DeformKernel2d((4, 4), 8, 8, 3, 1, 1, groups=8, rotation_groups=2)
    sd = m.state_dict()
    assert sd["inner_conv.weight"].shape == (8, 1, 4, 4)
    assert sd["rotation_conv.weight"].shape == (2 * 9 * 2, 8, 3, 3) and "rotation_conv.bias" in sd
    assert float(sd["inner_conv.weight"].abs().max()) <= 1.0 / 3 + 1e-6
    m = DeformKernelConv2d((4, 4), 8, 8, 3, 2, 1, groups=8)
    assert m.state_dict()["offset_conv.weight"].shape == (18, 8, 3, 3)
    m = DeformConv2d(8, 8, 3, 1, 1, groups=8)
    assert m.state_dict()["inner_conv.weight"].shape == (8, 1, 3, 3)
    m = GlobalDeformKernel2d((2, 2), 8, 8, groups=8)
    assert set(m.state_dict()) == {"weight", "fc.weight", "fc.bias"}
    assert m.fc_bias == [0.5, 0.5]
    with pytest.raises(ValueError):
        DeformKernel2d((4, 4), 4, 4, 5, 1, 0, groups=4).inner_conv._output_size(torch.zeros(1, 4, 3, 3))


def test_reference_layers_import_unchanged_on_top_of_this_package():
    """The reference's own modules/deform_kernel.py and modules/deform_conv.py, loaded from
    the reference tree (or its staged copy) as they are, resolve their imports against this package's ops.
    tests/test_reference_layers_gpu.py runs their forward and backward on a GPU."""
    from oracle import build_ref
    mods = build_ref.load_layers()
    if mods is None:
        pytest.skip("neither the reference tree nor its staged layer files (oracle/_ref/ref_layers) are present")
    try:
        from deformable_kernels.ops.deform_kernel.modules import SampleDepthwise
        layer = mods["deform_kernel"].DeformKernel2d((4, 4), 8, 8, 3, 1, 1, groups=8)
        assert isinstance(layer.inner_conv, SampleDepthwise)
        assert set(layer.state_dict()) == {"rotation_conv.weight", "rotation_conv.bias", "inner_conv.weight"}
        import torch
        with pytest.raises(NotImplementedError):      # reaches this package's op, which has no CPU path
            layer(torch.randn(1, 8, 6, 6))
        assert mods["deform_conv"].DeformConv2d(8, 8, 3, 1, 1, groups=8).inner_conv.weight.shape == (8, 1, 3, 3)
    finally:
        import sys
        for k in [k for k in sys.modules if k.startswith("deformable_kernels._ref_layers")]:
            sys.modules.pop(k, None)
