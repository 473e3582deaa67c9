#!/usr/bin/env python3
"""Build the reference's own CUDA extensions, unmodified, into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file or
anything it produces; only tests/, the golden-vector generator and bench.py's
reference-on-GPU side measurement load the two modules built here.

The reference sources are compiled where they lie (no copy is made, nothing is
patched).  The only help they get is ``ref_compat.h``, force-included ahead of
each translation unit, which restores one ATen overload that PyTorch 1.3 had and
current PyTorch dropped (the 9 + 3 ``AT_DISPATCH_...(x.type(), ...)`` sites in
csrc/filter_sample_depthwise_cuda_kernel.cu and csrc/nd_linear_sample_cuda_kernel.cu).

Outputs (git-ignored):
    oracle/_ref/filter_sample_depthwise_cuda.so   9 pybind functions, csrc/filter_sample_depthwise_cuda.cpp:540-569
    oracle/_ref/nd_linear_sample_cuda.so          3 pybind functions, csrc/nd_linear_sample_cuda.cpp:67-74

Usage:  python oracle/build_ref.py [reference_root]
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
EXTS = {
    "filter_sample_depthwise_cuda": [
        "csrc/filter_sample_depthwise_cuda.cpp",
        "csrc/filter_sample_depthwise_cuda_kernel.cu",
    ],
    "nd_linear_sample_cuda": [
        "csrc/nd_linear_sample_cuda.cpp",
        "csrc/nd_linear_sample_cuda_kernel.cu",
    ],
}


def reference_root(arg=None):
    return arg or os.environ.get("DK_REFERENCE_ROOT", "/root/reference")


def built(name):
    return os.path.join(OUT, name + ".so")


def build(root=None, verbose=False):
    """Compile both reference extensions for sm_100.  Returns the list of .so
    paths; raises if the reference tree is missing."""
    root = reference_root(root)
    csrc_root = os.path.join(root, "deformable_kernels", "ops", "deform_kernel")
    if not os.path.isdir(csrc_root):
        raise FileNotFoundError("reference tree not found at %s" % root)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils.cpp_extension import load

    compat = os.path.join(HERE, "ref_compat.h")
    outs = []
    for name, rel in EXTS.items():
        bdir = os.path.join(OUT, "_build_" + name)
        os.makedirs(bdir, exist_ok=True)
        srcs = [os.path.join(csrc_root, r) for r in rel]
        if os.path.exists(built(name)) and all(
            os.path.getmtime(built(name)) >= os.path.getmtime(s) for s in srcs + [compat]
        ):
            outs.append(built(name))
            continue
        load(
            name=name,
            sources=srcs,
            extra_cflags=["-O2", "-include", compat, "-w"],
            extra_cuda_cflags=["-O2", "-include", compat, "-w"],
            extra_include_paths=[os.path.join(csrc_root, "csrc")],
            build_directory=bdir,
            is_python_module=False,
            verbose=verbose,
        )
        src_so = os.path.join(bdir, name + ".so")
        os.replace(src_so, built(name))
        outs.append(built(name))
    return outs


LAYER_FILES = ("deform_kernel.py", "deform_conv.py")


def stage_layers(root=None):
    """Install the reference's two layer files (deformable_kernels/modules/deform_kernel.py and deform_conv.py) unmodified
    under oracle/_ref/ref_layers/, the way `pip install --target` would, so that the GPU tests can run the reference's own
    layers on top of this package's operators on a machine without the reference tree.  oracle/_ref/ is git-ignored."""
    import shutil
    src = os.path.join(reference_root(root), "deformable_kernels", "modules")
    if not os.path.isdir(src):
        raise FileNotFoundError("reference tree not found at %s" % reference_root(root))
    dst = os.path.join(OUT, "ref_layers")
    os.makedirs(dst, exist_ok=True)
    for f in LAYER_FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
    return dst


def layers_dir():
    """Directory holding the reference's layer files: the reference tree when present, else the staged copy, else None."""
    live = os.path.join(reference_root(), "deformable_kernels", "modules")
    if all(os.path.exists(os.path.join(live, f)) for f in LAYER_FILES):
        return live
    staged = os.path.join(OUT, "ref_layers")
    if all(os.path.exists(os.path.join(staged, f)) for f in LAYER_FILES):
        return staged
    return None


def load_layers():
    """The reference's layer modules, imported unchanged on top of this package's operators ({'deform_kernel': module,
    'deform_conv': module}), or None when neither the tree nor the staged copy is present.  `apex` is not installed here:
    a stand-in for apex.amp.float_function (the identity, which is what it is while amp is uninitialised) is put in
    sys.modules for the duration of the import."""
    import importlib.util
    import types
    mod_dir = layers_dir()
    if mod_dir is None:
        return None
    import deformable_kernels  # noqa: F401  (this package: the ops the layers import)
    amp = types.ModuleType("apex.amp")
    amp.float_function = lambda f: f
    apex = types.ModuleType("apex")
    apex.amp = amp
    saved = {k: sys.modules.get(k) for k in ("apex", "apex.amp")}
    sys.modules["apex"], sys.modules["apex.amp"] = apex, amp
    try:
        pkg = types.ModuleType("deformable_kernels._ref_layers")
        pkg.__path__ = [mod_dir]
        sys.modules["deformable_kernels._ref_layers"] = pkg
        mods = {}
        for name in ("deform_kernel", "deform_conv"):
            full = "deformable_kernels._ref_layers." + name
            spec = importlib.util.spec_from_file_location(full, os.path.join(mod_dir, name + ".py"))
            mod = importlib.util.module_from_spec(spec)
            sys.modules[full] = mod
            spec.loader.exec_module(mod)
            mods[name] = mod
        return mods
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def load_module(name):
    """Import one of the built pybind modules from oracle/_ref/ (torch must be
    imported first so that its shared libraries are resolvable)."""
    import importlib.util
    import torch  # noqa: F401

    path = built(name)
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    for p in build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True):
        print("built", p)
    print("staged", stage_layers(sys.argv[1] if len(sys.argv) > 1 else None))
