"""The reference's own layer classes, unmodified, running forward and backward on a GPU on top of this
package's operators, and the known-answer reduction of DeformConv2d to torchvision's deform_conv2d.

The layer files (deformable_kernels/modules/deform_kernel.py, deform_conv.py of the reference) are loaded
from the reference tree when it is present, else from the copy that oracle/build_ref.py stages under
oracle/_ref/ref_layers/ (git-ignored build output, like the reference's compiled extension beside it).
Each layer's result is compared with the pure-PyTorch composition oracle (oracle/torch_composition.py) given
the layer's own parameters (evaluated on the CPU in fp64, offset-producing convolution / linear layer included).
"""
import pytest
import torch
import torch.nn.functional as F

from dk_cases import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ref_layers():
    from oracle import build_ref
    mods = build_ref.load_layers()
    if mods is None:
        pytest.skip("the reference's layer files are on neither this machine's reference tree nor oracle/_ref/ref_layers "
                    "(staged by oracle/build_ref.py where the tree exists)")
    return mods


@pytest.fixture(autouse=True)
def exact_convolutions():
    """The offset-producing convolutions are stock cuDNN; keep them in full fp32 so that both sides see the same offsets."""
    old = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old


def _grads(y, dy, tensors):
    return torch.autograd.grad(y, tensors, dy)


def test_reference_local_layer_forward_backward(ref_layers):
    from oracle import torch_composition as TC
    torch.manual_seed(0)
    layer = ref_layers["deform_kernel"].DeformKernel2d((4, 4), 32, 32, 3, 2, 1, groups=32).to(DEV)
    with torch.no_grad():
        layer.rotation_conv.weight.normal_(0, 0.15)
        layer.rotation_conv.bias.normal_(0, 0.3)
    x = torch.randn(3, 32, 20, 18, device=DEV, requires_grad=True)
    y = layer(x)
    dy = torch.randn_like(y)
    params = [x, layer.inner_conv.weight, layer.rotation_conv.weight]
    got = _grads(y, dy, params)
    x2 = x.detach().cpu().double().requires_grad_(True)
    w2 = layer.inner_conv.weight.detach().cpu().double().requires_grad_(True)
    rw2 = layer.rotation_conv.weight.detach().cpu().double().requires_grad_(True)
    rot = F.conv2d(x2, rw2, layer.rotation_conv.bias.detach().cpu().double(), 2, 1)
    y2 = TC.sample_depthwise(x2, rot, w2, (3, 3), (2, 2), (1, 1), (1, 1), 1)
    want = _grads(y2, dy.cpu().double(), [x2, w2, rw2])
    assert rel_err(y, y2) < 1e-5
    for a, b, name in zip(got, want, ("grad x", "grad bank", "grad offset-conv weight")):
        assert rel_err(a, b) < 2e-5, name


def test_reference_dcn_layers_forward_backward(ref_layers):
    from oracle import torch_composition as TC
    torch.manual_seed(1)
    for cls, scope in ((ref_layers["deform_kernel"].DeformKernelConv2d, (4, 4)), (ref_layers["deform_conv"].DeformConv2d, None)):
        layer = (cls((4, 4), 16, 16, 3, 1, 1, groups=16) if scope else cls(16, 16, 3, 1, 1, groups=16)).to(DEV)
        with torch.no_grad():
            layer.offset_conv.weight.normal_(0, 0.2)
            layer.offset_conv.bias.normal_(0, 0.5)
        x = torch.randn(2, 16, 13, 15, device=DEV, requires_grad=True)
        y = layer(x)
        dy = torch.randn_like(y)
        got = _grads(y, dy, [x, layer.inner_conv.weight, layer.offset_conv.weight])
        x2 = x.detach().cpu().double().requires_grad_(True)
        w2 = layer.inner_conv.weight.detach().cpu().double().requires_grad_(True)
        ow2 = layer.offset_conv.weight.detach().cpu().double().requires_grad_(True)
        off = F.conv2d(x2, ow2, layer.offset_conv.bias.detach().cpu().double(), 1, 1)
        rot = torch.zeros(2, 18, 13, 15, dtype=torch.float64)
        y2 = TC.deform_sample_depthwise(x2, off, rot, w2, (3, 3), (1, 1), (1, 1), (1, 1), 1)
        want = _grads(y2, dy.cpu().double(), [x2, w2, ow2])
        assert rel_err(y, y2) < 1e-5, cls.__name__
        for a, b, name in zip(got, want, ("grad x", "grad bank", "grad offset-conv weight")):
            assert rel_err(a, b) < 2e-5, (cls.__name__, name)


def test_reference_global_layer_forward_backward(ref_layers):
    from oracle import torch_composition as TC
    torch.manual_seed(2)
    layer = ref_layers["deform_kernel"].GlobalDeformKernel2d((3, 3), 24, 24, kernel_size=1, groups=24).to(DEV)
    with torch.no_grad():
        layer.weight.normal_(0, 0.5)        # the reference leaves this parameter uninitialised
        layer.fc.weight.normal_(0, 0.4)
    x = torch.randn(5, 24, 9, 9, device=DEV, requires_grad=True)
    y = layer(x)
    dy = torch.randn_like(y)
    got = _grads(y, dy, [x, layer.weight, layer.fc.weight])
    x2 = x.detach().cpu().double().requires_grad_(True)
    w2 = layer.weight.detach().cpu().double().requires_grad_(True)
    fw2 = layer.fc.weight.detach().cpu().double().requires_grad_(True)
    coord = F.linear(x2.view(5, 24, -1).mean(2), fw2, layer.fc.bias.detach().cpu().double()) + torch.tensor(
        layer.fc_bias, dtype=torch.float64).unsqueeze(0)
    coord = torch.clamp(coord, 0, 2)
    k = TC.nd_linear_sample(w2.view(24, 3, 3), coord.view(5, 2))   # [5, 24]: the per-sample 1x1 depthwise kernel
    y2 = x2 * k.view(5, 24, 1, 1)
    want = _grads(y2, dy.cpu().double(), [x2, w2, fw2])
    assert rel_err(y, y2) < 1e-5
    for a, b, name in zip(got, want, ("grad x", "grad bank", "grad fc weight")):
        assert rel_err(a, b) < 2e-5, name


@pytest.mark.parametrize("stride", [1, 2])
def test_deform_conv2d_reduces_to_torchvision(stride):
    """Scope == kernel and no kernel-space offsets: the operator is torchvision.ops.deform_conv2d with one offset group
    (same [N, 2 k^2, Ho, Wo] (h, w)-interleaved offsets, same -1 < position < size rule), values and all three
    gradients, including the one with respect to the offsets.  torchvision runs on the CPU in fp64."""
    import torchvision
    from deformable_kernels.ops.deform_kernel.functions import deform_sample_depthwise
    torch.manual_seed(3)
    c, h, w = 12, 11, 14
    ho, wo = (h + 2 - 3) // stride + 1, (w + 2 - 3) // stride + 1
    x = torch.randn(2, c, h, w, dtype=torch.float64)
    wt = torch.randn(c, 1, 3, 3, dtype=torch.float64) * 0.4
    off = torch.randn(2, 18, ho, wo, dtype=torch.float64) * 2.0
    dy = torch.randn(2, c, ho, wo, dtype=torch.float64)
    ref_in = [t.clone().requires_grad_(True) for t in (x, off, wt)]
    want_y = torchvision.ops.deform_conv2d(ref_in[0], ref_in[1], ref_in[2], stride=stride, padding=1)
    want = torch.autograd.grad(want_y, ref_in, dy)
    for dtype, tol in ((torch.float64, 1e-11), (torch.float32, 1e-5)):
        mine_in = [t.to(dtype).to(DEV).requires_grad_(True) for t in (x, off, wt)]
        y = deform_sample_depthwise(mine_in[0], mine_in[1], None, mine_in[2], (3, 3), (stride, stride), (1, 1), (1, 1), 1)
        got = torch.autograd.grad(y, mine_in, dy.to(dtype).to(DEV))
        assert rel_err(y, want_y) < tol
        for a, b, name in zip(got, want, ("grad x", "grad offsets", "grad weight")):
            assert rel_err(a, b) < tol, (dtype, name)
