"""The training-step configuration (MobileNetV2 with every 3x3 depthwise convolution replaced by DeformKernel2d):
one forward + backward of the model through this library's kernels against the same model whose deformable-kernel
operator is played by the pure-PyTorch composition oracle, and the batch-split identity data parallelism relies on.
"""
import pytest
import torch

from dk_cases import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def exact_convolutions():
    old = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old


def _model():
    import bench
    torch.manual_seed(0)
    model, replaced = bench.build_mobilenet_dk()
    assert replaced == 17
    with torch.no_grad():      # offsets large enough to matter (bench initialises them at 0.01)
        for m in model.modules():
            if hasattr(m, "rotation_conv"):
                m.rotation_conv.weight.normal_(0, 0.05)
                m.rotation_conv.bias.normal_(0, 0.3)
    return model.to(DEV)


def _step(model, x, labels):
    model.zero_grad(set_to_none=True)
    torch.manual_seed(1234)      # the classifier's dropout draws the same mask in both runs
    loss = torch.nn.functional.cross_entropy(model(x), labels)
    loss.backward()
    grads = {n: p.grad.detach().clone() for n, p in model.named_parameters()
             if ("inner_conv.weight" in n or "rotation_conv.weight" in n) and p.grad is not None}
    return float(loss.detach()), grads


def test_mobilenet_dk_step_matches_the_composition(monkeypatch):
    """fp32, batch 4, 96 x 96 images: loss and the gradients of all 17 weight banks and offset-producing convolutions
    agree with the run in which sample_depthwise is oracle/torch_composition.py.  Batch-norm uses its running statistics:
    with batch statistics of four images this random-init network amplifies fp32 rounding differences 3-4x per block
    (measured: 1e-7 after the first deformable layer, order 1 after the twelfth, with either operator), so nothing
    could be compared."""
    from deformable_kernels.ops.deform_kernel.modules import filter_sample_depthwise as wrapper
    from oracle import torch_composition as TC
    model = _model().eval()
    x = torch.randn(4, 3, 96, 96, device=DEV)
    labels = torch.randint(0, 1000, (4,), device=DEV)
    loss_mine, g_mine = _step(model, x, labels)

    def composed(input, rotation, weight, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1), dilation=(1, 1), rotation_groups=1):
        y = TC.sample_depthwise(input.cpu(), rotation.cpu(), weight.cpu(), kernel_size, stride, padding, dilation, rotation_groups)
        return y.to(input.device)

    monkeypatch.setattr(wrapper, "sample_depthwise", composed)
    loss_ref, g_ref = _step(model, x, labels)
    assert abs(loss_mine - loss_ref) < 1e-4 * max(1.0, abs(loss_ref))
    assert len(g_mine) == 34 and set(g_mine) == set(g_ref)
    for name in g_mine:
        assert rel_err(g_mine[name], g_ref[name]) < 1e-4, name


def test_bank_gradients_of_batch_halves_add_up_to_the_full_batch():
    """What data parallelism relies on: per-sample outputs of the two batch halves concatenate to the full-batch result
    and the two partial bank gradients sum to the full-batch bank gradient (fp16 tensor-core path and fp32)."""
    from deformable_kernels.ops.deform_kernel.functions import sample_depthwise
    from deformable_kernels.sharding import shard_batch
    from dk_cases import make_case
    for dtype, tol, c, hw in ((torch.float16, 2e-3, 96, 56), (torch.float32, 1e-5, 24, 20)):
        case = make_case(6, c, hw, hw, rot_std=1.0, seed=80)
        full = [case[k].to(dtype).to(DEV) for k in ("input", "rotation", "grad_output")]
        w = case["weight"].to(dtype).to(DEV)

        def run(x, r, dy):
            x, r, ww = x.clone().requires_grad_(True), r.clone().requires_grad_(True), w.clone().requires_grad_(True)
            y = sample_depthwise(x, r, ww, **case["args"])
            return (y.detach(),) + torch.autograd.grad(y, [x, r, ww], dy)

        y, gx, gr, gw = run(*full)
        parts = [run(*shard_batch(full, rank, 2)) for rank in range(2)]
        assert rel_err(torch.cat([p[0] for p in parts]), y) < tol
        assert rel_err(torch.cat([p[1] for p in parts]), gx) < tol
        assert rel_err(torch.cat([p[2] for p in parts]), gr) < tol
        assert rel_err(parts[0][3].float() + parts[1][3].float(), gw) < tol
