"""The backward operators re-exported under the reference's names
(actnn/actnn/cpp_extension/backward_func.cc:81-91) and the conv / transposed-conv Functions
built on them, against PyTorch autograd (GPU).

Follows the reference's own tests/test_backward_func.py:212-385: same shapes, the forward
output and the three gradients of every convolution flavour are compared with ``F.conv*``.
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture()
def actnn(cuda_device):
    import actnn_b200
    from actnn_b200.conf import QuantizationConfig
    actnn_b200.config.__dict__.update(QuantizationConfig().__dict__)
    actnn_b200.set_optimization_level("L0")            # exact activations: gradients must match autograd
    tf32 = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False
    yield actnn_b200
    torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = tf32
    actnn_b200.config.__dict__.update(QuantizationConfig().__dict__)


def _run(func, data, weight, bias, *args):
    d = data.clone().requires_grad_()
    w = weight.clone().requires_grad_()
    b = bias.clone().requires_grad_()
    out = func(d, w, b, *args)
    out.backward(torch.ones_like(out))
    return out.detach(), d.grad, w.grad, b.grad


def _assert_same(ref, got, atol):
    for name, r, g in zip(("output", "grad_input", "grad_weight", "grad_bias"), ref, got):
        scale = max(1.0, float(r.abs().max()))
        assert float((r - g).abs().max()) <= atol * scale, name


CONV_CASES = [
    # dims, spatial, CI, CO, kernel, stride, padding, dilation, groups      (reference: test_backward_func.py:212-300)
    (1, (28,), 64, 128, 3, 1, 1, 1, 1),
    (2, (28, 28), 64, 128, 3, 1, 1, 1, 1),
    (3, (8, 8, 8), 16, 32, 3, 1, 1, 1, 1),
    (1, (30,), 8, 16, 5, 2, 2, 1, 2),                   # stride, groups
    (2, (17, 13), 12, 24, 3, 2, 0, 2, 3),               # ragged, dilation, groups
    (3, (6, 7, 5), 4, 8, 2, 1, 1, 1, 1),
]


@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: "conv%dd-%s" % (c[0], "x".join(map(str, c[1]))))
def test_conv_functions_match_autograd(actnn, cuda_device, case):
    dims, spatial, ci, co, k, stride, padding, dilation, groups = case
    g = torch.Generator().manual_seed(dims * 100 + ci)
    data = torch.randn(4, ci, *spatial, generator=g).to(cuda_device)
    weight = torch.randn(co, ci // groups, *([k] * dims), generator=g).to(cuda_device)
    bias = torch.rand(co, generator=g).to(cuda_device)
    stock = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[dims]
    ours = {1: actnn.ops.conv1d, 2: actnn.ops.conv2d, 3: actnn.ops.conv3d}[dims]
    ref = _run(stock, data, weight, bias, stride, padding, dilation, groups)
    got = _run(lambda d, w, b, *a: ours.apply(d, w, b, *a, None), data, weight, bias, stride, padding, dilation,
               groups)
    _assert_same(ref, got, 1e-4)


CONVT_CASES = [
    # dims, spatial, CI, CO, kernel, stride, padding, output_padding, groups, dilation   (test_backward_func.py:303-385)
    (1, (28,), 64, 32, 3, 1, 1, 0, 1, 1),
    (2, (14, 14), 64, 32, 3, 1, 1, 0, 1, 1),
    (3, (6, 6, 6), 16, 8, 3, 1, 1, 0, 1, 1),
    (1, (11,), 8, 12, 4, 2, 1, 1, 2, 1),                # stride with output padding, groups
    (2, (7, 9), 6, 9, 3, 2, 1, 1, 3, 1),
    (3, (4, 5, 3), 4, 6, 2, 2, 0, 0, 1, 1),
]


@pytest.mark.parametrize("case", CONVT_CASES, ids=lambda c: "convT%dd-%s" % (c[0], "x".join(map(str, c[1]))))
def test_conv_transpose_functions_match_autograd(actnn, cuda_device, case):
    dims, spatial, ci, co, k, stride, padding, output_padding, groups, dilation = case
    g = torch.Generator().manual_seed(dims * 1000 + ci)
    data = torch.randn(4, ci, *spatial, generator=g).to(cuda_device)
    weight = torch.randn(ci, co // groups, *([k] * dims), generator=g).to(cuda_device)
    bias = torch.rand(co, generator=g).to(cuda_device)
    stock = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[dims]
    ours = {1: actnn.ops.conv_transpose1d, 2: actnn.ops.conv_transpose2d, 3: actnn.ops.conv_transpose3d}[dims]
    ref = _run(stock, data, weight, bias, stride, padding, output_padding, groups, dilation)
    got = _run(lambda d, w, b, *a: ours.apply(d, w, b, *a, None), data, weight, bias, stride, padding,
               output_padding, groups, dilation)
    _assert_same(ref, got, 1e-4)


def test_reexported_convolution_backwards_directly(actnn, cuda_device):
    """``cudnn_convolution_backward`` / ``cudnn_convolution_transpose_backward`` with the reference's
    argument order (backward_func.cc:82-83) and its output_mask."""
    from actnn_b200.cpp_extension import backward_func as bf
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 6, 9, 9, generator=g).to(cuda_device).requires_grad_()
    w = torch.randn(8, 6, 3, 3, generator=g).to(cuda_device).requires_grad_()
    y = F.conv2d(x, w, None, 2, 1)
    gy = torch.randn_like(y)
    y.backward(gy)
    gi, gw = bf.cudnn_convolution_backward(x.detach(), gy, w.detach(), (1, 1), (2, 2), (1, 1), 1, False, False, False,
                                           [True, True])
    assert torch.allclose(gi, x.grad, atol=1e-4) and torch.allclose(gw, w.grad, atol=1e-4)
    gi, gw = bf.cudnn_convolution_backward(x.detach(), gy, w.detach(), (1, 1), (2, 2), (1, 1), 1, True, False, False,
                                           [True, False])
    assert torch.allclose(gi, x.grad, atol=1e-4) and gw is None

    xt = torch.randn(2, 6, 5, 5, generator=g).to(cuda_device).requires_grad_()
    wt = torch.randn(6, 4, 3, 3, generator=g).to(cuda_device).requires_grad_()
    yt = F.conv_transpose2d(xt, wt, None, 2, 1, 1)
    gyt = torch.randn_like(yt)
    yt.backward(gyt)
    gi, gw = bf.cudnn_convolution_transpose_backward(xt.detach(), gyt, wt.detach(), (1, 1), (1, 1), (2, 2), (1, 1), 1,
                                                     False, False, False, [True, True])
    assert torch.allclose(gi, xt.grad, atol=1e-4) and torch.allclose(gw, wt.grad, atol=1e-4)


@pytest.mark.parametrize("param_dtype", [torch.float16, torch.bfloat16])
def test_sync_batch_norm_halves_with_16_bit_affine_parameters(cuda_device, param_dtype):
    """``batch_norm_elemt`` / ``batch_norm_backward_reduce`` / ``batch_norm_backward_elemt`` when
    weight and bias are not float32 (a model moved with ``.half()``): the float32 copies the
    binding makes must stay alive across the call.  Against the ATen operators."""
    from actnn_b200.cpp_extension import backward_func as bf
    g = torch.Generator().manual_seed(11)
    N, C, H, W = 6, 20, 9, 7
    x = torch.randn(N, C, H, W, generator=g).to(param_dtype).to(cuda_device)
    gy = torch.randn(N, C, H, W, generator=g).to(param_dtype).to(cuda_device)
    w = (torch.rand(C, generator=g) + 0.5).to(param_dtype).to(cuda_device)
    b = torch.randn(C, generator=g).to(param_dtype).to(cuda_device)
    mean, invstd = torch.batch_norm_stats(x.float(), 1e-5)
    tol = 2e-3 if param_dtype == torch.float16 else 1.6e-2

    def close(a, ref, t=tol):
        return float((a.double() - ref.double()).abs().max()) <= t * max(1.0, float(ref.abs().max()))

    for _ in range(3):                      # repeated: a freed temporary would be reused by the next call
        y = bf.batch_norm_elemt(x, w, b, mean, invstd, 1e-5)
        y_t = torch.batch_norm_elemt(x.float(), w.float(), b.float(), mean, invstd, 1e-5)
        assert close(y, y_t)
        sum_dy, sum_dy_xmu, gw, gb = bf.batch_norm_backward_reduce(gy, x, mean, invstd, w, True, True, True)
        t = torch.batch_norm_backward_reduce(gy.float(), x.float(), mean, invstd, w.float(), True, True, True)
        assert close(sum_dy, t[0], 1e-3) and close(sum_dy_xmu, t[1], 1e-3)
        assert close(gw.float(), t[2]) and close(gb.float(), t[3])
        count = torch.tensor([N * H * W], dtype=torch.float32, device=cuda_device)
        dx = bf.batch_norm_backward_elemt(gy, x, mean, invstd, w, t[0], t[1], count)
        dx_t = torch.batch_norm_backward_elemt(gy.float(), x.float(), mean, invstd, w.float(), t[0], t[1], count.int())
        assert close(dx, dx_t)
