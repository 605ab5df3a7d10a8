"""Does the library's rounding noise behave like independent noise where it matters?

The reference checks its quantizer by the bias and the spread of a layer's weight gradient
over repeated draws (tests/test_conv_layer.py:10-39: ten draws, ``|mean(dW) - dW_true|`` and
``|std(dW)|``).  The same protocol here, twice: with the noise the kernels generate (one
Philox4x32-10 call stretched to eight words, one byte per element for 16-bit activations) and
with independent ``uniform(-0.5, 0.5)`` noise injected through the ``noise=`` argument.  The two
must agree: same spread (second-order statistics are what pairwise independence guarantees)
and a bias that is sampling error, not a systematic offset.
"""
import json

import pytest
import torch

pytestmark = pytest.mark.gpu

DRAWS = 48


def _weight_grad(x, gy, w):
    _, gw, _ = torch.ops.aten.convolution_backward(gy, x, w, None, [1, 1], [1, 1], [1, 1], False, [0, 0], 1,
                                                   [False, True, False])
    return gw.float()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_weight_gradient_bias_and_spread_match_independent_noise(cuda_device, dtype):
    from actnn_b200.cpp_extension import minimax, quantization as q
    g = torch.Generator(device=cuda_device).manual_seed(0)
    N, C, H, W, K = 10, 32, 28, 28, 16
    x = torch.relu(torch.randn(N, C, H, W, device=cuda_device, generator=g)).to(dtype)
    w = (torch.randn(K, C, 3, 3, device=cuda_device, generator=g) * 0.05).to(dtype)
    gy = (torch.randn(N, K, H, W, device=cuda_device, generator=g) * 1e-2).to(dtype)
    true = _weight_grad(x, gy, w)
    groups = x.view(N, -1, 256)
    mn, mx = minimax.minimax(groups.view(-1, 256))
    mn, mx = mn.view(N, -1, 1), mx.view(N, -1, 1)

    def draws(make_noise_args):
        grads = []
        for i in range(DRAWS):
            packed, scale = q.pack_single_precision(groups, mn, mx, 2, True, **make_noise_args(i))
            xh = q.unpack_single_precision(packed, 2, scale, mn, N, groups.shape[1], 256).view_as(x)
            grads.append(_weight_grad(xh, gy, w))
        grads = torch.stack(grads)
        return float((grads.mean(0) - true).norm()), float(grads.std(0).norm())

    lib_bias, lib_std = draws(lambda i: {"philox": (1234, 4 * i)})
    ind_bias, ind_std = draws(lambda i: {"noise": (torch.rand(groups.shape, device=cuda_device, generator=g) - 0.5)
                                         .to(dtype)})
    report = {"dtype": str(dtype), "draws": DRAWS, "grad_norm": float(true.norm()), "library_bias": lib_bias,
              "library_std": lib_std, "independent_bias": ind_bias, "independent_std": ind_std}
    print(json.dumps(report))
    # same spread as independent noise (the estimate of a norm of standard deviations over 48 draws
    # is good to a few per cent)
    assert abs(lib_std - ind_std) <= 0.08 * ind_std
    # the bias of the mean over DRAWS draws is sampling error: about std / sqrt(DRAWS), for both
    expected = ind_std / DRAWS ** 0.5
    assert lib_bias <= 1.5 * expected and ind_bias <= 1.5 * expected
