"""The Python layer on a GPU: quantize_activation / dequantize_activation against the
reference-generated fixtures, the schemes, the Q-layers and QModule."""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import actnn_oracle as O
from conftest import DTYPES, from_raw, load_cases, same_values

pytestmark = pytest.mark.gpu

ACT = load_cases("quantize_activation")


@pytest.fixture()
def actnn(cuda_device):
    import actnn_b200
    from actnn_b200.conf import QuantizationConfig
    fresh = QuantizationConfig()
    actnn_b200.config.__dict__.update(fresh.__dict__)
    actnn_b200.QScheme.layers.clear()
    actnn_b200.QBNScheme.layers.clear()
    actnn_b200.QScheme.prev_layer = None
    actnn_b200.config.perlayer = False
    yield actnn_b200
    actnn_b200.config.__dict__.update(fresh.__dict__)


def philox_state():
    torch.cuda.init()                                   # the generators exist only once CUDA is up
    gen = torch.cuda.default_generators[torch.cuda.current_device()]
    return gen.initial_seed(), gen.get_offset()


@pytest.mark.parametrize("case", sorted(ACT))
def test_quantize_activation_against_reference_fixtures(actnn, case):
    """Same inputs as the reference run; the noise is this library's Philox stream replayed on
    the CPU, so codes are compared with the oracle and bits / statistics with the fixture."""
    f = ACT[case]
    _, dname, which, shape = case.split("_")
    dt = DTYPES[dname]
    shape = tuple(int(s) for s in shape.split("x"))
    x = from_raw(f["x"], dt).view(shape)
    stat_dt = torch.bfloat16 if dt == torch.float32 else dt
    cfg = actnn.config
    if which == "conv":
        cfg.activation_compression_bits = [2, 8, 8]
        scheme = actnn.QScheme(None, num_locations=9)
        scheme.scales = torch.tensor(0.37)
    elif which == "bn":
        cfg.activation_compression_bits = [2, 8, 8]
        scheme = actnn.QBNScheme()
    else:
        cfg.activation_compression_bits = [4]
        scheme = None
    torch.manual_seed(5)
    seed, offset = philox_state()
    q = actnn.ops.quantize_activation(x.cuda(), scheme)
    q_input, q_bits, q_scale, q_min = q

    groups = O.to_groups(x)
    n, g, _ = groups.shape
    noise = O.philox_noise(groups.numel(), dt, seed, offset).view(groups.shape)
    mn, mx = O.group_minimax(groups)
    if scheme is None:
        assert q_bits == 4
        codes, oscale = O.quantize(groups, 4, mn, mx, noise)
        assert np.array_equal(q_input.cpu().numpy(), O.pack_single_layout(codes, 4))
    else:
        assert np.array_equal(q_bits.cpu().numpy(), f["bits"])          # the reference's greedy result
        if which == "conv":
            assert torch.allclose(scheme.C.cpu(), torch.from_numpy(f["C"]), rtol=3e-3)
        codes, oscale = O.quantize(groups, q_bits.cpu(), mn, mx, noise)
        assert np.array_equal(q_input.cpu().numpy(), O.pack_mixed_layout(codes, q_bits.cpu()))
    assert q_scale.dtype == stat_dt and q_min.dtype == stat_dt
    assert same_values(q_scale.cpu(), from_raw(f["scale"], stat_dt))    # independent of the noise
    assert same_values(q_min.cpu(), from_raw(f["min"], stat_dt))
    out = actnn.ops.dequantize_activation(q, shape, dt)
    expect = O.dequantize_activation((codes, None, oscale.to(stat_dt), mn.to(stat_dt)), shape, dtype=dt)
    assert out.dtype == dt and out.shape == shape and same_values(out.cpu(), expect)
    ref = from_raw(f["deq"], torch.float32 if dt == torch.bfloat16 else dt).view(shape).float()
    step = (mx.float() - mn.float()).max() / 1.0 + 1e-3                  # coarse: within one range
    assert float((out.cpu().float() - ref).abs().max()) <= float(step)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_conv2d_cuda_path_matches_simulate_path(actnn, dtype):
    """The reference's own differential test (tests/test_act_quantized_ops.py:360-400), at 8
    bits: outputs and gradients of conv2d.apply with config.simulate on and off agree."""
    cfg = actnn.config
    cfg.activation_compression_bits = [8]
    cfg.initial_bits = 8
    N, H, W, CI, CO = 4, 28, 28, 64, 64
    g = torch.Generator().manual_seed(0)
    data = torch.randn(N, CI, H, W, generator=g).to(dtype)
    weight = (torch.randn(CO, CI, 3, 3, generator=g) * 0.05).to(dtype)
    bias = torch.randn(CO, generator=g).to(dtype)
    scheme = actnn.QScheme(None)

    def run(simulate):
        cfg.simulate = simulate
        torch.manual_seed(0)
        d = data.cuda().requires_grad_()
        w = weight.cuda().requires_grad_()
        b = bias.cuda().requires_grad_()
        out = actnn.ops.conv2d.apply(d, w, b, 1, 1, 1, 1, scheme)
        out.backward(torch.ones_like(out))
        return [t.detach().float().cpu() for t in (out, d.grad, w.grad, b.grad)]

    ref, us = run(True), run(False)
    cfg.simulate = False
    for a, b in zip(ref, us):
        assert torch.allclose(a, b, rtol=2e-2, atol=2e-2 * float(a.abs().max()))


def test_qmodule_training_step_matches_exact_training_closely(actnn):
    """8-bit activations: gradients of a small CNN stay close to exact training."""
    torch.manual_seed(0)
    net = nn.Sequential(nn.Conv2d(3, 16, 3, padding=1), nn.BatchNorm2d(16), nn.ReLU(), nn.MaxPool2d(3, 2, 1),
                        nn.Conv2d(16, 32, 3, padding=1), nn.BatchNorm2d(32), nn.ReLU(),
                        nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(32, 10)).cuda()
    import copy
    exact = copy.deepcopy(net)
    actnn.config.activation_compression_bits = [8, 8, 8]
    q = actnn.QModule(net)
    q.train()
    exact.train()
    x = torch.randn(16, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (16,), device="cuda")
    F.cross_entropy(q(x), y).backward()
    F.cross_entropy(exact(x), y).backward()
    for (name, p), pe in zip(q.model.named_parameters(), exact.parameters()):
        assert p.grad is not None, name
        if float(pe.grad.norm()) < 1e-5:          # conv bias in front of batch norm: exact gradient is ~0
            continue
        err = (p.grad - pe.grad).norm() / (pe.grad.norm() + 1e-12)
        assert float(err) < 0.15, (name, float(err))
    # state dicts interchange with the unwrapped model
    assert set(q.state_dict().keys()) == set(exact.state_dict().keys())
    q.load_state_dict(exact.state_dict())
    q.eval()
    assert actnn.config.training is False
    with torch.no_grad():
        assert torch.allclose(q(x), exact.eval()(x), atol=1e-5)


@pytest.mark.parametrize("level", ["L0", "L1", "L2", "L3", "L4"])
def test_optimization_levels_train(actnn, level):
    actnn.set_optimization_level(level)
    actnn.config.perlayer = True
    torch.manual_seed(1)
    net = nn.Sequential(nn.Conv2d(4, 16, 3, padding=1), nn.BatchNorm2d(16), nn.ReLU(),
                        nn.Conv2d(16, 16, 3, padding=1), nn.BatchNorm2d(16), nn.ReLU(),
                        nn.Flatten(), nn.Linear(16 * 16 * 16, 5))
    q = actnn.QModule(net).cuda()
    q.train()
    opt = torch.optim.SGD(q.parameters(), lr=0.01, momentum=0.9)
    x = torch.randn(8, 4, 16, 16, device="cuda")
    y = torch.randint(0, 5, (8,), device="cuda")
    losses = []
    for _ in range(4):
        opt.zero_grad()
        loss = F.cross_entropy(q(x), y)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert all(np.isfinite(losses)) and losses[-1] < losses[0]


def test_saved_activation_is_smaller(actnn):
    """Compressed conv input at 2 bits + statistics takes about 1/7 of the float16 tensor."""
    x = torch.randn(32, 64, 28, 28, device="cuda", dtype=torch.float16)
    actnn.config.activation_compression_bits = [2, 8, 8]
    scheme = actnn.QScheme(None, num_locations=9)
    q = actnn.ops.quantize_activation(x, scheme)
    saved = actnn.compute_tensor_bytes([q[0], q[2], q[3]])
    ratio = x.numel() * 2 / saved
    assert 6.5 < ratio < 8.0, ratio
    assert int(q[1].sum()) == 2 * 32


def test_bf16_activation_round_trip(actnn):
    x = torch.randn(8, 32, 16, 16, device="cuda").relu().to(torch.bfloat16)
    actnn.config.activation_compression_bits = [4]
    q = actnn.ops.quantize_activation(x, None)
    y = actnn.ops.dequantize_activation(q, x.shape, x.dtype)
    assert y.dtype == torch.bfloat16
    groups = x.view(8, -1, 256).float()
    rng = (groups.max(2, keepdim=True)[0] - groups.min(2, keepdim=True)[0])
    err = (y.view(8, -1, 256).float() - groups).abs()
    assert bool((err <= rng / 15 * 1.02 + 1e-2 * groups.abs() + 1e-3).all())


def test_autocast_conv_runs_in_half(actnn):
    conv = actnn.QConv2d(8, 8, 3, padding=1).cuda()
    actnn.config.training = True
    x = torch.randn(4, 8, 16, 16, device="cuda", requires_grad=True)
    with torch.autocast("cuda", dtype=torch.float16):
        y = conv(x)
    assert y.dtype == torch.float16
    y.float().sum().backward()
    assert x.grad is not None and conv.weight.grad is not None and conv.weight.grad.dtype == torch.float32


# ------------------------------------------------------------------------------ per-layer widths
PERLAYER = load_cases("perlayer")


@pytest.mark.parametrize("case", sorted(PERLAYER))
def test_allocate_perlayer_matches_the_reference(actnn, case):
    """``QScheme.allocate_perlayer`` / ``QBNScheme.allocate_perlayer`` against the widths the
    reference's own code produced for the same sensitivities (qscheme.py:96-128,
    qbnscheme.py:54-60): the joint allocation over layers x samples, the one-width-per-layer
    branch (group bits == initial bits) and the batch norms that follow their conv layer."""
    f = PERLAYER[case]
    group_bits, initial_bits = (int(v) for v in f["cfg"])
    actnn.config.perlayer = True
    actnn.config.activation_compression_bits = [group_bits]
    actnn.config.initial_bits = initial_bits
    actnn.QScheme.layers.clear()
    actnn.QBNScheme.layers.clear()
    follows = set(int(i) for i in f["bn_follows"])
    bns = []
    for i in range(f["C"].shape[0]):
        layer = actnn.QScheme(None)
        layer.C = torch.from_numpy(f["C"][i]).cuda()
        layer.dim = int(f["dims"][i])
        if i in follows:
            bns.append(actnn.QBNScheme())
    actnn.QScheme.allocate_perlayer()
    actnn.QBNScheme.allocate_perlayer()
    got = np.array([float(layer.bits) for layer in actnn.QScheme.layers], dtype=np.float32)
    assert np.array_equal(got, f["bits"])
    assert np.array_equal(np.array([float(b.bits) for b in bns], dtype=np.float32), f["bn_bits"])
    if group_bits == initial_bits:                       # that branch also moves the starting width
        assert [int(layer.initial_bits) for layer in actnn.QScheme.layers] == [int(b) for b in f["bits"]]
    actnn.QScheme.layers.clear()
    actnn.QBNScheme.layers.clear()


def test_a_layer_allocated_one_bit_still_compresses(actnn):
    """The one-width-per-layer branch can hand a layer 1 bit as its STARTING width
    (``layer.initial_bits = b[i]``, qscheme.py:111); the reference's greedy then returns all
    ones.  The compress must accept that instead of failing in the middle of training."""
    actnn.config.activation_compression_bits = [1]
    actnn.config.initial_bits = 1
    layer = actnn.QScheme(None)
    x = torch.randn(6, 8, 16, 16, device="cuda")
    q = actnn.ops.quantize_activation(x, layer)
    assert q[1].tolist() == [1] * 6
    y = actnn.ops.dequantize_activation(q, x.shape, x.dtype)
    assert torch.isfinite(y).all()
    groups, b, _, _ = layer.compute_quantization_bits(x)
    assert b.tolist() == [1] * 6


# ------------------------------------------------------------------------------ ReLU that also yields the group ranges
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(6, 16, 16, 16), (3, 1024), (5, 256), (1, 2, 8, 16)])
def test_relu_with_minmax_equals_minimax_of_its_output(actnn, dtype, shape):
    from actnn_b200.cpp_extension import minimax, quantization as q
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=g).to(dtype).cuda()
    x.view(-1)[3] = float("nan")                                   # decodes to 0 like every non-positive input
    y0, mask0 = q.relu_forward(x)
    y, mask, mn, mx = q.relu_forward(x, with_minmax=True)
    assert torch.equal(y, y0) and torch.equal(mask, mask0)
    rmn, rmx = minimax.minimax(y.view(-1, 256))
    assert torch.equal(mn, rmn.view(-1)) and torch.equal(mx, rmx.view(-1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_conv_after_relu_compresses_the_same_with_and_without_the_relu_ranges(actnn, dtype):
    """QReLU -> QConv2d at level L3: with ``config.relu_minmax`` the convolution takes the ranges
    from the ReLU pass (one read of its input instead of two); what it saves, what it returns and
    what it computes must be bit-identical to the two-read path."""
    actnn.set_optimization_level("L3")
    torch.manual_seed(0)
    relu, first = actnn.QReLU(), actnn.QConv2d(16, 8, 3, padding=1).cuda().to(dtype)
    weights = first.state_dict()
    x0 = torch.randn(6, 16, 16, 16, device="cuda", dtype=dtype)
    gy = torch.randn(6, 8, 16, 16, device="cuda", dtype=dtype)
    gen = torch.cuda.default_generators[torch.cuda.current_device()]
    results = []
    for flag in (True, False):
        actnn.config.relu_minmax = flag
        actnn.QScheme.layers.clear()                             # a fresh layer: the per-layer widths adapt after a step
        conv = actnn.QConv2d(16, 8, 3, padding=1).cuda().to(dtype)
        conv.load_state_dict(weights)
        conv.scheme.scales = torch.tensor(0.37)
        gen.manual_seed(123)
        x = x0.clone().requires_grad_(True)
        h = relu(x)
        assert hasattr(h, "actnn_minmax") == flag
        saved = {}
        from actnn_b200 import ops
        real = ops.quantize_activation

        def spy(inp, scheme, minmax=None):
            out = real(inp, scheme, minmax=minmax)
            saved["minmax_used"] = minmax is not None
            saved["q"] = [t.clone() if isinstance(t, torch.Tensor) else t for t in out]
            return out

        ops.quantize_activation = spy
        try:
            y = conv(h)
        finally:
            ops.quantize_activation = real
        assert saved["minmax_used"] == flag
        y.backward(gy)
        results.append((y.detach(), x.grad, conv.weight.grad, *saved["q"]))
    for i, (a, b) in enumerate(zip(*results)):
        if i in (1, 2):            # gradients come from cuDNN, whose algorithm choice may differ between two calls
            assert torch.allclose(a.float(), b.float(), rtol=1e-4, atol=1e-5)
        else:
            assert torch.equal(a, b)
