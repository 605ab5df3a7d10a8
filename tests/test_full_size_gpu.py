"""The benchmark configurations at their full sizes (GPU).

The CPU oracle cannot walk 50-100 M elements in seconds, so at full size the kernels are held to
(1) the oracle on whole sample blocks cut from both ends of the tensor, bit for bit, with the
library's own Philox noise replayed on the CPU, and (2) properties that do not depend on size:
every decoded element within one quantisation step of its input, two independent stream layouts
decoding to the same bits, rounding that is unbiased, widths that spend the budget exactly."""
import numpy as np
import pytest
import torch

import actnn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext(cuda_device):
    from actnn_b200.cpp_extension import calc_precision, minimax, quantization
    return type("Ext", (), {"q": quantization, "mm": minimax, "cp": calc_precision})


def relu_normal(shape, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.relu(torch.randn(shape, device="cuda", generator=g)).to(dtype)


def test_uniform_2bit_float32_round_trip_64x64x56x56(ext):
    """Configuration 0: float32 [64, 64, 56, 56] ~ ReLU(N(0,1)), group 256, 2 bits per sample."""
    N, G, bits, B = 64, 64 * 56 * 56 // 256, 2, 3
    seed, offset = 0, 0
    x = relu_normal((N, G, 256), torch.float32, 0)
    packed, scale, mn = ext.q.compress_single_precision(x, bits, True, philox=(seed, offset),
                                                        stat_dtype=torch.bfloat16)
    assert packed.numel() == O.single_total_bytes(bits, N, G, 256)
    noise = ext.q.noise_fill(x.numel(), torch.float32, "cuda", seed, offset).view(N, G, 256)

    # (1) the first, a middle and the last block of 8/bits samples against the oracle, bit for bit
    # (the middle one lies where the persistent grid has wrapped around many times)
    wpt = 8 // bits
    block_bytes = G * 256
    for no in (0, (N // wpt) // 2 + 1, N // wpt - 1):
        rows = slice(no * wpt, (no + 1) * wpt)
        xs = x[rows].cpu()
        omn, omx = O.group_minimax(xs)
        codes, oscale = O.quantize(xs, bits, omn, omx, noise[rows].cpu())
        expect = O.pack_single_layout(codes, bits)[:block_bytes]
        got = packed[no * block_bytes:(no + 1) * block_bytes].cpu().numpy()
        assert np.array_equal(got, expect)
        assert torch.equal(scale[rows].cpu().float(), oscale.to(torch.bfloat16).float())
        assert torch.equal(mn[rows].cpu().float(), omn.to(torch.bfloat16).float())

    # (2a) every element decodes to within one step (+ the bfloat16 rounding of scale and min)
    deq = ext.q.unpack_single_precision(packed, bits, scale, mn, N, G, 256, out_dtype=torch.float32)
    step = 1.0 / scale.float()
    allowed = step * (1.0 + B * 2.0 ** -7) + mn.float().abs() * 2.0 ** -7 + 1e-6
    err = (deq - x).abs()
    assert bool((err <= allowed).all())
    # (2b) the mixed-width stream with every width = 2 decodes to the same bits
    gmn, gmx = ext.mm.minimax(x.view(-1, 256))
    gmn, gmx = gmn.view(N, G, 1), gmx.view(N, G, 1)
    widths = torch.full((N,), bits, dtype=torch.int32, device="cuda")
    pm, pscale, pmn = ext.q.pack_mixed_precision(x, gmn, gmx, widths, True, philox=(seed, offset),
                                                 stat_dtype=torch.bfloat16, return_min=True)
    deq_m = ext.q.unpack_mixed_precision(pm, widths, pscale, pmn, N, G, 256, out_dtype=torch.float32)
    assert torch.equal(deq_m, deq)
    # (2c) unbiased: the mean error is far inside one step
    assert abs(float((deq - x).double().mean())) < 2e-3 * float(step.double().mean())
    # (2d) deterministic rounding lands within half a step
    p0, s0, m0 = ext.q.compress_single_precision(x, bits, False, stat_dtype=torch.bfloat16)
    d0 = ext.q.unpack_single_precision(p0, bits, s0, m0, N, G, 256, out_dtype=torch.float32)
    allowed0 = (0.5 + B * 2.0 ** -7) / s0.float() + m0.float().abs() * 2.0 ** -7 + 1e-6
    assert bool(((d0 - x).abs() <= allowed0).all())


def test_adaptive_bfloat16_512x256x28x28(ext):
    """Configuration 2: bfloat16 [512, 256, 28, 28] ~ ReLU(N(0,1)), per-sample sensitivities
    ~ LogNormal(0,1), greedy widths at a 2.0-bit average, pack, unpack."""
    N, G, initial = 512, 256 * 28 * 28 // 256, 8
    seed, offset = 11, 4
    dt = torch.bfloat16
    x = relu_normal((N, G, 256), dt, 2)
    g = torch.Generator(device="cuda").manual_seed(3)
    sens = torch.exp(torch.randn(N, device="cuda", generator=g))
    mn, mx = ext.mm.minimax(x.view(-1, 256))
    mn, mx = mn.view(N, G, 1), mx.view(N, G, 1)
    C = ext.cp.sensitivity(mn, mx, N, 1.0) * sens
    widths, offsets = ext.cp.allocate_bits(C.contiguous(), initial, 2 * N, None, G, 256, with_offsets=True)

    # the budget is spent exactly, widths stay in range, and the CPU heap agrees on the same C
    w_cpu = widths.cpu()
    assert int(w_cpu.sum()) == 2 * N and int(w_cpu.min()) >= 1 and int(w_cpu.max()) <= initial
    expect_w = O.calc_precision(torch.full((N,), initial, dtype=torch.int32), C.cpu(),
                                torch.ones(N, dtype=torch.int32), float(2 * N))
    assert torch.equal(w_cpu, expect_w.to(torch.int32))
    off_cpu = offsets.cpu()
    assert torch.equal(off_cpu[1:] - off_cpu[:-1], w_cpu.long() * (G * 256 // 32))

    packed, scale, q_min = ext.q.pack_mixed_precision(x, mn, mx, widths, True, philox=(seed, offset),
                                                      word_offsets=offsets, total_bits=2 * N, return_min=True)
    assert packed.numel() == 2 * N * G * 256 // 32
    noise = ext.q.noise_fill(x.numel(), dt, "cuda", seed, offset).view(N, G, 256)

    # (1) two samples from each end and two from the middle (where the persistent grid has
    # wrapped around many times and tasks straddle sample boundaries) against the oracle, word for word
    for rows in (slice(0, 2), slice(N // 2 + 1, N // 2 + 3), slice(N - 2, N)):
        xs, ws = x[rows].cpu(), w_cpu[rows]
        omn, omx = O.group_minimax(xs)
        codes, oscale = O.quantize(xs, ws, omn, omx, noise[rows].cpu())
        expect = O.pack_mixed_layout(codes, ws)
        lo, hi = int(off_cpu[rows.start]), int(off_cpu[rows.stop])
        assert np.array_equal(packed[lo:hi].cpu().numpy(), expect)
        assert torch.equal(scale[rows].cpu().float(), oscale.float())

    # (2) every element decodes to within one step of its sample's width (+ bfloat16 rounding)
    deq = ext.q.unpack_mixed_precision(packed, widths, scale, q_min, N, G, 256, word_offsets=offsets, out_dtype=dt)
    step = 1.0 / scale.float()
    allowed = step * 1.02 + x.float().abs() * 2.0 ** -6 + 1e-6
    assert bool(((deq.float() - x.float()).abs() <= allowed).all())
    # samples with more bits are decoded more accurately
    per_sample = (deq.float() - x.float()).pow(2).mean(dim=(1, 2)).cpu()
    wide, narrow = per_sample[w_cpu >= 4], per_sample[w_cpu <= 1]
    if len(wide) and len(narrow):
        assert float(wide.mean()) < float(narrow.mean())


def test_conv3x3_relu_fp16_256x256x28x28():
    """Configuration 1: QConv2d 3x3 256->256 + QReLU, float16 [256, 256, 28, 28]; 2-bit saved
    input, 1-bit ReLU mask.  The forward pass and dX do not depend on the saved activation and
    must equal the uncompressed layers exactly; dW carries the quantisation noise."""
    import actnn_b200 as actnn
    from actnn_b200.conf import QuantizationConfig
    actnn.config.__dict__.update(QuantizationConfig().__dict__)
    try:
        actnn.set_optimization_level("L3")
        torch.manual_seed(0)
        ref = torch.nn.Sequential(torch.nn.Conv2d(256, 256, 3, 1, 1, bias=False), torch.nn.ReLU()).cuda().half()
        torch.nn.init.kaiming_normal_(ref[0].weight)
        ours = torch.nn.Sequential(actnn.QConv2d(256, 256, 3, 1, 1, bias=False), actnn.QReLU()).cuda().half()
        ours[0].weight.data.copy_(ref[0].weight.data)
        x = torch.randn(256, 256, 28, 28, device="cuda", dtype=torch.float16)
        gy = torch.randn(256, 256, 28, 28, device="cuda", dtype=torch.float16) * 1e-2
        xr, xo = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        # one step first: the gradient scale that feeds the width allocation starts at zero
        # (as in the reference, qscheme.py:36-40), which parks most samples at one bit
        ours(xo).backward(gy)
        xo.grad, ours[0].weight.grad = None, None
        before = torch.cuda.memory_allocated()
        yo = ours(xo)
        saved = torch.cuda.memory_allocated() - before - yo.numel() * 2
        yr = ref(xr)
        assert torch.equal(yo, yr)
        # 2 bits + statistics for the conv input, 1 bit for the mask, conv output kept for ReLU only transiently
        assert saved < x.numel() * 2 * 0.30
        yr.backward(gy)
        yo.backward(gy)
        assert torch.equal(xo.grad, xr.grad)
        dw, dw_ref = ours[0].weight.grad.float(), ref[0].weight.grad.float()
        rel = float((dw - dw_ref).norm() / dw_ref.norm())
        assert rel < 1.0, rel                               # 2-bit noise is of the order of the signal
        # the noise is unbiased: the mean gradient error is small against the mean magnitude
        assert abs(float((dw - dw_ref).mean())) < 0.05 * float(dw_ref.abs().mean())
    finally:
        actnn.config.__dict__.update(QuantizationConfig().__dict__)
