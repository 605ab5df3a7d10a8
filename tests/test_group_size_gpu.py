"""Group sizes other than 256 (the reference accepts any multiple of 32,
quantization_cuda_kernel.cu:94,186, and ``config.group_size`` exposes it): every codec entry
point against the CPU oracle, bit for bit, and one pass through the public glue (GPU)."""
import numpy as np
import pytest
import torch

import actnn_oracle as O
from conftest import same_values

pytestmark = pytest.mark.gpu

DTS = [torch.float32, torch.float16, torch.bfloat16]


@pytest.fixture(scope="module")
def ext(cuda_device):
    from actnn_b200.cpp_extension import calc_precision, minimax, quantization
    return type("Ext", (), {"q": quantization, "mm": minimax, "cp": calc_precision})


def _groups(n, g, gs, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n, g, gs, generator=gen) * torch.exp(torch.randn(n, 1, 1, generator=gen))
    return x.to(dtype)


@pytest.mark.parametrize("dtype", DTS)
@pytest.mark.parametrize("gs", [64, 128, 512, 96])
def test_mixed_stream_other_group_sizes(ext, gs, dtype):
    n, g = 5, 7
    x = _groups(n, g, gs, dtype, gs)
    bits = torch.tensor([1, 2, 3, 8, 5], dtype=torch.int32)
    mn, mx = O.group_minimax(x)
    noise = O.torch_noise(x.shape, dtype, torch.Generator().manual_seed(1))
    codes, scale = O.quantize(x, bits, mn, mx, noise)
    dmn, dmx = ext.mm.minimax(x.cuda().view(-1, gs))
    assert same_values(dmn.cpu().view(n, g, 1), mn) and same_values(dmx.cpu().view(n, g, 1), mx)
    packed, dscale = ext.q.pack_mixed_precision(x.cuda(), mn.cuda(), mx.cuda(), bits.cuda(), True, noise=noise.cuda())
    assert np.array_equal(packed.cpu().numpy(), O.pack_mixed_layout(codes, bits))
    assert same_values(dscale.cpu(), scale)
    out = ext.q.unpack_mixed_precision(packed, bits.cuda(), dscale, mn.cuda(), n, g, gs)
    assert same_values(out.cpu(), O.dequantize(codes, scale, mn))
    # generated noise: the stream of the flat element index, replayed on the CPU
    seed, offset = 99, 16
    pnoise = O.philox_noise(x.numel(), dtype, seed, offset).view(x.shape)
    pcodes, _ = O.quantize(x, bits, mn, mx, pnoise)
    packed2, _ = ext.q.pack_mixed_precision(x.cuda(), mn.cuda(), mx.cuda(), bits.cuda(), True, philox=(seed, offset))
    assert np.array_equal(packed2.cpu().numpy(), O.pack_mixed_layout(pcodes, bits))


@pytest.mark.parametrize("dtype", DTS)
@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("gs", [64, 512])
def test_single_stream_other_group_sizes(ext, gs, bits, dtype):
    n, g = 5, 3                                        # 5 is not a multiple of 8 / bits
    x = _groups(n, g, gs, dtype, gs + bits)
    mn, mx = O.group_minimax(x)
    noise = O.torch_noise(x.shape, dtype, torch.Generator().manual_seed(2))
    codes, scale = O.quantize(x, bits, mn, mx, noise)
    packed, dscale = ext.q.pack_single_precision(x.cuda(), mn.cuda(), mx.cuda(), bits, True, noise=noise.cuda())
    assert np.array_equal(packed.cpu().numpy(), O.pack_single_layout(codes, bits))
    assert same_values(dscale.cpu(), scale)
    fused, fscale, fmn = ext.q.compress_single_precision(x.cuda(), bits, True, noise=noise.cuda())
    assert torch.equal(fused, packed) and same_values(fscale.cpu(), scale) and same_values(fmn.cpu(), mn)
    out = ext.q.unpack_single_precision(packed, bits, dscale, mn.cuda(), n, g, gs)
    assert same_values(out.cpu(), O.dequantize(codes, scale, mn))


@pytest.mark.parametrize("gs", [64, 128])
def test_glue_and_one_call_compress_with_another_group_size(ext, gs):
    import actnn_b200 as actnn
    from actnn_b200.conf import QuantizationConfig
    actnn.config.__dict__.update(QuantizationConfig().__dict__)
    try:
        actnn.set_optimization_level("L3")
        actnn.config.group_size = gs
        actnn.config.perlayer = False
        torch.manual_seed(0)
        x = (torch.randn(6, 8, 7, 9) * torch.exp(torch.randn(6, 1, 1, 1))).cuda()      # 504 features: padded
        scheme = actnn.QScheme(None, num_locations=9)
        gen = torch.cuda.default_generators[0]
        gen.manual_seed(5)
        seed, offset = gen.initial_seed(), gen.get_offset()
        q = actnn.ops.quantize_activation(x, scheme)
        y = actnn.ops.dequantize_activation(q, x.shape, x.dtype)
        # the oracle on the same sensitivities and the same noise
        groups = O.to_groups(x.cpu(), gs)
        noise = O.philox_noise(groups.numel(), torch.float32, seed, offset).view(groups.shape)
        oq = O.quantize_activation(x.cpu(), 2, lambda gr: noise, group_size=gs, coeff=(9 / 4, torch.tensor(0.0) + 1.0))
        # QScheme starts with scale 0: the reference multiplies C by it; the greedy then only sees ties
        assert int(q[1].sum()) == 2 * 6
        assert y.shape == x.shape and torch.isfinite(y).all()
        step = 1.0 / q[2].float()
        gx = actnn.qscheme.to_groups(x)
        err = (actnn.qscheme.to_groups(y) - gx).abs()
        # one step, plus the bfloat16 rounding of the stored scale and minimum of float32 data
        assert bool((err <= step * 1.02 + 1e-6 + gx.abs().amax(dim=2, keepdim=True) * 2.0 ** -6).all())
        assert oq[0].shape == groups.shape
    finally:
        actnn.QScheme.layers.clear()
        actnn.config.__dict__.update(QuantizationConfig().__dict__)
