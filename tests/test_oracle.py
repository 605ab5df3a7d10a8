"""The oracle against the fixtures produced by the reference's own code (CPU only)."""
import numpy as np
import pytest
import torch

import actnn_oracle as O
from conftest import DTYPES, from_raw, load_cases, same_values

SIM = load_cases("quantize_simulate")
ACT = load_cases("quantize_activation")
GREEDY = load_cases("calc_precision")


@pytest.mark.parametrize("case", sorted(SIM))
def test_quantize_dequantize_match_reference_simulate(case):
    f = SIM[case]
    dt = DTYPES[case.split("_")[1]]
    x, mn, mx, noise = (from_raw(f[k], dt) for k in ("x", "mn", "mx", "noise"))
    bits = torch.from_numpy(f["bits"])
    codes, scale = O.quantize(x, bits, mn, mx, noise)
    assert np.array_equal(codes.numpy(), f["codes"].astype(np.int32))
    assert same_values(scale, from_raw(f["scale"], dt))
    deq = O.dequantize(codes, scale, mn)
    assert deq.dtype == dt and same_values(deq, from_raw(f["deq"], dt))


@pytest.mark.parametrize("case", sorted(ACT))
def test_quantize_activation_matches_reference(case):
    f = ACT[case]
    _, dname, which, shape = case.split("_")
    dt = DTYPES[dname]
    shape = tuple(int(s) for s in shape.split("x"))
    x = from_raw(f["x"], dt).view(shape)
    noise = from_raw(f["noise"], dt)
    stat_dt = torch.bfloat16 if dt == torch.float32 else dt
    if which == "conv":
        q = O.quantize_activation(x, 2, lambda g: noise, coeff=(9 / 4 / 1, torch.tensor(0.37)))
        assert np.array_equal(q[1].numpy(), f["bits"])
        _, _, _, _, C = O.scheme_bits(x, 2, coeff=(9 / 4 / 1, torch.tensor(0.37)))
        assert np.array_equal(C.numpy(), f["C"])
    elif which == "bn":
        q = O.quantize_activation(x, 2, lambda g: noise)
        assert np.array_equal(q[1].numpy(), f["bits"])
    else:
        q = O.quantize_activation(x, 4, lambda g: noise, scheme=False)
        assert q[1] == 4 and np.all(f["bits"] == 4)
    assert np.array_equal(q[0].numpy(), f["codes"].astype(np.int32))
    assert q[2].dtype == stat_dt and same_values(q[2], from_raw(f["scale"], stat_dt))
    assert same_values(q[3], from_raw(f["min"], stat_dt))
    # the reference widens bfloat16 statistics to float32, whatever the input dtype was
    out_dt = torch.float32 if dt == torch.bfloat16 else dt
    deq = O.dequantize_activation(q, shape)
    assert deq.dtype == out_dt and deq.shape == shape
    assert same_values(deq, from_raw(f["deq"], out_dt).view(shape))
    if dt == torch.bfloat16:
        native = O.dequantize_activation(q, shape, dtype=dt)
        assert native.dtype == dt
        assert torch.allclose(native.float(), deq, rtol=2e-2, atol=1e-2 * float(deq.abs().max()))


@pytest.mark.parametrize("case", sorted(GREEDY, key=lambda s: int(s[1:])))
def test_greedy_matches_reference_calc_precision(case):
    f = GREEDY[case]
    n = f["C"].size
    b = O.calc_precision(torch.ones(n, dtype=torch.int32) * 8, torch.from_numpy(f["C"]),
                         torch.from_numpy(f["w"]), float(f["target"][0]))
    assert np.array_equal(b.numpy(), f["b"].astype(np.int32))


def test_greedy_against_compiled_reference_when_present():
    import build_ref
    ref = build_ref.load_ref_calc_precision()
    if ref is None:
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    g = torch.Generator().manual_seed(11)
    for t in range(60):
        n = int(torch.randint(1, 300, (1,), generator=g))
        C = torch.exp(torch.randn(n, generator=g) * (1 + t % 4))
        if t % 6 == 0:
            C = torch.zeros(n)
        w = torch.ones(n, dtype=torch.int32)
        target = int((1 + 7 * float(torch.rand(1, generator=g))) * n)
        b0 = torch.ones(n, dtype=torch.int32) * 8
        assert torch.equal(ref.calc_precision(b0.clone(), C.clone(), w.clone(), target),
                           O.calc_precision(b0, C, w, target))


@pytest.mark.parametrize("bits", [[1, 2, 3, 8, 5], [4, 4], [7, 6, 1], [16, 2]])
@pytest.mark.parametrize("gs", [32, 64, 256])
def test_mixed_layout_matches_kernel_emulation(bits, gs):
    g = torch.Generator().manual_seed(sum(bits) + gs)
    b = torch.tensor(bits, dtype=torch.int32)
    codes = torch.stack([torch.randint(0, 2 ** int(k), (2, gs), generator=g) for k in bits]).int()
    words = O.pack_mixed_layout(codes, b)
    assert np.array_equal(words, O.emulate_pack_mixed_kernel(codes, b))
    assert torch.equal(O.unpack_mixed_layout(words, b, len(bits), 2, gs), codes)


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [1, 3, 8, 9])
def test_single_layout_matches_kernel_emulation(bits, n):
    g = torch.Generator().manual_seed(bits * 100 + n)
    codes = torch.randint(0, 2 ** bits, (n, 2, 64), generator=g).int()
    packed = O.pack_single_layout(codes, bits)
    assert packed.size == O.single_total_bytes(bits, n, 2, 64)
    assert np.array_equal(packed, O.emulate_pack_single_kernel(codes, bits))
    assert torch.equal(O.unpack_single_layout(packed, bits, n, 2, 64), codes)


def test_mixed_layout_is_a_lane_ballot_for_group_size_256():
    """With 256-element groups, word ``j*b + i`` bit ``t`` is bit ``i`` of element ``8t + j``."""
    b = 3
    codes = torch.randint(0, 8, (1, 1, 256), generator=torch.Generator().manual_seed(5)).int()
    words = O.pack_mixed_layout(codes, torch.tensor([b], dtype=torch.int32)).view(np.uint32)
    for j in range(8):
        for i in range(b):
            expect = sum(((int(codes[0, 0, 8 * t + j]) >> i) & 1) << t for t in range(32))
            assert int(words[j * b + i]) == expect


def test_philox_known_answers():
    """Known-answer vectors of Philox4x32-10 from the Random123 distribution."""
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, out in kat:
        got = O.philox4x32_10(np.array([ctr], dtype=np.uint32), key)[0]
        assert tuple(int(v) for v in got) == out


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_philox_noise_range_and_mean(dt):
    u = O.philox_noise(1 << 16, dt, seed=1234, offset=5).float()
    assert u.min() >= -0.5 and u.max() <= 0.5
    assert abs(float(u.mean())) < 5e-3
    assert not torch.equal(u, O.philox_noise(1 << 16, dt, seed=1234, offset=6).float())


def test_relu_and_maxpool_oracle_agree_with_torch():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 3, 9, 10, generator=g)
    y, mask = O.relu_forward(x)
    assert torch.equal(y, torch.relu(x))
    dy = torch.randn(x.shape, generator=g)
    assert torch.equal(O.relu_backward(dy, mask), dy * (x > 0))
    for k, s, p in [((3, 3), (2, 2), (1, 1)), ((2, 2), (2, 2), (0, 0)), ((3, 2), (1, 2), (1, 0))]:
        xr = x.clone().requires_grad_()
        ref = torch.nn.functional.max_pool2d(xr, k, s, p)
        out, idx = O.max_pool2d_forward(x, k, s, p)
        assert torch.equal(out, ref.detach())
        go = torch.randn(ref.shape, generator=g)
        ref.backward(go)
        assert torch.allclose(O.max_pool2d_backward(go, idx, x.shape, k, s, p), xr.grad, atol=1e-6)


# ------------------------------------------------------------------ batch norm
@pytest.mark.parametrize("shape", [(4, 3, 5, 7), (6, 5), (2, 4, 9)])
def test_batch_norm_oracle_matches_torch_cpu(shape):
    """The float64 restatement against PyTorch's own CPU batch norm and its autograd."""
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(shape, generator=g, dtype=torch.float64) * 2 + 3).requires_grad_(True)
    C = shape[1]
    w = torch.randn(C, generator=g, dtype=torch.float64).requires_grad_(True)
    b = torch.randn(C, generator=g, dtype=torch.float64).requires_grad_(True)
    rm, rv = torch.randn(C, generator=g, dtype=torch.float64), torch.rand(C, generator=g, dtype=torch.float64) + 0.5
    rm_t, rv_t = rm.clone(), rv.clone()
    y_t = torch.nn.functional.batch_norm(x, rm_t, rv_t, w, b, True, 0.1, 1e-5)
    gy = torch.randn(shape, generator=g, dtype=torch.float64)
    gx_t, gw_t, gb_t = torch.autograd.grad(y_t, (x, w, b), gy)
    y, mean, invstd, new_rm, new_rv = O.batch_norm_forward(x.detach(), w.detach(), b.detach(), rm, rv, 0.1, 1e-5)
    assert torch.allclose(y, y_t, rtol=1e-10, atol=1e-10)
    assert torch.allclose(new_rm, rm_t, rtol=1e-10, atol=1e-12) and torch.allclose(new_rv, rv_t, rtol=1e-10, atol=1e-12)
    gx, gw, gb = O.batch_norm_backward(x.detach(), gy, w.detach(), mean, invstd)
    assert torch.allclose(gx, gx_t, rtol=1e-9, atol=1e-10)
    assert torch.allclose(gw, gw_t, rtol=1e-9, atol=1e-10) and torch.allclose(gb, gb_t, rtol=1e-9, atol=1e-10)
