"""Parity of the CUDA kernels (through the C ABI) with the CPU oracle: bit-exact codes,
packed words / bytes and dequantized values on identical inputs and identical noise."""
import numpy as np
import pytest
import torch

import actnn_oracle as O
from conftest import DTYPES, ROOT, from_raw, load_cases, same_values

pytestmark = pytest.mark.gpu

SIM = load_cases("quantize_simulate")
GREEDY = load_cases("calc_precision")
DT = [torch.float32, torch.float16, torch.bfloat16]


@pytest.fixture(scope="module")
def ext(cuda_device):
    from actnn_b200.cpp_extension import calc_precision, minimax, quantization
    return type("Ext", (), {"q": quantization, "mm": minimax, "cp": calc_precision})


def dev(t):
    return t.cuda()


def make_input(shape, dtype, seed, kind="randn"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    if kind == "relu":
        x = torch.relu(x)
    elif kind == "scaled":
        x = x * torch.exp(torch.randn(shape[0], generator=g)).view(-1, *([1] * (len(shape) - 1)))
    return x.to(dtype)


# ------------------------------------------------------------------------------ minimax
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("rows,cols", [(1024, 256), (1023, 256), (1, 256), (5, 64), (33, 512), (7, 1024)])
def test_minimax(ext, dtype, rows, cols):
    x = make_input((rows, cols), dtype, rows + cols)
    mn, mx = ext.mm.minimax(dev(x))
    omn, omx = O.minimax(x)
    assert mn.dtype == dtype and same_values(mn.cpu(), omn) and same_values(mx.cpu(), omx)


def test_minimax_rejects_bad_shapes(ext):
    with pytest.raises(RuntimeError):
        ext.mm.minimax(torch.zeros(4, 32, device="cuda"))        # D > 32 required
    with pytest.raises(RuntimeError):
        ext.mm.minimax(torch.zeros(4, 100, device="cuda"))       # D % 32 == 0 required
    with pytest.raises(RuntimeError):
        ext.mm.minimax(torch.zeros(4, 256))                      # CPU tensor
    with pytest.raises(RuntimeError):
        ext.mm.minimax(torch.zeros(4, 512, device="cuda")[:, ::2])   # not contiguous
    with pytest.raises(RuntimeError):
        ext.mm.minimax(torch.zeros(4, 256, device="cuda", dtype=torch.float64))


# ------------------------------------------------------------------------------ golden vectors
@pytest.mark.parametrize("case", sorted(SIM))
def test_reference_golden_vectors(ext, case):
    """Inputs, noise and expected codes come from the reference's own simulate branch."""
    f = SIM[case]
    dt = DTYPES[case.split("_")[1]]
    x, mn, mx, noise = (from_raw(f[k], dt) for k in ("x", "mn", "mx", "noise"))
    bits = torch.from_numpy(f["bits"])
    codes = torch.from_numpy(f["codes"].astype(np.int32))
    n, g, gs = x.shape

    packed, scale = ext.q.pack_mixed_precision(dev(x), dev(mn), dev(mx), dev(bits), True, noise=dev(noise))
    assert packed.dtype == torch.int32 and scale.dtype == dt
    assert np.array_equal(packed.cpu().numpy(), O.pack_mixed_layout(codes, bits))
    assert same_values(scale.cpu(), from_raw(f["scale"], dt))
    deq = ext.q.unpack_mixed_precision(packed, dev(bits), scale, dev(mn), n, g, gs)
    assert deq.dtype == dt and same_values(deq.cpu(), from_raw(f["deq"], dt))

    b0 = int(bits[0])
    if bool((bits == b0).all()) and 8 % b0 == 0:
        packed8, scale8 = ext.q.pack_single_precision(dev(x), dev(mn), dev(mx), b0, True, noise=dev(noise))
        assert packed8.dtype == torch.int8
        assert np.array_equal(packed8.cpu().numpy(), O.pack_single_layout(codes, b0))
        assert same_values(scale8.cpu(), from_raw(f["scale"], dt))
        deq8 = ext.q.unpack_single_precision(packed8, b0, scale8, dev(mn), n, g, gs)
        assert same_values(deq8.cpu(), from_raw(f["deq"], dt))
        fused = ext.q.compress_single_precision(dev(x), b0, True, noise=dev(noise), return_max=True)
        assert np.array_equal(fused[0].cpu().numpy(), packed8.cpu().numpy())
        assert same_values(fused[1].cpu(), scale8.cpu())
        assert same_values(fused[2].cpu(), mn) and same_values(fused[3].cpu(), mx)


# ------------------------------------------------------------------------------ random cases vs oracle
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("n,g", [(9, 13), (1, 1), (4, 4), (17, 2)])
@pytest.mark.parametrize("stochastic", [True, False])
def test_mixed_precision_against_oracle(ext, dtype, n, g, stochastic):
    x = make_input((n, g, 256), dtype, 10 * n + g, "scaled")
    x[0, 0] = 0                                   # an all-zero group (common after ReLU)
    if n > 1:
        x[1, 0] = x[1, 0, 0]                      # a constant group
    bits = torch.tensor([(i % 8) + 1 for i in range(n)], dtype=torch.int32)
    mn, mx = O.group_minimax(x)
    noise = O.torch_noise(x.shape, dtype, torch.Generator().manual_seed(n)) if stochastic else None
    codes, oscale = O.quantize(x, bits, mn, mx, noise)
    ok = torch.isfinite(oscale.float()).expand_as(x)      # constant non-zero groups: see test below
    packed, scale = ext.q.pack_mixed_precision(dev(x), dev(mn), dev(mx), dev(bits), stochastic,
                                               noise=None if noise is None else dev(noise))
    got = O.unpack_mixed_layout(packed.cpu().numpy(), bits, n, g, 256)
    assert torch.equal(got[ok], codes[ok])
    assert packed.numel() == O.mixed_total_words(bits, g, 256)
    assert same_values(scale.cpu(), oscale)
    deq = ext.q.unpack_mixed_precision(packed, dev(bits), scale, dev(mn), n, g, 256)
    odeq = O.dequantize(got, oscale, mn)
    assert same_values(deq.cpu()[ok], odeq[ok])
    # float32 activations may keep bfloat16 statistics (the reference's storage format)
    if dtype == torch.float32:
        p2, s2, m2 = ext.q.pack_mixed_precision(dev(x), dev(mn), dev(mx), dev(bits), stochastic,
                                                noise=None if noise is None else dev(noise),
                                                stat_dtype=torch.bfloat16, return_min=True)
        assert torch.equal(p2, packed)
        assert same_values(s2.cpu(), oscale.to(torch.bfloat16)) and same_values(m2.cpu(), mn.to(torch.bfloat16))
        d2 = ext.q.unpack_mixed_precision(p2, dev(bits), s2, m2, n, g, 256, out_dtype=torch.float32)
        od2 = O.dequantize(got, oscale.to(torch.bfloat16).float(), mn.to(torch.bfloat16).float())
        assert d2.dtype == torch.float32 and same_values(d2.cpu()[ok], od2[ok])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("n,g", [(1, 32), (3, 36), (7, 44), (5, 100), (40, 32), (2, 1000)])
def test_flat_task_kernels_against_oracle(ext, dtype, n, g):
    """Shapes with G % 4 == 0 and G >= 32 take the flat kernels (32-group tasks cut into runs of
    one width, tasks claimed by the warps of a block, the last ones in halves): every width
    1..8, tasks that end inside a bundle row of lanes, samples that change width inside a task,
    fewer tasks than warps and more."""
    x = make_input((n, g, 256), dtype, 7 * n + g, "scaled")
    bits = torch.tensor([((3 * i) % 8) + 1 for i in range(n)], dtype=torch.int32)
    mn, mx = O.group_minimax(x)
    noise = O.torch_noise(x.shape, dtype, torch.Generator().manual_seed(g))
    codes, oscale = O.quantize(x, bits, mn, mx, noise)
    ok = torch.isfinite(oscale.float()).expand_as(x)
    packed, scale = ext.q.pack_mixed_precision(dev(x), dev(mn), dev(mx), dev(bits), True, noise=dev(noise))
    got = O.unpack_mixed_layout(packed.cpu().numpy(), bits, n, g, 256)
    assert torch.equal(got[ok], codes[ok])
    assert same_values(scale.cpu(), oscale)
    deq = ext.q.unpack_mixed_precision(packed, dev(bits), scale, dev(mn), n, g, 256)
    assert same_values(deq.cpu()[ok], O.dequantize(got, oscale, mn)[ok])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("g", [32, 3])                 # flat tasks / bundle kernel
def test_wide_widths_decode_like_the_division_for_any_scale(ext, dtype, g):
    """From 6 bits on every element is computed: code / scale + min, each step rounded.  With
    16-bit statistics the kernels take the reciprocal of a group's scale once and correct the
    product with two fused multiply-adds (exactly rounded for scales in [2^-60, 2^60]); any other
    scale -- zero, infinity, subnormal, huge -- must fall back to the division.  Random words,
    random and hostile scales, against the oracle's dequantize."""
    n = 12 if g == 32 else 6
    gen = torch.Generator().manual_seed(11 * g)
    bits = torch.tensor([6 + (i % 3) for i in range(n)], dtype=torch.int32)
    words = O.mixed_total_words(bits, g, 256)
    packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (words,), dtype=torch.int32, generator=gen)
    stat = torch.bfloat16 if dtype == torch.float32 else dtype
    scale = torch.exp(torch.randn(n, g, 1, generator=gen) * 3).to(stat)
    hostile = [0.0, float("inf"), 1e-30, 6e-8, 5e4, 3e38, 1.0, 255.0]
    for i, v in enumerate(hostile):
        scale[i % n, (i * 5) % g, 0] = v
    mn = torch.randn(n, g, 1, generator=gen).to(stat)
    codes = O.unpack_mixed_layout(packed.numpy(), bits, n, g, 256)
    want = O.dequantize(codes, scale.to(dtype) if dtype != torch.float32 else scale.float(),
                        mn.to(dtype) if dtype != torch.float32 else mn.float())
    got = ext.q.unpack_mixed_precision(dev(packed), dev(bits), dev(scale), dev(mn), n, g, 256,
                                       **({"out_dtype": torch.float32} if dtype == torch.float32 else {}))
    a, b = got.cpu().float(), want.float()
    same = (a == b) | (torch.isnan(a) & torch.isnan(b))
    assert bool(same.all()), (a[~same][:4], b[~same][:4])


def test_eight_bit_single_stream_decodes_like_the_division(ext):
    """The uniform 8-bit stream computes every element too (reciprocal + correction)."""
    gen = torch.Generator().manual_seed(3)
    n, g = 8, 6
    for dtype in (torch.float16, torch.bfloat16):
        packed = torch.randint(-128, 128, (n * g * 256,), dtype=torch.int8, generator=gen)
        scale = torch.exp(torch.randn(n, g, 1, generator=gen) * 3).to(dtype)
        scale[0, 0, 0], scale[1, 1, 0], scale[2, 2, 0] = 0.0, float("inf"), 6e-8
        mn = torch.randn(n, g, 1, generator=gen).to(dtype)
        codes = O.unpack_single_layout(packed.numpy(), 8, n, g, 256)
        want = O.dequantize(codes, scale, mn)
        got = ext.q.unpack_single_precision(dev(packed), 8, dev(scale), dev(mn), n, g, 256)
        a, b = got.cpu().float(), want.float()
        same = (a == b) | (torch.isnan(a) & torch.isnan(b))
        assert bool(same.all()), (a[~same][:4], b[~same][:4])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_constant_nonzero_group_decodes_to_its_value(ext, dtype):
    """(mx - mn) + 2e-6 rounds to zero for such a group in 16-bit types; the reference then
    produces NaN codes.  Here the codes are 0 and the group decodes to its constant."""
    x = torch.full((2, 1, 256), 3.0, dtype=dtype)
    bits = torch.tensor([2, 4], dtype=torch.int32)
    mn, mx = O.group_minimax(x)
    packed, scale = ext.q.pack_mixed_precision(dev(x), dev(mn), dev(mx), dev(bits), True)
    assert int(packed.abs().sum()) == 0
    deq = ext.q.unpack_mixed_precision(packed, dev(bits), scale, dev(mn), 2, 1, 256)
    assert same_values(deq.cpu(), x)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("n,g", [(8, 6), (5, 3), (1, 1), (9, 7)])
def test_single_precision_against_oracle(ext, dtype, bits, n, g):
    x = make_input((n, g, 256), dtype, 100 * bits + n + g, "relu")
    mn, mx = O.group_minimax(x)
    noise = O.torch_noise(x.shape, dtype, torch.Generator().manual_seed(bits))
    codes, oscale = O.quantize(x, bits, mn, mx, noise)
    expect = O.pack_single_layout(codes, bits)
    packed, scale = ext.q.pack_single_precision(dev(x), dev(mn), dev(mx), bits, True, noise=dev(noise))
    assert packed.numel() == O.single_total_bytes(bits, n, g, 256)
    assert np.array_equal(packed.cpu().numpy(), expect)
    assert same_values(scale.cpu(), oscale)
    stat = torch.bfloat16 if dtype == torch.float32 else dtype
    fp, fs, fm = ext.q.compress_single_precision(dev(x), bits, True, noise=dev(noise), stat_dtype=stat)
    assert np.array_equal(fp.cpu().numpy(), expect)
    assert same_values(fs.cpu(), oscale.to(stat)) and same_values(fm.cpu(), mn.to(stat))
    deq = ext.q.unpack_single_precision(fp, bits, fs, fm, n, g, 256, out_dtype=dtype)
    odeq = O.dequantize(codes, oscale.to(stat).to(dtype), mn.to(stat).to(dtype))
    assert deq.dtype == dtype and same_values(deq.cpu(), odeq)


# ------------------------------------------------------------------------------ Philox noise
@pytest.mark.parametrize("dtype", DT)
def test_philox_noise_matches_oracle_and_drives_the_pack(ext, dtype):
    n, g = 6, 5
    seed, offset = 0x1234_5678_9ABC, 40
    x = make_input((n, g, 256), dtype, 77, "relu")
    noise = ext.q.noise_fill(x.numel(), dtype, "cuda", seed, offset)
    assert same_values(noise.cpu(), O.philox_noise(x.numel(), dtype, seed, offset))
    mn, mx = O.group_minimax(x)
    bits = torch.tensor([1, 2, 3, 4, 2, 8], dtype=torch.int32)
    a, _ = ext.q.pack_mixed_precision(dev(x), dev(mn), dev(mx), dev(bits), True, philox=(seed, offset))
    b, _ = ext.q.pack_mixed_precision(dev(x), dev(mn), dev(mx), dev(bits), True, noise=noise.view(x.shape))
    assert torch.equal(a, b)
    codes, _ = O.quantize(x, bits, mn, mx, noise.cpu().view(x.shape))
    assert np.array_equal(a.cpu().numpy(), O.pack_mixed_layout(codes, bits))
    for w in (1, 2, 4, 8):
        c = ext.q.compress_single_precision(dev(x), w, True, philox=(seed, offset))[0]
        d = ext.q.compress_single_precision(dev(x), w, True, noise=noise.view(x.shape))[0]
        assert torch.equal(c, d)
    other = ext.q.noise_fill(x.numel(), dtype, "cuda", seed, offset + 4)
    assert not torch.equal(other, noise)


def test_default_noise_follows_torch_manual_seed(ext):
    x = dev(make_input((4, 3, 256), torch.float16, 5))
    torch.manual_seed(123)
    a = ext.q.compress_single_precision(x, 2)[0]
    b = ext.q.compress_single_precision(x, 2)[0]
    torch.manual_seed(123)
    c = ext.q.compress_single_precision(x, 2)[0]
    assert torch.equal(a, c) and not torch.equal(a, b)


# ------------------------------------------------------------------------------ greedy
@pytest.mark.parametrize("case", sorted(GREEDY, key=lambda s: int(s[1:])))
def test_greedy_golden_vectors(ext, case):
    f = GREEDY[case]
    C = torch.from_numpy(f["C"])
    w = torch.from_numpy(f["w"])
    unit = bool((w == 1).all())
    bits, _ = ext.cp.allocate_bits(dev(C), 8, float(f["target"][0]), None if unit else dev(w))
    assert np.array_equal(bits.cpu().numpy(), f["b"].astype(np.int32))
    # the drop-in entry point takes CPU tensors like the reference's
    b = ext.cp.calc_precision(torch.ones(C.numel(), dtype=torch.int32) * 8, C, w, float(f["target"][0]))
    assert np.array_equal(b.numpy(), f["b"].astype(np.int32))


@pytest.mark.parametrize("n", [3, 700, 1171, 5000])
@pytest.mark.parametrize("weighted", [False, True])
def test_greedy_random_against_oracle(ext, n, weighted):
    g = torch.Generator().manual_seed(n)
    C = torch.exp(torch.randn(n, generator=g) * 2)
    C[::7] = C[0]                                                  # ties
    w = torch.randint(1, 100000, (n,), generator=g, dtype=torch.int32) if weighted else None
    tot = int(w.sum()) if weighted else n
    for avg in (1.0, 2.0, 3.7, 8.0):
        target = int(avg * tot)
        ob = O.calc_precision(torch.ones(n, dtype=torch.int32) * 8, C,
                              w if weighted else torch.ones(n, dtype=torch.int32), target)
        bits, offs = ext.cp.allocate_bits(dev(C), 8, target, dev(w) if weighted else None, 5, 256,
                                          with_offsets=True)
        assert torch.equal(bits.cpu(), ob)
        expect = torch.cat([torch.zeros(1, dtype=torch.int64), ob.long().cumsum(0)]) * (5 * 256 // 32)
        assert torch.equal(offs.cpu(), expect)
        if not weighted:
            from actnn_b200.qscheme import total_bits_after_greedy
            assert int(ob.sum()) == total_bits_after_greedy(n, 8, target)


def test_bits_prefix(ext):
    bits = torch.randint(1, 9, (3000,), dtype=torch.int32)
    offs = ext.q.bits_prefix(dev(bits), 7, 256)
    expect = torch.cat([torch.zeros(1, dtype=torch.int64), bits.long().cumsum(0)]) * (7 * 256 // 32)
    assert torch.equal(offs.cpu(), expect)


@pytest.mark.parametrize("dtype", DT)
def test_sensitivity_against_oracle(ext, dtype):
    x = make_input((12, 16, 14, 14), dtype, 3, "scaled")
    groups, _, mn, mx, C = O.scheme_bits(x, 2, coeff=(9 / 4, torch.tensor(0.37)))
    n = x.shape[0]
    got = ext.cp.sensitivity(dev(mn), dev(mx), n, 256 / (14 * 14), 9 / 4,
                             torch.tensor([0.37], device="cuda"))
    assert torch.allclose(got.cpu(), C, rtol=2e-3 if dtype != torch.float32 else 1e-5)


# ------------------------------------------------------------------------------ ReLU / dropout / max-pool
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("shape", [(128, 56, 56, 31), (3,), (1, 1025), (4, 8, 32)])
def test_relu_forward_backward(ext, dtype, shape):
    x = make_input(shape, dtype, len(shape))
    y, mask = ext.q.relu_forward(dev(x))
    oy, omask = O.relu_forward(x)
    assert same_values(y.cpu(), oy)
    assert np.array_equal(mask.cpu().numpy(), omask)
    dy = make_input(shape, dtype, 9)
    dx = ext.q.relu_backward(dev(dy), mask)
    assert same_values(dx.cpu(), O.relu_backward(dy, omask))
    # through autograd, against F.relu as the reference's own test does
    a = dev(x).requires_grad_()
    ext.q.act_quantized_relu(a).backward(dev(dy))
    b = dev(x).requires_grad_()
    torch.relu(b).backward(dev(dy))
    assert same_values(a.grad.cpu(), b.grad.cpu())


@pytest.mark.parametrize("dtype", DT)
def test_dropout_forward_backward(ext, dtype):
    x = make_input((7, 1001), dtype, 4)
    p = 0.3
    seed, offset = 99, 8
    u = ext.q.dropout_uniform_fill(x.numel(), "cuda", seed, offset)
    assert same_values(u.cpu(), O.philox_dropout_uniform(x.numel(), seed, offset))
    y, mask = ext.q.dropout_forward(dev(x), p, philox=(seed, offset))
    y2, mask2 = ext.q.dropout_forward(dev(x), p, u=u)
    assert torch.equal(y, y2) and torch.equal(mask, mask2)
    oy, omask = O.dropout_forward(x, u.cpu().view(x.shape), p)
    assert np.array_equal(mask.cpu().numpy(), omask)
    tol = dict(rtol=1e-2, atol=1e-3) if dtype != torch.float32 else dict(rtol=1e-3, atol=1e-6)
    assert torch.allclose(y.cpu().float(), oy.float(), **tol)
    dy = make_input(x.shape, dtype, 6)
    dx = ext.q.dropout_backward(dev(dy), mask, p)
    assert torch.allclose(dx.cpu().float(), O.dropout_backward(dy, omask, p).float(), **tol)
    keep = O.unpack_bitmask(omask, x.numel()).float().mean()
    assert abs(float(keep) - (1 - p)) < 0.02


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("geom", [((4, 8, 28, 28), (3, 3), (2, 2), (1, 1), (1, 1)),
                                  ((2, 3, 17, 9), (2, 2), (2, 2), (0, 0), (1, 1)),
                                  ((1, 2, 12, 13), (3, 2), (1, 2), (1, 0), (1, 1)),
                                  ((2, 2, 15, 15), (3, 3), (2, 2), (1, 1), (2, 2)),
                                  ((2, 4, 16, 32), (3, 3), (2, 2), (1, 1), (1, 1)),     # vector stores
                                  ((2, 2, 16, 16), (2, 2), (1, 1), (0, 0), (1, 1)),     # stride 1: ten columns
                                  ((1, 3, 9, 40), (2, 3), (2, 3), (1, 1), (1, 1)),
                                  # rows of W % 8 == 0, stride 2: the row-segment kernels, every (K, P) variant,
                                  # vector and scalar loads / stores, window columns that leave the plane
                                  ((2, 3, 14, 32), (3, 3), (2, 2), (0, 0), (1, 1)),
                                  ((2, 3, 16, 24), (3, 3), (2, 2), (1, 1), (1, 1)),
                                  ((2, 3, 10, 32), (2, 2), (2, 2), (0, 0), (1, 1)),
                                  ((2, 3, 10, 16), (2, 2), (2, 2), (1, 1), (1, 1)),
                                  ((1, 2, 11, 40), (3, 3), (2, 2), (0, 1), (1, 1)),
                                  ((1, 2, 12, 8), (3, 3), (2, 2), (1, 0), (1, 1)),
                                  ((3, 5, 8, 8), (2, 2), (2, 2), (0, 1), (1, 1))])
def test_max_pool2d_forward_backward(ext, dtype, geom):
    shape, k, s, p, d = geom
    x = make_input(shape, dtype, sum(shape))
    y, idx = ext.q.max_pool2d_forward(dev(x), k, s, p, d)
    oy, oidx = O.max_pool2d_forward(x, k, s, p, d)
    assert same_values(y.cpu(), oy) and torch.equal(idx.cpu(), oidx)
    dy = make_input(tuple(y.shape), dtype, 11)
    dx = ext.q.max_pool2d_backward(dev(dy), idx, shape, k, s, p, d)
    # overlapping windows add up to four gradients per input; kernel and oracle sum them in
    # float32 in different orders, so allow the last unit of the result type
    odx = O.max_pool2d_backward(dy, oidx, shape, k, s, p, d)
    tol = dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else dict(rtol=8e-3, atol=1e-3)
    assert torch.allclose(dx.cpu().float(), odx.float(), **tol)
    assert torch.equal(dx.cpu() == 0, odx == 0)
    # against F.max_pool2d through autograd (reference test: 1e-4)
    a = dev(x).float().requires_grad_()
    torch.nn.functional.max_pool2d(a, k, s, p, d).backward(dev(dy).float())
    b = dev(x).requires_grad_()
    out = ext.q.act_quantized_max_pool2d(b, k, s, p, d, False, False)
    out.backward(dev(dy))
    assert torch.allclose(b.grad.float(), a.grad, atol=1e-2 if dtype != torch.float32 else 1e-4, rtol=1e-2)


def test_max_pool2d_rejects_what_the_reference_rejects(ext):
    x = torch.zeros(1, 1, 8, 8, device="cuda")
    with pytest.raises(RuntimeError):
        ext.q.act_quantized_max_pool2d(x, (4, 4), (1, 1), (0, 0), (1, 1), False, False)   # KH*KW >= 16
    with pytest.raises(RuntimeError):
        ext.q.act_quantized_max_pool2d(x, (2, 2), (2, 2), (0, 0), (1, 1), True, False)    # ceil_mode
    with pytest.raises(RuntimeError):
        ext.q.act_quantized_max_pool2d(x, (2, 2), (2, 2), (0, 0), (1, 1), False, True)    # return_indices


# ------------------------------------------------------------------------------ error contract
def test_pack_argument_errors(ext):
    x = torch.zeros(2, 2, 256, device="cuda", dtype=torch.float16)
    mn = torch.zeros(2, 2, 1, device="cuda", dtype=torch.float16)
    bits = torch.ones(2, device="cuda", dtype=torch.int32)
    with pytest.raises(RuntimeError):
        ext.q.pack_single_precision(x, mn, mn, 3, True)                 # 8 % bits != 0
    with pytest.raises(RuntimeError):
        ext.q.pack_mixed_precision(x, mn, mn, bits.long(), True)       # bits must be int32
    with pytest.raises(RuntimeError):
        ext.q.pack_mixed_precision(x.view(2, 512), mn, mn, bits, True)  # rank 3 required
    with pytest.raises(RuntimeError):
        ext.q.pack_mixed_precision(x.float(), mn, mn, bits, True)      # stats must share the dtype
    with pytest.raises(RuntimeError):
        ext.q.unpack_single_precision(torch.zeros(10, device="cuda", dtype=torch.int32), 2, mn, mn, 2, 2, 256)
    with pytest.raises(RuntimeError):                                  # misaligned view -> status from the C ABI
        flat = torch.zeros(2 * 2 * 256 + 8, device="cuda", dtype=torch.float16)
        ext.q.compress_single_precision(flat[1:1 + 1024].view(2, 2, 256), 2)


# ------------------------------------------------------------------------------ one-call adaptive compress
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("shape", [(12, 16, 16, 16), (5, 8, 16, 16), (16, 2048)])
def test_compress_mixed_one_call_equals_stepwise_and_oracle(ext, dtype, shape):
    x = make_input(shape, dtype, sum(shape), "scaled")
    n = shape[0]
    groups = O.to_groups(x)
    g = groups.shape[1]
    num_pixels = groups.numel() // n // shape[1]
    stat = torch.bfloat16 if dtype == torch.float32 else dtype
    grad = torch.tensor([0.37], device="cuda")
    seed, offset = 77, 16
    packed, bits, scale, mn, C = ext.q.compress_mixed_precision(
        dev(groups), 2 * n, 8, 256 / num_pixels, 9 / 4, grad, True, philox=(seed, offset), stat_dtype=stat)
    # stepwise path through the individual entry points
    dmn, dmx = ext.mm.minimax(dev(groups).view(-1, 256))
    C2 = ext.cp.sensitivity(dmn.view(n, g, 1), dmx.view(n, g, 1), n, 256 / num_pixels, 9 / 4, grad)
    bits2, offs2 = ext.cp.allocate_bits(C2, 8, 2 * n, None, g, 256, with_offsets=True)
    p2, s2, m2 = ext.q.pack_mixed_precision(dev(groups), dmn.view(n, g, 1), dmx.view(n, g, 1), bits2, True,
                                            philox=(seed, offset), word_offsets=offs2, total_bits=2 * n,
                                            stat_dtype=stat, return_min=True)
    assert torch.equal(C, C2) and torch.equal(bits, bits2) and torch.equal(packed.word_offsets, offs2)
    assert torch.equal(packed, p2) and torch.equal(scale, s2) and torch.equal(mn, m2)
    assert int(bits.sum()) == 2 * n and packed.numel() == 2 * n * g * 256 // 32
    # and against the oracle, replaying the Philox noise
    omn, omx = O.group_minimax(groups)
    obits = O.calc_precision(torch.ones(n, dtype=torch.int32) * 8, C.cpu(), torch.ones(n, dtype=torch.int32), 2 * n)
    assert torch.equal(bits.cpu(), obits)
    noise = O.philox_noise(groups.numel(), dtype, seed, offset).view(groups.shape)
    codes, oscale = O.quantize(groups, obits, omn, omx, noise)
    assert np.array_equal(packed.cpu().numpy(), O.pack_mixed_layout(codes, obits))
    assert same_values(scale.cpu(), oscale.to(stat)) and same_values(mn.cpu(), omn.to(stat))
    out = ext.q.unpack_mixed_precision(packed, bits, scale, mn, n, g, 256, out_dtype=dtype)
    assert same_values(out.cpu(), O.dequantize(codes, oscale.to(stat).to(dtype), omn.to(stat).to(dtype)))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("shape", [(16, 64, 28, 28), (3, 1001), (5, 7, 3, 3), (2, 200000)])
def test_sample_sumsq(ext, dtype, shape):
    """QScheme.set_scale's per-sample squared gradient norm (qscheme.py:50,54); float
    accumulation order differs from torch's, hence the relative tolerance 1e-3."""
    g = make_input(shape, dtype, sum(shape)) * 1e-2
    got = ext.cp.sample_sumsq(dev(g))
    ref = g.view(shape[0], -1).float().norm(dim=1).square()
    assert got.dtype == torch.float32 and torch.allclose(got.cpu(), ref, rtol=1e-3)
    sliced = dev(g)[1:]                                       # a view that does not start the allocation
    assert torch.allclose(ext.cp.sample_sumsq(sliced).cpu(), ref[1:], rtol=1e-3)


def test_staged_pack_matches_direct_pack():
    """The opt-in bulk-copy staged pack (ACTNN_STAGED_PACK=1, read when the library first
    packs) against the default kernel, in a child process; its wait counter must stay zero."""
    import os
    import subprocess
    import sys
    code = r"""
import ctypes, sys, torch
sys.path.insert(0, %r)
from actnn_b200 import _lib
from actnn_b200.cpp_extension import quantization as q
g = torch.Generator().manual_seed(5)
x = torch.relu(torch.randn(16, 12, 256, generator=g)).to(torch.float16).cuda()
out = []
for dtype in (torch.float16, torch.bfloat16, torch.float32):
    for bits in (1, 2, 4, 8):
        p, s, m = q.compress_single_precision(x.to(dtype), bits, True, philox=(7, 0))
        out.append(p.cpu())
torch.cuda.synchronize()
count = ctypes.c_uint32(123)
_lib.check(_lib.load().actnn_bulk_wait_failures(ctypes.byref(count)), "actnn_bulk_wait_failures")
assert count.value == 0, count.value
torch.save(out, sys.argv[1])
""" % ROOT
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        results = []
        for flag in ("0", "1"):
            path = os.path.join(tmp, "out%s.pt" % flag)
            env = dict(os.environ, ACTNN_STAGED_PACK=flag)
            subprocess.run([sys.executable, "-c", code, path], check=True, env=env, timeout=300)
            results.append(torch.load(path))
    assert len(results[0]) == 12
    for a, b in zip(*results):
        assert torch.equal(a, b)
