"""No entry point writes outside its outputs (GPU).

Every output buffer is carved out of a larger allocation with 256 guard bytes of 0xA5 on
both sides; after the call the guards must be untouched.  Shapes are the ragged ones: one
sample, sample counts that are not a multiple of 8 / bits, group counts that are not a
multiple of the bundle sizes (and ones that are, which take the fast kernels), element
counts that are not a multiple of the 1024-element step of the mask kernels.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

GUARD = 256
FILL = 0xA5


class Guarded:
    """A tensor of `numel` elements of `dtype` with guard bytes before and after it."""

    def __init__(self, numel, dtype, device):
        self.nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        padded = (self.nbytes + 255) // 256 * 256
        self.raw = torch.full((GUARD + padded + GUARD,), FILL, dtype=torch.uint8, device=device)
        self.t = self.raw[GUARD:GUARD + self.nbytes].view(dtype)

    def ptr(self):
        return self.t.data_ptr()

    def intact(self):
        head = self.raw[:GUARD]
        tail = self.raw[GUARD + self.nbytes:]
        return bool((head == FILL).all()) and bool((tail == FILL).all())


@pytest.fixture(scope="module")
def env(cuda_device):
    from actnn_b200 import _lib
    from actnn_b200.cpp_extension import quantization
    return _lib.load(), _lib, quantization, cuda_device


def _check(_lib, status, what, buffers):
    _lib.check(status, what)
    torch.cuda.synchronize()
    for name, b in buffers.items():
        assert b.intact(), "%s wrote outside %s" % (what, name)


SHAPES = [(1, 1), (3, 5), (5, 36), (7, 64), (2, 33)]        # (N, G): G % 4 != 0, G % 4 == 0 with G >= 32, ...
DTS = [torch.float32, torch.float16, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTS)
@pytest.mark.parametrize("shape", SHAPES)
def test_codec_entry_points_stay_inside_their_outputs(env, shape, dtype):
    lib, _lib, q, dev = env
    n, g = shape
    gs = 256
    sdt = torch.bfloat16 if dtype == torch.float32 else dtype
    D, S = _lib.dtype_id(dtype), _lib.dtype_id(sdt)
    gen = torch.Generator().manual_seed(n * 100 + g)
    x = torch.randn(n, g, gs, generator=gen).to(dtype).to(dev)
    st = torch.cuda.current_stream().cuda_stream

    mn, mx = Guarded(n * g, dtype, dev), Guarded(n * g, dtype, dev)
    _check(_lib, lib.actnn_minimax(x.data_ptr(), mn.ptr(), mx.ptr(), n * g, gs, D, st), "actnn_minimax",
           {"min": mn, "max": mx})

    for bits in (1, 2, 4, 8):
        nbytes = q.single_precision_bytes(bits, n, g, gs)
        packed, scale, smn, smx = (Guarded(nbytes, torch.int8, dev), Guarded(n * g, sdt, dev),
                                   Guarded(n * g, sdt, dev), Guarded(n * g, sdt, dev))
        _check(_lib, lib.actnn_compress_single(x.data_ptr(), bits, packed.ptr(), scale.ptr(), smn.ptr(), smx.ptr(), n,
                                               g, gs, D, S, 1, None, 5, 0, st), "actnn_compress_single",
               {"packed": packed, "scale": scale, "min": smn, "max": smx})
        packed2, scale2, smn2 = Guarded(nbytes, torch.int8, dev), Guarded(n * g, sdt, dev), Guarded(n * g, sdt, dev)
        _check(_lib, lib.actnn_pack_single(x.data_ptr(), mn.ptr(), mx.ptr(), bits, packed2.ptr(), scale2.ptr(),
                                           smn2.ptr(), n, g, gs, D, S, 1, None, 5, 0, st), "actnn_pack_single",
               {"packed": packed2, "scale": scale2, "min": smn2})
        out = Guarded(n * g * gs, dtype, dev)
        _check(_lib, lib.actnn_unpack_single(packed.ptr(), bits, scale.ptr(), smn.ptr(), out.ptr(), n, g, gs, D, S, st),
               "actnn_unpack_single", {"out": out})

    widths = torch.tensor([(i * 3) % 8 + 1 for i in range(n)], dtype=torch.int32, device=dev)
    offs = Guarded(n + 1, torch.int64, dev)
    _check(_lib, lib.actnn_bits_prefix(widths.data_ptr(), n, g, gs, offs.ptr(), st), "actnn_bits_prefix",
           {"word_offsets": offs})
    words = int(widths.sum()) * g * gs // 32
    pm, pscale, pmn = Guarded(words, torch.int32, dev), Guarded(n * g, sdt, dev), Guarded(n * g, sdt, dev)
    _check(_lib, lib.actnn_pack_mixed(x.data_ptr(), mn.ptr(), mx.ptr(), widths.data_ptr(), offs.ptr(), pm.ptr(),
                                      pscale.ptr(), pmn.ptr(), n, g, gs, D, S, 1, None, 5, 0, st), "actnn_pack_mixed",
           {"packed": pm, "scale": pscale, "min": pmn})
    out = Guarded(n * g * gs, dtype, dev)
    _check(_lib, lib.actnn_unpack_mixed(pm.ptr(), widths.data_ptr(), offs.ptr(), pscale.ptr(), pmn.ptr(), out.ptr(), n,
                                        g, gs, D, S, st), "actnn_unpack_mixed", {"out": out})

    # the one-call adaptive compress at a 3-bit average
    total = 3 * n
    cm = {"packed": Guarded(total * g * gs // 32, torch.int32, dev), "scale": Guarded(n * g, sdt, dev),
          "min": Guarded(n * g, sdt, dev), "bits": Guarded(n, torch.int32, dev),
          "word_offsets": Guarded(n + 1, torch.int64, dev), "C": Guarded(n, torch.float32, dev)}
    ws_bytes = lib.actnn_compress_mixed_workspace(n, g, D)
    cm["workspace"] = Guarded(ws_bytes, torch.uint8, dev)
    _check(_lib, lib.actnn_compress_mixed(x.data_ptr(), cm["packed"].ptr(), cm["scale"].ptr(), cm["min"].ptr(),
                                          cm["bits"].ptr(), cm["word_offsets"].ptr(), cm["C"].ptr(),
                                          cm["workspace"].ptr(), ws_bytes, n, g, gs, D, S, 1.0, 1.0, None, 8,
                                          float(total), 1, None, 5, 0, st), "actnn_compress_mixed", cm)
    assert int(cm["bits"].t.sum()) == total

    C = Guarded(n, torch.float32, dev)
    _check(_lib, lib.actnn_range_sqr(mn.ptr(), mx.ptr(), n, g, D, 1.0, 1.0, None, C.ptr(), st), "actnn_range_sqr",
           {"C": C})
    b_out, offs2 = Guarded(n, torch.int32, dev), Guarded(n + 1, torch.int64, dev)
    _check(_lib, lib.actnn_calc_precision(C.ptr(), None, n, 8, float(2 * n), b_out.ptr(), offs2.ptr(), g, gs, None, 0,
                                          st), "actnn_calc_precision", {"bits": b_out, "word_offsets": offs2})
    ss = Guarded(n, torch.float32, dev)
    _check(_lib, lib.actnn_sample_sumsq(x.data_ptr(), ss.ptr(), n, g * gs, D, st), "actnn_sample_sumsq", {"out": ss})
    nz = Guarded(n * g * gs, dtype, dev)
    _check(_lib, lib.actnn_noise_fill(nz.ptr(), n * g * gs, D, 3, 4, st), "actnn_noise_fill", {"noise": nz})


@pytest.mark.parametrize("dtype", DTS)
@pytest.mark.parametrize("numel", [1, 31, 1000, 1024 * 3 + 17, 65536 + 8])
def test_mask_entry_points_stay_inside_their_outputs(env, numel, dtype):
    lib, _lib, q, dev = env
    D = _lib.dtype_id(dtype)
    st = torch.cuda.current_stream().cuda_stream
    x = torch.randn(numel, generator=torch.Generator().manual_seed(numel)).to(dtype).to(dev)
    y, mask = Guarded(numel, dtype, dev), Guarded((numel + 31) // 32, torch.int32, dev)
    _check(_lib, lib.actnn_relu_forward(x.data_ptr(), y.ptr(), mask.ptr(), numel, D, st), "actnn_relu_forward",
           {"y": y, "mask": mask})
    dx = Guarded(numel, dtype, dev)
    _check(_lib, lib.actnn_relu_backward(x.data_ptr(), mask.ptr(), dx.ptr(), numel, D, st), "actnn_relu_backward",
           {"dx": dx})
    y2, mask2 = Guarded(numel, dtype, dev), Guarded((numel + 31) // 32, torch.int32, dev)
    _check(_lib, lib.actnn_dropout_forward(x.data_ptr(), y2.ptr(), mask2.ptr(), numel, 0.3, D, None, 9, 0, st),
           "actnn_dropout_forward", {"y": y2, "mask": mask2})
    dx2 = Guarded(numel, dtype, dev)
    _check(_lib, lib.actnn_dropout_backward(x.data_ptr(), mask2.ptr(), dx2.ptr(), numel, 0.3, D, st),
           "actnn_dropout_backward", {"dx": dx2})
    u = Guarded(numel, torch.float32, dev)
    _check(_lib, lib.actnn_dropout_uniform_fill(u.ptr(), numel, 9, 0, st), "actnn_dropout_uniform_fill", {"u": u})


@pytest.mark.parametrize("dtype", DTS)
@pytest.mark.parametrize("geom", [(1, 3, 7, 9, 3, 2, 1), (2, 5, 16, 16, 2, 2, 0), (3, 2, 11, 5, 3, 1, 1)])
def test_max_pool_entry_points_stay_inside_their_outputs(env, geom, dtype):
    lib, _lib, q, dev = env
    n, c, h, w, k, s, p = geom
    D = _lib.dtype_id(dtype)
    st = torch.cuda.current_stream().cuda_stream
    ho, wo = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
    x = torch.randn(n, c, h, w, generator=torch.Generator().manual_seed(h)).to(dtype).to(dev)
    y, idx = Guarded(n * c * ho * wo, dtype, dev), Guarded(n * c * ho * wo, torch.int8, dev)
    _check(_lib, lib.actnn_max_pool2d_forward(x.data_ptr(), y.ptr(), idx.ptr(), n, c, h, w, k, k, s, s, p, p, 1, 1, D,
                                              st), "actnn_max_pool2d_forward", {"y": y, "idx": idx})
    dx = Guarded(n * c * h * w, dtype, dev)
    _check(_lib, lib.actnn_max_pool2d_backward(y.ptr(), idx.ptr(), dx.ptr(), n, c, h, w, k, k, s, s, p, p, 1, 1, D, st),
           "actnn_max_pool2d_backward", {"dx": dx})


@pytest.mark.parametrize("dtype", DTS)
@pytest.mark.parametrize("shape", [(1, 1, 256), (3, 8, 288), (2, 5, 1280)])
def test_statistics_minmax_pass_stays_inside_its_outputs(env, shape, dtype):
    """actnn_batch_norm_stats_minimax and actnn_compress_mixed_prestat with guarded buffers."""
    lib, _lib, q, dev = env
    n, c, hw = shape
    if (c * hw) % 256:
        pytest.skip("geometry needs padding")
    D = _lib.dtype_id(dtype)
    sdt = torch.bfloat16 if dtype == torch.float32 else dtype
    S = _lib.dtype_id(sdt)
    st = torch.cuda.current_stream().cuda_stream
    g = c * hw // 256
    x = torch.randn(n, c, hw, generator=torch.Generator().manual_seed(hw)).to(dtype).to(dev)
    nbytes = lib.actnn_batch_norm_stats_minimax_workspace(n, c, hw)
    assert nbytes > 0
    bufs = {"min": Guarded(n * g, dtype, dev), "max": Guarded(n * g, dtype, dev), "mean": Guarded(c, torch.float32, dev),
            "invstd": Guarded(c, torch.float32, dev), "workspace": Guarded(nbytes, torch.uint8, dev)}
    _check(_lib, lib.actnn_batch_norm_stats_minimax(x.data_ptr(), bufs["min"].ptr(), bufs["max"].ptr(), None, None,
                                                    None, None, bufs["mean"].ptr(), bufs["invstd"].ptr(), n, c, hw,
                                                    0.1, 1e-5, D, bufs["workspace"].ptr(), nbytes, st),
           "actnn_batch_norm_stats_minimax", bufs)
    total = 2 * n
    cm = {"packed": Guarded(total * g * 256 // 32, torch.int32, dev), "scale": Guarded(n * g, sdt, dev),
          "min_out": Guarded(n * g, sdt, dev), "bits": Guarded(n, torch.int32, dev),
          "word_offsets": Guarded(n + 1, torch.int64, dev), "C": Guarded(n, torch.float32, dev),
          "ticket": Guarded(256, torch.uint8, dev)}
    _check(_lib, lib.actnn_compress_mixed_prestat(x.data_ptr(), bufs["min"].ptr(), bufs["max"].ptr(),
                                                  cm["packed"].ptr(), cm["scale"].ptr(), cm["min_out"].ptr(),
                                                  cm["bits"].ptr(), cm["word_offsets"].ptr(), cm["C"].ptr(),
                                                  cm["ticket"].ptr(), n, g, 256, D, S, 1.0, 1.0, None, 8, float(total),
                                                  1, None, 5, 0, st), "actnn_compress_mixed_prestat", cm)
    assert int(cm["bits"].t.sum()) == total
    # the variant with a kept ticket: same outputs, the ticket is zero before and after, twice in a row
    first = {k: v.t.clone() for k, v in cm.items() if k != "ticket"}
    assert int(cm["ticket"].t[:4].view(torch.int32)) == 0               # the call above left it at zero
    for _ in range(2):
        _check(_lib, lib.actnn_compress_mixed_prestat_kept(x.data_ptr(), bufs["min"].ptr(), bufs["max"].ptr(),
                                                           cm["packed"].ptr(), cm["scale"].ptr(), cm["min_out"].ptr(),
                                                           cm["bits"].ptr(), cm["word_offsets"].ptr(), cm["C"].ptr(),
                                                           cm["ticket"].ptr(), n, g, 256, D, S, 1.0, 1.0, None, 8,
                                                           float(total), 1, None, 5, 0, st),
               "actnn_compress_mixed_prestat_kept", cm)
        assert int(cm["ticket"].t[:4].view(torch.int32)) == 0
        for k, v in first.items():
            assert torch.equal(cm[k].t, v), k
