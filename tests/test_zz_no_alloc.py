"""`actnn_compress_mixed_static`: the adaptive compress for callers that cannot provide
scratch memory (a plug-in that is only handed pointers, a job with a fixed memory plan).
It must give exactly what `actnn_compress_mixed` gives with a caller workspace, call after
call, although all calls share one array inside the library.  Collected last on purpose."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, _lib, x, static, seed):
    n, g, gs = x.shape
    dev = x.device
    total = 2 * n
    out = {
        "packed": torch.zeros(total * g * gs // 32, dtype=torch.int32, device=dev),
        "scale": torch.zeros(n, g, 1, dtype=x.dtype, device=dev),
        "mn": torch.zeros(n, g, 1, dtype=x.dtype, device=dev),
        "bits": torch.zeros(n, dtype=torch.int32, device=dev),
        "offsets": torch.zeros(n + 1, dtype=torch.int64, device=dev),
        "C": torch.zeros(n, dtype=torch.float32, device=dev),
    }
    dt = _lib.dtype_id(x.dtype)
    stream = torch.cuda.current_stream().cuda_stream
    head = [x.data_ptr(), out["packed"].data_ptr(), out["scale"].data_ptr(), out["mn"].data_ptr(),
            out["bits"].data_ptr(), out["offsets"].data_ptr(), out["C"].data_ptr()]
    tail = [n, g, gs, dt, dt, 256 / 64.0, 9 / 4, None, 8, float(total), 1, None, seed, 8, stream]
    if static:
        _lib.check(lib.actnn_compress_mixed_static(*head, *tail), "actnn_compress_mixed_static")
    else:
        ws_bytes = lib.actnn_compress_mixed_workspace(n, g, dt)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        _lib.check(lib.actnn_compress_mixed(*head, ws.data_ptr(), ws_bytes, *tail), "actnn_compress_mixed")
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_static_scratch_variant_matches_the_workspace_variant_twice_in_a_row(cuda_device, dtype):
    from actnn_b200 import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(42)
    shapes = [(24, 16, 256), (7, 40, 256)]           # second call: other size, stale bytes left by the first
    for call, shape in enumerate(shapes):
        x = (torch.randn(*shape, generator=g) * torch.exp(torch.randn(shape[0], 1, 1, generator=g))).to(dtype)
        x = x.to(cuda_device)
        ref = _run(lib, _lib, x, static=False, seed=100 + call)
        got = _run(lib, _lib, x, static=True, seed=100 + call)
        for key in ref:                               # integer outputs and statistics: bit-exact
            assert torch.equal(ref[key], got[key]), (call, key)
        assert int(got["bits"].sum()) == 2 * shape[0]


def test_static_scratch_variant_allocates_nothing_and_takes_the_largest_size(cuda_device):
    """The largest problem that fits (1 Mi groups of float16: exactly the capacity), and the
    property the entry point exists for: across a call neither the driver's free memory nor
    torch's count of device allocations moves."""
    from actnn_b200 import _lib
    lib = _lib.load()
    n, g = 1024, 1024
    assert lib.actnn_compress_mixed_workspace(n, g, 1) == lib.actnn_compress_mixed_static_capacity()
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(n, g, 256, generator=gen).to(torch.float16).to(cuda_device)
    ref = _run(lib, _lib, x, static=False, seed=5)
    _run(lib, _lib, x, static=True, seed=5)              # first call on the device: looks the array up
    total = 2 * n
    out = {
        "packed": torch.zeros(total * g * 256 // 32, dtype=torch.int32, device=cuda_device),
        "scale": torch.zeros(n, g, 1, dtype=x.dtype, device=cuda_device),
        "mn": torch.zeros(n, g, 1, dtype=x.dtype, device=cuda_device),
        "bits": torch.zeros(n, dtype=torch.int32, device=cuda_device),
        "offsets": torch.zeros(n + 1, dtype=torch.int64, device=cuda_device),
        "C": torch.zeros(n, dtype=torch.float32, device=cuda_device),
    }
    dt = _lib.dtype_id(x.dtype)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    allocs_before = torch.cuda.memory_stats()["num_device_alloc"]
    st = lib.actnn_compress_mixed_static(
        x.data_ptr(), out["packed"].data_ptr(), out["scale"].data_ptr(), out["mn"].data_ptr(), out["bits"].data_ptr(),
        out["offsets"].data_ptr(), out["C"].data_ptr(), n, g, 256, dt, dt, 256 / 64.0, 9 / 4, None, 8, float(total), 1,
        None, 5, 8, stream)
    torch.cuda.synchronize()
    assert st == 0
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_stats()["num_device_alloc"] == allocs_before
    for key in ref:
        assert torch.equal(ref[key], out[key]), key


def test_static_scratch_variant_rejects_what_does_not_fit(cuda_device):
    from actnn_b200 import _lib
    lib = _lib.load()
    cap = lib.actnn_compress_mixed_static_capacity()
    assert cap == (4 << 20) + 256                     # 4 MiB of min / max and the ticket block
    n, g = 2048, 1024                                 # 2 Mi groups of float16: 8 MiB of min / max
    assert lib.actnn_compress_mixed_workspace(n, g, 1) > cap
    dummy = torch.zeros(64, device=cuda_device)
    st = lib.actnn_compress_mixed_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                         dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), n, g, 256, 1, 1,
                                         1.0, 1.0, None, 8, float(2 * n), 1, None, 0, 0, None)
    assert st == 8                                    # ACTNN_ERR_CAPACITY, nothing launched
    with pytest.raises(RuntimeError, match="capacity"):
        _lib.check(st, "actnn_compress_mixed_static")
