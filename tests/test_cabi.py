"""The C ABI without a GPU: the library loads, exports everything the header declares,
and rejects bad arguments on the host before anything would be launched."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "actnn_b200.h")


@pytest.fixture(scope="module")
def lib(built_library):
    from actnn_b200 import _lib
    return _lib.load()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(actnn_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from actnn_b200 import _lib
    names = declared_functions()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), "libactnn_b200.so does not export " + name
    bound = set(_lib.SIGNATURES) | {"actnn_status_string", "actnn_abi_version", "actnn_compress_mixed_workspace",
                                     "actnn_compress_mixed_static_capacity", "actnn_calc_precision_workspace",
                                     "actnn_batch_norm_workspace", "actnn_batch_norm_stats_minimax_workspace"}
    assert bound == set(names)


def test_every_entry_point_cites_the_reference():
    """The comment above each declaration names the reference file:line it replaces (or says
    that the reference has no counterpart)."""
    text = open(HEADER).read()
    for name in declared_functions():
        if name in ("actnn_status_string", "actnn_abi_version"):
            continue
        head = text[:re.search(r"\b(int|int64_t) " + name + r"\(", text).start()]
        section = head[head.rindex("/* ------"):]
        assert re.search(r"\.(cc|cu|py):\d+", section) or "counterpart" in section, name


def test_status_strings(lib):
    assert lib.actnn_abi_version() >= 1
    seen = {lib.actnn_status_string(i) for i in range(9)}
    assert len(seen) == 9 and lib.actnn_status_string(0) == b"ok"


def test_host_side_validation_needs_no_gpu(lib):
    OK, NULL, DTYPE, SHAPE, BITS, ALIGN, ARG = 0, 1, 2, 3, 4, 5, 6
    assert lib.actnn_minimax(None, None, None, 4, 30, 0, None) == SHAPE
    assert lib.actnn_minimax(None, None, None, 4, 32, 0, None) == SHAPE          # D > 32
    assert lib.actnn_minimax(None, None, None, 0, 256, 0, None) == OK            # empty input
    assert lib.actnn_minimax(None, None, None, 4, 256, 0, None) == NULL
    assert lib.actnn_minimax(16, 16, 16, 4, 256, 7, None) == DTYPE
    assert lib.actnn_minimax(8, 16, 16, 4, 256, 1, None) == ALIGN
    # pack / unpack
    assert lib.actnn_pack_single(None, None, None, 3, None, None, None, 1, 1, 256, 0, 0, 1, None, 0, 0, None) == BITS
    assert lib.actnn_pack_single(None, None, None, 2, None, None, None, 1, 1, 100, 0, 0, 1, None, 0, 0, None) == SHAPE   # not a multiple of 32
    assert lib.actnn_pack_single(None, None, None, 2, None, None, None, 1, 1, 256, 1, 0, 1, None, 0, 0, None) == DTYPE
    assert lib.actnn_pack_single(None, None, None, 2, None, None, None, 1, 1, 256, 0, 0, 1, None, 0, 0, None) == NULL
    assert lib.actnn_pack_mixed(None, None, None, None, None, None, None, None, -1, 1, 256, 0, 0, 1, None, 0, 0, None) == SHAPE
    assert lib.actnn_pack_mixed(None, None, None, None, None, None, None, None, 0, 1, 256, 0, 0, 1, None, 0, 0, None) == OK
    assert lib.actnn_pack_mixed(None, None, None, None, None, None, None, None, 2, 1, 256, 0, 0, 1, None, 0, 0, None) == NULL
    assert lib.actnn_unpack_mixed(None, None, None, None, None, None, 2, 1, 256, 2, 0, None) == DTYPE
    assert lib.actnn_unpack_single(None, 8, None, None, None, 2, 1, 256, 0, 2, None) == NULL
    # bit allocation
    assert lib.actnn_calc_precision(None, None, 4, 0, 8.0, None, None, 0, 256, None, 0, None) == BITS
    assert lib.actnn_calc_precision(None, None, 4, 8, float("nan"), None, None, 0, 256, None, 0, None) == ARG
    assert lib.actnn_calc_precision(None, None, 4, 8, 8.0, None, None, 0, 256, None, 0, None) == NULL
    assert lib.actnn_bits_prefix(None, 4, 1, 100, None, None) == NULL
    # mask ops
    assert lib.actnn_relu_forward(None, None, None, -1, 0, None) == SHAPE
    assert lib.actnn_relu_forward(None, None, None, 0, 0, None) == OK
    assert lib.actnn_relu_forward(None, None, None, 5, 0, None) == NULL
    assert lib.actnn_dropout_forward(None, None, None, 5, ctypes.c_float(1.5), 0, None, 0, 0, None) == ARG
    assert lib.actnn_max_pool2d_forward(None, None, None, 1, 1, 8, 8, 4, 4, 1, 1, 0, 0, 1, 1, 0, None) == ARG
    assert lib.actnn_max_pool2d_forward(None, None, None, 1, 1, 8, 8, 2, 2, 2, 2, 0, 0, 1, 1, 0, None) == NULL
    assert lib.actnn_noise_fill(None, 8, 0, 1, 2, None) == NULL
    # one-call adaptive compress: workspace size and capacity check
    assert lib.actnn_compress_mixed_workspace(4, 3, 1) == 2 * 256 + 256
    assert lib.actnn_compress_mixed_workspace(512, 784, 0) == 2 * 512 * 784 * 4 + 256
    assert lib.actnn_compress_mixed_workspace(-1, 3, 1) == -1
    args = [256] * 8 + [8, 4, 3, 256, 1, 1, 1.0, 1.0, None, 8, 8.0, 1, None, 0, 0, None]
    assert lib.actnn_compress_mixed(*args) == 8                      # ACTNN_ERR_CAPACITY: workspace too small
    args[8] = 1 << 20
    args[11] = 100                                                   # group size not a multiple of 32
    assert lib.actnn_compress_mixed(*args) == SHAPE


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    from actnn_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_calc_precision_has_no_cpu_path():
    import torch
    if torch.cuda.is_available():
        pytest.skip("only meaningful on a machine without a GPU")
    from actnn_b200.cpp_extension import calc_precision
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        calc_precision.calc_precision(torch.ones(4, dtype=torch.int32) * 8, torch.ones(4),
                                      torch.ones(4, dtype=torch.int32), 8)


def test_package_api_surface():
    import actnn_b200 as actnn
    for name in ("set_optimization_level", "QModule", "QConv1d", "QConv2d", "QConv3d", "QConvTranspose2d",
                 "QLinear", "QBatchNorm1d", "QBatchNorm2d", "QBatchNorm3d", "QSyncBatchNorm", "QReLU",
                 "QDropout", "QMaxPool2d", "QScheme", "QBNScheme", "config"):
        assert hasattr(actnn, name)
    from actnn_b200.cpp_extension import backward_func, calc_precision, minimax, quantization
    for fn in ("pack_mixed_precision", "unpack_mixed_precision", "pack_single_precision",
               "unpack_single_precision", "act_quantized_relu", "act_quantized_dropout",
               "act_quantized_max_pool2d"):
        assert callable(getattr(quantization, fn))
    assert callable(minimax.minimax) and callable(calc_precision.calc_precision)
    assert callable(backward_func.cudnn_convolution_backward)


def test_host_code_past_validation_returns_without_a_gpu(lib):
    """On a machine without a GPU the entry points get past their argument checks, fail to
    launch and say so; they must not spin or block in host code."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("would launch kernels on made-up pointers")
    LAUNCH = 7
    assert lib.actnn_calc_precision(256, None, 4, 8, 8.0, 256, None, 0, 256, None, 0, None) == LAUNCH
    assert lib.actnn_minimax(256, 256, 256, 8, 256, 1, None) == LAUNCH
    args = [256] * 8 + [1 << 20, 4, 32, 256, 1, 1, 1.0, 1.0, None, 8, 8.0, 1, None, 0, 0, None]
    assert lib.actnn_compress_mixed(*args) == LAUNCH


def test_fast_binding_exports_every_entry_point_and_validates_like_ctypes(lib):
    """The generated CPython wrappers (csrc/_actnn_fastcall.so) are the binding the package calls
    through; they must carry every entry point of the signature table and hand arguments over
    unchanged (checked on calls that return from host-side validation, so without a GPU)."""
    from actnn_b200 import _lib
    fast = _lib._fast_module()
    assert fast, "fast binding was not built"
    for name, letters in _lib._LETTERS.items():
        assert hasattr(fast, name), name
    assert fast.actnn_minimax(None, None, None, 4, 30, 0, None) == lib.actnn_minimax(None, None, None, 4, 30, 0, None) != 0
    assert fast.actnn_minimax(None, None, None, 0, 256, 0, None) == 0
    with pytest.raises(TypeError):
        fast.actnn_minimax(None, None, None, 0, 256, 0)
    with pytest.raises(TypeError):
        fast.actnn_minimax(None, None, None, 0.5, 256, 0, None)


def test_staged_pack_give_up_becomes_an_error(monkeypatch):
    """The binding turns a non-zero wait-failure counter of the opt-in staged pack into an error
    (host logic only: the library call and the stream are faked)."""
    import torch
    from actnn_b200 import _lib

    class FakeStream:
        def synchronize(self):
            pass

    counter = {"value": 0}

    def fake_call(name, tensor, address):
        assert name == "actnn_bulk_wait_failures"
        ctypes.c_uint32.from_address(address).value = counter["value"]

    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: FakeStream())
    monkeypatch.setattr(_lib, "call", fake_call)
    monkeypatch.setattr(_lib, "_staged_failures_seen", 0)
    x = torch.zeros(1)
    monkeypatch.delenv("ACTNN_STAGED_PACK", raising=False)
    counter["value"] = 5
    _lib.check_staged_pack(x, "actnn_pack_single")             # default pack: never checked
    monkeypatch.setenv("ACTNN_STAGED_PACK", "1")
    counter["value"] = 0
    _lib.check_staged_pack(x, "actnn_pack_single")
    counter["value"] = 3
    with pytest.raises(RuntimeError, match="3 warps"):
        _lib.check_staged_pack(x, "actnn_pack_single")
    _lib.check_staged_pack(x, "actnn_pack_single")             # the same three are not reported twice
