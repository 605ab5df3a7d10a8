"""ctypes binding of ``libactnn_b200.so`` (the C ABI declared in ``include/actnn_b200.h``).

This is the only place that touches the shared library.  There is no fallback of any
kind: if the library is missing or a call returns a non-zero status, a ``RuntimeError``
is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_uint64, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# ACTNN_B200_LIB: load another build of the library (same ABI) instead of the in-tree one
LIB_PATH = os.environ.get("ACTNN_B200_LIB") or os.path.join(_HERE, "csrc", "libactnn_b200.so")

F32, F16, BF16 = 0, 1, 2
_DTYPE_ID = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_CTYPES = {"P": c_void_p, "I": c_int, "L": c_int64, "U": c_uint64, "F": c_float, "D": c_double}

from ._signatures import SIGNATURES as _LETTERS  # noqa: E402

# name -> ctypes argument types, exactly as declared in include/actnn_b200.h
SIGNATURES = {name: [_CTYPES[c] for c in letters] for name, letters in _LETTERS.items()}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once; fail loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "actnn_b200: %s is missing. Build it with `python -m actnn_b200.csrc.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback." % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        lib.actnn_status_string.argtypes = [c_int]
        lib.actnn_status_string.restype = c_char_p
        lib.actnn_abi_version.argtypes = []
        lib.actnn_abi_version.restype = c_int
        lib.actnn_compress_mixed_workspace.argtypes = [c_int64, c_int64, c_int]
        lib.actnn_compress_mixed_workspace.restype = c_int64
        lib.actnn_calc_precision_workspace.argtypes = []
        lib.actnn_calc_precision_workspace.restype = c_int64
        lib.actnn_batch_norm_workspace.argtypes = [c_int64, c_int64, c_int64]
        lib.actnn_batch_norm_workspace.restype = c_int64
        lib.actnn_batch_norm_stats_minimax_workspace.argtypes = [c_int64, c_int64, c_int64]
        lib.actnn_batch_norm_stats_minimax_workspace.restype = c_int64
        lib.actnn_compress_mixed_static_capacity.argtypes = []
        lib.actnn_compress_mixed_static_capacity.restype = c_int64
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().actnn_status_string(status).decode()
        raise RuntimeError("%s failed: %s (status %d)" % (what, msg, status))


def dtype_id(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_ID[dtype]
    except KeyError:
        raise RuntimeError("actnn_b200: unsupported dtype %s" % dtype) from None


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_of_index(idx: int) -> int:
    if _raw_stream is not None:
        return _raw_stream(idx)
    return torch.cuda.current_stream(idx).cuda_stream


def stream_of(t: torch.Tensor) -> int:
    """The raw ``cudaStream_t`` of torch's current stream on the tensor's device."""
    if _raw_stream is not None:
        idx = t.device.index
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(t.device).cuda_stream


_scratch = {}


def scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """A uint8 scratch buffer of at least ``nbytes`` for kernels launched on the CURRENT stream
    of ``device``.  One grow-only buffer per (device, stream): the kernels that share it run in
    stream order, so the next user only starts when the previous one is done.  Saves a trip to
    the allocator in every layer of every step."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, stream_of_index(idx))
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(int(nbytes), 1 << 20)
        buf = _scratch[key] = torch.empty((size + 255) // 256 * 256, dtype=torch.uint8, device=device)
    return buf


_tickets = {}


def ticket(device: torch.device) -> torch.Tensor:
    """256 zeroed bytes per (device, current stream) that only ``actnn_compress_mixed_prestat_kept``
    uses: its kernels leave the ticket at zero, so it never needs clearing again."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, stream_of_index(idx))
    buf = _tickets.get(key)
    if buf is None:
        buf = _tickets[key] = torch.zeros(256, dtype=torch.uint8, device=device)
    return buf


_fns = {}
_fast = None
FAST_PATH = os.path.join(_HERE, "csrc", "_actnn_fastcall.so")


def _fast_module():
    """The generated CPython wrappers of the entry points (same library underneath, an order of
    magnitude less marshalling than ctypes); ``False`` when they were not built or another build
    of the library was requested."""
    global _fast
    if _fast is None:
        _fast = False
        if not os.environ.get("ACTNN_B200_LIB") and os.path.exists(FAST_PATH):
            import importlib.util
            load()                                            # libactnn_b200.so first: the wrappers link to it
            spec = importlib.util.spec_from_file_location("_actnn_fastcall", FAST_PATH)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _fast = mod
    return _fast


def call(name: str, tensor_for_device: torch.Tensor, *args) -> None:
    """Invoke ``name`` with the tensor's device current and check the status."""
    fn = _fns.get(name)
    if fn is None:
        fast = _fast_module()
        fn = _fns[name] = getattr(fast, name) if fast else getattr(load(), name)
    idx = tensor_for_device.device.index
    if idx is not None and idx != torch.cuda.current_device():
        with torch.cuda.device(idx):
            status = fn(*args)
    else:
        status = fn(*args)
    if status:
        check(status, name)


_staged_failures_seen = 0


def check_staged_pack(tensor: torch.Tensor, name: str) -> None:
    """With the opt-in staged single-stream pack (``ACTNN_STAGED_PACK=1``) a warp whose bounded
    wait for a bulk copy runs out leaves its part of the outputs unwritten and counts the event on
    the device.  The library call itself cannot know (it only enqueues), so the binding waits for
    the stream and reads the counter: a give-up becomes an error here instead of a silently
    corrupted activation.  The default pack has no waits and is not checked."""
    global _staged_failures_seen
    if os.environ.get("ACTNN_STAGED_PACK", "0") in ("", "0"):
        return
    import ctypes
    torch.cuda.current_stream(tensor.device).synchronize()
    count = ctypes.c_uint32(0)
    call("actnn_bulk_wait_failures", tensor, ctypes.addressof(count))
    if count.value > _staged_failures_seen:
        new = count.value - _staged_failures_seen
        _staged_failures_seen = count.value
        raise RuntimeError("%s: %d warps of the staged pack gave up waiting for a bulk copy; the packed "
                           "output is incomplete" % (name, new))


def next_philox(device: torch.device):
    """(seed, offset) from torch's default CUDA generator of ``device``; advances the offset
    so that ``torch.manual_seed`` reproduces a whole run, as the reference does with
    ``philox_engine_inputs`` (quantization_cuda_kernel.cu:115-121)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    gen = torch.cuda.default_generators[idx]
    seed, offset = gen.initial_seed(), gen.get_offset()
    gen.set_offset(offset + 4)
    return seed & 0xFFFFFFFFFFFFFFFF, offset
