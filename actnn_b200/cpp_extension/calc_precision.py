"""Greedy bit allocation on the GPU.

``calc_precision(b, C, w, target) -> b`` mirrors
actnn/actnn/cpp_extension/calc_precision.cc:9-50.  The reference runs a priority queue on
CPU tensors; here the same result comes from one CUDA kernel.  CPU tensors are accepted
(copied to the current device and back, as a drop-in must); CUDA tensors are processed in
place without any host synchronisation.  ``allocate_bits`` is the sync-free entry the
schemes use: it also returns the word offsets of the mixed-precision stream."""
import torch

from .. import _lib


def _uniform_initial_bits(b: torch.Tensor) -> int:
    first = int(b[0])
    if not bool((b == first).all()):
        raise RuntimeError("calc_precision: all entries of b must start from the same bit width")
    return first


def allocate_bits(C: torch.Tensor, initial_bits: int, target: float, w: torch.Tensor = None,
                  num_groups: int = 0, group_size: int = 256, with_offsets: bool = False):
    """``C`` float32 CUDA ``[N]`` -> ``(bits int32 [N], word_offsets int64 [N+1] or None)``."""
    if not C.is_cuda or C.dtype != torch.float32 or not C.is_contiguous():
        raise RuntimeError("C must be a contiguous float32 CUDA tensor!")
    n = C.numel()
    bits = torch.empty(n, dtype=torch.int32, device=C.device)
    offsets = torch.empty(n + 1, dtype=torch.int64, device=C.device) if with_offsets else None
    if w is not None and (not w.is_cuda or w.dtype != torch.int32 or not w.is_contiguous() or w.numel() != n):
        raise RuntimeError("w must be a contiguous int32 CUDA tensor of the same length as C!")
    # weighted or large problems run as multi-block launches over a small workspace
    ws = None
    if not with_offsets and (w is not None or n * (int(initial_bits) - 1) > 8192):
        ws = torch.empty(256, dtype=torch.uint8, device=C.device)
    _lib.call("actnn_calc_precision", C, C.data_ptr(), _lib.ptr(w), n, int(initial_bits), float(target),
              bits.data_ptr(), _lib.ptr(offsets), int(num_groups), int(group_size), _lib.ptr(ws),
              0 if ws is None else 256, _lib.stream_of(C))
    return bits, offsets


def sensitivity(mn: torch.Tensor, mx: torch.Tensor, n: int, range_factor: float, coeff: float = 1.0,
                grad_scale: torch.Tensor = None) -> torch.Tensor:
    """``C[n] = coeff * (float(norm(mx[n]-mn[n]))**2 * range_factor) [* grad_scale]`` in float32
    (actnn/actnn/qscheme.py:80-85, qbnscheme.py:42-45) with one kernel."""
    g = mn.numel() // max(n, 1)
    C = torch.empty(n, dtype=torch.float32, device=mn.device)
    if grad_scale is not None and (grad_scale.dtype != torch.float32 or not grad_scale.is_cuda
                                   or grad_scale.numel() != 1):
        raise RuntimeError("grad_scale must be a float32 CUDA tensor with one element!")
    _lib.call("actnn_range_sqr", mn, mn.data_ptr(), mx.data_ptr(), n, g, _lib.dtype_id(mn.dtype),
              float(range_factor), float(coeff), _lib.ptr(grad_scale), C.data_ptr(), _lib.stream_of(mn))
    return C


def sample_sumsq(grad: torch.Tensor) -> torch.Tensor:
    """``grad.view(N, -1).float().norm(dim=1).square()`` (actnn/actnn/qscheme.py:50,54) in one
    read of ``grad``: float32 ``[N]``."""
    if not grad.is_cuda or grad.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError("grad must be a floating-point CUDA tensor!")
    grad = grad.contiguous()
    n = grad.shape[0]
    out = torch.empty(n, dtype=torch.float32, device=grad.device)
    _lib.call("actnn_sample_sumsq", grad, grad.data_ptr(), out.data_ptr(), n, grad.numel() // max(n, 1),
              _lib.dtype_id(grad.dtype), _lib.stream_of(grad))
    return out


def calc_precision(b: torch.Tensor, C: torch.Tensor, w: torch.Tensor, target) -> torch.Tensor:
    for t, name in ((b, "b"), (C, "C"), (w, "w")):
        if not t.is_contiguous():
            raise RuntimeError("%s must be contiguous!" % name)
    if b.dtype != torch.int32 or w.dtype != torch.int32 or C.dtype != torch.float32:
        raise RuntimeError("calc_precision expects int32 b, float32 C and int32 w")
    if b.numel() == 0:
        return b
    on_cpu = not C.is_cuda
    if on_cpu:
        if not torch.cuda.is_available():
            raise RuntimeError("actnn_b200 needs a CUDA device; there is no CPU implementation")
        initial = _uniform_initial_bits(b)
        unit_w = bool((w == 1).all())
        dev = torch.device("cuda", torch.cuda.current_device())
        bits, _ = allocate_bits(C.to(dev), initial, float(target), None if unit_w else w.to(dev))
        b.copy_(bits)                      # the reference mutates b in place and returns it
        return b
    initial = _uniform_initial_bits(b)     # one host read, only on this compatibility entry
    bits, _ = allocate_bits(C, initial, float(target), w if w.is_cuda else w.to(C.device))
    b.copy_(bits)
    return b
