"""Pack / unpack and the mask-saving activations.

Mirror of actnn/actnn/cpp_extension/quantization.cc:46-206: same function names,
positional arguments and return types (``int32`` words for the mixed-precision stream,
``int8`` bytes for the single-precision one).  Keyword-only extras let the glue in
``actnn_b200.ops`` avoid every host synchronisation and inject rounding noise:

* ``noise``          tensor shaped like ``data`` with values in [-0.5, 0.5]; default: Philox
                     noise keyed by torch's CUDA generator;
* ``word_offsets`` / ``total_bits``   the prefix of ``bits`` and its sum when the caller
                     already knows them (otherwise one ``.item()`` as in the reference,
                     quantization_cuda_kernel.cu:97-98);
* ``stat_dtype``     ``torch.bfloat16`` to write scale (and ``mn_out``) of float32 data in the
                     reference's storage format (actnn/actnn/ops.py:115-116) directly.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import _lib
from ._checks import check_cuda_tensor

GROUP_SIZE = 256            # the size the fast kernels are written for; other multiples of 32 take a generic path
MAX_GROUP_SIZE = 8192


def _check_group_size(gs: int) -> None:
    if gs % 32 != 0 or gs <= 32:
        raise RuntimeError("Expected group_size % 32 == 0 (and group_size > 32) to be true, but got false.")
    if gs > MAX_GROUP_SIZE:
        raise RuntimeError("actnn_b200: group sizes above %d are not supported" % MAX_GROUP_SIZE)


def _noise_args(data: torch.Tensor, stochastic: bool, noise: Optional[torch.Tensor], philox):
    if not stochastic:
        return 0, 0, 0
    if noise is not None:
        check_cuda_tensor(noise, "noise", dtype=data.dtype)
        if noise.numel() != data.numel():
            raise RuntimeError("noise must have as many elements as data!")
        return noise.data_ptr(), 0, 0
    seed, offset = philox if philox is not None else _lib.next_philox(data.device)
    return 0, seed, offset


def _stat_dtype(data_dtype: torch.dtype, stat_dtype: Optional[torch.dtype]) -> torch.dtype:
    if stat_dtype is None or stat_dtype == data_dtype:
        return data_dtype
    if data_dtype == torch.float32 and stat_dtype == torch.bfloat16:
        return stat_dtype
    raise RuntimeError("statistics must have the data dtype (or bfloat16 for float32 data)")


# ------------------------------------------------------------------------------- mixed
def bits_prefix(bits: torch.Tensor, num_groups: int, group_size: int = GROUP_SIZE) -> torch.Tensor:
    """``word_offsets[n]`` = first int32 word of sample ``n``; last entry = total words."""
    check_cuda_tensor(bits, "bits", 1, torch.int32)
    n = bits.numel()
    offsets = torch.empty(n + 1, dtype=torch.int64, device=bits.device)
    _lib.call("actnn_bits_prefix", bits, bits.data_ptr(), n, num_groups, group_size, offsets.data_ptr(),
              _lib.stream_of(bits))
    return offsets


def pack_mixed_precision(data, min, max, bits, stochastic, *, noise=None, philox=None, word_offsets=None,
                         total_bits: Optional[int] = None, stat_dtype=None, return_min: bool = False):
    check_cuda_tensor(data, "data", 3)
    check_cuda_tensor(min, "min", 3, data.dtype)
    check_cuda_tensor(max, "max", 3, data.dtype)
    check_cuda_tensor(bits, "bits", 1, torch.int32)
    n, g, gs = data.shape
    if gs % 32 != 0:
        raise RuntimeError("Expected group_size % bits_per_int == 0 to be true, but got false.")
    _check_group_size(gs)
    if word_offsets is None:
        word_offsets = bits_prefix(bits, g, gs)
    if total_bits is None:
        # the reference-style call: one host read for the size (quantization_cuda_kernel.cu:97-98);
        # the same read checks the widths, which the kernels cannot refuse on their own
        lo, hi, words = (int(v) for v in torch.stack([bits.min().long(), bits.max().long(),
                                                      word_offsets[-1]]).tolist()) if n else (1, 1, 0)
        if lo < 1 or hi > 8:
            raise RuntimeError("pack_mixed_precision: bit widths must lie in 1..8, got %d..%d "
                               "(unsupported bit width)" % (lo, hi))
    else:
        words = (int(total_bits) * g * gs + 31) // 32
    sdt = _stat_dtype(data.dtype, stat_dtype)
    packed = torch.empty(words, dtype=torch.int32, device=data.device)
    scale = torch.empty((n, g, 1), dtype=sdt, device=data.device)
    mn_out = torch.empty((n, g, 1), dtype=sdt, device=data.device) if return_min else None
    nz, seed, offset = _noise_args(data, stochastic, noise, philox)
    _lib.call("actnn_pack_mixed", data, data.data_ptr(), min.data_ptr(), max.data_ptr(), bits.data_ptr(),
              word_offsets.data_ptr(), packed.data_ptr(), scale.data_ptr(), _lib.ptr(mn_out), n, g, gs,
              _lib.dtype_id(data.dtype), _lib.dtype_id(sdt), int(bool(stochastic)), nz, seed, offset,
              _lib.stream_of(data))
    packed.word_offsets = word_offsets          # lets the unpack skip the prefix kernel
    if return_min:
        return packed, scale, mn_out
    return packed, scale


def compress_mixed_precision(data, target_bits: int, initial_bits: int, range_factor: float, coeff: float = 1.0,
                             grad_scale=None, stochastic=True, *, noise=None, philox=None, stat_dtype=None,
                             minmax=None):
    """The adaptive compress of ``data [N, G, 256]`` in one native call: min/max,
    sensitivities, greedy allocation at ``target_bits`` total bits, pack.

    Equivalent to ``QScheme.compute_quantization_bits`` followed by ``pack_mixed_precision``
    (actnn/actnn/qscheme.py:57-94, ops.py:44-48) with no host synchronisation.
    ``minmax=(mn, mx)``: the per-group extrema when a previous pass already produced them
    (``backward_func.batch_norm_stats_minimax``); the activation is then read once, not twice.
    Returns ``(packed, bits, scale, min, C)``; ``packed.word_offsets`` is set."""
    check_cuda_tensor(data, "data", 3)
    n, g, gs = data.shape
    _check_group_size(gs)
    sdt = _stat_dtype(data.dtype, stat_dtype)
    total = min(initial_bits * n, max(int(target_bits), n))        # what the greedy ends with
    dev = data.device
    packed = torch.empty((total * g * gs + 31) // 32, dtype=torch.int32, device=dev)
    scale = torch.empty((n, g, 1), dtype=sdt, device=dev)
    mn = torch.empty((n, g, 1), dtype=sdt, device=dev)
    bits = torch.empty(n, dtype=torch.int32, device=dev)
    offsets = torch.empty(n + 1, dtype=torch.int64, device=dev)
    C = torch.empty(n, dtype=torch.float32, device=dev)
    if grad_scale is not None and (grad_scale.dtype != torch.float32 or not grad_scale.is_cuda
                                   or grad_scale.numel() != 1):
        raise RuntimeError("grad_scale must be a float32 CUDA tensor with one element!")
    nz, seed, offset = _noise_args(data, stochastic, noise, philox)
    if minmax is not None:
        gmn, gmx = minmax
        check_cuda_tensor(gmn, "min", dtype=data.dtype)
        check_cuda_tensor(gmx, "max", dtype=data.dtype)
        if gmn.numel() != n * g or gmx.numel() != n * g:
            raise RuntimeError("min / max must have one element per group!")
        workspace = _lib.ticket(dev)
        _lib.call("actnn_compress_mixed_prestat_kept", data, data.data_ptr(), gmn.data_ptr(), gmx.data_ptr(),
                  packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), bits.data_ptr(), offsets.data_ptr(),
                  C.data_ptr(), workspace.data_ptr(), n, g, gs, _lib.dtype_id(data.dtype), _lib.dtype_id(sdt),
                  float(range_factor), float(coeff), _lib.ptr(grad_scale), int(initial_bits), float(target_bits),
                  int(bool(stochastic)), nz, seed, offset, _lib.stream_of(data))
        packed.word_offsets = offsets
        bits.word_offsets = offsets
        bits.total_bits = total
        return packed, bits, scale, mn, C
    ws_bytes = 2 * ((n * g * data.element_size() + 255) // 256 * 256) + 256     # actnn_compress_mixed_workspace
    workspace = _lib.scratch(dev, ws_bytes)
    _lib.call("actnn_compress_mixed", data, data.data_ptr(), packed.data_ptr(), scale.data_ptr(), mn.data_ptr(),
              bits.data_ptr(), offsets.data_ptr(), C.data_ptr(), workspace.data_ptr(), ws_bytes, n, g, gs,
              _lib.dtype_id(data.dtype), _lib.dtype_id(sdt), float(range_factor), float(coeff),
              _lib.ptr(grad_scale), int(initial_bits), float(target_bits), int(bool(stochastic)), nz, seed, offset,
              _lib.stream_of(data))
    packed.word_offsets = offsets
    bits.word_offsets = offsets
    bits.total_bits = total
    return packed, bits, scale, mn, C


def unpack_mixed_precision(data, bits, scale, min, N, num_groups, group_size, *, word_offsets=None,
                           out_dtype=None):
    check_cuda_tensor(data, "data", 1, torch.int32)
    check_cuda_tensor(bits, "bits", 1, torch.int32)
    check_cuda_tensor(scale, "scale", 3)
    check_cuda_tensor(min, "min", 3, scale.dtype)
    if group_size % 32 != 0:
        raise RuntimeError("Expected group_size % 32 == 0 to be true, but got false.")
    _check_group_size(group_size)
    out_dtype = scale.dtype if out_dtype is None else out_dtype
    _stat_dtype(out_dtype, scale.dtype)
    if word_offsets is None:
        word_offsets = getattr(data, "word_offsets", None)
    if word_offsets is None:
        word_offsets = bits_prefix(bits, num_groups, group_size)
    out = torch.empty((N, num_groups, group_size), dtype=out_dtype, device=data.device)
    _lib.call("actnn_unpack_mixed", data, data.data_ptr(), bits.data_ptr(), word_offsets.data_ptr(),
              scale.data_ptr(), min.data_ptr(), out.data_ptr(), N, num_groups, group_size,
              _lib.dtype_id(out_dtype), _lib.dtype_id(scale.dtype), _lib.stream_of(data))
    return out


# ------------------------------------------------------------------------------- single
def single_precision_bytes(bits: int, n: int, num_groups: int, group_size: int) -> int:
    wpt = 8 // bits
    n_round = n + (wpt - n % wpt) % wpt
    return (bits * n_round * num_groups * group_size + 8) // 8


def _check_single_bits(bits):
    if not isinstance(bits, int) or bits <= 0 or 8 % bits != 0:
        raise RuntimeError("Expected 8 % bits == 0 to be true, but got false.")


def pack_single_precision(data, min, max, bits, stochastic, *, noise=None, philox=None, stat_dtype=None,
                          return_min: bool = False):
    check_cuda_tensor(data, "data", 3)
    check_cuda_tensor(min, "min", 3, data.dtype)
    check_cuda_tensor(max, "max", 3, data.dtype)
    _check_single_bits(bits)
    n, g, gs = data.shape
    _check_group_size(gs)
    sdt = _stat_dtype(data.dtype, stat_dtype)
    packed = torch.empty(single_precision_bytes(bits, n, g, gs), dtype=torch.int8, device=data.device)
    scale = torch.empty((n, g, 1), dtype=sdt, device=data.device)
    mn_out = torch.empty((n, g, 1), dtype=sdt, device=data.device) if return_min else None
    nz, seed, offset = _noise_args(data, stochastic, noise, philox)
    _lib.call("actnn_pack_single", data, data.data_ptr(), min.data_ptr(), max.data_ptr(), bits,
              packed.data_ptr(), scale.data_ptr(), _lib.ptr(mn_out), n, g, gs, _lib.dtype_id(data.dtype),
              _lib.dtype_id(sdt), int(bool(stochastic)), nz, seed, offset, _lib.stream_of(data))
    _lib.check_staged_pack(data, "actnn_pack_single")
    if return_min:
        return packed, scale, mn_out
    return packed, scale


def compress_single_precision(data, bits, stochastic=True, *, noise=None, philox=None, stat_dtype=None,
                              return_max: bool = False):
    """Fused min/max + stochastic rounding + pack in one read of ``data [N, G, 256]``.

    Equivalent to ``minimax`` followed by ``pack_single_precision``
    (actnn/actnn/ops.py:77-96, 44-48).  Returns ``(packed, scale, min[, max])``."""
    check_cuda_tensor(data, "data", 3)
    _check_single_bits(bits)
    n, g, gs = data.shape
    _check_group_size(gs)
    sdt = _stat_dtype(data.dtype, stat_dtype)
    packed = torch.empty(single_precision_bytes(bits, n, g, gs), dtype=torch.int8, device=data.device)
    scale = torch.empty((n, g, 1), dtype=sdt, device=data.device)
    mn = torch.empty((n, g, 1), dtype=sdt, device=data.device)
    mx = torch.empty((n, g, 1), dtype=sdt, device=data.device) if return_max else None
    nz, seed, offset = _noise_args(data, stochastic, noise, philox)
    _lib.call("actnn_compress_single", data, data.data_ptr(), bits, packed.data_ptr(), scale.data_ptr(),
              mn.data_ptr(), _lib.ptr(mx), n, g, gs, _lib.dtype_id(data.dtype), _lib.dtype_id(sdt),
              int(bool(stochastic)), nz, seed, offset, _lib.stream_of(data))
    _lib.check_staged_pack(data, "actnn_compress_single")
    if return_max:
        return packed, scale, mn, mx
    return packed, scale, mn


def unpack_single_precision(data, bits, scale, min, N, num_groups, group_size, *, out_dtype=None):
    check_cuda_tensor(data, "data", 1, torch.int8)
    check_cuda_tensor(scale, "scale", 3)
    check_cuda_tensor(min, "min", 3, scale.dtype)
    _check_single_bits(bits)
    _check_group_size(group_size)
    out_dtype = scale.dtype if out_dtype is None else out_dtype
    _stat_dtype(out_dtype, scale.dtype)
    out = torch.empty((N, num_groups, group_size), dtype=out_dtype, device=data.device)
    _lib.call("actnn_unpack_single", data, data.data_ptr(), bits, scale.data_ptr(), min.data_ptr(),
              out.data_ptr(), N, num_groups, group_size, _lib.dtype_id(out_dtype), _lib.dtype_id(scale.dtype),
              _lib.stream_of(data))
    return out


def noise_fill(numel: int, dtype: torch.dtype, device, seed: int, offset: int) -> torch.Tensor:
    """The noise ``pack_*`` draws for ``philox=(seed, offset)``, as a flat tensor."""
    out = torch.empty(numel, dtype=dtype, device=device)
    _lib.call("actnn_noise_fill", out, out.data_ptr(), numel, _lib.dtype_id(dtype), seed, offset,
              _lib.stream_of(out))
    return out


# ------------------------------------------------------------------------------- ReLU
def relu_forward(x: torch.Tensor, with_minmax: bool = False):
    """``(y, mask)``; with ``with_minmax`` (``x.numel() % 256 == 0``) also the min and the max of
    every 256 consecutive outputs, from the same pass: ``(y, mask, mn, mx)``."""
    y = torch.empty_like(x)
    mask = torch.empty((x.numel() + 31) // 32, dtype=torch.int32, device=x.device)
    if with_minmax:
        groups = x.numel() // 256
        mn = torch.empty(groups, dtype=x.dtype, device=x.device)
        mx = torch.empty(groups, dtype=x.dtype, device=x.device)
        _lib.call("actnn_relu_forward_minimax", x, x.data_ptr(), y.data_ptr(), mask.data_ptr(), mn.data_ptr(),
                  mx.data_ptr(), x.numel(), _lib.dtype_id(x.dtype), _lib.stream_of(x))
        return y, mask, mn, mx
    _lib.call("actnn_relu_forward", x, x.data_ptr(), y.data_ptr(), mask.data_ptr(), x.numel(),
              _lib.dtype_id(x.dtype), _lib.stream_of(x))
    return y, mask


def relu_backward(grad_output: torch.Tensor, mask: torch.Tensor):
    grad_output = grad_output.contiguous()
    grad_input = torch.empty_like(grad_output)
    _lib.call("actnn_relu_backward", grad_output, grad_output.data_ptr(), mask.data_ptr(),
              grad_input.data_ptr(), grad_output.numel(), _lib.dtype_id(grad_output.dtype),
              _lib.stream_of(grad_output))
    return grad_input


class _ActQuantizedReLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y, mask = relu_forward(x)
        ctx.save_for_backward(mask)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        return relu_backward(grad_output, mask)


class _ActQuantizedReLUMinmax(torch.autograd.Function):
    """The same op; the forward pass also returns the per-group extrema of its output."""

    @staticmethod
    def forward(ctx, x):
        y, mask, mn, mx = relu_forward(x, with_minmax=True)
        ctx.save_for_backward(mask)
        ctx.mark_non_differentiable(mn, mx)
        return y, mn, mx

    @staticmethod
    def backward(ctx, grad_output, _grad_mn, _grad_mx):
        (mask,) = ctx.saved_tensors
        return relu_backward(grad_output, mask)


def act_quantized_relu(input: torch.Tensor) -> torch.Tensor:
    check_cuda_tensor(input, "input")
    return _ActQuantizedReLU.apply(input)


def act_quantized_relu_with_minmax(input: torch.Tensor, group_size: int = 256):
    """``act_quantized_relu`` that hands the next layer the ranges it would otherwise compute with
    a pass of its own: the output carries ``(min, max)`` of every ``group_size`` consecutive
    elements of each sample in ``output.actnn_minmax`` (with the tensor version they belong to).
    Inputs whose samples are not whole groups of 256 contiguous elements take the plain op."""
    check_cuda_tensor(input, "input")
    n = input.shape[0] if input.dim() > 1 else 1
    if group_size != 256 or n == 0 or (input.numel() // n) % 256 != 0 or not input.is_contiguous():
        return _ActQuantizedReLU.apply(input)
    y, mn, mx = _ActQuantizedReLUMinmax.apply(input)
    y.actnn_minmax = (mn, mx, y._version)
    return y


# ------------------------------------------------------------------------------- dropout
def dropout_forward(x, p: float, *, u: Optional[torch.Tensor] = None, philox=None):
    y = torch.empty_like(x)
    mask = torch.empty((x.numel() + 31) // 32, dtype=torch.int32, device=x.device)
    if u is not None:
        check_cuda_tensor(u, "u", dtype=torch.float32)
        seed = offset = 0
    else:
        seed, offset = philox if philox is not None else _lib.next_philox(x.device)
    _lib.call("actnn_dropout_forward", x, x.data_ptr(), y.data_ptr(), mask.data_ptr(), x.numel(), float(p),
              _lib.dtype_id(x.dtype), _lib.ptr(u), seed, offset, _lib.stream_of(x))
    return y, mask


def dropout_backward(grad_output, mask, p: float):
    grad_output = grad_output.contiguous()
    grad_input = torch.empty_like(grad_output)
    _lib.call("actnn_dropout_backward", grad_output, grad_output.data_ptr(), mask.data_ptr(),
              grad_input.data_ptr(), grad_output.numel(), float(p), _lib.dtype_id(grad_output.dtype),
              _lib.stream_of(grad_output))
    return grad_input


def dropout_uniform_fill(numel: int, device, seed: int, offset: int) -> torch.Tensor:
    u = torch.empty(numel, dtype=torch.float32, device=device)
    _lib.call("actnn_dropout_uniform_fill", u, u.data_ptr(), numel, seed, offset, _lib.stream_of(u))
    return u


class _ActQuantizedDropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p):
        y, mask = dropout_forward(x, p)
        ctx.save_for_backward(mask)
        ctx.p = p
        return y

    @staticmethod
    def backward(ctx, grad_output):
        (mask,) = ctx.saved_tensors
        return dropout_backward(grad_output, mask, ctx.p), None


def act_quantized_dropout(input: torch.Tensor, dropout_p: float) -> torch.Tensor:
    check_cuda_tensor(input, "input")
    return _ActQuantizedDropout.apply(input, float(dropout_p))


# ------------------------------------------------------------------------------- max-pool
def _pool_args(kernel_size, stride, padding, dilation):
    for name, v in (("kernel_size", kernel_size), ("stride", stride), ("padding", padding),
                    ("dilation", dilation)):
        if len(v) != 2:
            raise RuntimeError("Expected %s.size() == 2 to be true, but got false." % name)
    return [int(a) for pair in (kernel_size, stride, padding, dilation) for a in pair]


def max_pool2d_forward(x, kernel_size, stride, padding, dilation):
    kh, kw, sh, sw, ph, pw, dh, dw = _pool_args(kernel_size, stride, padding, dilation)
    if kh * kw >= 16:
        raise RuntimeError("Expected kernel_size[0] * kernel_size[1] < 16 to be true, but got false.")
    if x.dim() != 4:
        raise RuntimeError("The dimension of input is not correct!")
    n, c, h, w = x.shape
    ho = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    wo = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    y = torch.empty((n, c, ho, wo), dtype=x.dtype, device=x.device)
    idx = torch.empty((n, c, ho, wo), dtype=torch.int8, device=x.device)
    _lib.call("actnn_max_pool2d_forward", x, x.data_ptr(), y.data_ptr(), idx.data_ptr(), n, c, h, w,
              kh, kw, sh, sw, ph, pw, dh, dw, _lib.dtype_id(x.dtype), _lib.stream_of(x))
    return y, idx


def max_pool2d_backward(grad_output, idx, input_shape, kernel_size, stride, padding, dilation):
    kh, kw, sh, sw, ph, pw, dh, dw = _pool_args(kernel_size, stride, padding, dilation)
    grad_output = grad_output.contiguous()
    n, c, h, w = input_shape
    grad_input = torch.empty(tuple(input_shape), dtype=grad_output.dtype, device=grad_output.device)
    _lib.call("actnn_max_pool2d_backward", grad_output, grad_output.data_ptr(), idx.data_ptr(),
              grad_input.data_ptr(), n, c, h, w, kh, kw, sh, sw, ph, pw, dh, dw,
              _lib.dtype_id(grad_output.dtype), _lib.stream_of(grad_output))
    return grad_input


class _ActQuantizedMaxPool2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kernel_size, stride, padding, dilation):
        y, idx = max_pool2d_forward(x, kernel_size, stride, padding, dilation)
        ctx.save_for_backward(idx)
        ctx.geometry = (tuple(x.shape), tuple(kernel_size), tuple(stride), tuple(padding), tuple(dilation))
        return y

    @staticmethod
    def backward(ctx, grad_output):
        (idx,) = ctx.saved_tensors
        shape, k, s, p, d = ctx.geometry
        return max_pool2d_backward(grad_output, idx, shape, k, s, p, d), None, None, None, None


def act_quantized_max_pool2d(input: torch.Tensor, kernel_size: Sequence[int], stride: Sequence[int],
                             padding: Sequence[int], dilation: Sequence[int], ceil_mode: bool,
                             return_indices: bool) -> torch.Tensor:
    check_cuda_tensor(input, "input")
    if ceil_mode:
        raise RuntimeError("Do not support ceil_mode")
    if return_indices:
        raise RuntimeError("Do not support return_indices")
    return _ActQuantizedMaxPool2d.apply(input, tuple(kernel_size), tuple(stride), tuple(padding),
                                        tuple(dilation))
