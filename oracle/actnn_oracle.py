"""CPU oracle for ActNN's activation compress / decompress path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it is the
checker used by the tests, by the smoke check and by the CPU-baseline / reference legs of
the benchmark.  It is a plain restatement, on CPU tensors, of what the reference computes:

* quantize / dequantize arithmetic: the reference's "simulate" branch,
  ``actnn/actnn/ops.py:23-41`` (quantize) and ``ops.py:56-57`` (dequantize), evaluated with
  the very same chain of torch operators so that every intermediate is rounded to the
  activation dtype exactly as PyTorch does it.  The only change is that the rounding noise
  is an argument instead of ``uniform_(-0.5, 0.5)`` (``ops.py:37``) and that the integer
  ``bits`` branch no longer hard-codes ``device='cuda'`` (``ops.py:28``).
* per-group min/max: ``torch.min/max(dim=1)``, which the reference's own test pins as the
  meaning of its minimax kernel (``tests/test_minimax.py:19-30``).
* bit-stream layouts: the index formulas of the reference's CUDA kernels,
  ``actnn/actnn/cpp_extension/quantization_cuda_kernel.cu:51-79`` (mixed precision, int32
  words) and ``:236-257`` (single precision, int8 bytes packed across the batch axis).
* grouping / padding / sensitivities: ``actnn/actnn/qscheme.py:57-94``,
  ``actnn/actnn/qbnscheme.py:21-52`` and ``ops.py:77-96``.
* greedy bit allocation: ``actnn/actnn/cpp_extension/calc_precision.cc:9-50``.
* glue: ``ops.py:99-139`` (bfloat16 storage of scale / min for float32 inputs, un-padding).
* mask ops: ``quantization_cuda_kernel.cu:411-508`` (ReLU), ``:514-627`` (dropout) and
  ``:633-754`` (max-pool) restated on whole tensors.

Parity status: PINNED.  ``tests/golden/make_golden.py`` executes the reference's own
``ops.py`` / ``qscheme.py`` / ``qbnscheme.py`` (simulate branch, CPU tensors) and its
``calc_precision.cc`` compiled unmodified, and stores their outputs as fixtures;
``tests/test_oracle.py`` checks every function here against those fixtures.  The two
bit-stream layouts exist in the reference only as CUDA index arithmetic and cannot be run
without its CUDA build, so for them the oracle is pinned by a second, literal
thread-by-thread emulation of those kernels (``emulate_*`` below) rather than by reference
output.
"""
from __future__ import annotations

import heapq
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

GROUP_SIZE = 256


# --------------------------------------------------------------------------------------
# min / max per group                                             (tests/test_minimax.py)
# --------------------------------------------------------------------------------------
def minimax(rows: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Row-wise min and max of a ``[R, D]`` tensor, in the tensor's dtype."""
    return torch.min(rows, 1)[0], torch.max(rows, 1)[0]


# --------------------------------------------------------------------------------------
# grouping / padding                           (qscheme.py:57-71, qbnscheme.py:21-35)
# --------------------------------------------------------------------------------------
def to_groups(x: torch.Tensor, group_size: int = GROUP_SIZE) -> torch.Tensor:
    """Flatten ``[N, ...]`` to ``[N, G, group_size]``, zero-padding each sample's tail."""
    n = x.shape[0]
    flat = x.reshape(n, -1)
    f = flat.shape[1]
    if f % group_size != 0:
        new_f = (f // group_size + 1) * group_size
        flat = torch.cat([flat, torch.zeros([n, new_f - f], dtype=x.dtype)], 1)
    return flat.reshape(n, -1, group_size)


def group_minimax(groups: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[N, G, gs]`` -> min, max of shape ``[N, G, 1]``."""
    n, g, gs = groups.shape
    mn, mx = minimax(groups.reshape(-1, gs))
    return mn.view(n, g, 1), mx.view(n, g, 1)


# --------------------------------------------------------------------------------------
# quantize / dequantize                                      (ops.py:23-41, ops.py:56-57)
# --------------------------------------------------------------------------------------
def bits_tensor(bits, n: int) -> torch.Tensor:
    if isinstance(bits, int):
        return torch.ones(n, dtype=torch.int32) * bits
    return bits.to(torch.int32)


def quantize(groups: torch.Tensor, bits, mn: torch.Tensor, mx: torch.Tensor,
             noise: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stochastic rounding of ``groups[N,G,gs]`` to per-sample ``bits``.

    ``noise`` has the shape and dtype of ``groups`` with values in [-0.5, 0.5]; ``None``
    means deterministic rounding (``config.stochastic = False``).
    Returns ``(codes int32 [N,G,gs], scale [N,G,1] in the dtype of groups)``.
    """
    n = groups.shape[0]
    bits = bits_tensor(bits, n)
    B = (2 ** bits - 1).view(n, 1, 1)
    mn = mn - 1e-6
    mx = mx + 1e-6
    scale = B / (mx - mn)
    out = (groups - mn) * scale
    if noise is not None:
        out = out + noise
    out = torch.relu(out)
    out = torch.min(out, B.float()).round_().int()
    return out, scale


def dequantize(codes: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """``codes / scale + mn`` with the *unshifted* minimum (ops.py:57)."""
    return codes / scale + mn


# --------------------------------------------------------------------------------------
# bit-stream layouts
# --------------------------------------------------------------------------------------
def mixed_total_words(bits: torch.Tensor, num_groups: int, group_size: int) -> int:
    total_bits = int(bits.to(torch.int64).sum()) * num_groups * group_size
    return (total_bits + 31) // 32


def pack_mixed_layout(codes: torch.Tensor, bits: torch.Tensor) -> np.ndarray:
    """Mixed-precision stream (quantization_cuda_kernel.cu:51-79): int32 words.

    Block ``(n, g)`` starts at word ``(P[n-1]*G*gs + bits[n]*g*gs) / 32`` with ``P`` the
    inclusive prefix sum of ``bits``; it spans ``W = gs*bits[n]/32`` words; bit ``i`` of
    element ``d`` lands in word ``(d*b+i) % W`` at bit position ``(d*b+i) // W``.
    """
    n, g, gs = codes.shape
    assert gs % 32 == 0
    bits_np = bits.numpy().astype(np.int64)
    codes_np = codes.numpy().astype(np.uint32)
    out = np.zeros(mixed_total_words(bits, g, gs), dtype=np.uint32)
    prefix = np.concatenate([[0], np.cumsum(bits_np)])
    d = np.arange(gs, dtype=np.int64)
    for s in range(n):
        b = int(bits_np[s])
        w = gs * b // 32
        base = int(prefix[s]) * g * gs // 32
        block = np.zeros((g, w), dtype=np.uint32)
        for i in range(b):
            pos = d * b + i
            word, shift = pos % w, pos // w
            bit = (codes_np[s] >> np.uint32(i)) & np.uint32(1)          # [g, gs]
            # several d map to one word with distinct shifts: accumulate with OR
            np.bitwise_or.at(block, (slice(None), word), bit << shift.astype(np.uint32))
        out[base:base + g * w] = block.reshape(-1)
    return out.view(np.int32)


def unpack_mixed_layout(words: np.ndarray, bits: torch.Tensor, n: int, g: int,
                        gs: int) -> torch.Tensor:
    """Inverse of :func:`pack_mixed_layout` (quantization_cuda_kernel.cu:156-169)."""
    bits_np = bits.numpy().astype(np.int64)
    words = np.asarray(words).view(np.uint32)
    prefix = np.concatenate([[0], np.cumsum(bits_np)])
    d = np.arange(gs, dtype=np.int64)
    codes = np.zeros((n, g, gs), dtype=np.uint32)
    for s in range(n):
        b = int(bits_np[s])
        w = gs * b // 32
        base = int(prefix[s]) * g * gs // 32
        block = words[base:base + g * w].reshape(g, w)
        for i in range(b):
            pos = d * b + i
            word, shift = pos % w, pos // w
            codes[s] |= ((block[:, word] >> shift.astype(np.uint32)) & np.uint32(1)) << np.uint32(i)
    return torch.from_numpy(codes.astype(np.int32))


def single_total_bytes(bits: int, n: int, num_groups: int, group_size: int) -> int:
    wpt = 8 // bits
    n_round = n + (wpt - n % wpt) % wpt
    return (bits * n_round * num_groups * group_size + 8) // 8


def pack_single_layout(codes: torch.Tensor, bits: int) -> np.ndarray:
    """Uniform-bit stream (quantization_cuda_kernel.cu:236-257): int8 bytes.

    Byte ``(no*G + g)*gs + d`` holds samples ``no*wpt + ni`` (``wpt = 8/bits``) at bit
    offset ``ni*bits``.  The reference allocates one spare trailing byte that it never
    writes; here it is zero.
    """
    assert 8 % bits == 0
    n, g, gs = codes.shape
    wpt = 8 // bits
    no = (n + wpt - 1) // wpt
    padded = np.zeros((no * wpt, g, gs), dtype=np.uint32)
    padded[:n] = codes.numpy().astype(np.uint32)
    padded = padded.reshape(no, wpt, g, gs)
    out = np.zeros(single_total_bytes(bits, n, g, gs), dtype=np.uint8)
    body = np.zeros((no, g, gs), dtype=np.uint32)
    for ni in range(wpt):
        body |= padded[:, ni] << np.uint32(ni * bits)
    out[:no * g * gs] = (body & 0xFF).astype(np.uint8).reshape(-1)
    return out.view(np.int8)


def unpack_single_layout(packed: np.ndarray, bits: int, n: int, g: int, gs: int) -> torch.Tensor:
    """Inverse of :func:`pack_single_layout` (quantization_cuda_kernel.cu:343-360)."""
    wpt = 8 // bits
    no = (n + wpt - 1) // wpt
    body = np.asarray(packed).view(np.uint8)[:no * g * gs].reshape(no, g, gs).astype(np.uint32)
    mask = np.uint32((1 << bits) - 1)
    codes = np.zeros((no * wpt, g, gs), dtype=np.uint32).reshape(no, wpt, g, gs)
    for ni in range(wpt):
        codes[:, ni] = (body >> np.uint32(ni * bits)) & mask
    return torch.from_numpy(codes.reshape(no * wpt, g, gs)[:n].astype(np.int32))


# Literal, thread-by-thread emulations of the reference kernels' index arithmetic.  Slow
# (pure Python loops); used only on tiny cases to pin the vectorised layouts above.
def emulate_pack_mixed_kernel(codes: torch.Tensor, bits: torch.Tensor) -> np.ndarray:
    n, g, gs = codes.shape
    bits_l = [int(b) for b in bits]
    prefix = np.cumsum(bits_l)
    out = [0] * mixed_total_words(bits, g, gs)
    for s in range(n):
        shared_len = gs * bits_l[s] // 32
        for grp in range(g):
            shared = [0] * shared_len
            for d in range(gs):
                val = int(codes[s, grp, d])
                offset = d * bits_l[s]
                for i in range(bits_l[s]):
                    shared[(offset + i) % shared_len] |= (1 & (val >> i)) << ((offset + i) // shared_len)
            global_offset = ((0 if s == 0 else int(prefix[s - 1])) * g * gs + bits_l[s] * grp * gs) // 32
            for k in range(shared_len):
                out[global_offset + k] = shared[k]
    return np.array(out, dtype=np.uint32).view(np.int32)


def emulate_pack_single_kernel(codes: torch.Tensor, bits: int) -> np.ndarray:
    n, g, gs = codes.shape
    wpt = 8 // bits
    out = np.zeros(single_total_bytes(bits, n, g, gs), dtype=np.uint8)
    for no in range((n + wpt - 1) // wpt):
        for grp in range(g):
            for d in range(gs):
                local = 0
                for ni in range(wpt):
                    s = no * wpt + ni
                    if s >= n:
                        break
                    local |= int(codes[s, grp, d]) << (ni * bits)
                out[(no * g + grp) * gs + d] = local & 0xFF
    return out.view(np.int8)


# --------------------------------------------------------------------------------------
# greedy bit allocation                                         (calc_precision.cc:9-50)
# --------------------------------------------------------------------------------------
def _greedy_delta(c: np.float32, b: int, w: int) -> np.float32:
    coeff_1 = ((1 << b) - 1) * ((1 << b) - 1)
    coeff_2 = ((1 << (b - 1)) - 1) * ((1 << (b - 1)) - 1)
    # float * double -> double; / int -> double; stored in a pair<float, int64>
    return np.float32(np.float64(c) * (1.0 / coeff_1 - 1.0 / coeff_2) / np.float64(w))


def calc_precision(b: torch.Tensor, C: torch.Tensor, w: torch.Tensor, target: float) -> torch.Tensor:
    """Greedy allocation with a max-heap of ``(float priority, index)`` pairs.

    ``std::priority_queue<std::pair<float,int64_t>>`` pops the lexicographically largest
    pair, so equal priorities resolve to the larger index.  ``heapq`` is a min-heap, hence
    the negated keys.  Returns a new tensor (the reference mutates ``b`` in place and
    returns it).
    """
    b_l = [int(v) for v in b]
    w_l = [int(v) for v in w]
    c_np = C.detach().to(torch.float32).numpy()
    with np.errstate(all="ignore"):
        heap = []
        b_sum = 0.0
        for i in range(len(b_l)):
            d = _greedy_delta(c_np[i], b_l[i], w_l[i])
            heap.append((-float(d), -i))
            b_sum += b_l[i] * w_l[i]
        heapq.heapify(heap)
        while b_sum > target:
            if not heap:      # the reference asserts here (compiled out under NDEBUG)
                break
            _, neg_i = heapq.heappop(heap)
            i = -neg_i
            b_l[i] -= 1
            b_sum -= w_l[i]
            if b_l[i] > 1:
                d = _greedy_delta(c_np[i], b_l[i], w_l[i])
                heapq.heappush(heap, (-float(d), -i))
    return torch.tensor(b_l, dtype=torch.int32)


# --------------------------------------------------------------------------------------
# per-sample sensitivities and bits            (qscheme.py:57-94, qbnscheme.py:21-52)
# --------------------------------------------------------------------------------------
def range_sqr(mn: torch.Tensor, mx: torch.Tensor, n: int, group_size: int, num_pixels: int) -> torch.Tensor:
    """``G * ||R_n||^2 / I`` (qscheme.py:80): norm in the stats' dtype, then float32."""
    return torch.norm((mx - mn).view(n, -1), dim=1).float().square() * (group_size / num_pixels)


def scheme_bits(x: torch.Tensor, avg_bits, initial_bits: int = 8, group_size: int = GROUP_SIZE,
                coeff: Optional[torch.Tensor] = None):
    """``QScheme/QBNScheme.compute_quantization_bits`` on CPU tensors.

    ``coeff`` is ``(num_locations / 4 / depthwise_groups, grad_scale)`` for conv / linear
    inputs, multiplied onto ``Range_sqr`` left to right as qscheme.py:84 does (python
    float first, then the gradient-scale tensor); ``None`` for batch-norm inputs, where
    ``C = Range_sqr`` (qbnscheme.py:45).
    Returns ``(groups, bits int32[N], mn, mx, C)``.
    """
    n = x.shape[0]
    num_pixels = x.reshape(n, -1).shape[1] // x.shape[1]
    groups = to_groups(x, group_size)
    mn, mx = group_minimax(groups)
    rs = range_sqr(mn, mx, n, group_size, num_pixels)
    C = (rs if coeff is None else coeff[0] * rs * coeff[1]).to(torch.float32)
    b = torch.ones(n, dtype=torch.int32) * initial_bits
    w = torch.ones(n, dtype=torch.int32)
    b = calc_precision(b, C, w, int(avg_bits * n))
    return groups, b, mn, mx, C


# --------------------------------------------------------------------------------------
# glue                                                                  (ops.py:99-139)
# --------------------------------------------------------------------------------------
def quantize_activation(x: torch.Tensor, bits, noise_fn, group_size: int = GROUP_SIZE,
                        coeff=None, scheme: bool = True, initial_bits: int = 8):
    """``quantize_activation`` with the simulate branch.

    ``scheme=True``: per-sample bits from the greedy at average ``bits``;
    ``scheme=False``: every sample gets the integer ``bits`` (ops.py:77-96).
    ``noise_fn(groups)`` returns the noise tensor (or ``None``).
    Returns ``(codes, q_bits, q_scale, q_min)`` with scale / min stored as bfloat16 when
    the input is float32 (ops.py:115-116).
    """
    if scheme:
        groups, q_bits, mn, mx, _ = scheme_bits(x, bits, initial_bits, group_size, coeff)
    else:
        groups = to_groups(x, group_size)
        mn, mx = group_minimax(groups)
        q_bits = bits
    codes, scale = quantize(groups, q_bits, mn, mx, noise_fn(groups))
    if x.dtype == torch.float32:
        return codes, q_bits, scale.to(torch.bfloat16), mn.to(torch.bfloat16)
    return codes, q_bits, scale, mn


def dequantize_activation(quantized, shape: Sequence[int], dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``dequantize_activation`` with the simulate branch (ops.py:121-139).

    The reference widens bfloat16 scale / min to float32 (ops.py:129-131) because that is
    how it stores the statistics of float32 inputs; it never met a bfloat16 activation (its
    extension rejects them), and for one it would therefore hand back a float32 tensor.
    ``dtype=None`` reproduces exactly that.  ``dtype=torch.bfloat16`` is this library's
    bfloat16 path: statistics stay bfloat16 and the same two operators run in bfloat16,
    like they do for float16.
    """
    codes, _, scale, mn = quantized
    if scale.dtype == torch.bfloat16 and dtype != torch.bfloat16:
        scale = scale.to(torch.float32)
        mn = mn.to(torch.float32)
    x = dequantize(codes, scale, mn)
    n = shape[0]
    f = int(np.prod(shape[1:]))
    return x.view(n, -1)[:, :f].reshape(*shape).contiguous()


# --------------------------------------------------------------------------------------
# mask ops
# --------------------------------------------------------------------------------------
def relu_forward(x: torch.Tensor) -> Tuple[torch.Tensor, np.ndarray]:
    """``y = x > 0 ? x : 0`` and the keep mask (quantization_cuda_kernel.cu:428-434).

    The reference never exposes its mask words, so the bit order is this library's own:
    bit ``k`` of byte ``e // 8`` is element ``e = 8*(e//8) + k`` of the flattened tensor
    (little-endian bit order), padded with zero bits to whole int32 words.
    """
    keep = x > 0
    y = torch.where(keep, x, torch.zeros_like(x))
    return y, pack_bitmask(keep)


def pack_bitmask(keep: torch.Tensor) -> np.ndarray:
    flat = keep.reshape(-1).numpy().astype(np.uint8)
    words = (flat.size + 31) // 32
    out = np.zeros(words * 4, dtype=np.uint8)
    packed = np.packbits(flat, bitorder="little")
    out[:packed.size] = packed
    return out.view(np.int32)


def unpack_bitmask(mask: np.ndarray, numel: int) -> torch.Tensor:
    bits = np.unpackbits(np.asarray(mask).view(np.uint8), bitorder="little")[:numel]
    return torch.from_numpy(bits.astype(bool))


def relu_backward(grad: torch.Tensor, mask: np.ndarray) -> torch.Tensor:
    """``dx = bit ? dy : 0`` (quantization_cuda_kernel.cu:479-486)."""
    keep = unpack_bitmask(mask, grad.numel()).view(grad.shape)
    return torch.where(keep, grad, torch.zeros_like(grad))


def dropout_forward(x: torch.Tensor, u: torch.Tensor, p: float) -> Tuple[torch.Tensor, np.ndarray]:
    """``keep = u > p``; ``y = keep ? x / (1 - p) : 0`` (quantization_cuda_kernel.cu:537-543).

    ``u`` is the injected uniform draw in float32.  The division is done in double and
    rounded to the tensor dtype, as the reference's ``data[id] / (1.0 - dropout_p)`` with a
    float ``dropout_p`` does.
    """
    p32 = np.float32(p)
    keep = u > float(p32)
    denom = 1.0 - float(p32)
    y = torch.where(keep, (x.double() / denom).to(x.dtype), torch.zeros_like(x))
    return y, pack_bitmask(keep)


def dropout_backward(grad: torch.Tensor, mask: np.ndarray, p: float) -> torch.Tensor:
    keep = unpack_bitmask(mask, grad.numel()).view(grad.shape)
    denom = 1.0 - float(np.float32(p))
    return torch.where(keep, (grad.double() / denom).to(grad.dtype), torch.zeros_like(grad))


def max_pool2d_forward(x: torch.Tensor, kernel, stride, padding, dilation=(1, 1)):
    """NCHW max-pool that keeps the window-local arg-max
    (quantization_cuda_kernel.cu:644-668): scan the window row-major, take a strictly
    larger value, index ``= kh*KW + kw``.  Window taps are ``dilation`` apart (the
    reference kernel ignores dilation; with dilation 1 the two coincide).
    """
    n, c, h, w = x.shape
    kh, kw = kernel
    sh, sw = stride
    ph, pw = padding
    dh, dw = dilation
    ho = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    wo = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    xp = torch.full((n, c, h + 2 * ph + dh * kh, w + 2 * pw + dw * kw), float("-inf"), dtype=torch.float32)
    xp[:, :, ph:ph + h, pw:pw + w] = x.float()
    best = torch.full((n, c, ho, wo), float("-inf"), dtype=torch.float32)
    idx = torch.zeros((n, c, ho, wo), dtype=torch.int8)
    for i in range(kh):
        for j in range(kw):
            tap = xp[:, :, i * dh:i * dh + sh * ho:sh, j * dw:j * dw + sw * wo:sw]
            better = tap > best
            best = torch.where(better, tap, best)
            idx = torch.where(better, torch.tensor(i * kw + j, dtype=torch.int8), idx)
    return best.to(x.dtype), idx


def max_pool2d_backward(grad: torch.Tensor, idx: torch.Tensor, input_shape, kernel, stride, padding,
                        dilation=(1, 1)) -> torch.Tensor:
    """Route each output gradient to its arg-max input (quantization_cuda_kernel.cu:712-724).
    Contributions to one input are summed in float32 and rounded once."""
    n, c, h, w = input_shape
    kh, kw = kernel
    sh, sw = stride
    ph, pw = padding
    dh, dw = dilation
    ho, wo = grad.shape[2], grad.shape[3]
    oh = torch.arange(ho).view(1, 1, ho, 1)
    ow = torch.arange(wo).view(1, 1, 1, wo)
    ih = oh * sh - ph + (idx.long() // kw) * dh
    iw = ow * sw - pw + (idx.long() % kw) * dw
    flat = (ih * w + iw).view(n, c, -1)
    dx = torch.zeros((n, c, h * w), dtype=torch.float32)
    dx.scatter_add_(2, flat, grad.float().view(n, c, -1))
    return dx.view(n, c, h, w).to(grad.dtype)


# --------------------------------------------------------------------------------------
# noise
# --------------------------------------------------------------------------------------
def batch_norm_forward(x: torch.Tensor, weight, bias, running_mean, running_var, momentum: float, eps: float):
    """Training-mode batch norm in float64: what ``cudnn_batch_norm`` computes at the
    reference's call site (ops.py:457-458).  Returns ``(y, save_mean, save_invstd,
    new_running_mean, new_running_var)``; y is rounded to x's dtype, the rest is float64."""
    C = x.shape[1]
    x64 = x.double().transpose(0, 1).reshape(C, -1)
    M = x64.shape[1]
    mean = x64.mean(dim=1)
    var = ((x64 - mean[:, None]) ** 2).mean(dim=1)
    invstd = 1.0 / torch.sqrt(var + eps)
    w = torch.ones(C, dtype=torch.float64) if weight is None else weight.double()
    b = torch.zeros(C, dtype=torch.float64) if bias is None else bias.double()
    shape = [1, C] + [1] * (x.dim() - 2)
    y = (x.double() - mean.view(shape)) * (invstd * w).view(shape) + b.view(shape)
    new_rm = new_rv = None
    if running_mean is not None:
        new_rm = (1 - momentum) * running_mean.double() + momentum * mean
    if running_var is not None:
        unbiased = var * (M / (M - 1)) if M > 1 else var
        new_rv = (1 - momentum) * running_var.double() + momentum * unbiased
    return y.to(x.dtype), mean, invstd, new_rm, new_rv


def batch_norm_backward(x: torch.Tensor, grad_out: torch.Tensor, weight, save_mean, save_invstd):
    """Gradients of training-mode batch norm in float64 (``cudnn_batch_norm_backward``,
    reference call site ops.py:492-493): ``(grad_input, grad_weight, grad_bias)``."""
    C = x.shape[1]
    shape = [1, C] + [1] * (x.dim() - 2)
    dims = [d for d in range(x.dim()) if d != 1]
    M = x.numel() // C
    mean, invstd = save_mean.double().view(shape), save_invstd.double().view(shape)
    w = torch.ones(C, dtype=torch.float64) if weight is None else weight.double()
    g = grad_out.double()
    xhat = (x.double() - mean) * invstd
    sum_dy = g.sum(dim=dims)
    sum_dy_xhat = (g * xhat).sum(dim=dims)
    dx = (w * save_invstd.double()).view(shape) * (g - sum_dy.view(shape) / M - xhat * sum_dy_xhat.view(shape) / M)
    return dx.to(x.dtype), sum_dy_xhat, sum_dy


def torch_noise(shape, dtype, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """``output.new(shape).uniform_(-0.5, 0.5)`` (ops.py:37) from a CPU generator."""
    return torch.empty(shape, dtype=dtype).uniform_(-0.5, 0.5, generator=generator)


_PHILOX_M0 = np.uint64(0xD2511F53)
_PHILOX_M1 = np.uint64(0xCD9E8D57)
_PHILOX_W0 = 0x9E3779B9
_PHILOX_W1 = 0xBB67AE85


def philox4x32_10(counter: np.ndarray, key: Tuple[int, int]) -> np.ndarray:
    """Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11)
    on an array of counters ``[..., 4]`` uint32 with one 64-bit key.  Vectorised numpy."""
    c = [counter[..., i].astype(np.uint64) for i in range(4)]
    k0, k1 = key[0] & 0xFFFFFFFF, key[1] & 0xFFFFFFFF
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ np.uint64(k0), lo1, hi0 ^ c[3] ^ np.uint64(k1), lo0]
        k0 = (k0 + _PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return np.stack([v.astype(np.uint32) for v in c], axis=-1)


def _philox_calls(count: int, seed: int, offset: int) -> np.ndarray:
    """Outputs ``[count, 4]`` uint32 of calls ``c = 0..count-1`` with counter
    ``(lo32(c), hi32(c), lo32(offset), hi32(offset))`` and key ``(lo32(seed), hi32(seed))``."""
    c = np.arange(count, dtype=np.uint64)
    ctr = np.stack([(c & np.uint64(0xFFFFFFFF)).astype(np.uint32), (c >> np.uint64(32)).astype(np.uint32),
                    np.full(count, offset & 0xFFFFFFFF, dtype=np.uint32),
                    np.full(count, (offset >> 32) & 0xFFFFFFFF, dtype=np.uint32)], axis=-1)
    return philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))


def _expand_call(r: np.ndarray) -> np.ndarray:
    """Eight words per call: the four outputs and ``v[i] + 0x9E3779B1 * v[(i + 1) % 4]`` mod 2^32."""
    nxt = np.roll(r, -1, axis=1).astype(np.uint64)
    derived = (r.astype(np.uint64) + nxt * np.uint64(0x9E3779B1)) & np.uint64(0xFFFFFFFF)
    return np.concatenate([r, derived.astype(np.uint32)], axis=1)


def philox_noise(numel: int, dtype: torch.dtype, seed: int, offset: int) -> torch.Tensor:
    """The rounding noise the CUDA pack kernels draw when no noise tensor is injected.

    Element ``e`` of the padded ``[N, G, 256]`` activation: flat group ``q = e // 256``,
    position ``d = e % 256``, lane ``t = d // 8``, ``j = d % 8``.  Each call's four output
    words are extended to eight (``_expand_call``).
    * float16 / bfloat16: call ``c = (q // 4) * 32 + t``; with ``h = q % 4`` and ``p = j % 4`` the
      word is ``w = e[2h + j // 4]``.  float16: ``k`` = bits 1..8 (``p`` even) or 17..24 (``p`` odd)
      of ``w`` rotated right by ``8 * (p // 2)``; bfloat16: ``k`` = byte ``2 * (p % 2) + p // 2`` of
      ``w``.  Noise ``(2k + 1 - 256) / 512``.
    * float32: call ``c = (q // 2) * 32 + t``; with ``h = q % 2``, 16-bit field ``j`` of the
      words ``e[4h .. 4h + 3]`` is ``k``; noise ``(2k + 1 - 65536) / 131072``.
    """
    e = np.arange(numel, dtype=np.int64)
    q, d = e // 256, e % 256
    t, j = d // 8, d % 8
    if dtype == torch.float32:
        c, h = (q // 2) * 32 + t, q % 2
        w = _expand_call(_philox_calls(int(c.max()) + 1 if numel else 0, seed, offset))
        k = (w[c, 4 * h + j // 2] >> (16 * (j % 2)).astype(np.uint32)) & np.uint32(0xFFFF)
        u = (2.0 * k.astype(np.float64) + 1 - 65536) / 131072
    else:
        c, h = (q // 4) * 32 + t, q % 4
        w = _expand_call(_philox_calls(int(c.max()) + 1 if numel else 0, seed, offset))
        word = w[c, 2 * h + j // 4].astype(np.uint64)
        p = j % 4
        if dtype == torch.float16:
            rot = (8 * (p // 2)).astype(np.uint64)
            word = ((word >> rot) | (word << (np.uint64(32) - rot))) & np.uint64(0xFFFFFFFF)
            k = (word >> (1 + 16 * (p % 2)).astype(np.uint64)) & np.uint64(0xFF)
        else:
            k = (word >> (8 * (2 * (p % 2) + p // 2)).astype(np.uint64)) & np.uint64(0xFF)
        u = (2.0 * k.astype(np.float64) + 1 - 256) / 512
    return torch.from_numpy(u.astype(np.float32)).to(dtype)


def philox_dropout_uniform(numel: int, seed: int, offset: int) -> torch.Tensor:
    """The uniforms in (0, 1] the CUDA dropout draws: call ``c = e // 8``, 16-bit field
    ``e % 8`` is ``k``, ``u = (k + 1) / 65536`` (float32)."""
    e = np.arange(numel, dtype=np.int64)
    c, j = e // 8, e % 8
    r = _philox_calls(int(c.max()) + 1 if numel else 0, seed, offset)
    k = (r[c, j // 2] >> (16 * (j % 2)).astype(np.uint32)) & np.uint32(0xFFFF)
    return torch.from_numpy(((k.astype(np.float64) + 1) / 65536).astype(np.float32))
