"""Backward operators under the names the reference re-exports
(actnn/actnn/cpp_extension/backward_func.cc:81-91).

PyTorch 2.x dropped ``cudnn_convolution_backward`` / ``cudnn_convolution_transpose_backward``
in favour of ``convolution_backward``; the two names are kept here with the reference's
argument order and are routed to that operator: the dense convolution math stays in cuDNN.

``cudnn_batch_norm`` / ``cudnn_batch_norm_backward`` keep the reference's names, arguments
and return values, but the training-mode work is done by this package's own kernels
(``actnn_batch_norm_forward`` / ``actnn_batch_norm_backward`` of the C ABI), which spread a
channel over many blocks instead of cuDNN's one block per channel.  ``batch_norm_stats``,
``batch_norm_elemt``, ``batch_norm_backward_reduce`` and ``batch_norm_backward_elemt`` are
the same kernels under the names of the ATen operators the reference's synchronised batch
norm calls (ops.py:515-603)."""
import torch

from .. import _lib

aten = torch.ops.aten


class _cudnn_benchmark:
    """``torch.backends.cudnn.benchmark = flag`` for the duration of a call; the global is only
    touched when it differs (the usual case, one setting for a whole run, costs nothing)."""

    def __init__(self, flag):
        self.flag = bool(flag)
        self.prev = None

    def __enter__(self):
        cur = torch.backends.cudnn.benchmark
        if cur != self.flag:
            self.prev = cur
            torch.backends.cudnn.benchmark = self.flag

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.backends.cudnn.benchmark = self.prev
        return False


def cudnn_convolution_backward(input, grad_output, weight, padding, stride, dilation, groups,
                               benchmark, deterministic, allow_tf32, output_mask):
    with _cudnn_benchmark(benchmark):
        gi, gw, _ = aten.convolution_backward(
            grad_output, input, weight, None, list(stride), list(padding), list(dilation), False,
            [0] * len(stride), groups, [bool(output_mask[0]), bool(output_mask[1]), False])
    return gi, gw


def cudnn_convolution_transpose_backward(input, grad_output, weight, padding, output_padding, stride,
                                         dilation, groups, benchmark, deterministic, allow_tf32,
                                         output_mask):
    with _cudnn_benchmark(benchmark):
        gi, gw, _ = aten.convolution_backward(
            grad_output, input, weight, None, list(stride), list(padding), list(dilation), True,
            list(output_padding), groups, [bool(output_mask[0]), bool(output_mask[1]), False])
    return gi, gw


def _as_f32(t):
    return None if t is None else (t if t.dtype == torch.float32 else t.float()).contiguous()


def _bn_dims(input):
    if input.dim() < 2:
        raise RuntimeError("batch_norm: expected an input of at least 2 dimensions, got %d" % input.dim())
    N, C = input.shape[0], input.shape[1]
    HW = input.numel() // (N * C) if N * C else 0
    return N, C, HW


def _bn_workspace(N, C, HW, device):
    """Scratch of the batch-norm kernels (they clear what must start at zero themselves), taken
    from the per-stream scratch buffer instead of the allocator."""
    nbytes = _lib.load().actnn_batch_norm_workspace(N, C, HW)
    return _lib.scratch(device, max(nbytes, 16)), nbytes


def cudnn_batch_norm(input, weight, bias, running_mean, running_var, training, exponential_average_factor,
                     epsilon):
    """Returns ``(output, save_mean, save_invstd, reserve)`` like ``at::cudnn_batch_norm``
    (reference call site: ops.py:457-458).  ``reserve`` is an empty byte tensor."""
    if not training:
        return aten.cudnn_batch_norm(input, weight, bias, running_mean, running_var, training,
                                     exponential_average_factor, epsilon)
    if not input.is_cuda:
        raise RuntimeError("cudnn_batch_norm: the input must be a CUDA tensor")
    x = input.contiguous()
    N, C, HW = _bn_dims(x)
    w32, b32 = _as_f32(weight), _as_f32(bias)
    for name, t in (("running_mean", running_mean), ("running_var", running_var)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise RuntimeError("cudnn_batch_norm: %s must be a contiguous float32 tensor" % name)
    y = torch.empty_like(x)
    save_mean = torch.empty(C, dtype=torch.float32, device=x.device)
    save_invstd = torch.empty(C, dtype=torch.float32, device=x.device)
    ws, nbytes = _bn_workspace(N, C, HW, x.device)
    _lib.call("actnn_batch_norm_forward", x, _lib.ptr(x), _lib.ptr(w32), _lib.ptr(b32), _lib.ptr(running_mean),
              _lib.ptr(running_var), _lib.ptr(y), _lib.ptr(save_mean), _lib.ptr(save_invstd), N, C, HW,
              float(exponential_average_factor), float(epsilon), _lib.dtype_id(x.dtype), _lib.ptr(ws), nbytes,
              _lib.stream_of(x))
    return y, save_mean, save_invstd, torch.empty(0, dtype=torch.uint8, device=x.device)


def cudnn_batch_norm_backward(input, grad_output, weight, running_mean, running_var, save_mean, save_var,
                              epsilon, reserve):
    """Returns ``(grad_input, grad_weight, grad_bias)`` like ``at::cudnn_batch_norm_backward``
    (reference call site: ops.py:492-493); ``save_var`` is the inverse standard deviation the
    forward saved."""
    if not input.is_cuda:
        raise RuntimeError("cudnn_batch_norm_backward: the input must be a CUDA tensor")
    x = input.contiguous()
    dy = grad_output.contiguous()
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    N, C, HW = _bn_dims(x)
    w32 = _as_f32(weight)
    dx = torch.empty_like(x)
    dweight = torch.empty(C, dtype=torch.float32, device=x.device)
    dbias = torch.empty(C, dtype=torch.float32, device=x.device)
    ws, nbytes = _bn_workspace(N, C, HW, x.device)
    _lib.call("actnn_batch_norm_backward", x, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(w32), _lib.ptr(save_mean),
              _lib.ptr(save_var), _lib.ptr(dx), _lib.ptr(dweight), _lib.ptr(dbias), N, C, HW,
              _lib.dtype_id(x.dtype), _lib.ptr(ws), nbytes, _lib.stream_of(x))
    if weight is not None and weight.dtype != torch.float32:
        dweight, dbias = dweight.to(weight.dtype), dbias.to(weight.dtype)
    return dx, dweight, dbias


def batch_norm_stats(input, eps, out=None):
    """``torch.batch_norm_stats``: per-channel ``(mean, invstd)`` of this rank's batch
    (reference call site: ops.py:515).  ``out``: an optional contiguous float32 buffer of at
    least ``2 * C`` elements that receives mean then invstd (the message a synchronised batch
    norm gathers), so that no concatenation is needed."""
    x = input.contiguous()
    N, C, HW = _bn_dims(x)
    if out is None:
        out = torch.empty(2 * C, dtype=torch.float32, device=x.device)
    elif out.dtype != torch.float32 or not out.is_contiguous() or out.numel() < 2 * C or out.device != x.device:
        raise RuntimeError("batch_norm_stats: out must be a contiguous float32 tensor of >= 2*C elements")
    ws, nbytes = _bn_workspace(N, C, HW, x.device)
    _lib.call("actnn_batch_norm_stats", x, _lib.ptr(x), out.data_ptr(), out.data_ptr() + 4 * C, N, C, HW, float(eps),
              _lib.dtype_id(x.dtype), _lib.ptr(ws), nbytes, _lib.stream_of(x))
    flat = out.view(-1)
    return flat[:C], flat[C:2 * C]


def batch_norm_stats_minimax(input, weight, bias, running_mean, running_var, momentum, eps, out=None):
    """Batch-norm statistics AND the codec's per-group min / max from one read of ``input``
    (the reference reads it once for each: ops.py:456-458 / :515 and qbnscheme.py:28-40).

    Returns ``(mn, mx, mean, invstd)`` -- ``mn`` / ``mx`` shaped ``[N, G, 1]`` in the input's
    dtype, ``mean`` / ``invstd`` float32 ``[C]`` -- or ``None`` when the geometry is not covered
    (then the caller takes the two-read path).  ``running_mean`` / ``running_var`` are updated
    when given; ``out``: optional float32 buffer of >= 2 * C elements for mean then invstd."""
    if not input.is_cuda or not input.is_contiguous() or input.dim() < 2:
        return None
    N, C, HW = _bn_dims(input)
    lib = _lib.load()
    nbytes = lib.actnn_batch_norm_stats_minimax_workspace(N, C, HW)
    if nbytes < 0:
        return None
    for t in (running_mean, running_var):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            return None
    G = C * HW // 256
    dev = input.device
    mn = torch.empty((N, G, 1), dtype=input.dtype, device=dev)
    mx = torch.empty((N, G, 1), dtype=input.dtype, device=dev)
    if out is None:
        out = torch.empty(2 * C, dtype=torch.float32, device=dev)
    elif out.dtype != torch.float32 or not out.is_contiguous() or out.numel() < 2 * C or out.device != dev:
        raise RuntimeError("batch_norm_stats_minimax: out must be a contiguous float32 tensor of >= 2*C elements")
    w32, b32 = _as_f32(weight), _as_f32(bias)
    ws = _lib.scratch(dev, nbytes)
    _lib.call("actnn_batch_norm_stats_minimax", input, _lib.ptr(input), mn.data_ptr(), mx.data_ptr(), _lib.ptr(w32),
              _lib.ptr(b32), _lib.ptr(running_mean), _lib.ptr(running_var), out.data_ptr(), out.data_ptr() + 4 * C,
              N, C, HW, float(momentum), float(eps), _lib.dtype_id(input.dtype), ws.data_ptr(), nbytes,
              _lib.stream_of(input))
    flat = out.view(-1)
    return mn, mx, flat[:C], flat[C:2 * C]


def batch_norm_elemt(input, weight, bias, mean, invstd, eps):
    """``torch.batch_norm_elemt``: normalise with given statistics (ops.py:554)."""
    x = input.contiguous()
    N, C, HW = _bn_dims(x)
    y = torch.empty_like(x)
    ws = _lib.scratch(x.device, max(16 * C, 16))
    # the converted copies must outlive the call: a pointer taken from a temporary would dangle
    w32, b32, m32, i32 = _as_f32(weight), _as_f32(bias), _as_f32(mean), _as_f32(invstd)
    _lib.call("actnn_batch_norm_elemt", x, _lib.ptr(x), _lib.ptr(w32), _lib.ptr(b32), _lib.ptr(m32), _lib.ptr(i32),
              _lib.ptr(y), N, C, HW, _lib.dtype_id(x.dtype), _lib.ptr(ws), 16 * C, _lib.stream_of(x))
    return y


def batch_norm_backward_reduce(grad_out, input, mean, invstd, weight, input_g, weight_g, bias_g, out=None):
    """``torch.batch_norm_backward_reduce``: ``(sum_dy, sum_dy_xmu, grad_weight, grad_bias)`` of this
    rank (ops.py:570-577).  ``out``: optional contiguous float32 ``[2 * C]`` buffer that receives
    sum_dy then sum_dy_xmu (the message a synchronised batch norm all-reduces)."""
    x = input.contiguous()
    dy = grad_out.contiguous()
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    N, C, HW = _bn_dims(x)
    if out is None:
        out = torch.empty(2 * C, dtype=torch.float32, device=x.device)
    elif out.dtype != torch.float32 or not out.is_contiguous() or out.numel() < 2 * C or out.device != x.device:
        raise RuntimeError("batch_norm_backward_reduce: out must be a contiguous float32 tensor of >= 2*C elements")
    grad_weight = torch.empty(C, dtype=torch.float32, device=x.device)
    ws, nbytes = _bn_workspace(N, C, HW, x.device)
    w32, m32, i32 = _as_f32(weight), _as_f32(mean), _as_f32(invstd)       # kept alive across the call
    _lib.call("actnn_batch_norm_backward_reduce", x, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(w32),
              _lib.ptr(m32), _lib.ptr(i32), out.data_ptr(), out.data_ptr() + 4 * C,
              _lib.ptr(grad_weight), N, C, HW, _lib.dtype_id(x.dtype), _lib.ptr(ws), nbytes, _lib.stream_of(x))
    flat = out.view(-1)
    sum_dy, sum_dy_xmu = flat[:C], flat[C:2 * C]
    grad_bias = sum_dy.clone() if bias_g else None             # the message buffer is all-reduced in place later
    if weight is not None and weight.dtype != torch.float32:
        grad_weight = grad_weight.to(weight.dtype)
        grad_bias = None if grad_bias is None else grad_bias.to(weight.dtype)
    return sum_dy, sum_dy_xmu, (grad_weight if weight_g else None), grad_bias


def batch_norm_backward_elemt(grad_out, input, mean, invstd, weight, sum_dy, sum_dy_xmu, count):
    """``torch.batch_norm_backward_elemt``: the input gradient from sums over all ranks; ``count``
    holds every rank's elements per channel and stays on the device (ops.py:594-603)."""
    x = input.contiguous()
    dy = grad_out.contiguous()
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    N, C, HW = _bn_dims(x)
    counts = count.reshape(-1).to(torch.float32).contiguous()
    dx = torch.empty_like(x)
    ws = _lib.scratch(x.device, max(16 * C, 16))
    w32, m32, i32 = _as_f32(weight), _as_f32(mean), _as_f32(invstd)       # kept alive across the call
    sdy, sdx = _as_f32(sum_dy), _as_f32(sum_dy_xmu)
    _lib.call("actnn_batch_norm_backward_elemt", x, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(w32),
              _lib.ptr(m32), _lib.ptr(i32), _lib.ptr(sdy),
              _lib.ptr(sdx), _lib.ptr(counts), counts.numel(), _lib.ptr(dx), N, C, HW,
              _lib.dtype_id(x.dtype), _lib.ptr(ws), 16 * C, _lib.stream_of(x))
    return dx


def native_batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps):
    return aten.native_batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps)


def native_batch_norm_backward(grad_out, input, weight, running_mean, running_var, save_mean, save_invstd,
                               train, eps, output_mask):
    return aten.native_batch_norm_backward(grad_out, input, weight, running_mean, running_var, save_mean,
                                           save_invstd, train, eps, list(output_mask))
