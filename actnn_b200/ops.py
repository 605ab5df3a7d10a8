"""Autograd operators that keep a compressed copy of their input for the backward pass,
and the compress / decompress glue they share.

Mirror of actnn/actnn/ops.py: ``quantize_activation`` / ``dequantize_activation``
(:99-139) and the Functions ``conv{1,2,3}d``, ``conv_transpose{1,2,3}d``, ``linear``,
``batch_norm``, ``sync_batch_norm``, ``adaptive_avg_pool2d`` (:145-628).  The dense math
(convolutions, batch-norm, matmuls) stays in cuDNN / cuBLAS / ATen exactly as in the
reference; what changes is the codec underneath:

* uniform-bit layers (no scheme) compress with ONE fused kernel that reads the activation
  once (min/max + stochastic rounding + pack);
* adaptive layers run minimax -> sensitivity -> greedy -> pack as four launches with no
  host synchronisation (the reference needs three syncs and a CPU heap per layer);
* float32 inputs get their bfloat16 scale / min written by the pack kernel and read by the
  unpack kernel directly (the reference converts with extra kernels, ops.py:115-116,129-131).
"""
import math
from collections import namedtuple

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.autograd.function import Function
from torch.nn.modules.utils import _pair, _single, _triple

from .conf import config
from .cpp_extension import backward_func as ext_backward_func
from .cpp_extension import minimax as ext_minimax  # noqa: F401  (kept under the name the reference imports)
from .cpp_extension import quantization as ext_quantization
from .qscheme import group_minimax, to_groups
from .utils import compute_tensor_bytes, empty_cache, get_memory_usage, swap_to_cpu, swap_to_gpu

QParams = namedtuple("QParams", ["range", "zero_point", "num_bits"])


# ---------------------------------------------------------------------------------------
# compress / decompress
# ---------------------------------------------------------------------------------------
def _simulate_quantize(data, bits, mn, mx):
    """The reference's pure-PyTorch debug branch (ops.py:23-41), kept behind
    ``config.simulate`` exactly as there.  Off by default; never used for speed."""
    N = data.shape[0]
    if isinstance(bits, int):
        bits = torch.ones(N, dtype=torch.int32, device=data.device) * bits
    B = (2 ** bits - 1).view(N, 1, 1)
    mn = mn - 1e-6
    mx = mx + 1e-6
    scale = B / (mx - mn)
    output = (data - mn) * scale
    if config.stochastic:
        output = output + output.new(output.shape).uniform_(-0.5, 0.5)
    output = F.relu(output)
    return torch.min(output, B.float()).round_().int(), scale


def quantize_and_pack(data, bits, mn, mx):
    """``data [N, G, gs]`` -> ``(packed, scale)``; ``bits`` an int (uniform) or an int32
    tensor (per sample).  Mirror of ops.py:22-52."""
    if config.simulate:
        return _simulate_quantize(data, bits, mn, mx)
    if isinstance(bits, int):
        output, scale = ext_quantization.pack_single_precision(data, mn, mx, bits, config.stochastic)
    else:
        output, scale = ext_quantization.pack_mixed_precision(
            data, mn, mx, bits, config.stochastic, word_offsets=getattr(bits, "word_offsets", None),
            total_bits=getattr(bits, "total_bits", None))
    if config.swap:
        output = swap_to_cpu(output)
    return output, scale


def dequantize_and_unpack(data, shape, bits, scale, mn, out_dtype=None):
    """Mirror of ops.py:55-74."""
    if config.simulate:
        return data / scale + mn
    if config.swap:
        data = swap_to_gpu(data)
    N = shape[0]
    num_features = math.prod(shape[1:])
    gs = config.group_size
    num_features = num_features + (gs - num_features % gs) % gs
    if isinstance(bits, int):
        return ext_quantization.unpack_single_precision(data, bits, scale, mn, N, num_features // gs, gs,
                                                        out_dtype=out_dtype)
    return ext_quantization.unpack_mixed_precision(data, bits, scale, mn, N, num_features // gs, gs,
                                                   out_dtype=out_dtype)


def no_scheme_compute_quantization_bits(input):
    """Uniform-bit layers: groups, the configured width and the group ranges (ops.py:77-96)."""
    groups, mn, mx = group_minimax(input)
    return groups, config.activation_compression_bits[0], mn, mx


def producer_minmax(input):
    """Per-group extrema that the op which produced ``input`` left on it (QReLU does), if they still
    describe it: same tensor version, contiguous, one value per 256 elements."""
    rec = getattr(input, "actnn_minmax", None)
    if rec is None:
        return None
    mn, mx, version = rec
    if input._version != version or not input.is_contiguous() or mn.numel() * 256 != input.numel() \
            or mn.dtype != input.dtype:
        return None
    return mn, mx


def quantize_activation(input, scheme, minmax=None):
    """Compress one activation; returns ``(q_input, q_bits, q_scale, q_min)`` (ops.py:99-118).

    ``minmax=(mn, mx)``: per-group extrema of ``input`` that a previous pass already produced
    (the batch-norm Functions get them with their statistics); only schemes whose ``compress``
    accepts them use them."""
    if not config.compress_activation:
        if config.swap:
            input = swap_to_cpu(input)
        return input, None, None, None

    stat_dtype = torch.bfloat16 if input.dtype == torch.float32 else input.dtype
    if config.simulate:
        if scheme:
            groups, q_bits, q_min, mx = scheme.compute_quantization_bits(input)
        else:
            groups, q_bits, q_min, mx = no_scheme_compute_quantization_bits(input)
        q_input, q_scale = quantize_and_pack(groups, q_bits, q_min, mx)
        return q_input, q_bits, q_scale.to(stat_dtype), q_min.to(stat_dtype)

    if scheme:
        if minmax is not None:
            fused = scheme.compress(input, stat_dtype, minmax=minmax)
        else:
            fused = scheme.compress(input, stat_dtype) if hasattr(scheme, "compress") else None
        if fused is not None:
            q_input, q_bits, q_scale, q_min = fused
        else:
            groups, q_bits, mn, mx = scheme.compute_quantization_bits(input)
            q_input, q_scale, q_min = ext_quantization.pack_mixed_precision(
                groups, mn, mx, q_bits, config.stochastic, word_offsets=getattr(q_bits, "word_offsets", None),
                total_bits=getattr(q_bits, "total_bits", None), stat_dtype=stat_dtype, return_min=True)
    else:
        q_bits = config.activation_compression_bits[0]
        if config.pergroup:
            # one pass over the activation: min/max, rounding and packing fused
            q_input, q_scale, q_min = ext_quantization.compress_single_precision(
                to_groups(input), q_bits, config.stochastic, stat_dtype=stat_dtype)
        else:
            groups, _, mn, mx = no_scheme_compute_quantization_bits(input)
            q_input, q_scale, q_min = ext_quantization.pack_single_precision(
                groups, mn, mx, q_bits, config.stochastic, stat_dtype=stat_dtype, return_min=True)
    if config.swap:
        q_input = swap_to_cpu(q_input)
    return q_input, q_bits, q_scale, q_min


def dequantize_activation(quantized, q_input_shape, dtype=None):
    """Rebuild the activation (ops.py:121-139).

    ``dtype`` is the dtype of the original activation when the caller knows it.  Without it
    the reference's rule applies: bfloat16 statistics mean a float32 activation
    (ops.py:129-131)."""
    if not config.compress_activation:
        ret = quantized[0]
        if config.swap:
            ret = swap_to_gpu(ret)
        return ret

    q_input, q_bits, q_scale, q_min = quantized
    if dtype is None:
        dtype = torch.float32 if q_scale.dtype == torch.bfloat16 else q_scale.dtype
    if config.simulate:
        if dtype != q_scale.dtype:
            q_scale, q_min = q_scale.to(dtype), q_min.to(dtype)
        input = dequantize_and_unpack(q_input, q_input_shape, q_bits, q_scale, q_min)
    else:
        input = dequantize_and_unpack(q_input, q_input_shape, q_bits, q_scale, q_min, out_dtype=dtype)

    N = q_input_shape[0]
    num_features = math.prod(q_input_shape[1:])
    input = input.view(N, -1)[:, :num_features]
    return input.reshape(*q_input_shape).contiguous()


# ---------------------------------------------------------------------------------------
# helpers shared by the Functions
# ---------------------------------------------------------------------------------------
conv2d_layer_ct = 0
bn_layer_ct = 0
total_act_mem = 0


def _autocast_inputs(*tensors):
    """Under ``torch.autocast`` run the op in the autocast dtype, as a built-in op would.
    Must be called before autocast is switched off for the body of the Function."""
    if not torch.is_autocast_enabled("cuda"):
        return tensors
    dt = torch.get_autocast_dtype("cuda")
    return tuple(t.to(dt) if isinstance(t, torch.Tensor) and t.is_floating_point() and t.is_cuda else t
                 for t in tensors)


def _debug_forward(tag, quantized):
    global conv2d_layer_ct, total_act_mem
    print("========== %s forward %d ==========" % (tag, conv2d_layer_ct))
    get_memory_usage(True)
    conv2d_layer_ct += 1
    total_act_mem += compute_tensor_bytes([t for t in quantized if isinstance(t, torch.Tensor)])
    print("Act mem: %.2f MB" % (total_act_mem / 1024 ** 2))


def _chunked_conv_backward(backward_op, input, grad_output, weight, args, needs):
    """Micro-batched backward that overwrites ``input`` with the input gradient chunk by chunk
    (the reference's "pipeline", ops.py:195-220)."""
    ws_mem = compute_tensor_bytes([grad_output, input, input])
    micro = int((ws_mem + config.pipeline_threshold) // config.pipeline_threshold)
    grad_weight = None
    for x, g in zip(torch.chunk(input, micro), torch.chunk(grad_output, micro)):
        gi, gw = backward_op(x, g, weight, *args, config.cudnn_benchmark_conv2d, False, False, needs)
        x[:] = gi
        grad_weight = gw if grad_weight is None else grad_weight + gw
    return input, grad_weight


class convnd(Function):
    @staticmethod
    def run_forward(n, forward_op, ctx, input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1,
                    scheme=None):
        input, weight, bias = _autocast_inputs(input, weight, bias)
        with torch.autocast("cuda", enabled=False):
            quantized = quantize_activation(input, scheme, minmax=producer_minmax(input) if scheme else None)
            ctx.scheme = scheme
            ctx.saved = quantized, weight, bias
            ctx.other_args = (input.shape, stride, padding, dilation, groups, input.dtype)
            empty_cache(config.empty_cache_threshold)
            if config.debug_memory_op_forward:
                _debug_forward("conv%dd" % n, quantized)
            return forward_op(input, weight, bias, stride, padding, dilation, groups)

    @staticmethod
    def run_backward(n, ctx, grad_output, bias_reduce_dims, aug):
        if ctx.scheme:
            ctx.scheme.set_scale(grad_output)
        q_input_shape, stride, padding, dilation, groups, in_dtype = ctx.other_args
        padding, stride, dilation = aug(padding), aug(stride), aug(dilation)
        quantized, weight, bias = ctx.saved
        input = dequantize_activation(quantized, q_input_shape, in_dtype)
        del quantized, ctx.saved
        empty_cache(config.empty_cache_threshold)
        if config.debug_memory_op_backward:
            global conv2d_layer_ct
            print("========== conv%dd backward %d ==========" % (n, conv2d_layer_ct))
            get_memory_usage(True)
            conv2d_layer_ct += 1
            print("WS: %.2f MB" % (compute_tensor_bytes([grad_output, input, input]) / 1024 ** 2))

        grad_output = grad_output.to(input.dtype)
        needs = [ctx.needs_input_grad[0], ctx.needs_input_grad[1]]
        use_pipeline = bool(config.pipeline_threshold) and all(needs) and \
            compute_tensor_bytes([grad_output, input, input]) > config.pipeline_threshold
        args = (padding, stride, dilation, groups)
        if use_pipeline:
            grad_input, grad_weight = _chunked_conv_backward(
                ext_backward_func.cudnn_convolution_backward, input, grad_output, weight, args, needs)
        else:
            grad_input, grad_weight = ext_backward_func.cudnn_convolution_backward(
                input, grad_output, weight, *args, config.cudnn_benchmark_conv2d, False, False, needs)
        grad_bias = grad_output.sum(bias_reduce_dims) if bias is not None and ctx.needs_input_grad[2] else None
        if ctx.scheme:
            ctx.scheme.if_allocate_perlayer()
        return grad_input, grad_weight, grad_bias, None, None, None, None, None


def _make_conv(n, forward_op, reduce_dims, aug):
    class _Conv(Function):
        @staticmethod
        def forward(ctx, input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, scheme=None):
            return convnd.run_forward(n, forward_op, ctx, input, weight, bias, stride, padding, dilation,
                                      groups, scheme)

        @staticmethod
        def backward(ctx, grad_output):
            return convnd.run_backward(n, ctx, grad_output, reduce_dims, aug)
    _Conv.__name__ = _Conv.__qualname__ = "conv%dd" % n
    return _Conv


conv1d = _make_conv(1, F.conv1d, [0, 2], _single)
conv2d = _make_conv(2, F.conv2d, [0, 2, 3], _pair)
conv3d = _make_conv(3, F.conv3d, [0, 2, 3, 4], _triple)


class conv_transposend(Function):
    @staticmethod
    def run_forward(n, forward_op, ctx, input, weight, bias=None, stride=1, padding=0, output_padding=0,
                    groups=1, dilation=1, scheme=None):
        input, weight, bias = _autocast_inputs(input, weight, bias)
        with torch.autocast("cuda", enabled=False):
            quantized = quantize_activation(input, scheme)
            ctx.scheme = scheme
            ctx.saved = quantized, weight, bias
            ctx.other_args = (input.shape, stride, padding, output_padding, dilation, groups, input.dtype)
            empty_cache(config.empty_cache_threshold)
            if config.debug_memory_op_forward:
                _debug_forward("conv%dd_transpose" % n, quantized)
            return forward_op(input, weight, bias, stride, padding, output_padding, groups, dilation)

    @staticmethod
    def run_backward(n, ctx, grad_output, bias_reduce_dims, aug):
        if ctx.scheme:
            ctx.scheme.set_scale(grad_output)
        q_input_shape, stride, padding, output_padding, dilation, groups, in_dtype = ctx.other_args
        padding, output_padding, stride, dilation = aug(padding), aug(output_padding), aug(stride), aug(dilation)
        quantized, weight, bias = ctx.saved
        input = dequantize_activation(quantized, q_input_shape, in_dtype)
        del quantized, ctx.saved
        empty_cache(config.empty_cache_threshold)
        if config.debug_memory_op_backward:
            global conv2d_layer_ct
            print("========== conv%dd_transpose backward %d ==========" % (n, conv2d_layer_ct))
            get_memory_usage(True)
            conv2d_layer_ct += 1
            print("WS: %.2f MB" % (compute_tensor_bytes([grad_output, input, input]) / 1024 ** 2))

        grad_output = grad_output.to(input.dtype)
        needs = [ctx.needs_input_grad[0], ctx.needs_input_grad[1]]
        use_pipeline = bool(config.pipeline_threshold) and all(needs) and \
            compute_tensor_bytes([grad_output, input, input]) > config.pipeline_threshold
        args = (padding, output_padding, stride, dilation, groups)
        if use_pipeline:
            grad_input, grad_weight = _chunked_conv_backward(
                ext_backward_func.cudnn_convolution_transpose_backward, input, grad_output, weight, args, needs)
        else:
            grad_input, grad_weight = ext_backward_func.cudnn_convolution_transpose_backward(
                input, grad_output, weight, *args, config.cudnn_benchmark_conv2d, False, False, needs)
        grad_bias = grad_output.sum(bias_reduce_dims) if bias is not None and ctx.needs_input_grad[2] else None
        if ctx.scheme:
            ctx.scheme.if_allocate_perlayer()
        return grad_input, grad_weight, grad_bias, None, None, None, None, None, None


def _make_conv_transpose(n, forward_op, reduce_dims, aug):
    class _ConvT(Function):
        @staticmethod
        def forward(ctx, input, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1,
                    scheme=None):
            return conv_transposend.run_forward(n, forward_op, ctx, input, weight, bias, stride, padding,
                                                output_padding, groups, dilation, scheme)

        @staticmethod
        def backward(ctx, grad_output):
            return conv_transposend.run_backward(n, ctx, grad_output, reduce_dims, aug)
    _ConvT.__name__ = _ConvT.__qualname__ = "conv_transpose%dd" % n
    return _ConvT


conv_transpose1d = _make_conv_transpose(1, F.conv_transpose1d, [0, 2], _single)
conv_transpose2d = _make_conv_transpose(2, F.conv_transpose2d, [0, 2, 3], _pair)
conv_transpose3d = _make_conv_transpose(3, F.conv_transpose3d, [0, 2, 3, 4], _triple)


class linear(Function):
    @staticmethod
    def forward(ctx, input, weight, bias=None, scheme=None):
        input, weight, bias = _autocast_inputs(input, weight, bias)
        with torch.autocast("cuda", enabled=False):
            quantized = quantize_activation(input, scheme)
            empty_cache(config.empty_cache_threshold)
            ctx.scheme = scheme
            ctx.saved = quantized, weight, bias
            ctx.other_args = (input.shape, input.dtype)
            return F.linear(input, weight, bias)

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.scheme:
            ctx.scheme.set_scale(grad_output)
        quantized, weight, bias = ctx.saved
        q_input_shape, in_dtype = ctx.other_args
        input = dequantize_activation(quantized, q_input_shape, in_dtype)
        del quantized, ctx.saved
        empty_cache(config.empty_cache_threshold)

        grad_output = grad_output.to(input.dtype)
        go = grad_output.reshape(-1, grad_output.shape[-1])
        x = input.reshape(-1, input.shape[-1])
        grad_input = go.mm(weight).view(q_input_shape)
        grad_weight = go.t().mm(x)
        grad_bias = go.sum(0) if bias is not None else None
        if ctx.scheme:
            ctx.scheme.if_allocate_perlayer()
        return grad_input, grad_weight, grad_bias, None


def _fused_bn_statistics(input, scheme, weight, bias, running_mean, running_var, momentum, eps, out=None):
    """Statistics of a training-mode batch norm together with the group min / max its compressed
    copy needs, from one read of ``input``; ``None`` when that pass does not apply (exact or
    simulated activations, per-tensor ranges, a scheme without the one-call compress, or a
    geometry the kernel does not cover)."""
    if not (config.compress_activation and config.pergroup and not config.simulate and scheme is not None
            and hasattr(scheme, "compress") and config.group_size == 256):
        return None
    return ext_backward_func.batch_norm_stats_minimax(input, weight, bias, running_mean, running_var, momentum, eps,
                                                      out=out)


class batch_norm(Function):
    @staticmethod
    def forward(ctx, input, running_mean, running_var, weight, bias, training, exponential_average_factor, eps,
                scheme):
        fused = None
        if training and input.is_cuda:
            input = input.contiguous()
            fused = _fused_bn_statistics(input, scheme, weight, bias, running_mean, running_var,
                                         exponential_average_factor, eps)
        if fused is not None:
            # one read of the input gave the statistics and the group ranges; the second read
            # packs, the third normalises (the reference reads it four times)
            mn, mx, save_mean, save_var = fused
            quantized = quantize_activation(input, scheme, minmax=(mn, mx))
        else:
            quantized = quantize_activation(input, scheme)
        empty_cache(config.empty_cache_threshold)
        if config.debug_memory_op_forward:
            global bn_layer_ct, total_act_mem
            print("========== bn forward %d ==========" % bn_layer_ct)
            get_memory_usage(True)
            bn_layer_ct += 1
            total_act_mem += compute_tensor_bytes([t for t in quantized if isinstance(t, torch.Tensor)])
            print("Act mem: %.2f MB" % (total_act_mem / 1024 ** 2))

        if fused is not None:
            output = ext_backward_func.batch_norm_elemt(input, weight, bias, save_mean, save_var, eps)
            reserve = torch.empty(0, dtype=torch.uint8, device=input.device)
        elif training:
            output, save_mean, save_var, reserve = ext_backward_func.cudnn_batch_norm(
                input, weight, bias, running_mean, running_var, training, exponential_average_factor, eps)
        else:
            output, save_mean, save_var = ext_backward_func.native_batch_norm(
                input, weight, bias, running_mean, running_var, training, exponential_average_factor, eps)
            reserve = None
        ctx.scheme = scheme
        ctx.other_args = (input.shape, input.dtype)
        ctx.saved = (quantized, weight, running_mean, running_var, save_mean, save_var, training, eps, reserve)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        quantized, weight, running_mean, running_var, save_mean, save_var, training, eps, reserve = ctx.saved
        q_input_shape, in_dtype = ctx.other_args
        input = dequantize_activation(quantized, q_input_shape, in_dtype)
        del quantized, ctx.saved
        empty_cache(config.empty_cache_threshold)
        if config.debug_memory_op_backward:
            global bn_layer_ct
            print("========== bn backward %d ==========" % bn_layer_ct)
            get_memory_usage(True)
            bn_layer_ct += 1

        if training:
            grad_input, grad_weight, grad_bias = ext_backward_func.cudnn_batch_norm_backward(
                input.contiguous(), grad_output.contiguous(), weight, running_mean, running_var, save_mean,
                save_var, eps, reserve)
        else:
            grad_input, grad_weight, grad_bias = ext_backward_func.native_batch_norm_backward(
                grad_output, input, weight, running_mean, running_var, save_mean, save_var, training, eps,
                [ctx.needs_input_grad[0], ctx.needs_input_grad[3], ctx.needs_input_grad[4]])
        if ctx.scheme:
            ctx.scheme.if_allocate_perlayer()
        return grad_input, None, None, grad_weight, grad_bias, None, None, None, None


class sync_batch_norm(Function):
    """Batch norm with statistics shared across the process group: an all_gather of
    ``[mean, invstd, count]`` forward and an all_reduce of ``[sum_dy, sum_dy_xmu]`` backward
    (reference: ops.py:505-614).  Both messages are a few KB; NCCL carries them."""

    @staticmethod
    def forward(self, input, weight, bias, running_mean, running_var, eps, momentum, process_group, world_size,
                scheme):
        input = input.contiguous()
        num_channels = input.shape[1]
        local_count = input.numel() // num_channels
        # the gathered message [mean, invstd, count] is written in place: no cat / stack
        combined = torch.empty(2 * num_channels + 1, dtype=torch.float32, device=input.device)
        # local statistics, with the group ranges of the compressed copy from the same read when possible
        fused = _fused_bn_statistics(input, scheme, None, None, None, None, 0.0, eps, out=combined)
        if fused is None:
            ext_backward_func.batch_norm_stats(input, eps, out=combined)
        combined[2 * num_channels:].fill_(local_count)
        gathered = torch.empty(world_size, 2 * num_channels + 1, dtype=torch.float32, device=input.device)
        dist.all_gather_into_tensor(gathered, combined, process_group, async_op=False)
        mean_all, invstd_all, count_all = torch.split(gathered, num_channels, dim=1)
        # every rank contributes at least one value per channel, so the reference's check
        # (ops.py:530-533) can only trip in a single-rank group: no device read is needed
        size = local_count if world_size == 1 else 2
        if size == 1:
            raise ValueError("Expected more than 1 value per channel when training, got input size {}".format(size))
        mean, invstd = torch.batch_norm_gather_stats_with_counts(
            input, mean_all, invstd_all, running_mean, running_var, momentum, eps, count_all.reshape(-1))

        self.saved = quantize_activation(input, scheme, minmax=None if fused is None else fused[:2])
        self.save_for_backward(weight, mean, invstd, count_all)
        self.scheme = scheme
        self.other_args = (input.shape, input.dtype)
        self.process_group = process_group
        return ext_backward_func.batch_norm_elemt(input, weight, bias, mean, invstd, eps)

    @staticmethod
    def backward(self, grad_output):
        grad_output = grad_output.contiguous()
        q_input_shape, in_dtype = self.other_args
        saved_input = dequantize_activation(self.saved, q_input_shape, in_dtype)
        del self.saved
        weight, mean, invstd, count_tensor = self.saved_tensors
        grad_input = None
        num_channels = saved_input.shape[1]
        combined = torch.empty(2 * num_channels, dtype=torch.float32, device=saved_input.device)
        sum_dy, sum_dy_xmu, grad_weight, grad_bias = ext_backward_func.batch_norm_backward_reduce(
            grad_output, saved_input, mean, invstd, weight, self.needs_input_grad[0], self.needs_input_grad[1],
            self.needs_input_grad[2], out=combined)
        if self.needs_input_grad[0]:
            dist.all_reduce(combined, dist.ReduceOp.SUM, self.process_group, async_op=False)
            grad_input = ext_backward_func.batch_norm_backward_elemt(
                grad_output, saved_input, mean, invstd, weight, sum_dy, sum_dy_xmu, count_tensor.reshape(-1))
        if weight is None or not self.needs_input_grad[1]:
            grad_weight = None
        if weight is None or not self.needs_input_grad[2]:
            grad_bias = None
        if self.scheme:
            self.scheme.if_allocate_perlayer()
        return grad_input, grad_weight, grad_bias, None, None, None, None, None, None, None


class adaptive_avg_pool2d(Function):
    """Global average pooling that saves only the input shape (ops.py:617-628)."""

    @staticmethod
    def forward(ctx, input, output_size):
        assert output_size == (1, 1)
        ctx.saved = input.shape
        return torch.mean(input, dim=[2, 3], keepdim=True)

    @staticmethod
    def backward(ctx, grad_output):
        input_shape = ctx.saved
        repeat_size = [int(x / y) for x, y in zip(input_shape, grad_output.shape)]
        return grad_output.repeat(repeat_size) / np.prod(repeat_size), None
