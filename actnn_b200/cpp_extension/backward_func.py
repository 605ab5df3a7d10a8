"""ATen backward operators under the names the reference re-exports
(actnn/actnn/cpp_extension/backward_func.cc:81-91).

PyTorch 2.x dropped ``cudnn_convolution_backward`` / ``cudnn_convolution_transpose_backward``
in favour of ``convolution_backward``; the two names are kept here with the reference's
argument order and are routed to that operator.  The dense math stays in cuDNN / ATen: this
module holds no kernels."""
import torch

aten = torch.ops.aten


def cudnn_convolution_backward(input, grad_output, weight, padding, stride, dilation, groups,
                               benchmark, deterministic, allow_tf32, output_mask):
    prev = torch.backends.cudnn.benchmark
    torch.backends.cudnn.benchmark = bool(benchmark)
    try:
        gi, gw, _ = aten.convolution_backward(
            grad_output, input, weight, None, list(stride), list(padding), list(dilation), False,
            [0] * len(stride), groups, [bool(output_mask[0]), bool(output_mask[1]), False])
    finally:
        torch.backends.cudnn.benchmark = prev
    return gi, gw


def cudnn_convolution_transpose_backward(input, grad_output, weight, padding, output_padding, stride,
                                         dilation, groups, benchmark, deterministic, allow_tf32,
                                         output_mask):
    prev = torch.backends.cudnn.benchmark
    torch.backends.cudnn.benchmark = bool(benchmark)
    try:
        gi, gw, _ = aten.convolution_backward(
            grad_output, input, weight, None, list(stride), list(padding), list(dilation), True,
            list(output_padding), groups, [bool(output_mask[0]), bool(output_mask[1]), False])
    finally:
        torch.backends.cudnn.benchmark = prev
    return gi, gw


def cudnn_batch_norm(input, weight, bias, running_mean, running_var, training, exponential_average_factor,
                     epsilon):
    return aten.cudnn_batch_norm(input, weight, bias, running_mean, running_var, training,
                                 exponential_average_factor, epsilon)


def cudnn_batch_norm_backward(input, grad_output, weight, running_mean, running_var, save_mean, save_var,
                              epsilon, reserve):
    return aten.cudnn_batch_norm_backward(input, grad_output, weight, running_mean, running_var, save_mean,
                                          save_var, epsilon, reserve)


def native_batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps):
    return aten.native_batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps)


def native_batch_norm_backward(grad_out, input, weight, running_mean, running_var, save_mean, save_invstd,
                               train, eps, output_mask):
    return aten.native_batch_norm_backward(grad_out, input, weight, running_mean, running_var, save_mean,
                                           save_invstd, train, eps, list(output_mask))
