"""Drop-in ``nn.Module`` layers that save compressed activations.

Same classes, constructor signatures and behaviour as actnn/actnn/layers.py:20-515: in
training mode (``config.training``) the forward goes through the autograd Functions of
``actnn_b200.ops``; otherwise the stock PyTorch layer runs.  ``QReLU``, ``QMaxPool2d`` and
``QDropout`` call the mask-saving kernels directly, at every optimisation level."""
import warnings
from typing import Optional

import torch
import torch.distributed
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.modules.pooling import _AvgPoolNd, _MaxPoolNd
from torch.nn.modules.utils import _pair, _single, _triple

from . import ops
from .conf import config
from .cpp_extension import quantization as ext_quantization
from .qbnscheme import QBNScheme
from .qscheme import QScheme


def _taps(kernel_size, ndim):
    if isinstance(kernel_size, int):
        return kernel_size ** ndim
    n = 1
    for k in kernel_size[:ndim]:
        n *= k
    return n


# ------------------------------------------------------------------------- convolutions
class _QConvMixin:
    _ndim = 2
    _fn = None
    _tuple = staticmethod(_pair)

    def _init_scheme(self, kernel_size, groups, group):
        if config.adaptive_conv_scheme:
            self.scheme = QScheme(self, num_locations=_taps(kernel_size, self._ndim), group=group,
                                  depthwise_groups=groups)
        else:
            self.scheme = None

    def forward(self, input):
        if not config.training:
            return super().forward(input)
        if self.padding_mode != "zeros":
            input = F.pad(input, self._reversed_padding_repeated_twice, mode=self.padding_mode)
            return self._fn.apply(input, self.weight, self.bias, self.stride, self._tuple(0), self.dilation,
                                  self.groups, self.scheme)
        return self._fn.apply(input, self.weight, self.bias, self.stride, self.padding, self.dilation,
                              self.groups, self.scheme)


class QConv1d(_QConvMixin, nn.Conv1d):
    _ndim, _fn, _tuple = 1, ops.conv1d, staticmethod(_single)

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, padding_mode="zeros", group=0):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                         padding_mode)
        self._init_scheme(kernel_size, groups, group)


class QConv2d(_QConvMixin, nn.Conv2d):
    _ndim, _fn, _tuple = 2, ops.conv2d, staticmethod(_pair)

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, padding_mode="zeros", group=0):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                         padding_mode)
        self._init_scheme(kernel_size, groups, group)


class QConv3d(_QConvMixin, nn.Conv3d):
    _ndim, _fn, _tuple = 3, ops.conv3d, staticmethod(_triple)

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, padding_mode="zeros", group=0):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                         padding_mode)
        self._init_scheme(kernel_size, groups, group)


class _QConvTransposeMixin(_QConvMixin):
    def forward(self, input, output_size=None):
        if not config.training:
            return super(_QConvMixin, self).forward(input, output_size)
        if self.padding_mode != "zeros":
            raise ValueError("Only `zeros` padding mode is supported for %s" % type(self).__name__[1:])
        num_spatial_dims = self._ndim
        output_padding = self._output_padding(input, output_size, self.stride, self.padding, self.kernel_size,
                                              num_spatial_dims, self.dilation)
        return self._fn.apply(input, self.weight, self.bias, self.stride, self.padding, output_padding,
                              self.groups, self.dilation, self.scheme)


class QConvTranspose1d(_QConvTransposeMixin, nn.ConvTranspose1d):
    _ndim, _fn = 1, ops.conv_transpose1d

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, groups=1,
                 bias=True, dilation=1, padding_mode="zeros", group=0):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, output_padding, groups, bias,
                         dilation, padding_mode)
        self._init_scheme(kernel_size, groups, group)


class QConvTranspose2d(_QConvTransposeMixin, nn.ConvTranspose2d):
    _ndim, _fn = 2, ops.conv_transpose2d

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, groups=1,
                 bias=True, dilation=1, padding_mode="zeros", group=0):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, output_padding, groups, bias,
                         dilation, padding_mode)
        self._init_scheme(kernel_size, groups, group)


class QConvTranspose3d(_QConvTransposeMixin, nn.ConvTranspose3d):
    _ndim, _fn = 3, ops.conv_transpose3d

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, groups=1,
                 bias=True, dilation=1, padding_mode="zeros", group=0):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, output_padding, groups, bias,
                         dilation, padding_mode)
        self._init_scheme(kernel_size, groups, group)


# ------------------------------------------------------------------------- linear
class QLinear(nn.Linear):
    num_layers = 0

    def __init__(self, input_features, output_features, bias=True, group=0):
        super().__init__(input_features, output_features, bias)
        self.scheme = QScheme(self, group=group) if config.adaptive_conv_scheme else None

    def forward(self, input):
        if config.training:
            return ops.linear.apply(input, self.weight, self.bias, self.scheme)
        return super().forward(input)


# ------------------------------------------------------------------------- batch norm
class _QBatchNormMixin:
    def _init_scheme(self, group):
        self.scheme = QBNScheme(group=group) if config.adaptive_bn_scheme else None

    def _averaging_factor(self):
        """Momentum for the running statistics; also counts the batch (nn.BatchNorm semantics)."""
        factor = 0.0 if self.momentum is None else self.momentum
        if self.training and self.track_running_stats and self.num_batches_tracked is not None:
            self.num_batches_tracked.add_(1)          # in place, as nn.BatchNorm does: no buffer re-registration
            factor = 1.0 / float(self.num_batches_tracked) if self.momentum is None else self.momentum
        return factor

    def _buffers_for(self):
        use = (not self.training) or self.track_running_stats
        return (self.running_mean if use else None), (self.running_var if use else None)

    def forward(self, input):
        if not config.training:
            return super().forward(input)
        self._check_input_dim(input)
        factor = self._averaging_factor()
        bn_training = True if self.training else (self.running_mean is None and self.running_var is None)
        running_mean, running_var = self._buffers_for()
        return ops.batch_norm.apply(input, running_mean, running_var, self.weight, self.bias, bn_training,
                                    factor, self.eps, self.scheme)


class QBatchNorm1d(_QBatchNormMixin, nn.BatchNorm1d):
    def __init__(self, num_features, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True, group=0):
        super().__init__(num_features, eps, momentum, affine, track_running_stats)
        self._init_scheme(group)


class QBatchNorm2d(_QBatchNormMixin, nn.BatchNorm2d):
    def __init__(self, num_features, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True, group=0):
        super().__init__(num_features, eps, momentum, affine, track_running_stats)
        self._init_scheme(group)


class QBatchNorm3d(_QBatchNormMixin, nn.BatchNorm3d):
    def __init__(self, num_features, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True, group=0):
        super().__init__(num_features, eps, momentum, affine, track_running_stats)
        self._init_scheme(group)


class QSyncBatchNorm(_QBatchNormMixin, nn.SyncBatchNorm):
    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 track_running_stats: bool = True, process_group=None, group=0) -> None:
        super().__init__(num_features, eps, momentum, affine, track_running_stats, process_group)
        self._init_scheme(group)

    def forward(self, input):
        if not input.is_cuda:
            raise ValueError("SyncBatchNorm expected input tensor to be on GPU")
        self._check_input_dim(input)
        factor = self._averaging_factor()
        bn_training = True if self.training else (self.running_mean is None and self.running_var is None)
        running_mean, running_var = self._buffers_for()

        need_sync = bn_training and torch.distributed.is_available() and torch.distributed.is_initialized()
        if need_sync:
            process_group = self.process_group or torch.distributed.group.WORLD
            world_size = torch.distributed.get_world_size(process_group)
            need_sync = world_size > 1
        if not need_sync:                      # single process: plain (quantized) batch norm
            return ops.batch_norm.apply(input, running_mean, running_var, self.weight, self.bias, bn_training,
                                        factor, self.eps, self.scheme)
        return ops.sync_batch_norm.apply(input, self.weight, self.bias, running_mean, running_var, self.eps,
                                         factor, process_group, world_size, self.scheme)


# ------------------------------------------------------------------------- mask-saving layers
class QReLU(nn.Module):
    def __init__(self, inplace=False):
        super().__init__()

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        # the layer after a ReLU is nearly always a convolution that compresses this output: let
        # the ReLU pass produce the group ranges that compression starts from
        if (config.training and config.compress_activation and config.adaptive_conv_scheme and config.pergroup
                and config.relu_minmax and not config.simulate):
            return ext_quantization.act_quantized_relu_with_minmax(input, config.group_size)
        return ext_quantization.act_quantized_relu(input)


class QDropout(nn.Dropout):
    def __init__(self, p=0.5):
        super().__init__(p=p)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self.training:
            return ext_quantization.act_quantized_dropout(input, self.p)
        return super().forward(input)


class QMaxPool2d(_MaxPoolNd):
    def __init__(self, kernel_size, stride=None, padding=0, dilation=1, return_indices=False, ceil_mode=False):
        super().__init__(kernel_size, stride, padding, dilation, return_indices, ceil_mode)
        self.kernel_size = _pair(kernel_size)
        self.stride = _pair(stride if stride is not None else kernel_size)
        self.padding = _pair(padding)
        self.dilation = _pair(dilation)

    def forward(self, input):
        return ext_quantization.act_quantized_max_pool2d(input, self.kernel_size, self.stride, self.padding,
                                                         self.dilation, self.ceil_mode, self.return_indices)


class QAvgPool2d(_AvgPoolNd):
    """As in the reference (layers.py:506-515), average pooling is REPLACED by the
    index-saving max pooling, with a warning: no memory-saving average-pool kernel exists."""
    __constants__ = ["kernel_size", "stride", "padding", "ceil_mode", "count_include_pad", "divisor_override"]

    def __init__(self, kernel_size, stride=None, padding=0, ceil_mode: bool = False,
                 count_include_pad: bool = True, divisor_override: Optional[int] = None) -> None:
        super().__init__()
        self.kernel_size = _pair(kernel_size)
        self.stride = _pair(stride if stride is not None else kernel_size)
        self.padding = _pair(padding)
        self.ceil_mode = ceil_mode
        self.count_include_pad = count_include_pad
        self.divisor_override = divisor_override

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        warnings.warn("avg_pool2d is replaced by max_pool2d, because the optimized cuda kernel "
                      "for avg_pool2d is not implemented.")
        return ext_quantization.act_quantized_max_pool2d(input, self.kernel_size, self.stride, self.padding,
                                                         (1, 1), self.ceil_mode, False)
