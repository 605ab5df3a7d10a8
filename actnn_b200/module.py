"""``QModule``: wrap a model and swap its ``nn`` layers for the compressed-activation ones.

Mirror of actnn/actnn/module.py:14-100.  Two additions: the replacement layers take over
the parameters and buffers of the layers they replace (the reference leaves them freshly
initialised), and ``nn.SyncBatchNorm`` is converted to ``QSyncBatchNorm`` (the reference
never converts it)."""
from collections import OrderedDict

import torch
import torch.nn as nn

from .conf import config
from .layers import (QAvgPool2d, QBatchNorm1d, QBatchNorm2d, QBatchNorm3d, QConv1d, QConv2d, QConv3d,
                     QConvTranspose1d, QConvTranspose2d, QConvTranspose3d, QDropout, QLinear, QMaxPool2d,
                     QReLU, QSyncBatchNorm)

_Q_TYPES = (QConv1d, QConv2d, QConv3d, QConvTranspose1d, QConvTranspose2d, QConvTranspose3d, QBatchNorm1d,
            QBatchNorm2d, QBatchNorm3d, QSyncBatchNorm, QReLU, QDropout, QLinear, QMaxPool2d, QAvgPool2d)
_CONV = {nn.Conv1d: QConv1d, nn.Conv2d: QConv2d, nn.Conv3d: QConv3d}
_CONV_T = {nn.ConvTranspose1d: QConvTranspose1d, nn.ConvTranspose2d: QConvTranspose2d,
           nn.ConvTranspose3d: QConvTranspose3d}
_BN = {nn.BatchNorm1d: QBatchNorm1d, nn.BatchNorm2d: QBatchNorm2d, nn.BatchNorm3d: QBatchNorm3d}


def _adopt_state(new: nn.Module, old: nn.Module) -> nn.Module:
    with torch.no_grad():
        for name, p in old.named_parameters(recurse=False):
            q = getattr(new, name, None)
            if q is not None and q.shape == p.shape:
                q.data = p.data.clone()
                q.requires_grad_(p.requires_grad)
        for name, b in old.named_buffers(recurse=False):
            q = getattr(new, name, None)
            if q is not None and b is not None and q.shape == b.shape:
                q.data = b.data.clone()
    new.train(old.training)
    return new


def _replacement(child: nn.Module):
    t = type(child)
    if t in _CONV:
        return _CONV[t](child.in_channels, child.out_channels, child.kernel_size, child.stride, child.padding,
                        child.dilation, child.groups, child.bias is not None, child.padding_mode)
    if t in _CONV_T:
        return _CONV_T[t](child.in_channels, child.out_channels, child.kernel_size, child.stride, child.padding,
                          child.output_padding, child.groups, child.bias is not None, child.dilation,
                          child.padding_mode)
    if t is nn.SyncBatchNorm and config.enable_quantized_bn:
        return QSyncBatchNorm(child.num_features, child.eps, child.momentum, child.affine,
                              child.track_running_stats, child.process_group)
    if t in _BN and config.enable_quantized_bn:
        return _BN[t](child.num_features, child.eps, child.momentum, child.affine, child.track_running_stats)
    if t is nn.Linear:
        return QLinear(child.in_features, child.out_features, child.bias is not None)
    if t is nn.ReLU:
        return QReLU()
    if t is nn.Dropout:
        return QDropout(child.p)
    if t is nn.MaxPool2d:
        return QMaxPool2d(child.kernel_size, child.stride, child.padding, child.dilation, child.return_indices,
                          child.ceil_mode)
    if t is nn.AvgPool2d:
        return QAvgPool2d(child.kernel_size, child.stride, child.padding, child.ceil_mode,
                          child.count_include_pad, child.divisor_override)
    return None


class QModule(nn.Module):
    def __init__(self, model):
        super().__init__()
        self.model = model
        QModule.convert_layers(model)

    @staticmethod
    def convert_layers(module):
        for name, child in module.named_children():
            if isinstance(child, _Q_TYPES):            # already converted
                continue
            new = _replacement(child)
            if new is None:
                if not isinstance(child, tuple(_CONV) + tuple(_CONV_T) + tuple(_BN) + (
                        nn.SyncBatchNorm, nn.Linear, nn.ReLU, nn.Dropout, nn.MaxPool2d, nn.AvgPool2d)):
                    QModule.convert_layers(child)
                continue
            ref = next(child.parameters(recurse=False), None)
            if ref is None:
                ref = next(child.buffers(recurse=False), None)
            if ref is not None:
                new = new.to(device=ref.device, dtype=ref.dtype if ref.is_floating_point() else None)
            setattr(module, name, _adopt_state(new, child))

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def train(self, mode: bool = True):
        config.training = mode
        return super().train(mode)

    def eval(self):
        config.training = False
        return super().eval()

    def load_state_dict(self, state_dict, strict: bool = True):
        # checkpoints are interchangeable with the unwrapped model: add the "model." prefix
        return super().load_state_dict(OrderedDict(("model." + k, v) for k, v in state_dict.items()), strict)

    def state_dict(self, destination=None, prefix="", keep_vars=False):
        ret = super().state_dict(destination=destination, prefix=prefix, keep_vars=keep_vars)
        return OrderedDict((k[len("model."):] if k.startswith("model.") else k, v) for k, v in ret.items())
