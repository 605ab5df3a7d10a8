"""Argument checks with the reference's error texts (ext_common.h:2-27)."""
import torch

FLOAT_TYPES = (torch.float32, torch.float16, torch.bfloat16)


def check_cuda_tensor(t, name, ndim=None, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor!" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous!" % name)
    if ndim is not None and t.dim() != ndim:
        raise RuntimeError("The dimension of %s is not correct!" % name)
    if dtype is None:
        if t.dtype not in FLOAT_TYPES:
            raise RuntimeError("The type of %s is not correct!" % name)
    elif t.dtype != dtype:
        raise RuntimeError("The type of %s is not correct!" % name)
