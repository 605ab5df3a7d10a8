"""Small helpers: host swap, memory accounting, experiment recorder
(reference: actnn/actnn/utils.py:10-80)."""
import json
import os
from collections import OrderedDict

import numpy as np
import torch


def swap_to_cpu(tensor: torch.Tensor):
    """Move a saved tensor to pinned host memory (reference: utils.py:10-16).

    With ``config.swap_arena`` (the default) the copy goes through the pooled arena of
    ``swap_arena.py`` on a copy stream and a ``SwappedTensor`` handle comes back; otherwise
    this is the reference's scheme: an asynchronous copy into freshly pinned memory."""
    from .conf import config
    if tensor.is_cuda and getattr(config, "swap_arena", True):
        from .swap_arena import arena_for
        return arena_for(tensor.device).to_host(tensor)
    host = torch.empty(tensor.shape, dtype=tensor.dtype, device="cpu", pin_memory=tensor.is_cuda)
    host.copy_(tensor, non_blocking=True)
    for attr in ("word_offsets",):
        if hasattr(tensor, attr):
            setattr(host, attr, getattr(tensor, attr))
    return host


def swap_to_gpu(saved):
    """The CUDA tensor behind what ``swap_to_cpu`` returned, usable on the current stream."""
    from .swap_arena import SwappedTensor
    if isinstance(saved, SwappedTensor):
        return saved.arena.to_device(saved)
    out = saved.cuda(non_blocking=True)
    offsets = getattr(saved, "word_offsets", None)
    if offsets is not None:
        out.word_offsets = offsets
    return out


def get_memory_usage(print_info: bool = False) -> int:
    """Bytes held by live tensors according to the caching allocator (device 0)."""
    allocated = torch.cuda.memory_allocated(0)
    if print_info:
        print("allocated: %.2f MB" % (allocated / 1024 / 1024), flush=True)
        print("reserved:  %.2f MB" % (torch.cuda.memory_reserved(0) / 1024 / 1024), flush=True)
    return allocated


_BYTES = {torch.float32: 4, torch.int32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int16: 2, torch.int8: 1}


def compute_tensor_bytes(tensors) -> int:
    """Total bytes of the float32/int32/16-bit/int8 tensors in ``tensors`` (others count 0)."""
    if not isinstance(tensors, (list, tuple)):
        tensors = [tensors]
    return int(sum(t.numel() * _BYTES.get(t.dtype, 0) for t in tensors))


def empty_cache(ratio) -> None:
    """Release cached blocks when less than ``ratio`` of the reserved memory is in use."""
    if ratio is None:
        return
    allocated = torch.cuda.memory_allocated(0)
    reserved = torch.cuda.memory_reserved(0)
    if reserved > 0 and allocated / reserved < ratio:
        torch.cuda.empty_cache()


def disable_cache_allocator() -> None:
    os.environ["PYTORCH_NO_CUDA_MEMORY_CACHING"] = "1"


def enable_cache_allocator() -> None:
    del os.environ["PYTORCH_NO_CUDA_MEMORY_CACHING"]


class GlobalExpRecorder:
    """Key/value store appended to a JSON-lines file."""

    def __init__(self):
        self.val_dict = OrderedDict()

    def record(self, key, value, float_round: int = 6) -> None:
        if isinstance(value, (np.int32, np.int64)):
            value = int(value)
        if isinstance(value, (float, np.float32, np.float64)):
            value = round(float(value), float_round)
        self.val_dict[key] = value

    def dump(self, filename: str) -> None:
        with open(filename, "a") as fout:
            fout.write(json.dumps(self.val_dict) + "\n")
        print("Save exp results to %s" % filename)

    def clear(self) -> None:
        self.val_dict.clear()


exp_recorder = GlobalExpRecorder()
