"""Host swap of saved activations (levels L4 / L5 / "swap") through a pooled pinned arena
and two copy streams.

The reference copies every packed activation into freshly pinned memory on the compute
stream and copies it back, again on the compute stream, when backward needs it
(actnn/actnn/utils.py:10-16, ops.py:50-51, 59-60): both transfers stall the kernels.  Here

* pinned memory is a stack over large slabs that are pinned once (pinning is the expensive
  part of the reference's scheme): saved tensors are produced in forward order and
  consumed in reverse;
* device-to-host copies run on a copy-out stream that waits for the producing kernel, so the
  next layer's forward overlaps them;
* host-to-device copies run on a copy-in stream and are issued early: when backward asks
  for one swapped tensor, the tensors saved just before it (the ones backward will want
  next) are already being fetched, up to ``prefetch_bytes``.

``swap_to_cpu`` returns a ``SwappedTensor`` handle; ``swap_to_gpu`` turns it back into a CUDA
tensor that is safe to use on the current stream.  Plain tensors pass through
``swap_to_gpu`` with ``.cuda(non_blocking=True)``, so the reference's behaviour is one
switch away (``config.swap_arena = False``)."""
from __future__ import annotations

import threading
import weakref
from typing import Callable, Dict, List

import torch


class PinnedStack:
    """Stack allocator over large pinned slabs.

    Saved activations are produced in forward order and consumed in reverse, so their host
    copies follow a stack discipline: ``push`` bumps a pointer, ``pop`` marks a block free and
    the pointer falls back over every free block on top.  What matters is the total of the
    live blocks, which a training step repeats exactly (the bit budget is fixed), not the
    individual sizes, which move with the per-layer bit allocation: after the first step no
    memory is pinned again (pinning costs about a millisecond per MiB).  Blocks freed out of
    order only delay the fall-back.  ``alloc(nbytes)`` creates a slab (pinned host memory in
    production, anything sliceable with ``numel()`` in tests)."""

    ALIGN = 512

    def __init__(self, alloc: Callable[[int], object], slab_bytes: int = 1 << 30):
        self._alloc = alloc
        self.slab_bytes = slab_bytes
        self._slabs: List[object] = []
        self._blocks: List[list] = []                     # [slab, offset, size, live] in push order
        self._lock = threading.Lock()
        self.allocated_bytes = 0
        self.live_bytes = 0
        self.peak_live_bytes = 0

    def push(self, nbytes: int):
        """Returns ``(buffer view of nbytes, token)``."""
        size = max(self.ALIGN, (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN)
        with self._lock:
            if self._blocks:
                slab, off, sz, _ = self._blocks[-1]
                off += sz
            else:
                slab, off = 0, 0
            while True:
                if slab >= len(self._slabs):
                    cap = max(self.slab_bytes, size)
                    self._slabs.append(self._alloc(cap))
                    self.allocated_bytes += cap
                if off + size <= self._slabs[slab].numel():
                    break
                slab, off = slab + 1, 0
            block = [slab, off, size, True]
            self._blocks.append(block)
            self.live_bytes += size
            self.peak_live_bytes = max(self.peak_live_bytes, self.live_bytes)
            return self._slabs[slab][off:off + nbytes], block

    def pop(self, token) -> None:
        with self._lock:
            if not token[3]:
                return
            token[3] = False
            self.live_bytes -= token[2]
            while self._blocks and not self._blocks[-1][3]:
                self._blocks.pop()

    def clear(self) -> None:
        with self._lock:
            self._slabs.clear()
            self._blocks.clear()
            self.allocated_bytes = self.live_bytes = 0


class SwappedTensor:
    """A saved tensor that lives in pinned host memory until backward fetches it."""
    __slots__ = ("arena", "index", "host", "token", "host_ready", "shape", "dtype", "device", "nbytes", "gpu",
                 "gpu_ready", "word_offsets", "__weakref__")

    def size(self):
        return self.shape

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def __del__(self):
        arena = self.arena
        if arena is not None:
            arena._drop(self)


class SwapArena:
    def __init__(self, device: torch.device, prefetch_bytes: int = 512 << 20, prefetch_count: int = 4):
        self.device = device
        self.pool = PinnedStack(lambda n: torch.empty(n, dtype=torch.uint8, pin_memory=True))
        self._last_read = None                           # the newest host-to-device copy (one stream: it orders all)
        self.copy_out = torch.cuda.Stream(device)
        self.copy_in = torch.cuda.Stream(device)
        self.prefetch_bytes = prefetch_bytes
        self.prefetch_count = prefetch_count
        self._live: Dict[int, "weakref.ReferenceType[SwappedTensor]"] = {}
        self._next = 0
        self._inflight = 0                               # bytes fetched ahead and not yet consumed

    # ------------------------------------------------------------------ device -> host
    def to_host(self, tensor: torch.Tensor) -> SwappedTensor:
        src = tensor.contiguous()
        nbytes = src.numel() * src.element_size()
        host, token = self.pool.push(nbytes)
        free_after = self._last_read                      # whoever read this memory before has been issued by now
        cur = torch.cuda.current_stream(self.device)
        produced = torch.cuda.Event()
        produced.record(cur)
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(produced)
            if free_after is not None:
                self.copy_out.wait_event(free_after)      # earlier host-to-device reads of this memory
            host.view(src.dtype).view(src.shape).copy_(src, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.copy_out)
        src.record_stream(self.copy_out)
        h = SwappedTensor()
        h.arena, h.index, h.host, h.token, h.host_ready = self, self._next, host, token, done
        h.shape, h.dtype, h.device, h.nbytes = tuple(src.shape), src.dtype, src.device, nbytes
        h.gpu, h.gpu_ready = None, None
        h.word_offsets = getattr(tensor, "word_offsets", None)
        self._live[h.index] = weakref.ref(h)
        self._next += 1
        return h

    # ------------------------------------------------------------------ host -> device
    def _issue(self, h: SwappedTensor) -> None:
        if h.gpu is not None or h.host is None:
            return
        with torch.cuda.stream(self.copy_in):
            self.copy_in.wait_event(h.host_ready)
            gpu = torch.empty(h.shape, dtype=h.dtype, device=h.device)
            gpu.copy_(h.host.view(h.dtype).view(h.shape), non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(self.copy_in)
        h.gpu, h.gpu_ready = gpu, ready
        self._last_read = ready
        self._inflight += h.nbytes

    def to_device(self, h: SwappedTensor) -> torch.Tensor:
        if h.host is None:
            raise RuntimeError("this swapped tensor was already fetched")
        self._issue(h)
        # backward walks the saved tensors newest first: fetch the next ones down the stack
        ahead, idx = 0, h.index - 1
        while ahead < self.prefetch_count and idx >= 0 and self._inflight < self.prefetch_bytes:
            ref = self._live.get(idx)
            nxt = ref() if ref is not None else None
            if nxt is not None and nxt.host is not None:
                self._issue(nxt)
                ahead += 1
            idx -= 1
            if h.index - idx > 4 * self.prefetch_count:
                break
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(h.gpu_ready)
        out = h.gpu
        out.record_stream(cur)
        if h.word_offsets is not None:
            out.word_offsets = h.word_offsets
        self._inflight -= h.nbytes
        self.pool.pop(h.token)
        h.host, h.gpu = None, None
        self._live.pop(h.index, None)
        return out

    def _drop(self, h: SwappedTensor) -> None:
        """A handle died without being fetched (forward without backward)."""
        try:
            self._live.pop(h.index, None)
            if h.host is not None:
                if h.gpu is not None:
                    self._inflight -= h.nbytes
                self.pool.pop(h.token)
                h.host = None
        except Exception:                                  # interpreter shutdown
            pass


_arenas: Dict[int, SwapArena] = {}


def arena_for(device: torch.device) -> SwapArena:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    a = _arenas.get(idx)
    if a is None:
        a = _arenas[idx] = SwapArena(torch.device("cuda", idx))
    return a


def reset_arenas() -> None:
    """Forget all arenas (frees the pinned pools once their tensors are gone)."""
    _arenas.clear()
