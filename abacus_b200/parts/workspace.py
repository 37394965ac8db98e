"""Scratch tensors of a step, kept between steps and shared by all layers.

`get(name, shape, dtype)` returns a view of a buffer that only ever grows (with guard words around it,
kernels/guards.py).
`generation` goes up whenever a buffer is replaced, so that whoever holds
addresses (a captured CUDA graph) knows they are stale.
"""
import torch

from ..kernels import guards


class Workspace:
    def __init__(self, device):
        self.device = device
        self.generation = 0
        self._buffers = {}
        self._views = {}

    def get(self, name, shape, dtype):
        view = self._views.get((name, shape, dtype)) if type(shape) is tuple else None
        if view is not None:
            return view
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            buf = guards.empty(max(count, 1), dtype, self.device, what=f"workspace {name}")
            self._buffers[key] = buf
            self.generation += 1
            self._views = {k: v for k, v in self._views.items() if (k[0], k[2]) != key}
        view = buf[:count].view(*shape)
        if type(shape) is tuple:
            if len(self._views) > 4096:
                self._views.clear()
            self._views[(name, shape, dtype)] = view
        return view

    def bytes(self):
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
