"""Scratch tensors of a step, kept between steps and shared by all layers.

`get(name, shape, dtype)` returns a view of a buffer that only ever grows.
`generation` goes up whenever a buffer is replaced, so that whoever holds
addresses (a captured CUDA graph) knows they are stale.
"""
import torch


class Workspace:
    def __init__(self, device):
        self.device = device
        self.generation = 0
        self._buffers = {}

    def get(self, name, shape, dtype):
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf[:count].view(*shape)

    def bytes(self):
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
