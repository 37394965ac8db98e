"""Rotary position encoding: the table of angles (src/model.c:116-124).

A position encoding of the rotary family gives the attention mixer
  tables(n_positions, device) -> (cos, sin), float32 [n_positions, rotary_dim / 2]
  rotary_dim, interleaved
and the q/k preparation kernel applies them. The angles are made on the host
in float32 with abacus's own expression, pos * (1 / theta^(2i / rotary_dim)).
"""
import numpy as np
import torch

from .base import POSITIONS


@POSITIONS.register("rotary")
class Rotary:
    def __init__(self, spec):
        if spec.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {spec.pairing!r} is neither half nor interleaved")
        if spec.rotary_dim < 2 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        self.interleaved = spec.pairing == "interleaved"
        self._tables = {}

    def tables(self, n_positions, device):
        key = str(device)
        have = self._tables.get(key)
        if have is None or have[0].shape[0] < n_positions:
            half = self.rotary_dim // 2
            i = np.arange(half, dtype=np.float32)
            inv = np.float32(1.0) / np.power(np.float32(self.spec.theta),
                                             (np.float32(2.0) * i) / np.float32(self.rotary_dim), dtype=np.float32)
            angle = (np.arange(n_positions, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
            have = (torch.from_numpy(np.cos(angle, dtype=np.float32)).to(device),
                    torch.from_numpy(np.sin(angle, dtype=np.float32)).to(device))
            self._tables[key] = have
        return have
