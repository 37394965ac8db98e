"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a seed.

Matrices are N(0, std), norm weights 1 + N(0, norm_std), all stored as bfloat16 like the checkpoints
tools/export.py converts. abacus gets such a model from a library's initialiser (tools/tiny.py:15-20);
here a value depends only on (seed, tensor name, element index): a tensor can be filled on the GPU in
one pass (csrc/utility.cu) or made on the host, whole or in slices, and both give the same bits.

The unit normal is a sum of twelve 16-bit uniforms drawn from three splitmix64-mixed counters: integer
arithmetic and two float32 roundings, nothing that two machines could round differently. Its variance
is 1 - 2^-32 and it stays within +-6.
"""
import hashlib
import json
import os

import numpy as np
import torch

from .safetensors_io import save_tensors

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1, _M2 = np.uint64(0xBF58476D1CE4E5B9), np.uint64(0x94D049BB133111EB)
_HOST_CHUNK = 1 << 22


def tensor_key(seed, name):
    """The 64-bit key of a tensor's random stream."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _mix64(x):
    x = x ^ (x >> np.uint64(30))
    x = x * _M1
    x = x ^ (x >> np.uint64(27))
    x = x * _M2
    return x ^ (x >> np.uint64(31))


def unit_normal(key, first, count):
    """z(key, i) for i in [first, first + count), float32: the host twin of csrc/utility.cu's unit_normal."""
    with np.errstate(over="ignore"):
        i = np.arange(first, first + count, dtype=np.uint64)
        total = np.zeros(count, dtype=np.int64)
        low = np.uint64(0xFFFF)
        for j in (1, 2, 3):
            h = _mix64(np.uint64(key) + _GAMMA * (np.uint64(3) * i + np.uint64(j)))
            total += ((h & low) + ((h >> np.uint64(16)) & low) + ((h >> np.uint64(32)) & low)
                      + (h >> np.uint64(48))).astype(np.int64)
    return (total - 393210).astype(np.float32) * np.float32(1.0 / 65536.0)


def normal_values(key, first, count, mean, amplitude):
    """mean + amplitude * z, each operation rounded to float32 (what the device kernel computes)."""
    return (np.float32(mean) + np.float32(amplitude) * unit_normal(key, first, count)).astype(np.float32)


def _moments(name, shape, std, norm_std, scales):
    """(mean, amplitude) of a tensor: 1-D tensors are norm weights, the rest matrices; `scales` multiplies both."""
    mean, amplitude = (1.0, norm_std) if len(shape) == 1 else (0.0, std)
    for key, factor in (scales or {}).items():
        if key in name:
            mean, amplitude = mean * factor, amplitude * factor
    return float(np.float32(mean)), float(np.float32(amplitude))


def random_tensor(name, shape, seed, std=0.02, norm_std=0.0, scales=None, device=None, dtype=torch.bfloat16):
    """One tensor by name: 1-D tensors are norm weights, the rest matrices.

    scales: optional {substring of a name: factor} applied to the distribution, for tests that want, say,
    sharper attention. device: None or "cpu" makes it on the host; a CUDA device fills it there with the
    kernel. Both give the same bits.
    """
    mean, amplitude = _moments(name, shape, std, norm_std, scales)
    key = tensor_key(seed, name)
    count = int(np.prod(shape)) if len(shape) else 1
    device = torch.device(device) if device is not None else torch.device("cpu")
    if device.type == "cuda":
        from ..kernels import ops
        out = torch.empty(tuple(shape), dtype=dtype, device=device)
        ops.fill_normal(out, key, mean, amplitude)
        return out
    out = torch.empty(count, dtype=dtype)
    for first in range(0, count, _HOST_CHUNK):
        n = min(_HOST_CHUNK, count - first)
        out[first:first + n] = torch.from_numpy(normal_values(key, first, n, mean, amplitude)).to(dtype)
    return out.reshape(tuple(shape))


def random_tensors(expected, seed, std=0.02, norm_std=0.0, scales=None, device=None):
    return {name: random_tensor(name, tuple(shape), seed, std, norm_std, scales, device)
            for name, shape in expected.items()}


def write_random_model(folder, config, seed, std=0.02, norm_std=0.0, scales=None):
    """Write config.json and model.safetensors for `config` (a typed configuration of a registered architecture)."""
    from ..config.registry import get_architecture
    arch = get_architecture(config.architecture)
    expected, _ = arch.tensor_names(config.to_spec(), None)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    save_tensors(os.path.join(folder, "model.safetensors"), random_tensors(expected, seed, std, norm_std, scales))
    return folder
