"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a seed.

Matrices are N(0, std), norm weights 1 + N(0, norm_std), all stored as
bfloat16 like the checkpoints tools/export.py converts. The values depend only
on (seed, tensor name), not on the order tensors are made in.
"""
import hashlib
import json
import os

import torch

from .safetensors_io import save_tensors


def _generator(seed, name):
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensor(name, shape, seed, std=0.02, norm_std=0.0, scales=None):
    """One tensor by name: 1-D tensors are norm weights, the rest matrices.

    scales: optional {substring of a name: factor} applied after drawing, for
    tests that want, say, sharper attention.
    """
    g = _generator(seed, name)
    if len(shape) == 1:
        t = torch.ones(shape, dtype=torch.float32)
        if norm_std:
            t += norm_std * torch.randn(shape, generator=g, dtype=torch.float32)
    else:
        t = std * torch.randn(shape, generator=g, dtype=torch.float32)
    for key, factor in (scales or {}).items():
        if key in name:
            t = t * factor
    return t.to(torch.bfloat16)


def random_tensors(expected, seed, std=0.02, norm_std=0.0, scales=None):
    return {name: random_tensor(name, tuple(shape), seed, std, norm_std, scales) for name, shape in expected.items()}


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
