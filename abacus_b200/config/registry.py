"""One registry from an architecture's name (config.json "architectures"[0]) to its model.

An architecture is an object with
  name                    the string config.json carries
  parse_config(dict)      -> a typed configuration with .to_spec() -> ModelSpec
  tensor_names(spec)      -> how safetensors names map onto the parts (see models/qwen3.py)
  info(spec)              -> the model's name and sizes in one line, for the command line's --info
Adding an architecture is one call of `register_architecture`; nothing else in
the package names a model.
"""
import json
import os


class ConfigError(ValueError):
    """A config.json that is unreadable, incomplete or asks for what is not built."""


_ARCHITECTURES = {}


def register_architecture(arch):
    _ARCHITECTURES[arch.name] = arch
    return arch


def architecture_names():
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name):
    _load_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; known: {', '.join(sorted(_ARCHITECTURES))}")
    return _ARCHITECTURES[name]


def _load_builtin():
    from .. import models  # noqa: F401  (registers the built-in architectures on import)


def read_config_json(folder):
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def architecture_of(raw):
    names = raw.get("architectures")
    if not names or not isinstance(names, list):
        raise ConfigError('config.json has no "architectures" list; known: ' + ", ".join(architecture_names()))
    return get_architecture(names[0])


def load_config(folder):
    """config.json of a model folder -> (architecture, typed configuration)."""
    raw = read_config_json(folder)
    arch = architecture_of(raw)
    return arch, arch.parse_config(raw)
