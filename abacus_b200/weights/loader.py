"""Weights by tensor name, checked against what the model's parts expect.

`expected` comes from the architecture (models/qwen3.py: the names of
tools/export.py:90-99). All faults of a folder are reported in one error:
missing names, names nothing asks for, and wrong shapes.
"""
from .safetensors_io import FolderReader, WeightError


def check_names(expected, available, optional=()):
    """expected {name: shape}; available {name: shape}. Raises one WeightError listing every fault."""
    missing = sorted(n for n in expected if n not in available)
    unexpected = sorted(n for n in available if n not in expected and n not in optional)
    wrong = sorted((n, tuple(available[n]), tuple(expected[n])) for n in expected
                   if n in available and tuple(available[n]) != tuple(expected[n]))
    if not (missing or unexpected or wrong):
        return
    lines = ["the weights do not fit the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " +
                     ", ".join(f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong))
    raise WeightError("\n".join(lines))


def load_folder(folder, expected_of):
    """Read a model folder's tensors.

    expected_of(names in the folder) -> ({name: shape}, optional names): the
    architecture may depend on what is there (a tied head has no lm_head.weight).
    Returns {name: CPU tensor}, each in its stored precision.
    """
    reader = FolderReader(folder)
    available = {n: reader.shape(n) for n in reader.names()}
    expected, optional = expected_of(set(available))
    check_names(expected, available, optional)
    return {name: reader.tensor(name) for name in expected}
