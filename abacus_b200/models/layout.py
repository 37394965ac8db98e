"""How an architecture's checkpoint names map onto the slots of the parts."""
from dataclasses import dataclass, field


@dataclass
class ModelLayout:
    """Tensor names of a model.

    embed, final_norm, head: names of the embedding table, the last norm's weight and the output
    matrix. layers[l] maps (part name within the block, slot) to a tensor name, where the part
    names are those of the block's parts() ("mixer_norm", "mixer", "ffn_norm", "ffn").
    """
    embed: str
    final_norm: str
    head: str
    layers: list = field(default_factory=list)
