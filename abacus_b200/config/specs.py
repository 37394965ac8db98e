"""Descriptions of the parts a model is put together from.

A spec is plain data: the sizes and constants one part needs, nothing about the
model it sits in. An architecture's configuration turns its config.json into a
`ModelSpec`: one `BlockSpec` per layer (so layers may differ), and a schedule,
the order in which layers run.

Every spec class carries a `kind`; the part registries (abacus_b200.parts) map
a kind to the class that implements it. A new kind of part brings its own spec
class; nothing here needs to know it.
"""
from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    """RMSNorm as src/model.c:164-169: w * (x / sqrt(mean(x^2) + eps))."""
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding as src/model.c:116-124, 173-181.

    pairing "half" rotates (i, i + rotary_dim/2); "interleaved" rotates (2i, 2i+1).
    rotary_dim may be smaller than the head size (the rest passes unchanged).
    """
    theta: float
    rotary_dim: int
    pairing: str = "half"
    kind: str = "rotary"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal attention as src/model.c:197-211, 247-259.

    window None: every earlier key; W: the last W keys, the token's own included.
    scale multiplies the scores (src/model.c:202 uses 1/sqrt(head_dim)).
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float
    qk_norm_eps: Optional[float]  # None: no per-head norm of q and k
    position: Optional[RotarySpec]
    window: Optional[int] = None
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(x)) * up(x)) as src/model.c:274-282, 307-309."""
    hidden: int
    inter: int
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its two norms, its mixer, its feed-forward and how they are wired.

    arrangement "pre_norm" is src/model.c:292-310: x += mixer(norm(x)); x += ffn(norm(x)).
    """
    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object
    arrangement: str = "pre_norm"

    @property
    def kind(self):
        return self.arrangement


@dataclass(frozen=True)
class ScheduleEntry:
    """One entry of the run order.

    layer: index into ModelSpec.layers (a layer may be named more than once).
    source: None if the mixer keeps keys/values or state of its own for this
    entry; else the index of an earlier entry whose cache it reads.
    """
    layer: int
    source: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden: int
    vocab: int
    layers: tuple
    schedule: tuple
    final_norm: object
    tied_head: bool
    max_positions: int
    stop_tokens: tuple = field(default_factory=tuple)
    frame: str = "plain"  # how tokens become the stream and the stream logits (parts/frame.py)

    @property
    def kind(self):  # the frame is built from the model's spec
        return self.frame
