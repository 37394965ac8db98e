"""What every part is, and the registries that map a spec's kind to its class.

A part is built from its spec alone (sizes and constants), declares the tensors
it needs as named slots with shapes, is bound to tensors once, and then runs on
the rows of a step. No part knows which model it is in or what its tensors are
called in a checkpoint: the architecture's layout maps slots to names.

Interfaces (duck-typed; these base classes only document them):

  Part.param_shapes() -> {slot: shape}
  Part.bind(params: {slot: tensor}, ctx: BuildContext)

  Norm.forward(x, y, out, rows=None, n_rows=None)
      x float32 [T, d] is the residual stream; y (or None) is added to it first
      (x is updated in place), then out = norm(x). With rows, only those rows
      are normed into out and x is left alone.
  Mixer.cache_need() -> cache.CacheNeed (keys/values per token, a window, and/or
      a per-sequence state of fixed shape)
  Mixer.forward(xn, out, batch, cache, ws)
      xn [T, d] in the compute dtype; out float32 [T, d] is what is added to
      the residual stream; batch is engine.batch.StepBatch; cache is the
      cache.EntryView of this schedule entry.
  FeedForward.forward(xn, out, batch, ws)
  Position: see parts/position.py.
  A part whose forward only launches device work (no decision on the host from the step's
  contents, no allocation) may set `capturable = True`; decode steps of a model whose parts
  all do are replayed as CUDA graphs. Without it the model runs step by step.
  Block.forward(x, y, batch, cache, ws) -> y': runs norms, mixer and
      feed-forward in its arrangement; y is the output still to be added to x.
  Frame: see parts/frame.py.
  Optional, on any part:
    step_weights() -> tensors the part reads once per step whatever the step's size (the bytes a decode step moves)
    capturable_prompts (mixers): False if steps of several tokens must not be replayed from a captured graph
    step_plans() (mixers): see engine/batch.py
"""
from dataclasses import dataclass

import torch


@dataclass
class BuildContext:
    device: torch.device
    dtype: torch.dtype  # torch.bfloat16: the serving path; torch.float32: everything in true 32-bit


class Registry:
    def __init__(self, what):
        self.what = what
        self._classes = {}

    def register(self, kind, cls=None):
        if cls is None:  # decorator form
            return lambda c: self.register(kind, c)
        self._classes[kind] = cls
        return cls

    def build(self, spec, **kw):
        kind = getattr(spec, "kind", None)
        if kind not in self._classes:
            raise KeyError(f"no {self.what} of kind {kind!r}; registered: {', '.join(sorted(self._classes))}")
        return self._classes[kind](spec, **kw)

    def kinds(self):
        return sorted(self._classes)


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block arrangement")
FRAMES = Registry("frame (embedding, last norm and output matrix)")


def to_device(t, ctx, dtype=None):
    """A parameter on the device; dtype None keeps the stored precision."""
    return t.to(device=ctx.device, dtype=dtype or t.dtype).contiguous()
