"""A model put together from parts, and its forward pass over the rows of a step.

The model is data: a frame (embedding, last norm, output matrix), a list of blocks (built from
BlockSpecs through the part registries) and a schedule, the order the blocks run in; an entry of
the schedule may name a block a second time or read the cache of an earlier entry.
The forward pass is abacus's forward_batch (src/model.c:286-313) followed by
the output matrix on the wanted rows only (src/model.c:322-325).
"""
import torch

from ..parts import BLOCKS, FRAMES, BuildContext, Workspace
from ..weights.loader import check_names


def build_blocks(spec):
    return [BLOCKS.build(b) for b in spec.layers]


def expected_tensors(spec, layout, available=None, blocks=None, frame=None):
    """({tensor name: shape}, names that may be present and are ignored) for a spec and a layout.

    The output matrix is tied to the embedding if the spec says so or if the checkpoint has no
    tensor for it (tools/export.py:81).
    """
    blocks = blocks or build_blocks(spec)
    frame = frame or FRAMES.build(spec)
    tied = spec.tied_head or (available is not None and layout.head not in available)
    names = {"embed": layout.embed, "final_norm": layout.final_norm, "head": layout.head}
    expected = {names[slot]: tuple(shape) for slot, shape in frame.param_shapes(tied).items()}
    for block, layer_names in zip(blocks, layout.layers):
        for part_name, part in block.parts().items():
            for slot, shape in part.param_shapes().items():
                expected[layer_names[(part_name, slot)]] = tuple(shape)
    return expected, ({layout.head} if tied else set())


class Model:
    def __init__(self, spec, layout, tensors, dtype, device):
        """tensors: {name: CPU or GPU tensor} holding at least what expected_tensors lists."""
        self.spec, self.layout = spec, layout
        self.ctx = BuildContext(device=torch.device(device), dtype=dtype)
        self.blocks = build_blocks(spec)
        self.frame = FRAMES.build(spec)
        expected, _ = expected_tensors(spec, layout, set(tensors), self.blocks, self.frame)
        check_names(expected, {n: tuple(t.shape) for n, t in tensors.items() if n in expected},
                    optional=set())
        ctx = self.ctx
        self.tied = layout.head not in expected
        names = {"embed": layout.embed, "final_norm": layout.final_norm, "head": layout.head}
        self.frame.bind({slot: tensors[names[slot]] for slot in self.frame.param_shapes(self.tied)}, ctx)
        for block, layer_names in zip(self.blocks, layout.layers):
            params = {pn: {slot: tensors[layer_names[(pn, slot)]] for slot in part.param_shapes()}
                      for pn, part in block.parts().items()}
            block.bind(params, ctx)
        self.schedule = list(spec.schedule)
        for i, e in enumerate(self.schedule):
            if e.source is not None and not (0 <= e.source < i and self.schedule[e.source].source is None):
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.source}, "
                                 "which must be an earlier entry with a cache of its own")
        self.ws = Workspace(self.ctx.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.ctx.device)

    def parts(self):
        """Every part of the model: the frame, then each block's."""
        yield self.frame
        for b in self.blocks:
            yield from b.parts().values()

    # what the cache must hold, entry by entry
    def cache_needs(self):
        return [self.blocks[e.layer].mixer.cache_need() if e.source is None else None for e in self.schedule]

    def cache_sources(self):
        return [e.source for e in self.schedule]

    def step_plans(self):
        """What the mixers want made on the host for every step (engine/batch.py), one of each name."""
        plans = {}
        for b in self.blocks:
            for p in getattr(b.mixer, "step_plans", lambda: [])():
                plans.setdefault(p.name, p)
        return list(plans.values())

    def prepare(self, max_positions):
        for b in self.blocks:
            prepare = getattr(b.mixer, "prepare", None)
            if prepare:
                prepare(max_positions, self.ctx.device)

    def weight_bytes_read_per_step(self):
        """Bytes of weights a decode step has to read once: what the parts say they read whatever the step's
        size (every matrix and norm, but of the embedding table only the rows looked up, which the caller counts)."""
        seen, total = set(), 0
        parts = [self.frame] + [part for e in self.schedule for part in self.blocks[e.layer].parts().values()]
        for part in parts:
            for t in getattr(part, "step_weights", lambda: [])():
                if t is not None and t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    def forward(self, batch, cache):
        """Logits float32 [batch.n_logit_rows, vocab] of the wanted rows of this step."""
        ws = self.ws
        x = self.frame.embed(batch, ws, self.status)
        y = None
        for i, entry in enumerate(self.schedule):
            y = self.blocks[entry.layer].forward(x, y, batch, cache.views[i], ws)
        return self.frame.logits(x, y, batch, ws)
