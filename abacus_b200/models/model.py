"""A model put together from parts, and its forward pass over the rows of a step.

The model is data: a list of blocks (built from BlockSpecs through the part
registries) and a schedule, the order the blocks run in; an entry of the
schedule may name a block a second time or read the cache of an earlier entry.
The forward pass is abacus's forward_batch (src/model.c:286-313) followed by
the output matrix on the wanted rows only (src/model.c:322-325).
"""
import torch

from ..kernels import ops
from ..parts import BLOCKS, NORMS, BuildContext, Linear, Workspace
from ..parts.base import to_device
from ..weights.loader import check_names


def build_blocks(spec):
    return [BLOCKS.build(b) for b in spec.layers]


def expected_tensors(spec, layout, available=None, blocks=None):
    """({tensor name: shape}, names that may be present and are ignored) for a spec and a layout.

    The output matrix is tied to the embedding if the spec says so or if the checkpoint has no
    tensor for it (tools/export.py:81).
    """
    blocks = blocks or build_blocks(spec)
    expected = {layout.embed: (spec.vocab, spec.hidden), layout.final_norm: (spec.final_norm.size,)}
    for block, names in zip(blocks, layout.layers):
        for part_name, part in block.parts().items():
            for slot, shape in part.param_shapes().items():
                expected[names[(part_name, slot)]] = tuple(shape)
    tied = spec.tied_head or (available is not None and layout.head not in available)
    optional = set()
    if tied:
        optional.add(layout.head)
    else:
        expected[layout.head] = (spec.vocab, spec.hidden)
    return expected, optional


class Model:
    def __init__(self, spec, layout, tensors, dtype, device):
        """tensors: {name: CPU or GPU tensor} holding at least what expected_tensors lists."""
        self.spec, self.layout = spec, layout
        self.ctx = BuildContext(device=torch.device(device), dtype=dtype)
        self.blocks = build_blocks(spec)
        expected, _ = expected_tensors(spec, layout, set(tensors), self.blocks)
        check_names(expected, {n: tuple(t.shape) for n, t in tensors.items() if n in expected},
                    optional=set())
        ctx = self.ctx
        self.embed = to_device(tensors[layout.embed], ctx, dtype)
        self.tied = layout.head not in expected
        self.head = Linear(self.embed if self.tied else to_device(tensors[layout.head], ctx, dtype))
        self.final_norm = NORMS.build(spec.final_norm)
        self.final_norm.bind({"weight": tensors[layout.final_norm]}, ctx)
        for block, names in zip(self.blocks, layout.layers):
            params = {pn: {slot: tensors[names[(pn, slot)]] for slot in part.param_shapes()}
                      for pn, part in block.parts().items()}
            block.bind(params, ctx)
        self.schedule = list(spec.schedule)
        for i, e in enumerate(self.schedule):
            if e.source is not None and not (0 <= e.source < i and self.schedule[e.source].source is None):
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.source}, "
                                 "which must be an earlier entry with a cache of its own")
        self.ws = Workspace(self.ctx.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.ctx.device)
        # a hint for whoever shares out attention's work among CTAs: the most heads any mixer runs per token
        self.attention_heads = max([getattr(getattr(b.mixer, "spec", None), "n_heads", 1) for b in self.blocks] + [1])

    # what the cache must hold, entry by entry
    def cache_needs(self):
        return [self.blocks[e.layer].mixer.cache_need() if e.source is None else None for e in self.schedule]

    def cache_sources(self):
        return [e.source for e in self.schedule]

    def prepare(self, max_positions):
        for b in self.blocks:
            prepare = getattr(b.mixer, "prepare", None)
            if prepare:
                prepare(max_positions, self.ctx.device)

    def weight_bytes_read_per_step(self):
        """Bytes of weights a decode step has to read once: every matrix and norm, but of the
        embedding table only the rows looked up (counted by the caller)."""
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        for e in self.schedule:
            b = self.blocks[e.layer]
            for part in b.parts().values():
                for v in vars(part).values():
                    if isinstance(v, Linear):
                        add(v.weight)
                    elif isinstance(v, torch.Tensor) and v.is_cuda and v.dim() == 1:
                        add(v)
        add(self.head.weight)
        add(self.final_norm.weight)
        return total

    def forward(self, batch, cache):
        """Logits float32 [batch.n_logit_rows, vocab] of the wanted rows of this step."""
        n, d, ws = batch.n_rows, self.spec.hidden, self.ws
        x = ws.get("x", (n, d), torch.float32)
        ops.embed(batch.tokens, self.embed, x, self.status)
        y = None
        for i, entry in enumerate(self.schedule):
            y = self.blocks[entry.layer].forward(x, y, batch, cache.views[i], ws)
        r = batch.n_logit_rows
        logits = ws.get("logits", (max(r, 1), self.spec.vocab), torch.float32)[:r]
        if r:
            xn = ws.get("xn_final", (r, d), self.ctx.dtype)
            self.final_norm.forward(x, y, xn, rows=batch.logit_rows, n_rows=r)
            self.head.forward(xn, logits, r)
        return logits
