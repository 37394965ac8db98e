"""The frame around the layers: how tokens become the residual stream and how the stream becomes logits.

"plain" is abacus's: x = float(embed[token]) with no scale (src/model.c:290-291); after the last layer
x += y, xn = norm(x) (src/model.c:311-312) and logits = xn . head^T on the wanted rows only
(src/model.c:322-325), the output matrix being the embedding table when the model ties them
(src/model.c:102-103). An architecture that scales its embeddings, caps its logits or norms elsewhere
registers another frame; the model's forward pass does not change.

A frame has
  param_shapes(tied) -> {slot: shape}     slots "embed", "final_norm", and "head" unless tied
  bind(params, ctx)
  embed(batch, ws, status) -> x           float32 [rows, hidden], the residual stream
  logits(x, y, batch, ws) -> float32 [batch.n_logit_rows, vocab]
  step_weights() -> tensors a step reads once whatever its size
"""
import torch

from ..kernels import ops
from .base import FRAMES, NORMS, to_device
from .linear import Linear


@FRAMES.register("plain")
class PlainFrame:
    capturable = True  # launches kernels only

    def __init__(self, spec):
        """spec: the ModelSpec (hidden, vocab, final_norm)."""
        self.hidden, self.vocab = spec.hidden, spec.vocab
        self.final_norm = NORMS.build(spec.final_norm)

    def param_shapes(self, tied):
        shapes = {"embed": (self.vocab, self.hidden), "final_norm": tuple(self.final_norm.param_shapes()["weight"])}
        if not tied:
            shapes["head"] = (self.vocab, self.hidden)
        return shapes

    def bind(self, params, ctx):
        self.ctx = ctx
        self.table = to_device(params["embed"], ctx, ctx.dtype)
        self.tied = "head" not in params
        self.head = Linear(self.table if self.tied else to_device(params["head"], ctx, ctx.dtype))
        self.final_norm.bind({"weight": params["final_norm"]}, ctx)

    def step_weights(self):
        # of the embedding table a step reads only the rows it looks up; the output matrix it reads whole
        return [self.head.weight, *self.final_norm.step_weights()]

    def embed(self, batch, ws, status):
        x = ws.get("x", (batch.n_rows, self.hidden), torch.float32)
        ops.embed(batch.tokens, self.table, x, status)
        return x

    def logits(self, x, y, batch, ws):
        r = batch.n_logit_rows
        out = ws.get("logits", (max(r, 1), self.vocab), torch.float32)[:r]
        if r:
            xn = ws.get("xn_final", (r, self.hidden), self.ctx.dtype)
            self.final_norm.forward(x, y, xn, rows=batch.logit_rows, n_rows=r)
            self.head.forward(xn, out, r)
        return out
