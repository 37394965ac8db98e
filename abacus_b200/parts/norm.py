"""RMSNorm fused with the residual add that precedes it (src/model.c:238-244, 164-169)."""
import torch

from ..kernels import ops
from .base import NORMS, to_device


@NORMS.register("rmsnorm")
class RMSNorm:
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        self.spec = spec
        self.weight = None

    def param_shapes(self):
        return {"weight": (self.spec.size,)}

    def bind(self, params, ctx):
        self.weight = to_device(params["weight"], ctx, torch.float32)

    def step_weights(self):
        return [self.weight]

    def forward(self, x, y, out, rows=None, n_rows=None):
        ops.add_rmsnorm(x, y, self.weight, out, self.spec.eps, rows=rows, n_rows=n_rows)
        return out
