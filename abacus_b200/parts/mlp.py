"""Gated feed-forward: down(silu(gate(x)) * up(x)) (src/model.c:274-282, 307-309).

gate and up are one stacked matrix, as in src/model.c:98.
"""
import torch

from ..kernels import ops
from .base import FEED_FORWARDS, to_device
from .linear import ROWS_KERNEL_UP_TO, Linear


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP:
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not built (only silu)")
        self.spec = spec

    def param_shapes(self):
        s = self.spec
        return {"gate": (s.inter, s.hidden), "up": (s.inter, s.hidden), "down": (s.hidden, s.inter)}

    def bind(self, params, ctx):
        self.ctx = ctx
        self.gate_up = Linear(to_device(torch.cat([params["gate"], params["up"]], dim=0), ctx, ctx.dtype))
        self.down = Linear(to_device(params["down"], ctx, ctx.dtype))

    def forward(self, xn, out, batch, ws):
        n, inter = batch.n_rows, self.spec.inter
        act = ws.get("act", (n, inter), self.ctx.dtype)
        if n <= ROWS_KERNEL_UP_TO and ops.gemm_rows_takes(xn, self.gate_up.weight, act, n):
            ops.gemm_rows_swiglu(xn, self.gate_up.weight, act, n)  # a handful of rows: product and activation in one
        else:
            gate_up = ws.get("gate_up", (n, 2 * inter), self.ctx.dtype)
            self.gate_up.forward(xn, gate_up, n)
            ops.swiglu(gate_up, act)
        self.down.forward(act, out, n)
        return out
