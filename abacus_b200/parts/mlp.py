"""Gated feed-forward: down(silu(gate(x)) * up(x)) (src/model.c:274-282, 307-309).

gate and up are one matrix, as in src/model.c:98. In bfloat16, when the inner size allows, its rows come
in turns of 128 (gate of features 0-127, up of the same, gate of 128-255, ...): a 256-column tile of the
tensor-core product then holds both halves of 128 features, and the activation runs in its epilogue.
"""
import torch

from ..kernels import ops
from .base import FEED_FORWARDS, to_device
from .linear import Linear, rows_kernel_wins


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

    TURN = 128  # rows of gate, then of up, where the layout comes in turns

    def bind(self, params, ctx):
        self.ctx = ctx
        inter, gate, up = self.spec.inter, params["gate"], params["up"]
        self.block = self.TURN if ctx.dtype == torch.bfloat16 and inter % self.TURN == 0 else inter
        turns = inter // self.block
        stacked = torch.stack([gate.reshape(turns, self.block, -1), up.reshape(turns, self.block, -1)], dim=1)
        self.gate_up = Linear(to_device(stacked.reshape(2 * inter, -1).contiguous(), ctx, ctx.dtype))
        self.down = Linear(to_device(params["down"], ctx, ctx.dtype))

    def step_weights(self):
        return [self.gate_up.weight, self.down.weight]

    def forward(self, xn, out, batch, ws):
        n, inter = batch.n_rows, self.spec.inter
        act = ws.get("act", (n, inter), self.ctx.dtype)
        w = self.gate_up.weight
        if rows_kernel_wins(n, w, gated=True) and ops.gemm_rows_takes(xn, w, act, n):
            ops.gemm_rows_swiglu(xn, w, act, n, self.block)  # a handful of rows: product and activation in one
        elif ops.gemm_tc_swiglu_takes(xn, w, act, n, self.block):
            ops.gemm_tc_swiglu(xn, w, act, n)  # a prompt: the activation in the product's epilogue
        else:
            gate_up = ws.get("gate_up", (n, 2 * inter), self.ctx.dtype)
            self.gate_up.forward(xn, gate_up, n)
            ops.swiglu(gate_up, act, self.block)
        self.down.forward(act, out, n)
        return out
