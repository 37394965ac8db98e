"""Grouped-query causal attention over the paged cache (src/model.c:197-211, 247-259).

The mixer owns the q/k/v and output projections, the optional per-head norm of
q and k, and a position encoding; its sizes, scale, eps and window come from
its spec. q, k and v are one stacked matrix, as in src/model.c:88-93.
"""
import os

import torch

from ..cache.need import CacheNeed
from ..kernels import ops
from .attention_plan import AttentionLists, AttentionStepPlan
from .base import MIXERS, POSITIONS, to_device
from .linear import Linear


# A decode step's attention kernel can norm and rotate q and k and write the new key and value to the cache itself: a
# launch less in every layer. ABACUS_DECODE_PREPARES=0 keeps the preparation a kernel of its own (for comparison).
DECODE_PREPARES = os.environ.get("ABACUS_DECODE_PREPARES", "1") != "0"
# The q/k/v product of a long prompt step can do the same in its epilogue (heads of 128): a kernel and a pass over
# q, k and v less. ABACUS_PRODUCT_PREPARES=0 keeps the preparation a kernel of its own (for comparison).
PRODUCT_PREPARES = os.environ.get("ABACUS_PRODUCT_PREPARES", "1") != "0"


@MIXERS.register("attention")
class Attention:
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} query heads do not divide into {s.n_kv_heads} kv heads")
        if s.head_dim % 8 or s.head_dim > 256:
            raise ValueError(f"head_dim {s.head_dim}: the attention kernels take multiples of 8 up to 256")
        self.position = POSITIONS.build(s.position) if s.position is not None else None
        self.q_size, self.kv_size = s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
        self.cos = self.sin = None
        # a step of several tokens of a windowed layer is checked on the host (it may have to be refused): such
        # steps cannot be replayed from a captured graph; single-token steps can
        self.capturable_prompts = s.window is None
        self.lists = AttentionStepPlan(s.n_heads)  # the prefill kernels' tiles and work list, made per step

    def step_plans(self):
        """What this mixer wants made on the host for every step and sent with the step's indices."""
        return [self.lists]

    def step_weights(self):
        """The tensors a step reads once whatever its size (for the bytes a decode step must move)."""
        return [self.qkv_proj.weight, self.o_proj.weight, self.q_norm, self.k_norm]

    def param_shapes(self):
        s = self.spec
        shapes = {"wq": (self.q_size, s.hidden), "wk": (self.kv_size, s.hidden), "wv": (self.kv_size, s.hidden),
                  "wo": (s.hidden, self.q_size)}
        if s.qk_norm_eps is not None:
            shapes.update(q_norm=(s.head_dim,), k_norm=(s.head_dim,))
        return shapes

    def bind(self, params, ctx):
        self.ctx = ctx
        wqkv = torch.cat([params["wq"], params["wk"], params["wv"]], dim=0)
        self.qkv_proj = Linear(to_device(wqkv, ctx, ctx.dtype))
        self.q_proj = Linear(self.qkv_proj.weight[:self.q_size])  # for entries that read another entry's cache
        self.o_proj = Linear(to_device(params["wo"], ctx, ctx.dtype))
        self.q_norm = to_device(params["q_norm"], ctx, torch.float32) if "q_norm" in params else None
        self.k_norm = to_device(params["k_norm"], ctx, torch.float32) if "k_norm" in params else None

    def cache_need(self):
        s = self.spec
        return CacheNeed(n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.cos, self.sin = self.position.tables(max_positions, device)

    def forward(self, xn, out, batch, cache, ws):
        s = self.spec
        n = batch.n_rows
        qkv = ws.get("qkv", (n, self.q_size + 2 * self.kv_size), self.ctx.dtype)
        att = ws.get("att", (n, self.q_size), self.ctx.dtype)
        writes = cache.owns_storage
        rotary_dim = self.position.rotary_dim if self.position else 0
        interleaved = self.position.interleaved if self.position else False
        # A windowed cache keeps only the last keys; a prompt longer than that reads its keys from
        # this step's own rows, which hold all of them when the sequences start at position 0.
        from_step = s.window is not None and not batch.is_decode
        w = self.qkv_proj.weight
        prepared = False  # by the product's own kernel: a prompt's heads in its epilogue
        if (PRODUCT_PREPARES and writes and not batch.is_decode and not from_step and w.dtype == torch.bfloat16
                and ops.gemm_tc_qkv_takes(xn, w, qkv, n, s.n_heads, s.n_kv_heads, s.head_dim, cache.kv, self.q_norm,
                                          self.k_norm, self.cos, self.sin, rotary_dim, interleaved)):
            ops.gemm_tc_qkv(xn, w, qkv, s.n_heads, s.n_kv_heads, batch, self.q_norm, self.k_norm, s.qk_norm_eps,
                            self.cos, self.sin, cache.kv, n)
            prepared = True
        elif writes:
            self.qkv_proj.forward(xn, qkv, n)
        else:  # keys and values are another entry's: only q is needed
            self.q_proj.forward(xn, qkv[:, :self.q_size], n)
        prepare = None
        if prepared:
            pass
        elif (DECODE_PREPARES and batch.is_decode and cache.kv is not None
                and ops.attention_decode_prepares(qkv, s.n_heads, s.n_kv_heads, s.head_dim, cache.kv, self.q_norm,
                                                  self.k_norm, self.cos, self.sin, rotary_dim, interleaved)):
            prepare = dict(q_norm=self.q_norm, k_norm=self.k_norm, eps=s.qk_norm_eps, cos=self.cos, sin=self.sin, keep=writes)
        else:
            ops.qkv_prep(qkv, s.n_heads, s.n_kv_heads, s.head_dim, batch, self.q_norm, self.k_norm, s.qk_norm_eps,
                         self.cos, self.sin, rotary_dim, interleaved, cache.kv if writes else None, q_only=not writes)
        if from_step and (batch.any_continuation or not writes):
            raise ops.KernelRefused("windowed attention takes several tokens of a sequence only at its start, "
                                    "and only with keys of its own")
        mine = batch.plan.get(self.lists.name)
        ops.attention(qkv, att, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, batch, cache.kv,
                      from_step=from_step, ws=ws, lists=AttentionLists(mine) if mine is not None else None, prepare=prepare)
        self.o_proj.forward(att, out, n)
        return out
