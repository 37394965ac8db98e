"""The step function in C (csrc/step.cu), bound to a model once and called once per step.

A step is a few hundred kernel launches. Launched from Python one by one each costs some ten microseconds
of interpreter and ctypes; for a small model that is as long as the GPU works on them. `CStep` describes
the model to the C walker in plain structures (the parts' sizes, constants and device pointers, the
launchers' addresses) and from then on a step is one foreign call. abacus's forward() is C for the same
reason it is short: a fixed order of a dozen calls per layer (src/model.c:286-327).

It serves models whose parts are all the library's own in abacus's arrangement (`CStep.serves`); any other
model runs through the parts' forward() as before, and so does every model with ABACUS_C_STEP=0. Both
ways launch the same kernels with the same arguments; tests hold them to the same bits.
"""
import ctypes
import os

import torch

from ..kernels import ops
from ..kernels.build import load_module
from ..parts.attention import DECODE_PREPARES, PRODUCT_PREPARES, Attention
from ..parts.attention_plan import AttentionLists
from ..parts.block import PreNormBlock
from ..parts.frame import PlainFrame
from ..parts.mlp import GatedMLP
from ..parts.norm import RMSNorm

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
ENABLED = os.environ.get("ABACUS_C_STEP", "1") != "0"

# (field of AbkFns, kernel library, exported launcher) in the order of csrc/step.cu
LAUNCHERS = [("embed", "elementwise", "abk_embed"), ("add_rmsnorm", "elementwise", "abk_add_rmsnorm"),
             ("swiglu", "elementwise", "abk_swiglu"), ("qkv_prep", "elementwise", "abk_qkv_prep"),
             ("gemm_simt", "gemm_simt", "abk_gemm_simt"), ("gemm_rows", "gemm_rows", "abk_gemm_rows"),
             ("gemm_rows_swiglu", "gemm_rows", "abk_gemm_rows_swiglu"), ("gemm_tc", "gemm_tc", "abk_gemm_tc"),
             ("gemm_tc_swiglu", "gemm_tc", "abk_gemm_tc_swiglu"),
             ("attention_generic", "attention_generic", "abk_attention_generic"),
             ("attention_prefill", "attention_mma", "abk_attention_prefill"),
             ("attention_prefill_tc", "attention_tc", "abk_attention_prefill_tc"),
             ("attention_decode_ring", "attention_decode_ring", "abk_attention_decode_ring"),
             ("attention_decode", "attention_decode", "abk_attention_decode"),
             ("attention_decode_ring_prepare", "attention_decode_ring", "abk_attention_decode_ring_prepare"),
             ("gemm_tc_qkv", "gemm_tc", "abk_gemm_tc_qkv")]


class Fns(ctypes.Structure):
    _fields_ = [(name, P) for name, _, _ in LAUNCHERS]


class Linear(ctypes.Structure):
    _fields_ = [("w", P), ("ldw", L), ("n", I), ("k", I), ("dtype", I), ("pad", I)]


class Norm(ctypes.Structure):
    _fields_ = [("w", P), ("eps", F), ("size", I)]


class AttentionS(ctypes.Structure):
    _fields_ = [("qkv", Linear), ("q_only", Linear), ("o", Linear), ("q_norm", P), ("k_norm", P), ("cos", P), ("sin", P),
                ("eps", F), ("scale", F), ("n_heads", I), ("n_kv_heads", I), ("head_dim", I), ("window", I),
                ("rotary_dim", I), ("interleaved", I), ("table_positions", I), ("lists", I)]


class Mlp(ctypes.Structure):
    _fields_ = [("gate_up", Linear), ("down", Linear), ("inter", I), ("block", I)]


class Block(ctypes.Structure):
    _fields_ = [("norm1", Norm), ("norm2", Norm), ("att", AttentionS), ("mlp", Mlp)]


class Entry(ctypes.Structure):
    _fields_ = [("k", P), ("v", P), ("table", P), ("pool_rows", L), ("block", I), ("owns", I), ("table_width", I),
                ("ring_pages", I), ("tokens_per_page", I), ("pad", I)]


class ModelS(ctypes.Structure):
    _fields_ = [("fns", P), ("blocks", P), ("entries", P), ("embed", P), ("final_norm", Norm), ("head", Linear),
                ("status", P), ("gemm_scratch", P), ("gemm_tickets", P), ("kernel_status", P), ("halves", P),
                ("halves_tickets", P), ("attention_tickets", P), ("dtype", I), ("hidden", I), ("vocab", I),
                ("n_blocks", I), ("n_entries", I), ("halves_pairs", I), ("attention_ticket_count", I), ("decode_prepares", I),
                ("product_prepares", I)]


class Lists(ctypes.Structure):
    _fields_ = [("tiles64", P), ("work", P), ("n_tiles64", I), ("n_work", I), ("n_halved", I), ("pad", I)]


class Step(ctypes.Structure):
    _fields_ = [(n, P) for n in ("tokens", "token_seq", "token_pos", "seq_slot", "seq_start", "seq_pos0", "seq_len_after",
                                 "logit_rows", "lists", "x", "branch", "logits", "attention_partials", "xn", "qkv", "att",
                                 "act", "gate_up", "xn_final")]
    _fields_ += [("partial_floats", L)] + [(n, I) for n in ("n_rows", "n_logit_rows", "is_decode", "any_continuation",
                                                            "max_len_after", "position_bound", "n_lists", "pad")]


REFUSALS = {-101: "windowed attention takes several tokens of a sequence only at its start, and only with keys of its own",
            -102: "the step halves more attention tiles than the kernel's scratch memory holds",
            -103: "more (row, kv head) pairs than decode attention has tickets for",
            -104: "the workspace for decode attention's partial results is too small"}


def _ptr(t):
    return t.data_ptr() if t is not None else None


def _dt(dtype):
    return ops.BF16 if dtype == torch.bfloat16 else ops.F32


def _linear(lin):
    w = lin.weight
    return Linear(_ptr(w), w.stride(0), w.shape[0], w.shape[1], _dt(w.dtype), 0)


class CStep:
    @staticmethod
    def serves(model):
        """Whether every part of the model is one the C walker knows: the plain frame, pre-norm blocks of RMSNorm,
        the attention mixer and the gated feed-forward (their exact classes: a subclass may do anything)."""
        if not ENABLED or type(model.frame) is not PlainFrame or type(model.frame.final_norm) is not RMSNorm:
            return False
        for b in model.blocks:
            if type(b) is not PreNormBlock or type(b.mixer) is not Attention or type(b.ffn) is not GatedMLP:
                return False
            if type(b.mixer_norm) is not RMSNorm or type(b.ffn_norm) is not RMSNorm:
                return False
        return model.ctx.dtype in (torch.bfloat16, torch.float32) and model.ctx.device.type == "cuda"

    def __init__(self, model, cache):
        self.model, self.cache = model, cache
        self.lib = load_module("step")
        sizes = [Fns, Linear, Norm, AttentionS, Mlp, Block, Entry, ModelS, Lists, Step]
        for i, s in enumerate(sizes):
            if self.lib.abk_step_sizeof(I(i)) != ctypes.sizeof(s):
                raise RuntimeError(f"the C step function's structure {s.__name__} is {self.lib.abk_step_sizeof(I(i))} bytes "
                                   f"there and {ctypes.sizeof(s)} here")
        device, dtype = model.ctx.device, model.ctx.dtype
        # only the kernel libraries this model can reach are loaded (and, in a fresh checkout, compiled)
        needed = self.libraries(model)
        self.fns = Fns(*[ctypes.cast(getattr(load_module(lib), name), P).value if lib in needed else None
                         for _, lib, name in LAUNCHERS])
        self.plan_names = [p.name for p in model.step_plans()]
        blocks = (Block * len(model.blocks))()
        for i, b in enumerate(model.blocks):
            a, f, s = b.mixer, b.ffn, b.mixer.spec
            pos = a.position
            blocks[i] = Block(
                Norm(_ptr(b.mixer_norm.weight), b.mixer_norm.spec.eps, b.mixer_norm.spec.size),
                Norm(_ptr(b.ffn_norm.weight), b.ffn_norm.spec.eps, b.ffn_norm.spec.size),
                AttentionS(_linear(a.qkv_proj), _linear(a.q_proj), _linear(a.o_proj), _ptr(a.q_norm), _ptr(a.k_norm),
                           _ptr(a.cos), _ptr(a.sin), s.qk_norm_eps or 0.0, s.scale, s.n_heads, s.n_kv_heads, s.head_dim,
                           s.window or 0, pos.rotary_dim if pos else 0, 1 if (pos and pos.interleaved) else 0,
                           a.cos.shape[0] if a.cos is not None else 0, self.plan_names.index(a.lists.name)),
                Mlp(_linear(f.gate_up), _linear(f.down), f.spec.inter, f.block))
        entries = (Entry * len(model.schedule))()
        for i, e in enumerate(model.schedule):
            view = cache.views[i]
            kv = view.kv
            entries[i] = Entry(_ptr(kv.k) if kv else None, _ptr(kv.v) if kv else None, _ptr(kv.page_table) if kv else None,
                               kv.k.shape[0] * kv.k.shape[1] * kv.k.shape[2] if kv else 0, e.layer,
                               1 if view.owns_storage else 0, kv.table_width if kv else 0, kv.ring_pages if kv else 0,
                               kv.tokens_per_page if kv else 1, 0)
        sc = ops._Scratch.of(device)
        frame = model.frame
        bf16 = dtype == torch.bfloat16
        any128 = bf16 and any(b.mixer.spec.head_dim == 128 and b.mixer.spec.window is None for b in model.blocks)
        specs = [b.mixer.spec for b in model.blocks]
        # decode attention on the CUDA cores keeps partial results in the workspace (head size 256, or groups beyond 16)
        self.simt_decode = [s for s in specs if bf16 and s.head_dim in (64, 128, 256)
                            and (s.head_dim == 256 or s.n_heads // s.n_kv_heads > 16)]
        tickets = sc.attention_tickets if self.simt_decode else None
        self.blocks, self.entries = blocks, entries  # (kept alive: the C side holds their addresses)
        self.struct = ModelS(
            ctypes.addressof(self.fns), ctypes.addressof(blocks), ctypes.addressof(entries), _ptr(frame.table),
            Norm(_ptr(frame.final_norm.weight), frame.final_norm.spec.eps, frame.final_norm.spec.size), _linear(frame.head),
            _ptr(model.status), _ptr(sc.gemm_floats) if bf16 else None, _ptr(sc.gemm_tickets) if bf16 else None, _ptr(sc.status),
            _ptr(sc.attention_halves) if any128 else None, _ptr(sc.attention_halves_tickets) if any128 else None,
            _ptr(tickets), _dt(dtype), model.spec.hidden, model.spec.vocab, len(model.blocks),
            len(model.schedule), sc.attention_halves_pairs, tickets.numel() if tickets is not None else 0,
            1 if DECODE_PREPARES else 0, 1 if PRODUCT_PREPARES else 0)
        self.qkv_width = max((s.n_heads + 2 * s.n_kv_heads) * s.head_dim for s in specs)
        self.att_width = max(s.n_heads * s.head_dim for s in specs)
        self.inter = max(b.ffn.spec.inter for b in model.blocks)
        self.table_positions = min([b.mixer.cos.shape[0] for b in model.blocks if b.mixer.cos is not None] or [1 << 30])
        self.step, self.lists = Step(), (Lists * max(1, len(self.plan_names)))()
        # the tensors whose addresses the structures hold stay alive as long as this object does
        self.keep = [frame.table, frame.head.weight, frame.final_norm.weight, model.status]
        for b in model.blocks:
            a, f = b.mixer, b.ffn
            self.keep += [b.mixer_norm.weight, b.ffn_norm.weight, a.qkv_proj.weight, a.o_proj.weight, a.q_norm, a.k_norm,
                          a.cos, a.sin, f.gate_up.weight, f.down.weight]

    @staticmethod
    def libraries(model):
        """The kernel libraries a model's steps can reach, by the rules of csrc/step.cu."""
        needed = {"elementwise", "gemm_simt", "attention_generic"}
        if model.ctx.dtype != torch.bfloat16:
            return needed
        needed |= {"gemm_rows", "gemm_tc"}
        for b in model.blocks:
            s = b.mixer.spec
            group = s.n_heads // s.n_kv_heads
            if s.head_dim in (64, 128) and group <= 16:
                needed.add("attention_decode_ring")
            elif s.head_dim in (64, 128, 256):
                needed.add("attention_decode")
            if s.window is None and s.head_dim == 128:
                needed.add("attention_tc")
            if s.window is None and s.head_dim == 64:
                needed.add("attention_mma")
        return needed

    def run(self, batch):
        """Logits float32 [batch.n_logit_rows, vocab] of the wanted rows of this step: Model.forward in one call."""
        model, ws, s = self.model, self.model.ws, self.step
        n, d, dtype, r = batch.n_rows, model.spec.hidden, model.ctx.dtype, batch.n_logit_rows
        if batch.max_position >= self.table_positions:
            raise ops.KernelError(f"position {batch.max_position} is beyond the rotary table of {self.table_positions} positions")
        bound = getattr(batch, "position_bound", None) or 0
        if batch.is_decode and bound and batch.max_len_after > bound:
            raise ops.KernelError(f"a row at position {batch.max_len_after - 1} is beyond the bound {bound}")
        for i, name in enumerate(self.plan_names):
            view = batch.plan.get(name)
            if view is None:
                self.lists[i] = Lists(None, None, 0, 0, 0, 0)
                continue
            mine = AttentionLists(view)
            tiles, work = mine.tiles(64), mine.work
            self.lists[i] = Lists(tiles.data_ptr(), work.data_ptr(), tiles.shape[0], work.shape[0], mine.n_halved, 0)
        logits = ws.get("logits", (max(r, 1), model.spec.vocab), torch.float32)[:r]
        partial_floats = 0
        if batch.is_decode and self.simt_decode:
            chunks = -(-(bound or batch.max_len_after) // 128)
            partial_floats = max(n * sp.n_heads * chunks * (sp.head_dim + 2) for sp in self.simt_decode)
        for name in ("tokens", "token_seq", "token_pos", "seq_slot", "seq_start", "seq_pos0", "seq_len_after", "logit_rows"):
            setattr(s, name, getattr(batch, name).data_ptr())
        s.lists = ctypes.addressof(self.lists)
        s.x = ws.get("x", (n, d), torch.float32).data_ptr()
        s.branch = ws.get("branch", (n, d), torch.float32).data_ptr()
        s.logits = logits.data_ptr() if r else ws.get("logits", (1, model.spec.vocab), torch.float32).data_ptr()
        s.attention_partials = ws.get("attention_partials", (partial_floats,), torch.float32).data_ptr() if partial_floats else None
        s.xn = ws.get("xn", (n, d), dtype).data_ptr()
        s.qkv = ws.get("qkv", (n, self.qkv_width), dtype).data_ptr()
        s.att = ws.get("att", (n, self.att_width), dtype).data_ptr()
        s.act = ws.get("act", (n, self.inter), dtype).data_ptr()
        s.gate_up = ws.get("gate_up", (n, 2 * self.inter), dtype).data_ptr()
        s.xn_final = ws.get("xn_final", (max(r, 1), d), dtype).data_ptr()
        s.partial_floats = partial_floats
        s.n_rows, s.n_logit_rows, s.is_decode, s.any_continuation = n, r, int(batch.is_decode), int(batch.any_continuation)
        s.max_len_after, s.position_bound, s.n_lists = batch.max_len_after, bound, len(self.plan_names)
        rc = self.lib.abk_step(ctypes.byref(self.struct), ctypes.byref(s), ops._stream())
        if rc:
            where = self.lib.abk_last_error().decode()
            if rc in REFUSALS:
                raise ops.KernelRefused(f"{REFUSALS[rc]} ({where})")
            if rc < 0:
                raise ops.KernelRefused(f"a kernel refused its sizes: {where}")
            raise ops.KernelError(f"{where}: CUDA error {rc} at launch")
        ops.LAUNCHES += self.lib.abk_step_launches()
        return logits
