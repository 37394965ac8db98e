"""The step function: a batch of sequences, their next tokens, the logits at the wanted places.

An Engine holds a model, its cache and the slots of the live sequences. A step
runs only the tokens it is given, as one batch, against what earlier steps left
in the cache: whole prompts of unequal lengths in one step, then one token per
sequence. This is abacus's forward(tokens, n, pos, logits, n_logits)
(src/model.c:315-327) for a batch of sequences instead of one.
"""
import os

import numpy as np

import torch

from ..cache import SequenceCache
from ..config.registry import load_config
from ..models.model import Model
from ..weights.loader import load_folder
from .batch import Sequence, StepBatch
from .cstep import CStep
from .graphs import DecodeGraphs, PromptGraphs

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "f32": torch.float32}


class StepError(ValueError):
    """A step that asks for what cannot be run (context full, unknown slot, no tokens)."""


def _device():
    if not torch.cuda.is_available():
        raise RuntimeError("abacus_b200 runs on a CUDA GPU (sm_100a); none is visible and there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def load_model(folder, dtype="bfloat16", device=None):
    """A Model from a folder with config.json and *.safetensors; the class is chosen by config.json."""
    dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
    arch, config = load_config(folder)
    spec = config.to_spec()
    layout = arch.layout(spec)
    tensors = load_folder(folder, lambda available: arch.tensor_names(spec, available))
    model = Model(spec, layout, tensors, dtype, device or _device())
    model.config = config
    model.folder = os.path.abspath(folder)
    return model


_ONE_TOKEN, _WANT_IT = np.zeros(1, dtype=np.int64), [0]


def capturable(model):
    """(single-token steps, steps of several tokens): whether the model's steps may be replayed from captured
    graphs. A captured graph replays device work only: a part whose forward decides anything on the host from the
    step's contents cannot be captured, and parts say so: `capturable = True` on every part for single-token
    steps; for steps of several tokens also no mixer with `capturable_prompts = False`."""
    parts = list(model.parts())
    decode = all(getattr(part, "capturable", False) for part in parts)
    return decode, decode and all(getattr(part, "capturable_prompts", True) for part in parts)


class Engine:
    def __init__(self, model, max_tokens, max_slots=None, max_context=None, use_graphs=True):
        self.model = model
        spec = model.spec
        context = min(max_context or spec.max_positions, spec.max_positions)
        self.cache = SequenceCache(model.cache_needs(), model.cache_sources(), max_tokens, model.ctx.dtype,
                                   model.ctx.device, max_slots=max_slots, max_context=context)
        self.max_context = self.cache.max_context
        model.prepare(self.max_context)
        self.vocab = spec.vocab
        # the step function in C where the model is made of the library's own parts, else the parts' forward()
        self.cstep = CStep(model, self.cache) if CStep.serves(model) else None
        decode_graphs, prompt_graphs = capturable(model)
        self.graphs = DecodeGraphs(self) if use_graphs and decode_graphs else None
        prompts = use_graphs and prompt_graphs and os.environ.get("ABACUS_PROMPT_GRAPHS", "1") != "0"
        self.prompt_graphs = PromptGraphs(self) if prompts else None
        self._step_batch = None

    # ------------------------------------------------------------ sequences
    def open(self):
        """A slot for a new sequence."""
        return self.cache.open_slot()

    def close(self, slot):
        """The sequence is finished: what it holds is given back."""
        self.cache.close_slot(slot)

    def length(self, slot):
        return self.cache.length[slot]

    # ------------------------------------------------------------ the step
    def plan(self, entries):
        """entries: [(slot, tokens, want)] -> [Sequence]; checks them and makes room in the cache."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        seqs, seen = [], set()
        for slot, tokens, want in entries:
            if slot not in self.cache.length:
                raise StepError(f"slot {slot} is not open")
            if slot in seen:
                raise StepError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            tokens = np.asarray(tokens, dtype=np.int64).reshape(-1)
            if not tokens.size:
                raise StepError(f"slot {slot}: a step must bring at least one token")
            if tokens.min() < 0 or tokens.max() >= self.vocab:
                bad = tokens[(tokens < 0) | (tokens >= self.vocab)]
                raise StepError(f"slot {slot}: token {int(bad[0])} is outside the vocabulary of {self.vocab}")
            seqs.append(Sequence(slot, tokens, self.cache.length[slot], [int(w) for w in want]))
        self.cache.reserve_all([(s.slot, s.start + len(s.tokens)) for s in seqs])
        return seqs

    def step(self, entries):
        """Run one step; returns float32 logits [wanted rows, vocab] on the device, in the order of
        the entries and of each entry's `want`."""
        seqs = self.plan(entries)
        if self.graphs is not None and self.graphs.takes(seqs):  # a plain decode step: replay its graph
            graph = self.graphs.get(seqs)
            logits = graph.run(seqs)
            self.last_batch = graph.batch
        elif self.prompt_graphs is not None and self.prompt_graphs.takes(seqs):  # a shape of prompts seen before
            logits, self.last_batch = self.prompt_graphs.run(seqs)
        else:
            batch = self._room_for(sum(len(s.tokens) for s in seqs), len(seqs), sum(len(s.want) for s in seqs))
            batch.fill(seqs, exact=True)
            logits = self.forward(batch)
            self.last_batch = batch
        for s in seqs:
            self.cache.advance(s.slot, len(s.tokens))
        return logits

    def forward(self, batch):
        """The model's forward pass over a filled step: in one call to C where that serves the model."""
        if self.cstep is not None:
            return self.cstep.run(batch)
        return self.model.forward(batch, self.cache)

    def step_ahead(self, slots, tokens_dev):
        """A decode step (one token per sequence, its logits wanted) whose tokens are on the device, for instance
        where a sampler has just put them: the host need not have seen them. tokens_dev int32 [len(slots)], in the
        order of `slots`. Returns the logits like step(), or None if this engine runs such steps only from the
        host (no captured graphs), in which case nothing has happened."""
        if self.graphs is None:
            return None
        seqs = [Sequence(slot, _ONE_TOKEN, self.cache.length[slot], _WANT_IT) for slot in slots]
        if len(set(slots)) != len(slots) or not self.graphs.takes(seqs):
            return None
        self.cache.reserve_all([(s.slot, s.start + 1) for s in seqs])
        graph = self.graphs.get(seqs)
        logits = graph.run(seqs, tokens_dev=tokens_dev)
        self.last_batch = graph.batch
        for s in seqs:
            self.cache.advance(s.slot, 1)
        return logits

    def _room_for(self, n_rows, n_seqs, n_logits):
        """The engine's StepBatch for steps outside a graph; replaced by a larger one when a step outgrows it
        (pinned memory is slow to get, so it is not made anew for every step)."""
        b = self._step_batch
        if b is None or n_rows > b.cap_rows or n_seqs > b.cap_seqs or n_logits > b.cap_logits:
            grow = lambda n, least: max(least, 1 << max(0, int(n) - 1).bit_length())
            b = StepBatch(grow(max(n_rows, b.cap_rows if b else 0), 256), grow(max(n_seqs, b.cap_seqs if b else 0), 16),
                          grow(max(n_logits, b.cap_logits if b else 0), 64), self.model.ctx.device,
                          plans=self.model.step_plans())
            self._step_batch = b
        return b

    def check_status(self):
        """Raise if a kernel reported a fault (a bounded wait that ran out, a token out of range)."""
        from ..kernels import ops
        shared = ops.kernel_status(self.model.ctx.device)
        status = self.model.status.tolist() + shared.tolist()
        if any(status):
            self.model.status.zero_()
            shared.zero_()
            raise RuntimeError(f"a kernel reported a fault (a token outside the vocabulary, or a wait that "
                               f"ran out): status words {status}")
