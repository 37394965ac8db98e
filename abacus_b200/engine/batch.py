"""The rows of one step, as the kernels see them.

A step carries, for each sequence, its next tokens (a whole prompt, or one
token), flattened into rows. Token-parallel kernels see only the rows; the
mixers and the cache write also read which sequence and position a row belongs
to. All index arrays of a step live in one int32 buffer, filled on the host and
sent to the device in one copy.

Rows beyond the step's tokens (padding up to a fixed size, for a captured
graph) carry sequence index -1; kernels skip them and no result depends on them.

A mixer whose kernels need more than these arrays (work lists, tiles, whatever it
derives from the step's sequences on the host) brings a *step plan*: an object with
    name                              what the mixer looks its part of the step up by
    layout(n_rows, n_seqs) -> layout  an object with `.words`, the int32 words the plan needs at most in a
                                      StepBatch with this room, and whatever else the plan wants to remember
                                      about such a StepBatch (offsets of its lists)
    fill(layout, sequences, words, is_decode, exact) -> info
                                      writes its words (a numpy view of the host buffer) and returns
                                      what the mixer wants to know on the host (counts and the like)
The plan's words travel in the same buffer, at an address that is fixed for the StepBatch's
life (a captured graph holds it); `batch.plan[name]` gives the mixer its words on the device
with its layout and the info of the last fill. Nothing here knows what any plan holds.
"""
from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class Sequence:
    """One sequence's share of a step."""
    slot: int
    tokens: list  # its next tokens
    start: int  # how many tokens the slot already holds
    want: list  # places among `tokens` whose logits are wanted


@dataclass
class PlanView:
    """A step plan's part of a filled StepBatch."""
    plan: object
    layout: object
    words: torch.Tensor  # int32, on the device, at a fixed address
    info: object         # what the plan's fill returned


CORE = ["tokens", "token_seq", "token_pos", "seq_slot", "seq_start", "seq_pos0", "seq_len_after", "logit_rows"]


class StepBatch:
    """Device-side index arrays of a step, with room for n_rows rows and n_seqs sequences."""

    def __init__(self, n_rows, n_seqs, n_logit_rows, device, plans=()):
        """plans: the step plans of the model's mixers (see above), each under a name of its own."""
        self.device = torch.device(device)
        self.cap_rows, self.cap_seqs, self.cap_logits = n_rows, n_seqs, max(1, n_logit_rows)
        self.plans = {}
        for p in plans:
            self.plans.setdefault(p.name, p)
        sizes = [n_rows, n_rows, n_rows, n_seqs, n_seqs + 1, n_seqs, n_seqs, self.cap_logits]
        self._layouts = {name: p.layout(n_rows, n_seqs) for name, p in self.plans.items()}
        sizes += [max(1, int(self._layouts[name].words)) for name in self.plans]
        offsets = np.concatenate([[0], np.cumsum([-(-s // 4) * 4 for s in sizes])])  # 16-byte aligned parts
        self._host = torch.zeros(int(offsets[-1]), dtype=torch.int32)
        if self.device.type == "cuda":
            self._host = self._host.pin_memory()
        self._dev = torch.zeros(int(offsets[-1]), dtype=torch.int32, device=self.device)
        names = CORE + [f"plan:{name}" for name in self.plans]
        self._h, self._parts = {}, {}
        for name, off, size in zip(names, offsets[:-1], sizes):
            self._h[name] = self._host[int(off):int(off) + size].numpy()
            self._parts[name] = self._dev[int(off):int(off) + size]
        for name in CORE:
            setattr(self, name, self._parts[name])
        self.plan = {}
        self.n_rows = n_rows
        self.n_tokens = self.n_seqs = self.n_logit_rows = 0
        self.max_position = 0
        self.max_len_after = 0
        self.is_decode = False
        self.any_continuation = False
        self._sent = None

    def fill(self, sequences, pad_logits=False, exact=False):
        """Write the step described by `sequences` (list of Sequence) and send it to the device.
        pad_logits: logits are made for as many rows as this StepBatch has room for (a captured graph
        needs a fixed number); the rows beyond the wanted ones repeat row 0 and are ignored.
        exact: the step has as many rows, sequences and logit rows as `sequences` bring, not as many as
        there is room for (an engine keeps one StepBatch for steps of every size)."""
        h = self._h
        if self._sent is not None:
            self._sent.synchronize()  # the last copy must have read the host buffer before it is rewritten
        n_tokens = sum(len(s.tokens) for s in sequences)
        n_logits = sum(len(s.want) for s in sequences)
        if n_tokens > self.cap_rows or len(sequences) > self.cap_seqs or n_logits > self.cap_logits:
            raise ValueError("step is larger than this StepBatch")
        h["token_seq"][:] = -1
        h["tokens"][:] = 0
        h["token_pos"][:] = 0
        h["seq_slot"][:] = 0
        h["logit_rows"][:] = 0
        h["seq_pos0"][:] = 0
        h["seq_len_after"][:] = 0
        row, lr = 0, 0
        for i, s in enumerate(sequences):
            n = len(s.tokens)
            h["tokens"][row:row + n] = s.tokens
            h["token_seq"][row:row + n] = i
            h["token_pos"][row:row + n] = np.arange(s.start, s.start + n)
            h["seq_slot"][i] = s.slot
            h["seq_start"][i] = row
            h["seq_pos0"][i] = s.start
            h["seq_len_after"][i] = s.start + n
            for wpos in s.want:
                if not 0 <= wpos < n:
                    raise ValueError(f"wanted place {wpos} is outside the {n} tokens given")
                h["logit_rows"][lr] = row + wpos
                lr += 1
            row += n
        h["seq_start"][len(sequences):] = row
        self.n_tokens, self.n_seqs, self.n_logit_rows = n_tokens, len(sequences), n_logits
        if pad_logits:
            self.n_logit_rows = self.cap_logits
        if exact:
            self.n_rows = n_tokens
            n_seqs = len(sequences)
            for name, n in (("tokens", n_tokens), ("token_seq", n_tokens), ("token_pos", n_tokens), ("seq_slot", n_seqs),
                            ("seq_start", n_seqs + 1), ("seq_pos0", n_seqs), ("seq_len_after", n_seqs),
                            ("logit_rows", max(1, n_logits))):
                setattr(self, name, self._parts[name][:n])
        self.sequences = list(sequences)  # host view, for mixers that walk the sequences themselves
        self.is_decode = all(len(s.tokens) == 1 for s in sequences)
        for name, p in self.plans.items():
            info = p.fill(self._layouts[name], self.sequences, h[f"plan:{name}"], self.is_decode, exact)
            self.plan[name] = PlanView(p, self._layouts[name], self._parts[f"plan:{name}"], info)
        self.max_position = max((s.start + len(s.tokens) - 1 for s in sequences), default=0)
        self.max_len_after = self.max_position + 1
        self.any_continuation = any(s.start > 0 for s in sequences)
        self._dev.copy_(self._host, non_blocking=True)
        if self.device.type == "cuda":
            self._sent = torch.cuda.Event()
            self._sent.record()
        return self

    def advance_on_device(self):
        """Every sequence moves one position on (a decode step follows a decode step); the tokens are
        left as they are on the device. The host's view follows."""
        from ..kernels import ops
        ops.advance_decode(self)
        for s in self.sequences:
            s.start += 1
        self.max_position += 1
        self.max_len_after += 1
        self.any_continuation = True
        return self
