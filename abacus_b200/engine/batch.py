"""The rows of one step, as the kernels see them.

A step carries, for each sequence, its next tokens (a whole prompt, or one
token), flattened into rows. Token-parallel kernels see only the rows; the
attention kernels and the cache write also read which sequence and position a
row belongs to. All index arrays of a step live in one int32 buffer, filled on
the host and sent to the device in one copy.

Rows beyond the step's tokens (padding up to a fixed size, for a captured
graph) carry sequence index -1; kernels skip them and no result depends on them.
The same holds for the work lists of the prefill attention kernels (tiles of
64 and of 128 query rows; for the kernel that halves long tiles, a list of
CTAs' work in which such a tile stands twice, once per half of its keys), which
travel in the same buffer.
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


TILE_ROWS = (64, 128)  # query rows per tile of the prefill attention kernels
PAIRED_ROWS = 128       # the tile size of the kernel that halves long tiles
WORK_INTS = 8           # a CTA's work: sequence, first row, part (0 whole, 1 earlier keys, 2 later keys), then the
                        # sequence's first row in the step, first position, new tokens and slot, so that one load tells all
CTA_SLOTS = 2 * 148     # CTAs of that kernel the device holds at once
HALVED_PAIRS = 384      # (tile, head) pairs that kernel has scratch memory for when it halves tiles


class StepBatch:
    """Device-side index arrays of a step, with room for n_rows rows and n_seqs sequences."""

    def __init__(self, n_rows, n_seqs, n_logit_rows, device, attention_heads=1):
        """attention_heads: how many heads the prefill attention runs per tile (a hint for sharing out its work)."""
        self.device = torch.device(device)
        self.attention_heads = attention_heads
        self.cap_rows, self.cap_seqs, self.cap_logits = n_rows, n_seqs, max(1, n_logit_rows)
        self.cap_tiles = {r: n_rows // r + n_seqs + 1 for r in TILE_ROWS}  # no step of this size has more
        sizes = [n_rows, n_rows, n_rows, n_seqs, n_seqs + 1, n_seqs, n_seqs, self.cap_logits]
        sizes += [2 * self.cap_tiles[r] for r in TILE_ROWS]
        self.cap_work = 2 * self.cap_tiles[PAIRED_ROWS]  # every tile may stand twice
        self.n_halved = 0
        sizes += [WORK_INTS * self.cap_work]
        offsets = np.concatenate([[0], np.cumsum([-(-s // 4) * 4 for s in sizes])])  # 16-byte aligned parts
        self._host = torch.zeros(int(offsets[-1]), dtype=torch.int32)
        if self.device.type == "cuda":
            self._host = self._host.pin_memory()
        self._dev = torch.zeros(int(offsets[-1]), dtype=torch.int32, device=self.device)
        names = ["tokens", "token_seq", "token_pos", "seq_slot", "seq_start", "seq_pos0", "seq_len_after", "logit_rows"]
        names += [f"tiles{r}" for r in TILE_ROWS] + ["work"]
        self._h, self._parts = {}, {}
        for name, off, size in zip(names, offsets[:-1], sizes):
            self._h[name] = self._host[int(off):int(off) + size].numpy()
            self._parts[name] = self._dev[int(off):int(off) + size]
            setattr(self, name, self._parts[name])
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
        self._tiles, self.tile_pages = {}, {}
        self.is_decode = all(len(s.tokens) == 1 for s in sequences)
        for r in TILE_ROWS:
            h[f"tiles{r}"][:] = -1
            if not self.is_decode:
                self._write_tiles(r, exact)
        h["work"][:] = -1
        if not self.is_decode:
            self._write_work(exact)
        self.max_position = max((s.start + len(s.tokens) - 1 for s in sequences), default=0)
        self.max_len_after = self.max_position + 1
        self.any_continuation = any(s.start > 0 for s in sequences)
        self._dev.copy_(self._host, non_blocking=True)
        if self.device.type == "cuda":
            self._sent = torch.cuda.Event()
            self._sent.record()
        return self

    def _tiles_of(self, rows_per_tile):
        """(sequence, first row among its new tokens) of every tile of `rows_per_tile` query rows, int32 [tiles, 2]."""
        seq = np.concatenate([np.full(-(-len(s.tokens) // rows_per_tile), i, dtype=np.int32)
                              for i, s in enumerate(self.sequences)])
        row = np.concatenate([np.arange(0, len(s.tokens), rows_per_tile, dtype=np.int32) for s in self.sequences])
        keys = np.array([s.start for s in self.sequences], dtype=np.int64)[seq] + row
        # tiles that see the most keys first: the long ones start early and the short ones fill the tail
        order = np.argsort(-keys, kind="stable")
        last = np.minimum(row + rows_per_tile, np.array([len(s.tokens) for s in self.sequences], dtype=np.int64)[seq])
        self.tile_pages[rows_per_tile] = (keys + last - row - 1) // 64 + 1  # pages of 64 keys each tile sees
        return np.stack([seq[order], row[order]], axis=1)

    def _write_tiles(self, rows_per_tile, exact):
        name = f"tiles{rows_per_tile}"
        tiles = self._tiles_of(rows_per_tile)
        self._h[name][:tiles.size] = tiles.reshape(-1)
        n = len(tiles) if exact else self.cap_tiles[rows_per_tile]  # a captured graph has a fixed number: the rest say -1
        self._tiles[rows_per_tile] = self._parts[name][:2 * n].view(n, 2)

    def _write_work(self, exact):
        """The work list of the prefill attention kernel that halves long tiles. A kernel lasts as long as its
        longest CTA, and the tiles of a prompt see from one page of keys to all of them. CTAs with the most
        pages come first."""
        tiles = self._tiles_of(PAIRED_ROWS)
        seq, row = tiles[:, 0].astype(np.int64), tiles[:, 1].astype(np.int64)
        start = np.array([s.start for s in self.sequences], dtype=np.int64)[seq]
        new = np.array([len(s.tokens) for s in self.sequences], dtype=np.int64)[seq]
        pages = (start + np.minimum(row + PAIRED_ROWS, new) - 1) // 64 + 1
        # With fewer CTAs than the device holds at once, the longest tiles stand twice (each time with half of
        # their pages) as long as the CTAs still fit, give or take a few: then the kernel's longest CTA is shorter.
        # (measured on 2,048 tokens and 16 heads: 5 % over the device's places is best, 43 us -> 37 us; 20 % over is no gain)
        heads = self.attention_heads
        spare = 1.05 * CTA_SLOTS - len(pages) * heads
        k = min(int(np.ceil(spare / heads)) if spare > 0 else 0, HALVED_PAIRS // heads, len(pages))
        split = np.zeros(len(pages), dtype=bool)
        for i in np.argsort(-pages, kind="stable")[:k]:
            split[i] = pages[i] >= 8
        halved = {int(i): k for k, i in enumerate(np.flatnonzero(split))}
        self.n_halved = len(halved)
        entries = [((pages[i] + 1) // 2, i, 1) for i in halved] + [(pages[i] // 2, i, 2) for i in halved]
        entries += [(pages[i], i, 0) for i in range(len(pages)) if not split[i]]
        entries.sort(key=lambda t: -t[0])  # the CTAs with the most pages first
        first_row = np.array([0] + list(np.cumsum([len(s.tokens) for s in self.sequences])), dtype=np.int64)
        slots = np.array([s.slot for s in self.sequences], dtype=np.int64)
        work = np.full((len(entries), WORK_INTS), -1, dtype=np.int32)
        for k, (_, i, part) in enumerate(entries):
            work[k] = (seq[i], row[i], part, first_row[seq[i]], start[i], new[i], slots[seq[i]], halved.get(i, 0))
        self._h["work"][:work.size] = work.reshape(-1)
        n = len(work) if exact else self.cap_work
        self.work = self._parts["work"][:WORK_INTS * n].view(n, WORK_INTS)

    def query_tiles(self, rows_per_tile=64):
        """The work list of a prefill attention kernel: (sequence, first row among its new tokens) for every
        tile of `rows_per_tile` query rows of the step, int32 [tiles, 2] on the device; a tile whose sequence is
        -1 is padding. Tiles of 64 and 128 rows come with the step's one copy; other sizes are sent when asked for."""
        if rows_per_tile not in self._tiles:
            self._tiles[rows_per_tile] = torch.from_numpy(self._tiles_of(rows_per_tile)).to(self.device)
        return self._tiles[rows_per_tile]

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
