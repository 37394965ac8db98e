"""What the attention mixer adds to a step: the work lists of its prefill kernels.

A step that brings several tokens of some sequence is cut into tiles of query rows (64 for the
warp-level kernel, 128 for the tensor-memory one). The kernels walk these lists instead of working
the tiles out themselves; a tile whose sequence is -1 is padding. For the tensor-memory kernel the
list names the work of CTAs: a kernel lasts as long as its longest CTA, and the tiles of a prompt
see from one page of keys to all of them, so the longest tiles stand twice, each time with half of
their pages, as long as the CTAs still fit the device at once.

This is a step plan in the sense of engine/batch.py: the engine carries its words to the device
with the step's other indices and knows nothing of what they hold.
"""
import numpy as np

TILE_ROWS = (64, 128)  # query rows per tile of the prefill attention kernels
PAIRED_ROWS = 128       # the tile size of the kernel that halves long tiles
WORK_INTS = 8           # a CTA's work: sequence, first row, part (0 whole, 1 earlier keys, 2 later keys), then the
                        # sequence's first row in the step, first position, new tokens and slot, so that one load tells all
HALVED_PAIRS = 384      # (tile, head) pairs that kernel has scratch memory for when it halves tiles
CTAS_PER_SM = 2         # CTAs of that kernel an SM holds
_sm_count = {}


def sm_count():
    """SMs of the current GPU (148 on a B200); 148 where there is none (the lists are also made on the CPU, in tests)."""
    import torch
    if not torch.cuda.is_available():
        return 148
    device = torch.cuda.current_device()
    if device not in _sm_count:
        _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[device]


class AttentionLists:
    """The lists of one filled step, as the mixer reads them (device tensors are views of the step's buffer)."""

    def __init__(self, plan_view):
        self.n_halved = plan_view.info["n_halved"]
        self._layout, self._words, self._counts = plan_view.layout, plan_view.words, plan_view.info["counts"]

    def tiles(self, rows_per_tile):
        """(sequence, first row among its new tokens) of every tile, int32 [tiles, 2] on the device."""
        off = self._layout.offset[f"tiles{rows_per_tile}"]
        n = self._counts[f"tiles{rows_per_tile}"]
        return self._words[off:off + 2 * n].view(n, 2)

    @property
    def work(self):
        off, n = self._layout.offset["work"], self._counts["work"]
        return self._words[off:off + WORK_INTS * n].view(n, WORK_INTS)


class _Layout:
    """Where the lists lie in a StepBatch with room for n_rows rows and n_seqs sequences."""

    def __init__(self, n_rows, n_seqs):
        self.cap_tiles = {r: n_rows // r + n_seqs + 1 for r in TILE_ROWS}  # no step of this size has more
        self.cap_work = 2 * self.cap_tiles[PAIRED_ROWS]                    # every tile may stand twice
        self.offset, at = {}, 0
        for name, size in [(f"tiles{r}", 2 * self.cap_tiles[r]) for r in TILE_ROWS] + [("work", WORK_INTS * self.cap_work)]:
            self.offset[name] = at
            at += -(-size // 4) * 4  # 16-byte aligned
        self.words = at


class AttentionStepPlan:
    """heads: how many query heads the mixer runs per tile (it decides how many tiles can be halved).
    cta_slots: CTAs of the tile-halving kernel the device holds at once; by default two per SM of the current GPU."""

    def __init__(self, heads, cta_slots=None):
        self.heads, self.cta_slots = int(heads), cta_slots
        self.name = f"attention_lists_{self.heads}"

    def layout(self, n_rows, n_seqs):
        return _Layout(n_rows, n_seqs)

    def fill(self, layout, sequences, words, is_decode, exact):
        words[:] = -1
        counts = {f"tiles{r}": 0 if exact else layout.cap_tiles[r] for r in TILE_ROWS}
        counts["work"] = 0 if exact else layout.cap_work
        info = {"n_halved": 0, "counts": counts, "tile_pages": {}}
        if is_decode:  # one token each: the decode kernels need no lists
            return info
        for r in TILE_ROWS:
            tiles, pages = tiles_of(sequences, r)
            off = layout.offset[f"tiles{r}"]
            words[off:off + tiles.size] = tiles.reshape(-1)
            info["tile_pages"][r] = pages
            if exact:
                counts[f"tiles{r}"] = len(tiles)
        work, n_halved = self._work_list(sequences)
        off = layout.offset["work"]
        words[off:off + work.size] = work.reshape(-1)
        info["n_halved"] = n_halved
        if exact:
            counts["work"] = len(work)
        return info

    def _work_list(self, sequences):
        """The work list of the prefill attention kernel that halves long tiles. CTAs with the most pages come first."""
        tiles, _ = tiles_of(sequences, PAIRED_ROWS)
        seq, row = tiles[:, 0].astype(np.int64), tiles[:, 1].astype(np.int64)
        start = np.array([s.start for s in sequences], dtype=np.int64)[seq]
        new = np.array([len(s.tokens) for s in sequences], dtype=np.int64)[seq]
        pages = (start + np.minimum(row + PAIRED_ROWS, new) - 1) // 64 + 1
        # With fewer CTAs than the device holds at once, the longest tiles stand twice (each time with half of
        # their pages) as long as the CTAs still fit, give or take a few: then the kernel's longest CTA is shorter.
        # (measured on 2,048 tokens and 16 heads: 5 % over the device's places is best, 43 us -> 37 us; 20 % over is no gain)
        heads = self.heads
        slots = self.cta_slots if self.cta_slots is not None else CTAS_PER_SM * sm_count()
        spare = 1.05 * slots - len(pages) * heads
        k = min(int(np.ceil(spare / heads)) if spare > 0 else 0, HALVED_PAIRS // heads, len(pages))
        split = np.zeros(len(pages), dtype=bool)
        for i in np.argsort(-pages, kind="stable")[:k]:
            split[i] = pages[i] >= 8
        halved = {int(i): k for k, i in enumerate(np.flatnonzero(split))}
        entries = [((pages[i] + 1) // 2, i, 1) for i in halved] + [(pages[i] // 2, i, 2) for i in halved]
        entries += [(pages[i], i, 0) for i in range(len(pages)) if not split[i]]
        entries.sort(key=lambda t: -t[0])  # the CTAs with the most pages first
        first_row = np.array([0] + list(np.cumsum([len(s.tokens) for s in sequences])), dtype=np.int64)
        slot_of = np.array([s.slot for s in sequences], dtype=np.int64)
        work = np.full((len(entries), WORK_INTS), -1, dtype=np.int32)
        for k, (_, i, part) in enumerate(entries):
            work[k] = (seq[i], row[i], part, first_row[seq[i]], start[i], new[i], slot_of[seq[i]], halved.get(i, 0))
        return work, len(halved)


def tiles_of(sequences, rows_per_tile):
    """((sequence, first row among its new tokens) of every tile of `rows_per_tile` query rows, int32 [tiles, 2], the
    tiles that see the most keys first; pages of 64 keys each tile sees, in the sequences' order)."""
    seq = np.concatenate([np.full(-(-len(s.tokens) // rows_per_tile), i, dtype=np.int32) for i, s in enumerate(sequences)])
    row = np.concatenate([np.arange(0, len(s.tokens), rows_per_tile, dtype=np.int32) for s in sequences])
    keys = np.array([s.start for s in sequences], dtype=np.int64)[seq] + row
    # tiles that see the most keys first: the long ones start early and the short ones fill the tail
    order = np.argsort(-keys, kind="stable")
    last = np.minimum(row + rows_per_tile, np.array([len(s.tokens) for s in sequences], dtype=np.int64)[seq])
    pages = (keys + last - row - 1) // 64 + 1
    return np.stack([seq[order], row[order]], axis=1), pages
