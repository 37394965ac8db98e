"""The cache: a slot for each live sequence, keys and values for each schedule entry that keeps
its own, and a fixed-size state per sequence for mixers that have one.

Storage is paged: a page holds `TOKENS_PER_PAGE` consecutive positions of one sequence for one
kv head, [tokens, head_dim] contiguous, so a decode kernel streams whole pages. Entries with the
same need (kv heads, head size, window) form a group with pools of their own,
[entries, pages, kv heads, tokens per page, head_dim] for keys and for values, one page table
[slots, pages per sequence] and one free list. A windowed group keeps only as many pages per
sequence as its window can touch and uses them as a ring.

abacus keeps one sequence, [layers][seq_len][kv_dim] float32 (src/model.c:112-113, 256-258);
the slot, the pages and the groups are this library's own.
"""
from dataclasses import dataclass

import torch

from ..kernels import guards
from .need import CacheNeed
from .pages import CacheFull, FreeList, PageBook

TOKENS_PER_PAGE = 64


@dataclass
class LayerKV:
    """What the kernels need to find a sequence's keys and values for one schedule entry."""
    k: torch.Tensor  # [pages, kv heads, tokens per page, head_dim]
    v: torch.Tensor
    page_table: torch.Tensor  # int32 [slots, table_width]
    table_width: int
    ring_pages: int
    tokens_per_page: int
    window: object


@dataclass
class EntryView:
    owns_storage: bool  # False: the entry reads the cache of another entry
    kv: object  # LayerKV or None
    state: object  # float32 [slots, *state_shape] or None


class _Group:
    def __init__(self, need, entries, n_pages, max_slots, max_context, dtype, device):
        tpp = TOKENS_PER_PAGE
        self.need, self.entries = need, entries
        self.ring_pages = 0 if need.window is None else (need.window + tpp - 2) // tpp + 1
        per_seq = -(-max_context // tpp)
        if self.ring_pages:
            per_seq = min(per_seq, self.ring_pages)
            n_pages = min(n_pages, max_slots * self.ring_pages)
        self.table_width = max(1, min(per_seq, n_pages))
        self.book = PageBook(n_pages, tpp, self.ring_pages)
        shape = (len(entries), n_pages, need.n_kv_heads, tpp, need.head_dim)
        self.k = guards.zeros(shape, dtype, device, what="cache keys")  # guard words around the pools
        self.v = guards.zeros(shape, dtype, device, what="cache values")
        # pageable on purpose: a copy from pageable memory is staged before copy_ returns, so the
        # host may rewrite a row (a slot used again) while earlier steps are still in flight
        self.table_host = torch.zeros((max_slots, self.table_width), dtype=torch.int32)
        self.table = torch.zeros((max_slots, self.table_width), dtype=torch.int32, device=device)


class SequenceCache:
    """needs: one CacheNeed (or None) per schedule entry; sources: per entry, None or the entry it reads."""

    def __init__(self, needs, sources, max_tokens, dtype, device, max_slots=None, max_context=None):
        tpp = TOKENS_PER_PAGE
        self.device, self.dtype = torch.device(device), dtype
        self.n_pages = max(1, -(-max_tokens // tpp))
        self.max_slots = max_slots or min(self.n_pages, 4096)
        self.max_context = min(max_context or self.n_pages * tpp, self.n_pages * tpp)
        self.slots = FreeList(self.max_slots, "cache slot")
        self.length = {}
        self.groups, self._of_entry, self.states = [], {}, {}
        by_need = {}
        for e, (need, source) in enumerate(zip(needs, sources)):
            if source is not None or need is None:
                continue
            if need.n_kv_heads > 0:
                key = (need.n_kv_heads, need.head_dim, need.window)
                by_need.setdefault(key, []).append(e)
            if need.state_shape:
                self.states[e] = guards.zeros((self.max_slots, *need.state_shape), torch.float32, device,
                                              what=f"state of entry {e}")
        for (hkv, hd, window), entries in by_need.items():
            g = _Group(CacheNeed(hkv, hd, window), entries, self.n_pages, self.max_slots, self.max_context, dtype,
                       self.device)
            self.groups.append(g)
            for i, e in enumerate(entries):
                self._of_entry[e] = (g, i)
        self.sources = list(sources)
        self.views = [self._view(e) for e in range(len(needs))]

    def _view(self, e):
        owner = e if self.sources[e] is None else self.sources[e]
        kv = None
        if owner in self._of_entry:
            g, i = self._of_entry[owner]
            kv = LayerKV(g.k[i], g.v[i], g.table, g.table_width, g.ring_pages, TOKENS_PER_PAGE, g.need.window)
        return EntryView(self.sources[e] is None, kv, self.states.get(owner))

    # ------------------------------------------------------------ slots
    def open_slot(self):
        """A slot for a new sequence: no tokens, state zeroed."""
        slot = self.slots.take()
        self.length[slot] = 0
        for g in self.groups:
            g.book.open(slot)
        for state in self.states.values():
            state[slot].zero_()
        return slot

    def close_slot(self, slot):
        """Give the slot and all it holds back."""
        self.slots.give_back(slot)
        del self.length[slot]
        for g in self.groups:
            g.book.close(slot)

    def pages_short(self, slot, new_length):
        """How many pages the group that is shortest of them lacks for the slot to grow to new_length (0: it fits)."""
        short = 0
        for g in self.groups:
            want = g.book.pages_for(new_length) - len(g.book.of_slot[slot])
            short = max(short, want - g.book.pages.n_free)
        return short

    def reserve(self, slot, new_length):
        """Room for the sequence to grow to new_length tokens; page tables on the device follow. All groups
        get their pages or none does: a refused call leaves the cache as it was."""
        if new_length > self.max_context:
            raise CacheFull(f"context is full: {new_length} tokens, the cache holds {self.max_context} per sequence")
        short = self.pages_short(slot, new_length)
        if short > 0:
            raise CacheFull(f"the cache lacks {short} free pages of {TOKENS_PER_PAGE} tokens for slot {slot} to hold "
                            f"{new_length} tokens")
        for g in self.groups:
            added = g.book.grow(slot, new_length)
            if added:
                for logical, page in added:
                    g.table_host[slot, logical] = page
                g.table[slot].copy_(g.table_host[slot])

    def reserve_all(self, wanted):
        """reserve() for several slots at once, [(slot, new_length)]: either every one gets its room or the cache
        is left as it was (a step is refused whole, not from its third sequence on)."""
        for slot, new_length in wanted:
            if new_length > self.max_context:
                raise CacheFull(f"context is full: {new_length} tokens, the cache holds {self.max_context} per sequence")
        for g in self.groups:
            need = sum(max(0, g.book.pages_for(n) - len(g.book.of_slot[slot])) for slot, n in wanted)
            if need > g.book.pages.n_free:
                raise CacheFull(f"the cache has {g.book.pages.n_free} free pages of {TOKENS_PER_PAGE} tokens; this step "
                                f"needs {need} more")
        for slot, new_length in wanted:
            self.reserve(slot, new_length)

    def advance(self, slot, n_new):
        self.length[slot] += n_new

    @property
    def free_pages(self):
        return min((g.book.pages.n_free for g in self.groups), default=0)

    def bytes(self):
        total = sum(2 * g.k.numel() * g.k.element_size() for g in self.groups)
        return total + sum(s.numel() * 4 for s in self.states.values())
