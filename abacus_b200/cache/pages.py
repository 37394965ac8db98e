"""Host-side bookkeeping of the cache: which pages and slots are free, and who holds what.

Nothing here touches the GPU, so its invariants (no page or slot lost, held
twice or freed twice) are tested on the CPU.
"""


class CacheFull(RuntimeError):
    """More tokens or sequences are live than the cache was sized for."""


class FreeList:
    """Hands out integers 0..n-1, lowest first; takes them back; refuses a double free."""

    def __init__(self, n, what):
        self.n, self.what = n, what
        self._free = list(range(n - 1, -1, -1))
        self._held = set()

    def take(self):
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are in use)")
        i = self._free.pop()
        self._held.add(i)
        return i

    def give_back(self, i):
        if i not in self._held:
            raise ValueError(f"{self.what} {i} is not in use (freed twice, or never taken)")
        self._held.remove(i)
        self._free.append(i)
        # keep "lowest first" so that reuse is deterministic
        self._free.sort(reverse=True)

    @property
    def n_free(self):
        return len(self._free)

    @property
    def held(self):
        return frozenset(self._held)


class PageBook:
    """The pages of one cache group: per slot, the list of pages that hold its tokens.

    A group with ring_pages > 0 keeps at most that many pages per slot; position p
    lives in logical page (p // tokens_per_page) % ring_pages.
    """

    def __init__(self, n_pages, tokens_per_page, ring_pages=0):
        self.tokens_per_page, self.ring_pages = tokens_per_page, ring_pages
        self.pages = FreeList(n_pages, "cache page")
        self.of_slot = {}

    def open(self, slot):
        if slot in self.of_slot:
            raise ValueError(f"slot {slot} is already open")
        self.of_slot[slot] = []

    def pages_for(self, length):
        n = -(-length // self.tokens_per_page)
        return min(n, self.ring_pages) if self.ring_pages else n

    def grow(self, slot, length):
        """Make room for `length` tokens in all; returns [(logical index, page)] newly added."""
        have = self.of_slot[slot]
        want = self.pages_for(length)
        if want - len(have) > self.pages.n_free:
            raise CacheFull(f"the cache has {self.pages.n_free} free pages of {self.tokens_per_page} tokens; "
                            f"slot {slot} needs {want - len(have)} more to hold {length} tokens")
        added = []
        while len(have) < want:
            page = self.pages.take()
            added.append((len(have), page))
            have.append(page)
        return added

    def close(self, slot):
        for page in self.of_slot.pop(slot):
            self.pages.give_back(page)
