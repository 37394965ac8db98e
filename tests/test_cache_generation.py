"""The cache's bookkeeping and the generation loop's decisions: host logic, no GPU."""
import random

import pytest
import torch

from abacus_b200.cache import CacheFull, CacheNeed, FreeList, PageBook, SequenceCache, TOKENS_PER_PAGE
from abacus_b200.engine.generate import Generator, LiveBatch, Request, plan_batches
from abacus_b200.sampling import stream_seed


def test_free_list_never_loses_or_doubles():
    fl = FreeList(5, "slot")
    held = [fl.take() for _ in range(5)]
    assert sorted(held) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheFull):
        fl.take()
    fl.give_back(3)
    with pytest.raises(ValueError, match="twice"):
        fl.give_back(3)
    with pytest.raises(ValueError):
        fl.give_back(99)
    assert fl.take() == 3 and fl.n_free == 0


def test_page_book_random_walk_keeps_its_invariants():
    rnd = random.Random(0)
    book = PageBook(40, 64)
    lengths, next_slot = {}, 0
    for _ in range(2000):
        if lengths and rnd.random() < 0.3:
            slot = rnd.choice(list(lengths))
            book.close(slot)
            del lengths[slot]
        elif lengths and rnd.random() < 0.6:
            slot = rnd.choice(list(lengths))
            want = lengths[slot] + rnd.randint(1, 200)
            try:
                book.grow(slot, want)
                lengths[slot] = want
            except CacheFull:
                pass
        else:
            book.open(next_slot)
            lengths[next_slot] = 0
            next_slot += 1
        owned = [p for pages in book.of_slot.values() for p in pages]
        assert len(owned) == len(set(owned)), "a page is held twice"
        assert set(owned) == set(book.pages.held), "held pages and owners disagree"
        assert len(owned) + book.pages.n_free == 40, "a page was lost"
        for slot, n in lengths.items():
            assert len(book.of_slot[slot]) == -(-n // 64)


def test_ring_pages_bound_a_windowed_group():
    book = PageBook(10, 64, ring_pages=2)
    book.open(0)
    assert book.grow(0, 64) == [(0, book.of_slot[0][0])]
    book.grow(0, 65)
    assert len(book.of_slot[0]) == 2
    assert book.grow(0, 5000) == [] and len(book.of_slot[0]) == 2


def test_sequence_cache_groups_slots_and_state():
    needs = [CacheNeed(2, 16), CacheNeed(2, 16, window=24), CacheNeed(2, 16), None, CacheNeed(0, 0, state_shape=(3, 5))]
    sources = [None, None, None, 0, None]
    cache = SequenceCache(needs, sources, max_tokens=640, dtype=torch.float32, device="cpu", max_context=512)
    assert cache.n_pages == 10 and len(cache.groups) == 2
    full = [g for g in cache.groups if g.need.window is None][0]
    ring = [g for g in cache.groups if g.need.window is not None][0]
    assert full.k.shape == (2, 10, 2, TOKENS_PER_PAGE, 16) and full.entries == [0, 2]
    assert ring.ring_pages == 2 and ring.table_width == 2  # a window of 24 keys touches at most 2 pages of 64
    assert cache.views[3].owns_storage is False and cache.views[3].kv.k.data_ptr() == cache.views[0].kv.k.data_ptr()
    assert cache.views[4].kv is None and cache.views[4].state.shape == (cache.max_slots, 3, 5)
    a, b = cache.open_slot(), cache.open_slot()
    cache.reserve(a, 130)
    cache.reserve(b, 64)
    assert full.table[a, :3].tolist() == full.book.of_slot[a] and len(full.book.of_slot[a]) == 3
    assert len(ring.book.of_slot[a]) == 2
    cache.states[4][a] += 1.0
    with pytest.raises(CacheFull, match="context is full"):
        cache.reserve(a, 513)
    with pytest.raises(CacheFull, match="free pages"):
        cache.reserve(b, 64 * 8)
    cache.close_slot(a)
    with pytest.raises(ValueError):
        cache.close_slot(a)
    c = cache.open_slot()
    assert c == a and cache.length[c] == 0 and float(cache.states[4][c].abs().sum()) == 0.0  # state starts at zero
    cache.reserve(c, 64 * 6)  # the pages of `a` are free again
    assert full.book.pages.n_free == 10 - 6 - 1


def test_a_refused_reserve_leaves_every_group_as_it_was():
    """Two groups, the windowed one first; the group of all keys is the one that runs out. A refusal must not leave
    the windowed group with pages that its table on the device never heard of, and a step that does not fit for its
    last sequence must not keep the pages of its first."""
    needs = [CacheNeed(2, 16, window=100), CacheNeed(2, 16)]
    cache = SequenceCache(needs, [None, None], max_tokens=64 * 6, dtype=torch.float32, device="cpu", max_slots=4)
    ring, full = cache.groups
    assert ring.need.window == 100 and full.need.window is None
    a, b = cache.open_slot(), cache.open_slot()
    cache.reserve(a, 64 * 4)
    before = (list(ring.book.of_slot[b]), ring.book.pages.n_free, full.book.pages.n_free)
    with pytest.raises(CacheFull):
        cache.reserve(b, 64 * 3)  # the full group has 2 pages left
    assert (list(ring.book.of_slot[b]), ring.book.pages.n_free, full.book.pages.n_free) == before
    cache.close_slot(a)
    cache.reserve(b, 64 * 3)
    assert ring.table[b, :len(ring.book.of_slot[b])].tolist() == ring.book.of_slot[b]
    assert full.table[b, :3].tolist() == full.book.of_slot[b]
    c = cache.open_slot()
    before = (full.book.pages.n_free, ring.book.pages.n_free, len(full.book.of_slot[b]), len(full.book.of_slot[c]))
    with pytest.raises(CacheFull):
        cache.reserve_all([(b, 64 * 4), (c, 64 * 3)])  # b alone would fit, both do not
    assert (full.book.pages.n_free, ring.book.pages.n_free, len(full.book.of_slot[b]), len(full.book.of_slot[c])) == before
    cache.reserve_all([(b, 64 * 4), (c, 64 * 2)])
    assert full.book.pages.n_free == 0


def test_no_request_starts_its_random_stream_at_zero():
    """xorshift64 never leaves state 0, so no (seed, request) pair may start there, seed 0 included."""
    golden = 0x9E3779B97F4A7C15
    assert stream_seed(0, 0) != 0
    for i in range(1, 50):
        assert stream_seed((i * golden) % (1 << 64), i) != 0  # the seeds that would cancel request i's offset
        assert stream_seed(5, i) == (5 ^ (i * golden)) % (1 << 64)
    assert stream_seed(5, 0) == 5  # request 0 draws what abacus would with --seed 5


def test_window_ring_size():
    for window, pages in [(1, 1), (2, 2), (64, 2), (65, 2), (66, 3), (128, 3), (130, 4)]:
        cache = SequenceCache([CacheNeed(1, 16, window=window)], [None], 64 * 64, torch.float32, "cpu")
        # the keys pos-window+1..pos lie in at most `pages` pages of 64 for every pos
        worst = max(pos // 64 - max(0, pos - window + 1) // 64 + 1 for pos in range(0, 700))
        assert cache.groups[0].ring_pages == pages and worst <= pages


# ------------------------------------------------------------------ the loop's decisions

def reqs(lengths, max_new):
    return [Request(i, list(range(1, n + 1)), max_new) for i, n in enumerate(lengths)]


def test_plan_batches_respects_tokens_slots_and_order():
    r = reqs([5, 11, 17, 100, 3], 30)  # pages: 1, 1, 1, 3, 1
    assert [[x.index for x in b] for b in plan_batches(r, 64 * 3, 8, 512)] == [[0, 1, 2], [3], [4]]
    assert [[x.index for x in b] for b in plan_batches(r, 64 * 100, 2, 512)] == [[0, 1], [2, 3], [4]]
    assert [[x.index for x in b] for b in plan_batches(r, 64 * 100, 8, 512, batch_size=4)] == [[0, 1, 2, 3], [4]]
    with pytest.raises(ValueError, match="cache"):
        plan_batches(reqs([300], 0), 64 * 2, 8, 512)
    with pytest.raises(ValueError, match="longer than the context"):
        plan_batches(reqs([600], 0), 64 * 100, 8, 512)
    with pytest.raises(ValueError, match="empty"):
        plan_batches(reqs([0], 4), 64, 8, 512)


def test_live_batch_stops_lengths_and_context():
    r = reqs([3, 4, 5, 2], 3)
    for i, x in enumerate(r):
        x.slot = 10 + i
    live = LiveBatch(r, stop_tokens=[99], max_context=7)
    assert live.first_step() == [(10, [1, 2, 3], [2]), (11, [1, 2, 3, 4], [3]), (12, [1, 2, 3, 4, 5], [4]), (13, [1, 2], [1])]
    done, nxt = live.take([7, 99, 8, 9])
    assert [x.index for x in done] == [1] and r[1].finish_reason == "stop" and r[1].output == []
    assert nxt == [(10, [7], [0]), (12, [8], [0]), (13, [9], [0])]
    done, nxt = live.take([7, 8, 99])  # request 2 now holds 5 + 2 = 7 tokens: its context is full
    assert {x.index: x.finish_reason for x in done} == {2: "context", 3: "stop"}
    assert nxt == [(10, [7], [0])]
    done, nxt = live.take([5])
    assert r[0].finish_reason == "length" and r[0].output == [7, 7, 5] and nxt == []
    zero = reqs([2], 0)
    zero[0].slot = 1
    live = LiveBatch(zero, [], 10)
    done, nxt = live.take([4])
    assert zero[0].output == [] and zero[0].finish_reason == "length" and nxt == []


class FakeEngine:
    """Stands in for the engine: records steps, hands out slots lowest-first, 'logits' are made so that
    the sampler below returns (last token + 1) % 50."""

    class Cache:
        n_pages, max_slots = 4, 2

    def __init__(self):
        self.cache, self.max_context = self.Cache(), 64
        self.free, self.steps, self.opened = [1, 0], [], []

    def open(self):
        s = self.free.pop()
        self.opened.append(s)
        return s

    def close(self, slot):
        assert slot not in self.free
        self.free.append(slot)
        self.free.sort(reverse=True)

    def step(self, entries):
        self.steps.append([(s, list(t)) for s, t, _ in entries])
        self.last_batch = type("B", (), {"seq_slot": None})()
        return torch.tensor([[float(t[-1])] for _, t, _ in entries])


class FakeSampler:
    device = "cpu"

    def states(self, idx):
        return torch.tensor([stream_seed(1, i) % (1 << 62) for i in idx], dtype=torch.int64)

    def sample(self, logits, states, index=None):
        return ((logits[:, 0].to(torch.int64) + 1) % 50).to(torch.int32)


def test_generator_runs_batch_after_batch_and_reuses_slots():
    eng = FakeEngine()
    gen = Generator(eng, FakeSampler(), stop_tokens=[13])
    out = gen.generate([[10], [3, 4], [11, 12], [40]], max_new_tokens=4)
    assert [r.output for r in out] == [[11, 12], [5, 6, 7, 8], [], [41, 42, 43, 44]]
    assert [r.finish_reason for r in out] == ["stop", "length", "stop", "length"]
    assert gen.stats["batches"] == 2 and eng.opened == [0, 1, 0, 1] and eng.free == [1, 0]
    # first batch: both prompts whole, then one token each, then only the longer-running one
    assert eng.steps[0] == [(0, [10]), (1, [3, 4])] and eng.steps[1] == [(0, [11]), (1, [5])]
    assert eng.steps[2] == [(0, [12]), (1, [6])] and eng.steps[3] == [(1, [7])]
    # the stop token of request 0 (13) was neither kept nor run; request 2 stopped at once
    assert eng.steps[4] == [(0, [11, 12]), (1, [40])] and eng.steps[5] == [(1, [41])]


class FakeEngineAhead(FakeEngine):
    """The same, but it can run a decode step from tokens it is handed as a tensor, as the real engine does from
    tokens on the device; it notes which steps came that way."""

    def __init__(self):
        super().__init__()
        self.ahead = []

    def step_ahead(self, slots, tokens):
        self.ahead.append(len(self.steps))
        return self.step([(s, [int(t)], [0]) for s, t in zip(slots, tokens.tolist())])


def test_generator_runs_ahead_and_drops_the_rows_of_sequences_that_stopped():
    """With an engine that can step from tokens the host has not seen, the loop launches the next step before
    it reads the tokens. Outputs and finish reasons are those of the loop that waits; a step launched ahead
    carries the row of a sequence whose token then stopped it, and that row is dropped; no step is launched
    ahead when a sequence is about to end by its length."""
    eng, plain_eng = FakeEngineAhead(), FakeEngine()
    prompts = [[10], [3, 4], [11, 12], [40]]
    out = Generator(eng, FakeSampler(), stop_tokens=[13]).generate(prompts, max_new_tokens=4)
    want = Generator(plain_eng, FakeSampler(), stop_tokens=[13]).generate(prompts, max_new_tokens=4)
    assert [r.output for r in out] == [r.output for r in want] == [[11, 12], [5, 6, 7, 8], [], [41, 42, 43, 44]]
    assert [r.finish_reason for r in out] == [r.finish_reason for r in want]
    assert eng.opened == [0, 1, 0, 1] and eng.free == [1, 0]
    # first batch: the prompts; a step ahead with 11 and 5; one with 12 and 6; then 13 stops request 0 after the step
    # with 13 and 7 was launched: its row for request 0 is dropped and request 1 goes on alone (its last token by
    # the host's way, since it ends by its length)
    assert eng.steps[:4] == [[(0, [10]), (1, [3, 4])], [(0, [11]), (1, [5])], [(0, [12]), (1, [6])], [(0, [13]), (1, [7])]]
    assert eng.ahead[:3] == [1, 2, 3]
    # second batch: request 2 is stopped by its first token while the step ahead (with 13 and 41) is under way
    assert eng.steps[4] == [(0, [11, 12]), (1, [40])] and eng.steps[5] == [(0, [13]), (1, [41])]
    assert [len(st) for st in eng.steps[6:]] == [1, 1]
