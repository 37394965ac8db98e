"""The index arrays of a step (engine/batch.py), on the CPU: rows and padding; a step plan's words travelling with
them; and the attention mixer's own plan (parts/attention_plan.py), the tiles and the work list that its prefill
kernels walk. The kernels trust these lists; what they must hold is checked here against a reconstruction from the
sequences alone."""
import numpy as np
import pytest

from abacus_b200.engine.batch import Sequence, StepBatch
from abacus_b200.parts.attention_plan import (HALVED_PAIRS, PAIRED_ROWS, TILE_ROWS, WORK_INTS, AttentionLists,
                                              AttentionStepPlan)

CTA_SLOTS = 2 * 148  # the places the tests give the tile-halving kernel: two CTAs on each of a B200's SMs


def random_step(rng, n_seqs, longest):
    seqs = []
    for slot in rng.permutation(64)[:n_seqs]:
        n = int(rng.integers(1, longest + 1))
        start = int(rng.choice([0, 0, 5, 64, 700]))
        want = sorted(set(int(w) for w in rng.integers(0, n, int(rng.integers(0, 4)))))
        seqs.append(Sequence(int(slot), [int(t) for t in rng.integers(0, 1000, n)], start, want))
    return seqs


def test_rows_and_padding_of_a_step():
    rng = np.random.default_rng(0)
    for trial in range(20):
        seqs = random_step(rng, int(rng.integers(1, 7)), 300)
        rows = sum(len(s.tokens) for s in seqs)
        b = StepBatch(rows + 9, len(seqs) + 2, sum(len(s.want) for s in seqs) + 1, "cpu").fill(seqs)
        assert (b.n_tokens, b.n_seqs, b.n_rows) == (rows, len(seqs), rows + 9)
        at, wanted = 0, []
        for i, s in enumerate(seqs):
            n = len(s.tokens)
            assert b.tokens[at:at + n].tolist() == s.tokens and set(b.token_seq[at:at + n].tolist()) == {i}
            assert b.token_pos[at:at + n].tolist() == list(range(s.start, s.start + n))
            assert (int(b.seq_slot[i]), int(b.seq_start[i]), int(b.seq_pos0[i]), int(b.seq_len_after[i])) == \
                   (s.slot, at, s.start, s.start + n)
            wanted += [at + w for w in s.want]
            at += n
        assert set(b.token_seq[rows:].tolist()) == {-1}  # padding rows belong to no sequence
        assert b.seq_start[len(seqs):].tolist() == [rows] * 3
        assert b.logit_rows[:len(wanted)].tolist() == wanted and b.n_logit_rows == len(wanted)
        assert b.max_position == max(s.start + len(s.tokens) - 1 for s in seqs)
        assert b.any_continuation == any(s.start > 0 for s in seqs)
        exact = StepBatch(rows + 9, len(seqs) + 2, len(wanted) + 1, "cpu").fill(seqs, exact=True)
        assert exact.n_rows == rows and exact.tokens.shape[0] == rows and exact.seq_slot.shape[0] == len(seqs)


def test_a_step_that_does_not_fit_or_wants_a_place_it_does_not_bring_is_refused():
    b = StepBatch(10, 2, 2, "cpu")
    with pytest.raises(ValueError):
        b.fill([Sequence(0, [1] * 11, 0, [])])
    with pytest.raises(ValueError):
        b.fill([Sequence(0, [1], 0, []), Sequence(1, [1], 0, []), Sequence(2, [1], 0, [])])
    with pytest.raises(ValueError):
        b.fill([Sequence(0, [1, 2, 3], 0, [3])])


def test_a_decode_step_has_no_tiles():
    plan = AttentionStepPlan(4, cta_slots=CTA_SLOTS)
    b = StepBatch(8, 8, 8, "cpu", plans=[plan]).fill([Sequence(i, [7], 100 + i, [0]) for i in range(5)])
    lists = AttentionLists(b.plan[plan.name])
    assert b.is_decode and set(lists.work.reshape(-1).tolist()) == {-1} and lists.n_halved == 0
    for r in TILE_ROWS:
        assert set(lists.tiles(r).reshape(-1).tolist()) == {-1}


class CountingPlan:
    """A step plan of a toy mixer: for every sequence, how many tokens it brings and where it starts."""
    name = "counting"

    class Layout:
        def __init__(self, n_seqs):
            self.words = 2 * n_seqs

    def layout(self, n_rows, n_seqs):
        return self.Layout(n_seqs)

    def fill(self, layout, sequences, words, is_decode, exact):
        words[:] = -7
        for i, s in enumerate(sequences):
            words[2 * i], words[2 * i + 1] = len(s.tokens), s.start
        return {"sequences": len(sequences), "decode": is_decode}


def test_a_step_plan_travels_with_the_step():
    """The engine knows nothing of what a plan holds: it gives the plan its words in the step's one buffer, at a fixed
    place, and hands the mixer what the plan returned."""
    counting, lists = CountingPlan(), AttentionStepPlan(2, cta_slots=CTA_SLOTS)
    b = StepBatch(300, 4, 4, "cpu", plans=[counting, lists, counting])  # the same name twice: one part of the buffer
    assert list(b.plans) == ["counting", lists.name]
    seqs = [Sequence(3, [1] * 200, 0, [199]), Sequence(1, [2] * 5, 64, [])]
    b.fill(seqs)
    view = b.plan["counting"]
    assert view.words.tolist() == [200, 0, 5, 64, -7, -7, -7, -7] and view.info == {"sequences": 2, "decode": False}
    at = view.words.data_ptr()
    b.fill([Sequence(0, [9], 10, [0])])
    assert b.plan["counting"].words.data_ptr() == at and b.plan["counting"].words.tolist()[:2] == [1, 10]
    assert b.plan["counting"].info["decode"] and b.tokens[:1].tolist() == [9]
    assert (b._dev == b._host).all()  # the plans' words went to the device in the step's own copy


def expected_tiles(seqs, rows_per_tile):
    return {(i, r0) for i, s in enumerate(seqs) for r0 in range(0, len(s.tokens), rows_per_tile)}


def pages_seen(s, r0, rows_per_tile):
    return (s.start + min(r0 + rows_per_tile, len(s.tokens)) - 1) // 64 + 1


@pytest.mark.parametrize("heads", [1, 3, 16, 40])
def test_tiles_and_work_list_cover_every_row_once(heads):
    rng = np.random.default_rng(heads)
    halved_somewhere = False
    for trial in range(30):
        seqs = random_step(rng, int(rng.integers(1, 6)), int(rng.choice([40, 300, 2500])))
        if all(len(s.tokens) == 1 for s in seqs):
            continue
        rows = sum(len(s.tokens) for s in seqs)
        plan = AttentionStepPlan(heads, cta_slots=CTA_SLOTS)
        b = StepBatch(rows + 5, len(seqs) + 1, 16, "cpu", plans=[plan]).fill(seqs)
        lists = AttentionLists(b.plan[plan.name])
        for r in TILE_ROWS:
            tiles = lists.tiles(r).numpy()
            real = tiles[tiles[:, 0] >= 0]
            assert len(real) == len(expected_tiles(seqs, r)) == len({tuple(t) for t in real.tolist()})
            assert {tuple(t) for t in real.tolist()} == expected_tiles(seqs, r)
            assert (tiles[len(real):] == -1).all()  # padding behind, never between
            seen = [seqs[i].start + r0 for i, r0 in real.tolist()]
            assert seen == sorted(seen, reverse=True)  # the tiles that see the most keys first
        work = lists.work.numpy()
        real = work[work[:, 0] >= 0]
        assert (work[len(real):] == -1).all() and work.shape[1] == WORK_INTS
        first_row = np.cumsum([0] + [len(s.tokens) for s in seqs])
        parts, lengths = {}, []
        for seq, r0, part, row_of_seq, pos0, n_new, slot, halved_id in real.tolist():
            s = seqs[seq]
            assert (row_of_seq, pos0, n_new, slot) == (int(first_row[seq]), s.start, len(s.tokens), s.slot)
            parts.setdefault((seq, r0), []).append((part, halved_id))
            pages = pages_seen(s, r0, PAIRED_ROWS)
            lengths.append(pages if part == 0 else (pages + 1) // 2 if part == 1 else pages // 2)
        assert set(parts) == expected_tiles(seqs, PAIRED_ROWS)
        assert lengths == sorted(lengths, reverse=True)  # the CTAs with the most pages first
        ids = []
        for (seq, r0), ps in parts.items():
            if len(ps) == 1:
                assert ps[0][0] == 0  # a whole tile stands once
            else:  # a halved tile stands twice, earlier and later keys, under one id; only long tiles are halved
                assert sorted(p for p, _ in ps) == [1, 2] and ps[0][1] == ps[1][1]
                assert pages_seen(seqs[seq], r0, PAIRED_ROWS) >= 8
                ids.append(ps[0][1])
        assert sorted(ids) == list(range(len(ids))) and lists.n_halved == len(ids)
        assert len(ids) * heads <= HALVED_PAIRS  # what the kernel has scratch memory for
        if ids:
            halved_somewhere = True
            # tiles are halved only into places the device would otherwise leave empty, give or take a few
            assert len(real) * heads <= 1.05 * CTA_SLOTS + heads
    assert halved_somewhere or heads == 40


# ------------------------------------------------------------------ which captured graph a step goes to

def test_buckets_of_captured_steps():
    from abacus_b200.engine.graphs import ROW_BUCKETS, POSITION_STEP, prompt_bucket, row_bucket
    assert [row_bucket(n) for n in (1, 2, 3, 8, 9, 17, 64, 65, 256)] == [1, 2, 4, 8, 16, 24, 64, 96, 256]
    assert row_bucket(257) is None and list(ROW_BUCKETS) == sorted(ROW_BUCKETS) and POSITION_STEP % 64 == 0
    for n in list(range(1, 300)) + [1000, 2048, 2049, 5000, 100000]:
        b = prompt_bucket(n)
        assert b >= n and b >= 16 and (b & (b - 1) == 0 or b % 128 == 0)
        assert b <= max(16, 2 * n) and (n <= 128 or b - n < max(128, n // 8) + 1)  # never much padding
        assert prompt_bucket(b) == b  # a bucket is its own bucket


class FakeContext:
    device = "cpu"


class FakePart:
    def __init__(self, **flags):
        self.__dict__.update(flags)


class FakeModel:
    ctx = FakeContext()

    def __init__(self, parts=()):
        self._parts = list(parts)

    def parts(self):
        return iter(self._parts)

    def step_plans(self):
        return []


class FakeEngine:
    def __init__(self):
        self.model = FakeModel()
        self.max_context = 4096


def test_which_models_are_captured():
    """A model's steps are replayed from graphs only if every part says that its forward pass launches device work
    alone; steps of several tokens also only if no mixer objects (a windowed attention layer does: it checks such steps
    on the host)."""
    from abacus_b200.engine.engine import capturable
    sure = FakePart(capturable=True)
    assert capturable(FakeModel([sure, sure])) == (True, True)
    assert capturable(FakeModel([sure, FakePart()])) == (False, False)  # a part that does not say so is not
    assert capturable(FakeModel([sure, FakePart(capturable=True, capturable_prompts=False)])) == (True, False)
    from abacus_b200.config.specs import AttentionSpec
    from abacus_b200.parts import MIXERS
    spec = dict(hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, scale=0.25, qk_norm_eps=None, position=None)
    assert MIXERS.build(AttentionSpec(**spec)).capturable_prompts
    assert not MIXERS.build(AttentionSpec(**spec, window=24)).capturable_prompts


def test_which_steps_are_captured():
    from abacus_b200.engine.graphs import DecodeGraphs, PromptGraphs
    prompts = [Sequence(0, [1] * 700, 0, [699]), Sequence(1, [1] * 33, 0, [32])]
    decode = [Sequence(i, [5], 40 + i, [0]) for i in range(5)]
    graphs = PromptGraphs(FakeEngine())
    assert not graphs.takes(decode)  # one token each: the decode graphs' business
    assert not graphs.takes(prompts)  # a shape seen once is not worth a capture
    assert graphs.takes(prompts)  # the second time it is
    same_shape = [Sequence(3, [2] * 650, 0, [0]), Sequence(4, [2] * 90, 0, [1])]
    assert graphs.key(same_shape) == graphs.key(prompts) == (768, 2, 2)
    other = [Sequence(3, [2] * 650, 0, [0, 1, 2]), Sequence(4, [2] * 90, 0, [1])]
    assert graphs.key(other) == (768, 2, 4) and not graphs.takes(other)
    d = DecodeGraphs(FakeEngine())
    assert d.takes(decode) and not d.takes(prompts)
    assert not d.takes([Sequence(0, [5], 3, [])])  # a decode row whose logits nobody wants is not the captured shape
    assert not d.takes([Sequence(i, [5], 3, [0]) for i in range(257)])
    g = d.get(decode)
    assert (g.rows, g.position_bound) == (8, 1024) and d.get(decode) is g
    far = [Sequence(0, [5], 1024, [0])]
    assert d.get(far).position_bound == 2048 and d.get(far).rows == 1
