"""Each part alone, a model whose schedule names a layer twice or shares a cache, generation through
the entry point, and a toy mixer with state of its own that is registered from here."""
import math
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from helpers import BF16_REL_MAX, TINY, assert_logits, make_model_folder, random_tokens, tiny_config
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = [("float32", torch.float32), ("bfloat16", torch.bfloat16)]


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def ctx_of(dtype):
    from abacus_b200.parts import BuildContext
    return BuildContext(device=torch.device("cuda", 0), dtype=dtype)


def one_sequence_batch(n, start=0, slot=0):
    from abacus_b200.engine.batch import Sequence, StepBatch
    return StepBatch(n, 1, 0, "cuda").fill([Sequence(slot, [0] * n, start, [])])


def test_norm_part():
    from abacus_b200.config import NormSpec
    from abacus_b200.parts import NORMS
    rng = np.random.default_rng(0)
    w = (1 + 0.2 * rng.standard_normal(100)).astype(np.float32)
    norm = NORMS.build(NormSpec(size=100, eps=1e-4))
    assert norm.param_shapes() == {"weight": (100,)}
    norm.bind({"weight": torch.tensor(plain.bf16_round(w)).to(torch.bfloat16)}, ctx_of(torch.bfloat16))
    assert norm.weight.dtype == torch.float32  # norm weights are used in float32 whatever they are stored in
    x = rng.standard_normal((4, 100)).astype(np.float32)
    out = torch.empty(4, 100, device="cuda")
    norm.forward(dev(x), None, out)
    np.testing.assert_allclose(out.cpu().numpy(), plain.rmsnorm(x, plain.bf16_round(w), 1e-4), rtol=2e-5, atol=2e-6)


def test_rotary_part_tables():
    from abacus_b200.config import RotarySpec
    from abacus_b200.parts import POSITIONS
    rot = POSITIONS.build(RotarySpec(theta=1e6, rotary_dim=48))
    cos, sin = rot.tables(300, torch.device("cuda", 0))
    c, s = plain.rope_table(300, 48, 1e6)
    np.testing.assert_array_equal(cos.cpu().numpy(), c)  # both follow src/model.c:121 in float32
    np.testing.assert_array_equal(sin.cpu().numpy(), s)
    with pytest.raises(ValueError):
        POSITIONS.build(RotarySpec(theta=1e4, rotary_dim=7))


@pytest.mark.parametrize("dname, dtype", DTYPES)
def test_mlp_part(dname, dtype):
    from abacus_b200.config import GatedMLPSpec
    from abacus_b200.parts import FEED_FORWARDS, Workspace
    rng = np.random.default_rng(1)
    d, inter, n = 72, 200, 9
    w = {k: plain.bf16_round(0.1 * rng.standard_normal(s)) for k, s in
         [("gate", (inter, d)), ("up", (inter, d)), ("down", (d, inter))]}
    x = plain.bf16_round(rng.standard_normal((n, d)))
    ffn = FEED_FORWARDS.build(GatedMLPSpec(hidden=d, inter=inter))
    assert ffn.param_shapes() == {"gate": (inter, d), "up": (inter, d), "down": (d, inter)}
    ffn.bind({k: torch.tensor(v).to(torch.bfloat16) for k, v in w.items()}, ctx_of(dtype))
    out = torch.empty(n, d, device="cuda")
    ffn.forward(dev(x, dtype), out, one_sequence_batch(n), Workspace(torch.device("cuda", 0)))
    r = plain.bf16_round if dtype == torch.bfloat16 else (lambda a: a)
    gate_up = r(np.concatenate([plain.linear(x, w["gate"]), plain.linear(x, w["up"])], -1))
    want = plain.linear(r(plain.swiglu(gate_up)), w["down"])
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-4 if dtype == torch.float32 else 2e-2,
                               atol=1e-5 if dtype == torch.float32 else 2e-3)


@pytest.mark.parametrize("dname, dtype", DTYPES)
def test_attention_part_and_block(dname, dtype):
    """An attention mixer alone (with a cache of its own), then a whole block around it."""
    from abacus_b200.cache import SequenceCache
    from abacus_b200.config import AttentionSpec, BlockSpec, GatedMLPSpec, NormSpec, RotarySpec
    from abacus_b200.parts import BLOCKS, Workspace
    rng = np.random.default_rng(2)
    d, hq, hkv, hd, inter, n, eps = 56, 4, 2, 24, 88, 75, 1e-5
    spec = BlockSpec(
        mixer_norm=NormSpec(d, eps),
        mixer=AttentionSpec(hidden=d, n_heads=hq, n_kv_heads=hkv, head_dim=hd, scale=1 / math.sqrt(hd),
                            qk_norm_eps=eps, position=RotarySpec(theta=5e4, rotary_dim=hd)),
        ffn_norm=NormSpec(d, eps), ffn=GatedMLPSpec(d, inter))
    block = BLOCKS.build(spec)
    shapes = {pn: part.param_shapes() for pn, part in block.parts().items()}
    assert shapes["mixer"]["wq"] == (hq * hd, d) and shapes["mixer"]["k_norm"] == (hd,)
    w = {pn: {slot: plain.bf16_round((0.15 * rng.standard_normal(s)) if len(s) == 2 else
                                     (2 + 0.2 * rng.standard_normal(s))) for slot, s in sh.items()}
         for pn, sh in shapes.items()}
    block.bind({pn: {k: torch.tensor(v).to(torch.bfloat16) for k, v in ws.items()} for pn, ws in w.items()}, ctx_of(dtype))
    cache = SequenceCache([block.mixer.cache_need()], [None], 256, dtype, "cuda", max_context=256)
    block.mixer.prepare(256, torch.device("cuda", 0))
    ws = Workspace(torch.device("cuda", 0))
    r = plain.bf16_round if dtype == torch.bfloat16 else (lambda a: a)
    x0 = rng.standard_normal((n, d)).astype(np.float32)
    # plain: the block as src/model.c:292-310 runs it
    cos, sin = plain.rope_table(n, hd, 5e4)
    m = w["mixer"]
    xn = r(plain.rmsnorm(x0, w["mixer_norm"]["weight"], eps))
    q = r(plain.linear(xn, m["wq"])).reshape(n, hq, hd)
    k = r(plain.linear(xn, m["wk"])).reshape(n, hkv, hd)
    v = r(plain.linear(xn, m["wv"])).reshape(n, hkv, hd)
    q, k = r(plain.rope(plain.rmsnorm(q, m["q_norm"], eps), cos, sin)), r(plain.rope(plain.rmsnorm(k, m["k_norm"], eps), cos, sin))
    att = r(plain.attention(q, k, v, rnd=plain.bf16_round if dtype == torch.bfloat16 else None).reshape(n, hq * hd))
    mix = plain.linear(att, m["wo"])
    x1 = x0 + mix
    xn2 = r(plain.rmsnorm(x1, w["ffn_norm"]["weight"], eps))
    gu = r(np.concatenate([plain.linear(xn2, w["ffn"]["gate"]), plain.linear(xn2, w["ffn"]["up"])], -1))
    ffn = plain.linear(r(plain.swiglu(gu)), w["ffn"]["down"])
    if dtype == torch.float32:
        def near(got, want):
            np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-4)
    else:  # the bound of helpers.assert_logits: 2 % of the largest value
        def near(got, want):
            np.testing.assert_allclose(got, want, rtol=0, atol=BF16_REL_MAX * np.abs(want).max())
    # the mixer alone: 60 tokens, then 15 more one by one
    slot = cache.open_slot()
    outs = []
    for a, b in [(0, 60)] + [(i, i + 1) for i in range(60, n)]:
        cache.reserve(slot, b)
        out = torch.empty(b - a, d, device="cuda")
        block.mixer.forward(dev(xn[a:b], dtype), out, one_sequence_batch(b - a, a, slot), cache.views[0], ws)
        cache.advance(slot, b - a)
        outs.append(out.cpu().numpy())
    near(np.concatenate(outs), mix)
    cache.close_slot(slot)
    # the block: residual stream in, residual stream and pending output out
    slot = cache.open_slot()
    cache.reserve(slot, n)
    x = dev(x0)
    y = block.forward(x, None, one_sequence_batch(n, 0, slot), cache.views[0], ws)
    near(x.cpu().numpy(), x1)
    near(y.cpu().numpy(), ffn)


# ------------------------------------------------------------------ schedules

@pytest.mark.parametrize("dname, dtype", DTYPES)
def test_schedule_names_a_layer_twice_and_shares_a_cache(tmp_path, dname, dtype):
    """The run order is data: layer 0 runs twice (each run with keys of its own), and the last entry
    reads the keys and values of the first instead of making its own."""
    from abacus_b200.config import ScheduleEntry, load_config
    from abacus_b200.engine import Engine
    from abacus_b200.models import Model
    from abacus_b200.weights import load_folder
    import dataclasses
    folder = make_model_folder(tmp_path, "B")
    arch, cfg = load_config(folder)
    spec = dataclasses.replace(cfg.to_spec(), schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                                        ScheduleEntry(2, source=0)))
    tensors = load_folder(folder, lambda names: arch.tensor_names(spec, names))
    engine = Engine(Model(spec, arch.layout(spec), tensors, dtype, torch.device("cuda", 0)), max_tokens=256)
    assert len(engine.cache.groups[0].entries) == 3  # entries 0, 1 and 2 keep keys; entry 3 borrows
    pcfg, pw = plain.load(folder)
    ids = random_tokens(np.random.default_rng(4), 50, pcfg["vocab"])
    want = plain.forward(pcfg, pw, ids, rnd=plain.bf16_round if dtype == torch.bfloat16 else None,
                         schedule=[(0, None), (1, None), (0, None), (2, 0)])
    slot = engine.open()
    got = [engine.step([(slot, ids[:30], list(range(30)))]).cpu().numpy()]
    for i in range(30, 50):
        got.append(engine.step([(slot, ids[i:i + 1], [0])]).cpu().numpy())
    assert_logits(np.concatenate(got), want, dname, "schedule")


@pytest.mark.parametrize("dname, dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_prompt_steps_of_a_shape_seen_before_are_replayed(tmp_path, name, dname, dtype):
    """A step that brings prompts is captured the second time its shape (rows, sequences, wanted rows, each
    rounded up) comes by, and replayed after that. With other tokens, other lengths inside the same bucket and
    other slots every replay gives what the plain implementation gives; and every step, also those in which
    the sequences go on by several tokens, gives what an engine without graphs gives for it (the padding of a
    captured step changes no result)."""
    from abacus_b200.engine import Engine, load_model
    folder = make_model_folder(tmp_path, name)
    model = load_model(folder, dname)
    engine, eager = Engine(model, max_tokens=4096), Engine(model, max_tokens=4096, use_graphs=False)
    pcfg, pw = plain.load(folder)
    rng = np.random.default_rng(11)

    def want_and_noise(tokens):  # the plain logits in this dtype, and the rounding noise they carry (helpers.assert_logits)
        exact = plain.forward(pcfg, pw, tokens)
        if dtype == torch.bfloat16:
            want = plain.forward(pcfg, pw, tokens, rnd=plain.bf16_round)
            return want, float(np.abs(want - exact).max())
        return exact, float(np.abs(exact - plain.forward64(pcfg, pw, tokens)).max())

    def both(entries_of):
        got = engine.step(entries_of(slots)).cpu().numpy()
        ref = eager.step(entries_of(eager_slots)).cpu().numpy()
        close = 1e-5 if dtype == torch.float32 else 4e-3  # of the largest logit: the same kernels on the same rows
        assert np.abs(got - ref).max() <= close * np.abs(ref).max(), "a replayed step differs from the step run as it is"
        return got

    for round_, lengths in enumerate([(150, 70), (141, 90), (160, 60), (129, 101)]):  # 220-231 rows: one bucket
        ids = [random_tokens(rng, n, pcfg["vocab"]) for n in lengths]
        slots, eager_slots = [engine.open() for _ in lengths], [eager.open() for _ in lengths]
        got = both(lambda ss: [(s, t, [0, len(t) - 1]) for s, t in zip(ss, ids)])
        for i, t in enumerate(ids):
            want, noise = want_and_noise(t)
            assert_logits(got[2 * i:2 * i + 2], want[[0, len(t) - 1]], dname, f"{name} round {round_} sequence {i}", noise)
        if round_ == 3:  # the sequences go on by several tokens each: another shape, met twice
            for again in range(2):
                more = [random_tokens(rng, 40, pcfg["vocab"]) for _ in lengths]
                both(lambda ss: [(s, m, [39]) for s, m in zip(ss, more)])
        for s, e in zip(slots, eager_slots):
            engine.close(s), eager.close(e)
    engine.check_status()
    assert engine.prompt_graphs.captured == 2 and engine.prompt_graphs.replayed == 4 and eager.prompt_graphs is None


@pytest.mark.parametrize("sizes, lens, embed_scale", [
    (dict(hidden_size=1024, intermediate_size=3072, num_attention_heads=16, tie_word_embeddings=True), (2048, 700), 4.0),
    (dict(hidden_size=2560, intermediate_size=9728, num_attention_heads=32, tie_word_embeddings=True), (1100, 300), 2.5),
    (dict(hidden_size=4096, intermediate_size=12288, num_attention_heads=32, tie_word_embeddings=False), (900, 260), 2.0),
], ids=["0.6b", "4b", "8b"])
def test_layers_of_the_measured_size(tmp_path, sizes, lens, embed_scale):
    """Two layers with the sizes of a measured configuration (the Qwen3-0.6B, 4B and 8B shapes: widths 1024, 2560 and
    4096, 16 or 32 query heads on 8 kv heads of 128, inner sizes 3072, 9728 and 12288, the last with an output matrix
    of its own), a long prompt beside a shorter one, then decode steps: the step takes the ways that tiny models do not
    (the persistent tensor-core product and, for the down projections whose K is beyond it, the per-tile one; SwiGLU
    in the epilogue; attention tiles halved between CTAs; groups of 2 and of 4; the rows kernels with clusters), the
    second time from a captured graph. bfloat16 against the plain implementation."""
    from abacus_b200.config import Qwen3Config
    from abacus_b200.engine import Engine, load_model
    from abacus_b200.weights import write_random_model
    from helpers import SHARP
    raw = dict(sizes, num_hidden_layers=2, num_key_value_heads=8, head_dim=128, vocab_size=3000, max_position_embeddings=4096,
               rope_theta=1e6, rms_norm_eps=1e-6, architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    folder = os.path.join(str(tmp_path), "wide")
    # (the factors that sharpen the tiny models, with the embedding's and the output matrix's turned down: at these
    # widths they alone would make logits of twenty and more, where the tiny models have five to eight)
    write_random_model(folder, Qwen3Config.from_dict(raw), seed=5, norm_std=0.05,
                       scales=dict(SHARP, embed_tokens=embed_scale, lm_head=embed_scale))
    pcfg, pw = plain.load(folder)
    rng = np.random.default_rng(3)
    extra = 2
    ids = [random_tokens(rng, n + extra, pcfg["vocab"]) for n in lens]
    exact = [plain.forward(pcfg, pw, t) for t in ids]
    want = [plain.forward(pcfg, pw, t, rnd=plain.bf16_round) for t in ids]
    noise = [float(np.abs(w - e).max()) for w, e in zip(want, exact)]
    engine = Engine(load_model(folder, "bfloat16"), max_tokens=2 * 4096)
    for turn in range(2):
        slots = [engine.open() for _ in ids]
        places = [[0, 100, n // 2, n - 1] for n in lens]
        got = engine.step([(s, t[:n], list(range(n))) for s, t, n in zip(slots, ids, lens)]).cpu().numpy()
        first = 0
        for i, (n, w) in enumerate(zip(lens, places)):
            mine = got[first:first + n]
            first += n
            assert_logits(mine[w], want[i][w], "bfloat16", f"turn {turn} prompt {i}", noise[i])
            # Every other row: a tile of rows gone wrong (a race between a CTA's warps, a page taken twice) is off by
            # several times the rounding noise that the plain implementation itself shows on this input, and need
            # not touch the four places above.
            off = np.abs(mine - want[i][:n]).max(axis=1)
            assert off.max() <= noise[i], f"turn {turn} prompt {i}: row {off.argmax()} is off by {off.max():.3g}"
        for step in range(extra):
            got = engine.step([(s, t[n + step:n + step + 1], [0]) for s, t, n in zip(slots, ids, lens)]).cpu().numpy()
            for i, n in enumerate(lens):
                assert_logits(got[i:i + 1], want[i][n + step:n + step + 1], "bfloat16", f"turn {turn} decode {step} of {i}", noise[i])
        for s in slots:
            engine.close(s)
    engine.check_status()
    assert engine.prompt_graphs.replayed == 1


# ------------------------------------------------------------------ generation through the entry point

@pytest.mark.parametrize("dname", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dname):
    """The workloads that are measured: unequal prompts, greedy; more requests than one batch holds, a stop token."""
    from abacus_b200 import LM
    folder = make_model_folder(tmp_path, name)
    cfg, w = plain.load(folder)
    rng = np.random.default_rng(11)
    prompts = [random_tokens(rng, n, cfg["vocab"]) for n in (5, 11, 17, 1, 40)]
    rnd = plain.bf16_round if dname == "bfloat16" else None
    free = plain.generate(cfg, w, prompts[1], 12, rnd=rnd)
    stop = free[6]  # a token that request 1 will reach: it must end there, without it
    want = [plain.generate(cfg, w, p, 12, stop=(stop,), rnd=rnd) for p in prompts]
    lm = LM(folder, dtype=dname, max_tokens=64 * 3)  # room for three requests: two batches
    got = lm.generate(prompts, max_new_tokens=12, temperature=0.0, stop_tokens=[stop])
    assert lm.last_stats["batches"] == 2
    if dname == "float32":
        assert got == want
    else:
        # In bfloat16 a near-tie may fall the other way, after which the texts differ for good. So each
        # token the engine chose must be a maximum of the plain logits for the engine's own text,
        # up to the bfloat16 tolerance of the logits.
        from helpers import BF16_REL_MAX
        for p_, g in zip(prompts, got):
            if not g:
                continue
            logits = plain.forward(cfg, w, p_ + g, rnd=rnd)[len(p_) - 1:len(p_) + len(g) - 1]
            slack = 2 * BF16_REL_MAX * np.abs(logits).max()
            for i, tok in enumerate(g):
                assert logits[i, tok] >= logits[i].max() - slack, (i, tok)
        assert sum(g == x for g, x in zip(got, want)) >= 3  # and most requests agree outright
    assert len(got[1]) <= 6 and stop not in got[1]


def test_sampled_generation_is_seeded_and_independent_of_batching(tmp_path):
    """The second measured configuration's workload: temperature 0.8, seeded. A request draws the same tokens alone
    as in a batch, because its random stream is its own."""
    from abacus_b200 import LM
    folder = make_model_folder(tmp_path, "B")
    cfg, w = plain.load(folder)
    rng = np.random.default_rng(12)
    prompts = [random_tokens(rng, n, cfg["vocab"]) for n in (1, 7, 23, 40)]
    lm = LM(folder, dtype="float32", max_tokens=64 * 4)
    a = lm.generate(prompts, max_new_tokens=16, temperature=0.8, seed=5)
    b = lm.generate(prompts, max_new_tokens=16, temperature=0.8, seed=5, batch_size=1)
    c = lm.generate(prompts, max_new_tokens=16, temperature=0.8, seed=6)
    assert a == b and a != c and all(len(x) == 16 for x in a)
    # request 0 draws what abacus's loop would: xorshift64 from `seed` itself (src/main.c:52)
    assert a[0] == plain.generate(cfg, w, prompts[0], 16, temp=0.8, seed=5)


# ------------------------------------------------------------------ a toy mixer with state of its own

@dataclass(frozen=True)
class RunningMeanSpec:
    hidden: int
    kind: str = "toy_running_mean"


class TokensSoFar:
    """The toy mixer's step plan (engine/batch.py): for every row of the step, how many tokens its sequence holds up
    to and including it. Made on the host from the step's sequences, carried to the device with the step's indices."""
    name = "toy_tokens_so_far"

    class Layout:
        def __init__(self, n_rows):
            self.words = n_rows

    def layout(self, n_rows, n_seqs):
        return self.Layout(n_rows)

    def fill(self, layout, sequences, words, is_decode, exact):
        words[:] = 1  # padding rows divide by one
        row = 0
        for s in sequences:
            n = len(s.tokens)
            words[row:row + n] = np.arange(s.start + 1, s.start + n + 1)
            row += n
        return row


class RunningMean:
    """out_t = W . mean(xn_0..xn_t): the state per sequence is the running sum (fixed size, no keys); the divisors
    come from a step plan of its own."""
    counts = TokensSoFar()

    def __init__(self, spec):
        self.spec = spec

    def step_plans(self):
        return [self.counts]

    def param_shapes(self):
        return {"w": (self.spec.hidden, self.spec.hidden)}

    def bind(self, params, ctx):
        self.w = params["w"].to(device=ctx.device, dtype=torch.float32)

    def cache_need(self):
        from abacus_b200.cache import CacheNeed
        return CacheNeed(state_shape=(self.spec.hidden,))

    def forward(self, xn, out, batch, cache, ws):
        mine = batch.plan[self.counts.name]
        assert mine.info == batch.n_tokens  # what the plan's fill returned comes back with its words
        so_far = mine.words.float()[:, None]
        row = 0
        for s in batch.sequences:  # a ragged step: walk each sequence's rows from its own state
            n = len(s.tokens)
            cum = cache.state[s.slot] + torch.cumsum(xn[row:row + n].float(), dim=0)
            out[row:row + n] = (cum / so_far[row:row + n]) @ self.w.T
            cache.state[s.slot] = cum[-1]
            row += n
        return out


def test_a_toy_mixer_is_registered_built_and_stepped(tmp_path):
    """Nothing in the package is changed: the mixer, its spec, its configuration and its architecture
    are all defined here, layers alternate between it and attention, and cuts and slot reuse agree."""
    from abacus_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, NormSpec, RotarySpec,
                                    ScheduleEntry, register_architecture)
    from abacus_b200.engine import Engine
    from abacus_b200.models import Model, ModelLayout, expected_tensors
    from abacus_b200.parts import MIXERS
    from abacus_b200.weights import random_tensors
    MIXERS.register("toy_running_mean", RunningMean)
    d, vocab, hd = 48, 97, 16

    class ToyArchitecture:
        name = "ToyForCausalLM"

        def spec(self):
            att = AttentionSpec(hidden=d, n_heads=3, n_kv_heads=1, head_dim=hd, scale=hd ** -0.5, qk_norm_eps=None,
                                position=RotarySpec(theta=1e4, rotary_dim=hd))
            blocks = tuple(BlockSpec(NormSpec(d, 1e-5), mixer, NormSpec(d, 1e-5), GatedMLPSpec(d, 64))
                           for mixer in (RunningMeanSpec(d), att, RunningMeanSpec(d)))
            return ModelSpec("ToyForCausalLM", d, vocab, blocks, tuple(ScheduleEntry(i) for i in range(3)),
                             NormSpec(d, 1e-5), True, 200)

        def layout(self, spec):
            layers = []
            for l, b in enumerate(spec.layers):
                from abacus_b200.parts import BLOCKS
                layers.append({(pn, slot): f"layers.{l}.{pn}.{slot}" for pn, part in BLOCKS.build(b).parts().items()
                               for slot in part.param_shapes()})
            return ModelLayout("embed", "norm", "head", layers)

    arch = register_architecture(ToyArchitecture())
    spec = arch.spec()
    layout = arch.layout(spec)
    expected, _ = expected_tensors(spec, layout)
    tensors = random_tensors(expected, seed=3, std=0.2, norm_std=0.1)
    model = Model(spec, layout, tensors, torch.float32, torch.device("cuda", 0))
    engine = Engine(model, max_tokens=64 * 4)
    assert sorted(engine.cache.states) == [0, 2] and len(engine.cache.groups) == 1
    # the step carries the toy mixer's plan beside the attention layer's, each once
    assert sorted(p.name for p in model.step_plans()) == ["attention_lists_3", "toy_tokens_so_far"]

    def plain_toy(ids):
        w = {k: v.float().numpy() for k, v in tensors.items()}
        n = len(ids)
        x = plain.embed(ids, w["embed"])
        cos, sin = plain.rope_table(n, hd, 1e4)
        for l in range(3):
            p = f"layers.{l}."
            xn = plain.rmsnorm(x, w[p + "mixer_norm.weight"], 1e-5)
            if l == 1:
                q = plain.rope(plain.linear(xn, w[p + "mixer.wq"]).reshape(n, 3, hd), cos, sin)
                k = plain.rope(plain.linear(xn, w[p + "mixer.wk"]).reshape(n, 1, hd), cos, sin)
                v = plain.linear(xn, w[p + "mixer.wv"]).reshape(n, 1, hd)
                mix = plain.linear(plain.attention(q, k, v).reshape(n, 3 * hd), w[p + "mixer.wo"])
            else:
                mean = np.cumsum(xn, axis=0, dtype=np.float32) / np.arange(1, n + 1, dtype=np.float32)[:, None]
                mix = plain.linear(mean, w[p + "mixer.w"])
            x = x + mix
            xn = plain.rmsnorm(x, w[p + "ffn_norm.weight"], 1e-5)
            gu = np.concatenate([plain.linear(xn, w[p + "ffn.gate"]), plain.linear(xn, w[p + "ffn.up"])], -1)
            x = x + plain.linear(plain.swiglu(gu), w[p + "ffn.down"])
        return plain.linear(plain.rmsnorm(x, w["norm"], 1e-5), w["embed"])

    rng = np.random.default_rng(5)
    seqs = [random_tokens(rng, n, vocab) for n in (20, 9, 33)]
    want = [plain_toy(s) for s in seqs]
    for round_ in range(2):  # the second round runs in slots (and states) the first has used
        slots = [engine.open() for _ in seqs]
        cut = [12, 9, 5]
        got = engine.step([(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
        at = 0
        for i, c in enumerate(cut):
            assert_logits(got[at:at + c], want[i][:c], "float32", f"toy prompt {i}")
            at += c
        live = [i for i in range(3) if cut[i] < len(seqs[i])]
        engine.close(slots[1])
        k = 0
        while live:
            got = engine.step([(slots[i], [seqs[i][cut[i] + k]], [0]) for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                assert_logits(got[j:j + 1], want[i][cut[i] + k:cut[i] + k + 1], "float32", f"toy decode {i}")
            k += 1
            for i in [i for i in live if cut[i] + k == len(seqs[i])]:
                engine.close(slots[i])
            live = [i for i in live if cut[i] + k < len(seqs[i])]


# ------------------------------------------------------------------ a toy feed-forward with routing, a toy position encoding

@dataclass(frozen=True)
class TopOneExpertsSpec:
    hidden: int
    inter: int
    n_experts: int
    kind: str = "toy_top_one_experts"


class TopOneExperts:
    """Each token goes to the expert its router scores highest; the expert's gated MLP, times the softmax
    weight of that score. Every expert runs on every row and the router picks: a row's result depends on
    nothing but the row."""

    def __init__(self, spec):
        self.spec = spec

    def param_shapes(self):
        s = self.spec
        return {"router": (s.n_experts, s.hidden), "gate": (s.n_experts * s.inter, s.hidden),
                "up": (s.n_experts * s.inter, s.hidden), "down": (s.n_experts * s.hidden, s.inter)}

    def bind(self, params, ctx):
        s = self.spec
        f = lambda t, *shape: t.to(device=ctx.device, dtype=torch.float32).reshape(*shape)
        self.router = f(params["router"], s.n_experts, s.hidden)
        self.gate, self.up = f(params["gate"], s.n_experts, s.inter, s.hidden), f(params["up"], s.n_experts, s.inter, s.hidden)
        self.down = f(params["down"], s.n_experts, s.hidden, s.inter)

    def forward(self, xn, out, batch, ws):
        n = batch.n_rows
        x = xn[:n].float()
        weights = torch.softmax(x @ self.router.T, dim=-1)
        top, chosen = weights.max(dim=-1)
        g, u = torch.einsum("td,eid->tei", x, self.gate), torch.einsum("td,eid->tei", x, self.up)
        every = torch.einsum("tei,edi->ted", torch.nn.functional.silu(g) * u, self.down)
        out[:n] = every[torch.arange(n, device=x.device), chosen] * top[:, None]
        return out


@dataclass(frozen=True)
class SlowedRotarySpec:
    rotary_dim: int
    theta: float
    slow: float
    kind: str = "toy_slowed_rotary"


class SlowedRotary:
    """Rotary angles whose lower half of the frequencies turns `slow` times slower, on interleaved pairs of the
    first rotary_dim elements of a head: another table for the same kernel."""

    def __init__(self, spec):
        self.spec, self.rotary_dim, self.interleaved = spec, spec.rotary_dim, True

    def angles(self, n_positions):
        half = self.rotary_dim // 2
        inv = 1.0 / self.spec.theta ** (2.0 * np.arange(half) / self.rotary_dim)
        inv[half // 2:] /= self.spec.slow
        return (np.arange(n_positions)[:, None] * inv[None, :]).astype(np.float32)

    def tables(self, n_positions, device):
        a = self.angles(n_positions)
        return torch.from_numpy(np.cos(a)).to(device), torch.from_numpy(np.sin(a)).to(device)


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_are_registered_built_and_stepped():
    """Nothing in the package is changed: a feed-forward that routes each token to one of three experts and a
    position encoding with a table of its own are defined above, registered, put into layers beside the gated
    MLP, and stepped whole, cut and one token at a time, in slots that were used before."""
    from abacus_b200.config import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, NormSpec, ScheduleEntry,
                                    register_architecture)
    from abacus_b200.engine import Engine
    from abacus_b200.models import Model, ModelLayout, expected_tensors
    from abacus_b200.parts import BLOCKS, FEED_FORWARDS, POSITIONS
    from abacus_b200.weights import random_tensors
    FEED_FORWARDS.register("toy_top_one_experts", TopOneExperts)
    POSITIONS.register("toy_slowed_rotary", SlowedRotary)
    d, vocab, hd, rot, heads, eps = 40, 83, 24, 16, 2, 1e-5
    position = SlowedRotarySpec(rotary_dim=rot, theta=100.0, slow=4.0)

    class RoutedArchitecture:
        name = "ToyRoutedForCausalLM"

        def spec(self):
            att = AttentionSpec(hidden=d, n_heads=heads, n_kv_heads=1, head_dim=hd, scale=hd ** -0.5, qk_norm_eps=None,
                                position=position)
            ffns = (TopOneExpertsSpec(d, 24, 3), GatedMLPSpec(d, 56), TopOneExpertsSpec(d, 16, 3))
            blocks = tuple(BlockSpec(NormSpec(d, eps), att, NormSpec(d, eps), ffn) for ffn in ffns)
            return ModelSpec("ToyRoutedForCausalLM", d, vocab, blocks, tuple(ScheduleEntry(i) for i in range(3)),
                             NormSpec(d, eps), True, 200)

        def layout(self, spec):
            layers = [{(pn, slot): f"layers.{l}.{pn}.{slot}" for pn, part in BLOCKS.build(b).parts().items()
                       for slot in part.param_shapes()} for l, b in enumerate(spec.layers)]
            return ModelLayout("embed", "norm", "head", layers)

    arch = register_architecture(RoutedArchitecture())
    spec = arch.spec()
    layout = arch.layout(spec)
    expected, _ = expected_tensors(spec, layout)
    tensors = random_tensors(expected, seed=11, std=0.3, norm_std=0.1)
    engine = Engine(Model(spec, layout, tensors, torch.float32, torch.device("cuda", 0)), max_tokens=64 * 4)
    w = {k: v.float().numpy() for k, v in tensors.items()}

    def rotate(x, cos, sin):  # interleaved pairs (2i, 2i+1) of the first `rot` elements of every head
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        c, s = cos[:, None, :], sin[:, None, :]
        turned = np.stack([a * c - b * s, b * c + a * s], axis=-1).reshape(*x.shape[:-1], rot)
        return np.concatenate([turned, x[..., rot:]], axis=-1).astype(np.float32)

    picks = []

    def plain_routed(ids):
        n = len(ids)
        x = plain.embed(ids, w["embed"])
        angle = SlowedRotary(position).angles(n)
        cos, sin = np.cos(angle), np.sin(angle)
        for l, block in enumerate(spec.layers):
            p = f"layers.{l}."
            xn = plain.rmsnorm(x, w[p + "mixer_norm.weight"], eps)
            q = rotate(plain.linear(xn, w[p + "mixer.wq"]).reshape(n, heads, hd), cos, sin)
            k = rotate(plain.linear(xn, w[p + "mixer.wk"]).reshape(n, 1, hd), cos, sin)
            v = plain.linear(xn, w[p + "mixer.wv"]).reshape(n, 1, hd)
            x = x + plain.linear(plain.attention(q, k, v).reshape(n, heads * hd), w[p + "mixer.wo"])
            xn = plain.rmsnorm(x, w[p + "ffn_norm.weight"], eps)
            if isinstance(block.ffn, TopOneExpertsSpec):
                e, inter = block.ffn.n_experts, block.ffn.inter
                scores = np.stack([plain.softmax(row) for row in plain.linear(xn, w[p + "ffn.router"])])
                y = np.zeros_like(x)
                for t in range(n):
                    c = int(scores[t].argmax())
                    picks.append(c)
                    gate, up = w[p + "ffn.gate"].reshape(e, inter, d)[c], w[p + "ffn.up"].reshape(e, inter, d)[c]
                    gu = np.concatenate([plain.linear(xn[t:t + 1], gate), plain.linear(xn[t:t + 1], up)], -1)
                    y[t] = plain.linear(plain.swiglu(gu), w[p + "ffn.down"].reshape(e, d, inter)[c])[0] * scores[t, c]
                x = x + y
            else:
                gu = np.concatenate([plain.linear(xn, w[p + "ffn.gate"]), plain.linear(xn, w[p + "ffn.up"])], -1)
                x = x + plain.linear(plain.swiglu(gu), w[p + "ffn.down"])
        return plain.linear(plain.rmsnorm(x, w["norm"], eps), w["embed"])

    rng = np.random.default_rng(6)
    seqs = [random_tokens(rng, n, vocab) for n in (26, 7, 40)]
    want = [plain_routed(s) for s in seqs]
    assert len(set(picks)) == 3  # every expert is somebody's
    for round_ in range(2):  # the second round runs in slots the first has used
        slots = [engine.open() for _ in seqs]
        cut = [15, 7, 3]
        got = engine.step([(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
        at = 0
        for i, c in enumerate(cut):
            assert_logits(got[at:at + c], want[i][:c], "float32", f"routed prompt {i}")
            at += c
        engine.close(slots[1])
        live, k = [0, 2], 0
        while live:
            got = engine.step([(slots[i], [seqs[i][cut[i] + k]], [0]) for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                assert_logits(got[j:j + 1], want[i][cut[i] + k:cut[i] + k + 1], "float32", f"routed decode {i}")
            k += 1
            for i in [i for i in live if cut[i] + k == len(seqs[i])]:
                engine.close(slots[i])
            live = [i for i in live if cut[i] + k < len(seqs[i])]
