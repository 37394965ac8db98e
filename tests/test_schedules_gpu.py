"""Schedules of steps that the replay tests do not reach, each against the plain implementation: the command
line's text path, a decode that crosses the bound its captured graph was made for, a step that mixes a sequence
bringing many tokens with sequences bringing one, more one-token sequences than the largest captured step
holds, and sequences that go on by several tokens at once."""
import json
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import ROOT, SHARP, TINY, assert_logits, random_tokens
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def folder_of(tmp_path, name, **changes):
    """A model folder of tiny configuration `name` with some keys of its config.json changed."""
    from abacus_b200.config import Qwen3Config
    from abacus_b200.weights import write_random_model
    t = TINY[name]
    raw = dict(t["cfg"], architectures=["Qwen3ForCausalLM"], model_type="qwen3", **changes)
    return write_random_model(os.path.join(str(tmp_path), "m"), Qwen3Config.from_dict(raw), seed=t["seed"],
                              norm_std=t["norm_std"], scales=SHARP)


def test_command_line_text_tokenize_and_bench(tmp_path):
    """`abacus FOLDER -p TEXT`: chat template, tokenizer, generation, pieces printed as they come, special tokens left
    out, the speed line on stderr (src/main.c:165-186); --raw; --tokenize (src/main.c:146-149); --bench (src/main.c:65-82).
    The folder has the synthetic tokenizer of tests/golden/ and a model whose vocabulary holds its ids."""
    from abacus_b200.api import CHAT_TEMPLATE
    from abacus_b200.tokenizer import Tokenizer
    folder = folder_of(tmp_path, "A", vocab_size=460, eos_token_id=459)
    shutil.copy(os.path.join(GOLDEN, "tokenizer_synthetic.json"), os.path.join(folder, "tokenizer.json"))
    tok = Tokenizer.from_file(os.path.join(folder, "tokenizer.json"))
    cfg, w = plain.load(folder)
    stops = sorted(set(tok.stop_ids()) | {459})
    exe = [sys.executable, os.path.join(ROOT, "bin", "abacus"), folder, "--fp32"]

    def run(*args, env=None):
        done = subprocess.run([*exe, *args], check=True, capture_output=True, env=env)
        return done.stdout.decode("utf-8", errors="replace"), done.stderr.decode()

    text = "Why is the sea salty?"
    for raw in (False, True):
        ids = tok.encode(text if raw else CHAT_TEMPLATE.format(text))
        want = plain.generate(cfg, w, ids, 12, stop=stops)
        out, err = run("-p", text, "--temp", "0", "-n", "12", *(["--raw"] if raw else []))
        assert out == tok.decode(want), (raw, out, want)
        assert f"prompt {len(ids)} tokens, " in err and f"| generated {len(want)} tokens, " in err and "tok/s" in err
    # sampled: the same seed draws the same text, and what request 0 draws is what abacus's loop would (src/main.c:52)
    ids = tok.encode(CHAT_TEMPLATE.format(text))
    want = plain.generate(cfg, w, ids, 10, temp=0.9, seed=11, stop=stops)
    assert run("-p", text, "--temp", "0.9", "--seed", "11", "-n", "10")[0] == tok.decode(want)
    out, _ = run("--tokenize", "It's 2026, and the engine writes <|im_end|> tokens.")
    assert [int(t) for t in out.split()] == tok.encode("It's 2026, and the engine writes <|im_end|> tokens.")
    # the switches: no captured prompt steps, no captured steps' C walker; the same ids either way
    ids = " ".join(str(t) for t in tok.encode(CHAT_TEMPLATE.format(text)))
    plain_ids = " ".join(str(t) for t in plain.generate(cfg, w, [int(t) for t in ids.split()], 9))
    for switch in ({}, {"ABACUS_PROMPT_GRAPHS": "0"}, {"ABACUS_C_STEP": "0"}, {"ABACUS_PROMPT_GRAPHS": "0", "ABACUS_C_STEP": "0"}):
        assert run("--ids", ids, "-n", "9", env=dict(os.environ, **switch))[0].strip() == plain_ids, switch
    res = json.loads(run("--bench", "64", "8", "--batch", "3")[0])
    assert res["pp"] == 64 and res["tg"] == 8 and res["batch"] == 3 and res["prefill_tok_s"] > 0 and res["decode_tok_s"] > 0


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("D", "bfloat16")])
def test_decode_across_the_bound_of_a_captured_graph(tmp_path, name, dtype):
    """A decode graph is captured for positions below a bound that goes in steps of 1,024. A sequence that decodes
    from position 1,015 to 1,035 leaves one graph and enters the next in the middle of a request."""
    from abacus_b200.engine import Engine, load_model
    from abacus_b200.engine.graphs import POSITION_STEP
    folder = folder_of(tmp_path, name, max_position_embeddings=1152)
    cfg, w = plain.load(folder)
    rng = np.random.default_rng(5)
    first, last = POSITION_STEP - 9, POSITION_STEP + 11
    ids = [random_tokens(rng, last + 1, cfg["vocab"]), random_tokens(rng, last + 1 - 400, cfg["vocab"])]
    rnd = plain.bf16_round if dtype == "bfloat16" else None
    exact = [plain.forward(cfg, w, t) for t in ids]
    want = [plain.forward(cfg, w, t, rnd=rnd) if rnd else e for t, e in zip(ids, exact)]
    noise = [float(np.abs(a - e).max()) if rnd else float(np.abs(e - plain.forward64(cfg, w, t)).max())
             for a, e, t in zip(want, exact, ids)]
    engine = Engine(load_model(folder, dtype), max_tokens=2 * 1152)
    slots = [engine.open(), engine.open()]
    starts = [first, first - 400]  # the second sequence is 400 positions behind: it stays below the bound
    got = engine.step([(s, t[:n], [n - 1]) for s, t, n in zip(slots, ids, starts)]).cpu().numpy()
    for i in range(2):
        assert_logits(got[i:i + 1], want[i][starts[i] - 1:starts[i]], dtype, f"prompt {i}", noise[i])
    bounds = set()
    for k in range(last - first + 1):
        got = engine.step([(s, [t[n + k]], [0]) for s, t, n in zip(slots, ids, starts)]).cpu().numpy()
        bounds.add(engine.last_batch.position_bound)
        for i in range(2):
            assert_logits(got[i:i + 1], want[i][starts[i] + k:starts[i] + k + 1], dtype, f"decode {k} of {i}", noise[i])
    assert len(bounds) == 2, bounds  # two graphs served the request
    engine.check_status()


@pytest.mark.parametrize("name, dtype", [("B", "float32"), ("D", "bfloat16"), ("A", "bfloat16")])
def test_steps_that_mix_many_tokens_with_single_ones_and_go_on_by_several(tmp_path, name, dtype):
    """After their prompts, one sequence brings 30 tokens beside two that bring one; then all three go on by several
    tokens each (5, 1, 17), twice, so that the second time the step's shape is replayed from a captured graph."""
    from abacus_b200.engine import Engine, load_model
    folder = folder_of(tmp_path, name)
    cfg, w = plain.load(folder)
    rng = np.random.default_rng(8)
    prompts, more = [40, 70, 9], [[30, 5, 5], [1, 1, 1], [1, 17, 17]]
    ids = [random_tokens(rng, p + sum(m), cfg["vocab"]) for p, m in zip(prompts, more)]
    rnd = plain.bf16_round if dtype == "bfloat16" else None
    exact = [plain.forward(cfg, w, t) for t in ids]
    want = [plain.forward(cfg, w, t, rnd=rnd) if rnd else e for t, e in zip(ids, exact)]
    noise = [float(np.abs(a - e).max()) if rnd else float(np.abs(e - plain.forward64(cfg, w, t)).max())
             for a, e, t in zip(want, exact, ids)]
    engine = Engine(load_model(folder, dtype), max_tokens=64 * 8)
    slots = [engine.open() for _ in ids]
    at = [0, 0, 0]
    for counts in [prompts] + [list(c) for c in zip(*more)]:
        entries = [(s, t[a:a + n], list(range(n))) for s, t, a, n in zip(slots, ids, at, counts)]
        got = engine.step(entries).cpu().numpy()
        row = 0
        for i, n in enumerate(counts):
            assert_logits(got[row:row + n], want[i][at[i]:at[i] + n], dtype, f"sequence {i} at {at[i]} + {n}", noise[i])
            row += n
            at[i] += n
    engine.check_status()
    assert engine.prompt_graphs is None or engine.prompt_graphs.replayed >= 1


def test_more_single_token_sequences_than_a_captured_step_holds(tmp_path):
    """300 sequences of one token each in one step, then a second token each: beyond the largest captured decode step
    (256 rows), so the step runs as it is."""
    from abacus_b200.engine import Engine, load_model
    folder = folder_of(tmp_path, "A")
    cfg, w = plain.load(folder)
    rng = np.random.default_rng(9)
    n = 300
    ids = [random_tokens(rng, 2, cfg["vocab"]) for _ in range(n)]
    from abacus_b200.engine.graphs import row_bucket
    assert row_bucket(n) is None
    exact = np.stack([plain.forward(cfg, w, t) for t in ids])  # [n, 2, vocab]
    for dtype in ("float32", "bfloat16"):
        engine = Engine(load_model(folder, dtype), max_tokens=64 * n, max_slots=n)
        slots = [engine.open() for _ in range(n)]
        if dtype == "bfloat16":
            want = np.stack([plain.forward(cfg, w, t, rnd=plain.bf16_round) for t in ids])
            noise = float(np.abs(want - exact).max())
        else:
            want = exact
            noise = max(float(np.abs(e - plain.forward64(cfg, w, t)).max()) for e, t in zip(exact, ids))
        for k in range(2):
            got = engine.step([(s, [t[k]], [0]) for s, t in zip(slots, ids)]).cpu().numpy()
            assert got.shape == (n, cfg["vocab"])
            assert_logits(got, want[:, k], dtype, f"{dtype} token {k}", noise=noise)
        for s in slots:
            engine.close(s)
        engine.check_status()


def test_a_wait_that_runs_out_becomes_an_exception_and_the_engine_goes_on(tmp_path):
    """Every wait of a kernel on a barrier is bounded; when one runs out the kernel sets a status word and returns, and
    Engine.check_status() turns the word into an exception. Here a kernel whose only wait nothing can satisfy (a barrier
    that expects bytes nobody sends) is given a limit of two milliseconds: it returns, the word is set, check_status
    raises and clears it, and the next step gives the logits it gave before. Nothing faults and nothing hangs."""
    import time

    import torch
    from abacus_b200.engine import Engine, load_model
    from abacus_b200.kernels import ops
    folder = folder_of(tmp_path, "D")
    engine = Engine(load_model(folder, "bfloat16"), max_tokens=256)
    tokens = random_tokens(np.random.default_rng(1), 70, TINY["D"]["cfg"]["vocab_size"])
    slot = engine.open()
    before = engine.step([(slot, tokens, [69])]).cpu().numpy()
    engine.close(slot)
    engine.check_status()
    ops.set_wait_limit_ns(2_000_000)
    try:
        start = time.perf_counter()
        ops.wait_that_runs_out(ops.kernel_status(torch.device("cuda", 0)))
        torch.cuda.synchronize()
        assert time.perf_counter() - start < 0.2  # two milliseconds, not the quarter of a second of the default
    finally:
        ops.set_wait_limit_ns(250_000_000)
    with pytest.raises(RuntimeError, match="a wait that ran out"):
        engine.check_status()
    engine.check_status()  # the words were cleared
    slot = engine.open()
    again = engine.step([(slot, tokens, [69])]).cpu().numpy()
    engine.close(slot)
    engine.check_status()
    assert np.array_equal(before, again)


@pytest.mark.parametrize("name, dtype", [("B", "float32"), ("C", "float32"), ("C2", "bfloat16"), ("D", "bfloat16"), ("A", "bfloat16")])
def test_the_step_function_in_c_launches_what_the_parts_would(tmp_path, name, dtype):
    """A step is one call to the C walker (csrc/step.cu) where the model is made of the library's own parts, and a walk
    through the parts' forward() otherwise. Both must pick the same kernels with the same arguments: prompts of unequal
    lengths, a continuation by several tokens and decode steps give the same bits either way, with and without
    captured graphs. (A windowed layer refuses the continuation on both ways, with the same words.)"""
    from abacus_b200.engine import Engine, load_model
    from abacus_b200.kernels import ops
    folder = folder_of(tmp_path, name)
    model = load_model(folder, dtype)
    rng = np.random.default_rng(4)
    vocab = TINY[name]["cfg"]["vocab_size"]
    prompts = [random_tokens(rng, n, vocab) for n in (70, 3, 131)]
    more = [random_tokens(rng, n, vocab) for n in (9, 2, 1)]
    windowed = any(t == "sliding_attention" for t in TINY[name]["cfg"].get("layer_types", []))

    def run(engine):
        out, slots = [], [engine.open() for _ in prompts]  # (a step's logits live in the workspace: copied at once)
        out.append(engine.step([(s, p, [0, len(p) - 1]) for s, p in zip(slots, prompts)]).clone())
        try:
            out.append(engine.step([(s, m, list(range(len(m)))) for s, m in zip(slots, more)]).clone())
        except ops.KernelRefused as e:
            assert windowed and "windowed attention" in str(e)
            for s in slots:  # what the refused step reserved stays reserved: start over in fresh slots
                engine.close(s)
            slots = [engine.open() for _ in prompts]
            out.append(engine.step([(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).clone())
        for k in range(3):
            out.append(engine.step([(s, [int(t)], [0]) for s, t in zip(slots, rng_tokens[k])]).clone())
        for s in slots:
            engine.close(s)
        engine.check_status()
        return out

    rng_tokens = [random_tokens(rng, 3, vocab) for _ in range(3)]
    results = []
    for use_graphs in (False, True):
        for c_step in (True, False):
            engine = Engine(model, max_tokens=64 * 9, use_graphs=use_graphs)
            assert engine.cstep is not None
            if not c_step:
                engine.cstep = None
            results.append(run(engine) + (run(engine) if use_graphs else []))  # twice: the second time from captured graphs
    for other in results[1:]:
        for a, b in zip(results[0], other):
            assert torch.equal(a, b)



def test_preparing_q_k_v_in_the_neighbouring_kernels_changes_no_bit(tmp_path, monkeypatch):
    """In bfloat16 the step between the q/k/v product and attention (per-head norm, rotation, cache write) runs in the
    product's epilogue for long prompt steps and inside the attention kernel for decode steps. With both switched off
    it is a kernel of its own. Prompts of 300 and 281 tokens, a continuation by 270 and 1 tokens and decode steps give
    the same bits either way, through the C walker and through the parts."""
    from abacus_b200.engine import Engine, cstep, load_model
    from abacus_b200.kernels import ops
    from abacus_b200.parts import attention
    folder = folder_of(tmp_path, "D")
    model = load_model(folder, "bfloat16")
    rng = np.random.default_rng(6)
    vocab = TINY["D"]["cfg"]["vocab_size"]
    prompts = [random_tokens(rng, n, vocab) for n in (300, 281)]
    more = [random_tokens(rng, n, vocab) for n in (270, 1)]
    single = [random_tokens(rng, 2, vocab) for _ in range(4)]

    def run(engine):
        out, slots = [], [engine.open() for _ in prompts]
        out.append(engine.step([(s, p, [0, len(p) - 1]) for s, p in zip(slots, prompts)]).clone())
        out.append(engine.step([(s, m, [len(m) - 1]) for s, m in zip(slots, more)]).clone())
        for k in range(4):
            out.append(engine.step([(s, [int(t)], [0]) for s, t in zip(slots, single[k])]).clone())
        for s in slots:
            engine.close(s)
        engine.check_status()
        return out

    results, launches = [], []
    for fused in (True, False):
        for module in (attention, cstep):
            monkeypatch.setattr(module, "DECODE_PREPARES", fused)
            monkeypatch.setattr(module, "PRODUCT_PREPARES", fused)
        for c_step in (True, False):
            engine = Engine(model, max_tokens=64 * 24, use_graphs=False)
            if not c_step:
                engine.cstep = None
            before = ops.LAUNCHES
            results.append(run(engine))
            launches.append(ops.LAUNCHES - before)
    for other in results[1:]:
        for a, b in zip(results[0], other):
            assert torch.equal(a, b)
    # the preparation's own kernel is one launch more per layer and step: 2 layers x 6 steps
    assert launches[0] == launches[1] and launches[2] == launches[3] == launches[0] + 2 * 6, launches
