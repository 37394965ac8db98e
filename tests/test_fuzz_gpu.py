"""Random configurations, random batches and random cuts: the engine against the plain implementation.

The other tests run four hand-made configurations. Here a seeded generator draws forty more (head sizes 16
to 256, one to four kv heads with groups of one to seven, widths, inner sizes and vocabularies that are no
powers of two, one or two layers, tied and untied heads, windows on every other layer), each with a batch
of one to five prompts of unequal lengths followed by a few decode steps in which the shorter requests end
earlier. Every case runs twice in the same engine, so that slots, pages and captured step shapes come
round again. Both dtypes; the bounds are those of helpers.assert_logits, unchanged.

Why no deeper models here. In bfloat16 the engine and the plain model round the same tensors at the same
places, and the probabilities of the second product to the same bits (a reference that is a whole power
of two, see plain.attention). What is left are float32 sums taken in another order, which flip the
rounding of about one stored value in three thousand; one flipped value of a row flips about a twentieth
of the next stored tensor's values in that row (measured on one-layer models). After two layers most
values have met a flip, engine and plain model are two independent roundings of the same model, and their
distance measures bfloat16, not the engine: with three layers 4 of 4,000 comparisons lay over the bound
(by up to 1.8), with one or two layers none of 8,000. A fault of the cache, a batch or a kernel's edge
shows at any depth; depth itself is what the replay tests' four-layer configuration is for.
"""
import os
import tempfile

import numpy as np
import pytest

from helpers import SHARP, assert_logits, random_tokens
from plain import qwen3_plain as plain

N_CASES = 40
PROMPT_LENGTHS = [1, 2, 5, 33, 64, 65, 130, 200, 300]


def draw_case(index):
    """(config.json contents, dtype, weight seed, prompt lengths, decode steps per request, rng) of case `index`."""
    rng = np.random.default_rng(7000 + index)
    hd = int(rng.choice([16, 32, 48, 64, 64, 80, 128, 128, 128, 256]))
    kvh = int(rng.choice([1, 2, 3, 4]))
    group = int(rng.choice([1, 2, 3, 4, 7]))
    layers = int(rng.choice([1, 2, 2]))
    cfg = dict(hidden_size=int(rng.choice([64, 96, 136, 192, 264])), intermediate_size=int(rng.choice([128, 104, 256, 272, 384])),
               num_hidden_layers=layers, num_attention_heads=kvh * group, num_key_value_heads=kvh, head_dim=hd,
               vocab_size=int(rng.choice([256, 389, 515, 1000, 2311])), max_position_embeddings=1024,
               rope_theta=float(rng.choice([1e4, 1e6])), rms_norm_eps=float(rng.choice([1e-6, 1e-5])),
               tie_word_embeddings=bool(rng.integers(0, 2)), architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    if rng.random() < 0.25 and layers >= 2:
        cfg.update(layer_types=[("sliding_attention" if i % 2 else "full_attention") for i in range(layers)],
                   sliding_window=int(rng.choice([24, 64, 100])), use_sliding_window=True)
    dtype = "bfloat16" if index % 3 else "float32"
    n_req = int(rng.integers(1, 6))
    lengths = [int(rng.choice(PROMPT_LENGTHS)) for _ in range(n_req)]
    decode = [int(rng.integers(0, 10)) for _ in range(n_req)]
    return cfg, dtype, int(rng.integers(0, 1000)), lengths, decode, rng


def run_case(index):
    """Runs case `index`; returns the list of comparisons that failed (as text)."""
    import torch
    from abacus_b200.config import Qwen3Config
    from abacus_b200.engine import Engine, load_model
    from abacus_b200.weights import write_random_model
    cfg, dtype, weight_seed, lengths, decode, rng = draw_case(index)
    what = (f"case {index}: head {cfg['head_dim']} heads {cfg['num_attention_heads']}/{cfg['num_key_value_heads']} "
            f"width {cfg['hidden_size']} inner {cfg['intermediate_size']} layers {cfg['num_hidden_layers']} "
            f"vocab {cfg['vocab_size']} window {cfg.get('sliding_window')} {dtype} prompts {lengths} decode {decode}")
    failures = []
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(os.path.join(tmp, "m"), Qwen3Config.from_dict(cfg), seed=weight_seed, norm_std=0.05,
                                    scales=SHARP)
        pcfg, pw = plain.load(folder)
        engine = Engine(load_model(folder, dtype), max_tokens=sum(-(-(n + d) // 64) * 64 for n, d in zip(lengths, decode)))
    rnd = plain.bf16_round if dtype == "bfloat16" else None

    def compare(got, want, noise, where):
        try:
            assert_logits(got, want, dtype, where, noise)
        except AssertionError as e:
            failures.append(f"{what} :: {e}")

    for repeat in range(2):
        ids = [random_tokens(rng, n + d, cfg["vocab_size"]) for n, d in zip(lengths, decode)]
        exact = [plain.forward(pcfg, pw, t) for t in ids]
        want = [plain.forward(pcfg, pw, t, rnd=rnd) if rnd else e for t, e in zip(ids, exact)]
        noise = [float(np.abs(w - e).max()) if rnd else float(np.abs(e - plain.forward64(pcfg, pw, t)).max())
                 for w, e, t in zip(want, exact, ids)]
        slots = [engine.open() for _ in ids]
        got = engine.step([(s, t[:n], [0, n - 1]) for s, t, n in zip(slots, ids, lengths)]).cpu().numpy()
        for i, n in enumerate(lengths):
            compare(got[2 * i:2 * i + 2], want[i][[0, n - 1]], noise[i], f"round {repeat} prompt {i}")
        for step in range(max(decode)):
            live = [i for i in range(len(ids)) if step < decode[i]]
            entries = [(slots[i], ids[i][lengths[i] + step:lengths[i] + step + 1], [0]) for i in live]
            got = engine.step(entries).cpu().numpy()
            for j, i in enumerate(live):
                compare(got[j:j + 1], want[i][lengths[i] + step:lengths[i] + step + 1], noise[i],
                        f"round {repeat} request {i} decode step {step}")
            for i in live:
                if step == decode[i] - 1:
                    engine.close(slots[i])
                    slots[i] = None
        for s in slots:
            if s is not None:
                engine.close(s)
    engine.check_status()
    del engine
    torch.cuda.empty_cache()
    return failures


@pytest.mark.gpu
def test_random_configurations_batches_and_cuts():
    failures = []
    for index in range(N_CASES):
        failures += run_case(index)
    assert not failures, f"{len(failures)} comparisons outside the bounds:\n" + "\n".join(failures[:20])
