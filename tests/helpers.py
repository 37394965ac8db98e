"""Shared by the tests: the tiny configurations, model folders in temporary places, a driver for
bin/trace_run, and the comparison rules."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Four tiny configurations of the architecture that differ in every size and option.
#   A: the first measured configuration in small (tied head, group of 2, norm weights 1).
#   B: the second in small (untied head, group of 3, head size decoupled from the width, prime vocabulary).
#   C: one kv head per query head, head size 48, a window of 24 keys on every other layer.
TINY = {
    "A": dict(cfg=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, vocab_size=256, max_position_embeddings=512,
                       rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
              seed=0, norm_std=0.0),
    "B": dict(cfg=dict(hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=6,
                       num_key_value_heads=2, head_dim=32, vocab_size=389, max_position_embeddings=384,
                       rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
              seed=1, norm_std=0.1),
    "C": dict(cfg=dict(hidden_size=80, intermediate_size=112, num_hidden_layers=4, num_attention_heads=5,
                       num_key_value_heads=5, head_dim=48, vocab_size=300, max_position_embeddings=448,
                       rope_theta=500000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
                       layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
                       sliding_window=24, use_sliding_window=True),
              seed=2, norm_std=0.05),
    # D: the head size (128) and group (2) of the Qwen3 checkpoints, which the faster bfloat16 kernels take
    "D": dict(cfg=dict(hidden_size=192, intermediate_size=272, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=128, vocab_size=515, max_position_embeddings=640,
                       rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
              seed=3, norm_std=0.02),
}
# C's first two layers (one with all keys, one windowed). The bfloat16 replay uses this one: engine and plain model
# round the same tensors at the same places, but float32 sums taken in another order flip the rounding of about one
# stored value in three thousand, a flipped value flips about a twentieth of the next tensor's row, and from the third
# layer on the two are independent roundings of the same model whose distance measures bfloat16, not the engine.
# Measured over 8 weight seeds each: every replay passes at two layers, 7 of 8 at three, 4 or 5 of 8 at four, with
# or without windows and with either attention kernel. The four layers stay where they say something: in float32.
TINY["C2"] = dict(TINY["C"], cfg=dict(TINY["C"]["cfg"], num_hidden_layers=2,
                                      layer_types=["full_attention", "sliding_attention"]))
# B with its vocabulary padded to a multiple of 8, which abacus's int8 engine needs of every matrix
# (src/matmul.c:100-103): the form of B that abacus itself can load (tests/golden/).
TINY["B392"] = dict(TINY["B"], cfg=dict(TINY["B"]["cfg"], vocab_size=392))
# Random N(0, 0.02) weights give nearly flat attention, in which a lost key changes little. These
# factors on the q/k norm weights and on the value/output matrices make scores a few units wide
# and the logits of order one, so that one wrong key, position or slot shows in the logits.
SHARP = {"q_norm": 2.5, "k_norm": 2.5, "v_proj": 4.0, "o_proj": 4.0, "down_proj": 3.0, "embed_tokens": 8.0,
         "lm_head": 8.0}


def tiny_config(name):
    from abacus_b200.config import Qwen3Config
    raw = dict(TINY[name]["cfg"], architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    return Qwen3Config.from_dict(raw)


def make_model_folder(tmp, name, scales=SHARP):
    """Write config.json and model.safetensors of tiny configuration `name` under tmp; returns the folder."""
    from abacus_b200.weights import write_random_model
    folder = os.path.join(str(tmp), f"tiny{name}")
    t = TINY[name]
    write_random_model(folder, tiny_config(name), seed=t["seed"], norm_std=t["norm_std"], scales=scales)
    return folder


def weights_digest(folder):
    """A hash of a model folder's tensors by name, whatever order the file keeps them in."""
    import hashlib
    from plain import qwen3_plain as plain
    h = hashlib.sha256()
    for name, t in sorted(plain.read_safetensors(os.path.join(folder, "model.safetensors")).items()):
        h.update(name.encode() + str(t.shape).encode() + np.ascontiguousarray(t).tobytes())
    return h.hexdigest()


def random_tokens(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, n)]


class TraceRun:
    """bin/trace_run as a child process: one step in, wait for "done", read the logits file."""

    def __init__(self, model, dtype, out, max_tokens, env=None):
        self.out = str(out)
        self.proc = subprocess.Popen(
            [sys.executable, TRACE_RUN, "--model", model, "--dtype", dtype, "--out", self.out, "--max-tokens",
             str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.n = 0

    def step(self, entries, end=()):
        """entries: [(id, tokens, want)]. Returns float32 [wanted, vocab] or None."""
        sid = self.n
        self.n += 1
        line = json.dumps({"step": sid, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w in entries],
                           "end": list(end)})
        self.proc.stdin.write(line + "\n")
        self.proc.stdin.flush()
        reply = self.proc.stdout.readline().strip()
        if reply != f"done {sid}":
            self.proc.stdin.close()
            self.proc.wait()
            raise RuntimeError(f"trace_run answered {reply!r} to step {sid} (exit {self.proc.returncode})")
        path = os.path.join(self.out, f"{sid}.f32")
        if not any(w for _, _, w in entries):
            assert not os.path.exists(path)
            return None
        return np.fromfile(path, dtype="<f4")

    def close(self):
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        assert code == 0, f"trace_run exited with {code}"


# ------------------------------------------------------------------ comparison rules
# float32: the engine and the plain implementation do the same float32 arithmetic in different
# orders. Their distance is bounded by a small absolute/relative term plus the rounding noise that
# float32 itself shows on that input: `noise` = max |plain float32 - plain float64|. The sharpened
# weights above amplify rounding (measured: up to 1.4e-4 on four-layer configuration C), and a
# limit below the reference's own noise would test nothing but luck.
F32_ATOL, F32_RTOL, F32_NOISE = 5e-5, 5e-5, 3.0
# bfloat16: against the plain implementation with its stored tensors rounded to bfloat16 at the
# same places. What is left is single-ulp rounding flips and their propagation, a fraction of
# the rounding noise of bfloat16 itself: `noise` = max |plain with bfloat16 storage - plain float32|
# (measured: 0.2 to 1.3 on logits of scale 6 to 7). The limit is 2 % of the largest logit or a
# quarter of that noise, whichever is larger, and a small KL divergence.
BF16_REL_MAX, BF16_NOISE, BF16_KL = 0.02, 0.25, 2e-3


def log_softmax64(x):
    x = x.astype(np.float64)
    x = x - x.max(axis=-1, keepdims=True)
    return x - np.log(np.exp(x).sum(axis=-1, keepdims=True))


def assert_logits(got, want, dtype, what="", noise=0.0):
    got, want = np.asarray(got, dtype=np.float32), np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: logits are not finite"
    diff = np.abs(got - want)
    if dtype == "float32":
        bad = diff > F32_ATOL + F32_RTOL * np.abs(want) + F32_NOISE * noise
        assert not bad.any(), (f"{what}: float32 logits differ by up to {diff.max():.3g} "
                               f"(first bad row {np.argwhere(bad)[0][0]} of {got.shape[0]}, noise {noise:.3g})")
    else:
        scale = np.abs(want).max()
        limit = max(BF16_REL_MAX * scale, BF16_NOISE * noise)
        rows = diff.max(axis=-1)
        assert rows.max() <= limit, (f"{what}: bfloat16 logits differ by {rows.max():.3g} at row {rows.argmax()} "
                                     f"(limit {limit:.3g}, scale {scale:.3g}, noise {noise:.3g})")
        lp, lq = log_softmax64(want), log_softmax64(got)
        kl = (np.exp(lp) * (lp - lq)).sum(-1)
        assert kl.max() <= BF16_KL, f"{what}: KL {kl.max():.3g} at row {kl.argmax()} (limit {BF16_KL})"
