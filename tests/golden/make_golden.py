#!/usr/bin/env python3
"""Makes tests/golden/tiny<NAME>_abacus.json and .npy: logits of abacus's own engine on tiny random models.

usage: python tests/golden/make_golden.py /path/to/abacus   (the reference's source tree)

abacus's engine compiles here on the CPU (its Makefile's compile line), and its converter
tools/export.py turns a folder with config.json, model.safetensors and a stub tokenizer.json into
its model file. The engine in the tree is int8 in every linear layer (src/model.c:93-103), so its
logits carry quantisation noise: they anchor the architecture (norm placement, per-head norms
before the rotation, the rotation's pairing, the head grouping, tied and untied output matrix), not
the last digits. tests/test_plain.py compares the plain implementation with these logits.
Two tiny configurations are used: A, and B with its vocabulary padded from 389 to 392 (untied head,
groups of 3, a head size decoupled from the width, eps 1e-5, norm weights that are not 1). Every matrix
of these has rows % 8 == 0 and cols % 32 == 0, which the int8 engine needs (src/matmul.c:100-103).
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from helpers import TINY, make_model_folder, weights_digest  # noqa: E402

CASES = {"A": (7, 17), "B392": (8, 40)}  # configuration -> (seed of the token ids, how many)


def main():
    ref = sys.argv[1]
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "abacus")
        srcs = sorted(os.path.join(ref, "src", n) for n in os.listdir(os.path.join(ref, "src")) if n.endswith(".c"))
        subprocess.run(["cc", "-O2", "-march=native", "-std=c11", "-D_GNU_SOURCE", "-pthread", "-o", exe, *srcs, "-lm"],
                       check=True)  # Makefile:13-14
        for name, (seed, count) in CASES.items():
            folder = make_model_folder(tmp, name)
            vocab = TINY[name]["cfg"]["vocab_size"]
            with open(os.path.join(folder, "tokenizer.json"), "w") as f:  # what tools/export.py:54-69, 88 needs
                json.dump({"model": {"vocab": {}, "merges": []},
                           "added_tokens": [{"content": "<|endoftext|>", "id": vocab - 2},
                                            {"content": "<|im_end|>", "id": vocab - 1}]}, f)
            model_bin = os.path.join(tmp, f"{name}.bin")
            subprocess.run([sys.executable, os.path.join(ref, "tools", "export.py"), folder, model_bin], check=True)
            ids = [int(t) for t in np.random.default_rng(seed).integers(0, vocab - 2, count)]
            dump = os.path.join(tmp, "logits.f32")
            subprocess.run([exe, model_bin, "-t", "1", "--ids", " ".join(map(str, ids)), "--dump-logits", dump,
                            "--from", "1", "--chunk", "0"], check=True)  # src/main.c:85-102: positions >= from - 1
            logits = np.fromfile(dump, dtype="<f4").reshape(len(ids), vocab)
            info = subprocess.run([exe, model_bin, "--info"], check=True, capture_output=True, text=True).stdout.strip()
            digest = weights_digest(folder)
            np.save(os.path.join(HERE, f"tiny{name}_abacus.npy"), logits.astype(np.float32))
            with open(os.path.join(HERE, f"tiny{name}_abacus.json"), "w") as f:
                json.dump({"ids": ids, "info": info, "weights_sha256": digest, "config": name}, f)
            print(info, logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
