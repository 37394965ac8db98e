#!/usr/bin/env python3
"""Makes tests/golden/tokenizer_synthetic.json and tokenizer_abacus.json: token ids of abacus's own tokenizer.

usage: python tests/golden/make_tokenizer_golden.py /path/to/abacus   (the reference's source tree)

abacus checks its tokenizer by identical ids (tools/check.py:56-61). Its `--tokenize TEXT` mode
(src/main.c:146-149) needs only a model file, and tools/export.py:54-69 takes any tokenizer.json. So this script
(1) trains a small byte-level BPE (real merges, a few hundred) on a handful of sentences written for the purpose,
in the alphabet of tools/export.py:15-25, and writes it as tokenizer_synthetic.json with the added tokens of a
Qwen chat model; (2) builds abacus, converts tiny configuration A with that tokenizer, and stores the ids abacus
gives for the cases below. tests/test_tokenizer_cli.py holds abacus_b200.tokenizer to these ids.
Cases marked "unicode" are ones where abacus's coarse classes beyond ASCII (src/tokenizer.c:73-88) and Unicode's
own categories part ways on purpose; abacus's ids are stored for them too, and the test says what differs.
"""
import collections
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from abacus_b200.tokenizer import _byte_decoder, next_word  # noqa: E402
from helpers import make_model_folder  # noqa: E402

CORPUS = [
    "The engine reads a folder of weights and writes the next token.",
    "It's not that we don't care; they've said they'll do it, and I'm sure she'd agree.",
    "There were 12 boxes, 340 crates and 5,678 barrels in the harbour on 3 May 2026.",
    "def step(tokens, cache):\n    for t in tokens:\n        cache.append(t)\n    return cache[-1]\n",
    "A table\thas columns\tand rows;   some cells are empty.\r\nThe next line starts here.",
    "Why is the sea salty? Because rivers carry minerals to it, and the water leaves them behind.",
    "the the the and and of of to to in in is is that that it it was was for for on on",
    "Token ids: [1, 2, 3] -> {\"a\": 1.5e-3, \"b\": null} # a comment!",
    "中文的句子没有空格。日本語の文も同じです。한국어 문장은 띄어쓰기가 있습니다.",
    "Élodie a mangé une crêpe à Zürich; señor Núñez pidió café.",
    "Смотри: это кириллица, а это ελληνικά.",
    "emoji 🙂 and 🚀🚀 count as symbols, like © and € and → do.",
    "WE'LL SEE. I'VE HEARD. HE'S GONE. THEY'RE HERE.",
    "   leading spaces, trailing spaces   ",
    "x = y + 1;  // two  spaces   three",
    "The next token is written when the engine has read the weights; the weights are read once.",
    "They said the harbour was empty, but the boxes and the crates were there, and the barrels too.",
    "A sentence with numbers like 2026, 340 and 12, and another sentence with the same numbers: 2026, 340, 12.",
    "return the cache; append the token; for every token in the tokens, append it to the cache.",
]
# Sequences over which abacus's classes and Unicode's differ: learned as whole chunks (split at blanks only), so that
# the vocabulary holds merges that only one way of cutting words can reach.
CROSS = ["\u0663\u0664 \u0663\u0664 \u0663\u0664 \u0663\u0664", "\u5168\u89d2\u3000\u7a7a\u767d \u5168\u89d2\u3000\u7a7a\u767d \u5168\u89d2\u3000\u7a7a\u767d",
         "e\u0301te e\u0301te e\u0301te e\u0301te"]
ADDED = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>"]
N_MERGES = 360

CASES = [
    ("ascii", "Hello, world! The engine writes the next token."),
    ("ascii", "It's not that I don't care; they've said WE'LL see, and she'd agree."),
    ("ascii", "In 2026 there were 12 boxes and 5,678 barrels."),
    ("ascii", "a   b \t c\n\n\nd  \n e"),
    ("ascii", "def f(x):\n    return x[-1] + 1.5e-3  # done"),
    ("ascii", "trailing spaces   "),
    ("ascii", "   leading"),
    ("ascii", "tabs\tand\r\nnew lines"),
    ("ascii", "'s't're've'm'll'd 'S 'x '"),
    ("beyond", "中文的句子没有空格。日本語も。"),
    ("beyond", "Élodie a mangé une crêpe à Zürich."),
    ("beyond", "это кириллица, а это ελληνικά"),
    ("beyond", "emoji 🙂 and 🚀🚀, © and € and →"),
    ("added", "<|im_start|>user\nWhy is the sea salty?<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n"),
    ("added", "text<|endoftext|>more<|im_end|><|im_end|> tail"),
    ("added", "<|im_start|"),
    ("unicode", "\u0663\u0664 apples"),       # Arabic-Indic digits: Unicode N*, abacus counts them as letters
    ("beyond", "\u5168\u89d2\u3000\u7a7a\u767d"),         # U+3000 before letters: white space or symbol, the same word either way
    ("unicode", "éte"),        # a combining accent: Unicode M*, not a letter; abacus counts it as one
]


def train():
    enc = {b: ch for ch, b in _byte_decoder().items()}
    vocab = {enc[b]: b for b in range(256)}
    words = collections.Counter()
    for line in CORPUS:
        i = 0
        while i < len(line):
            j = next_word(line, i)
            words[tuple(enc[b] for b in line[i:j].encode("utf-8"))] += 1
            i = j
    for line in CROSS:
        for chunk in line.split(" "):
            words[tuple(enc[b] for b in chunk.encode("utf-8"))] += 1
    merges = []
    for _ in range(N_MERGES):
        pairs = collections.Counter()
        for w, c in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += c
        if not pairs:
            break
        (a, b), count = min(pairs.items(), key=lambda kv: (-kv[1], kv[0]))
        if count < 2:
            break
        merges.append(f"{a} {b}")
        vocab[a + b] = len(vocab)
        merged = collections.Counter()
        for w, c in words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            merged[tuple(out)] += c
        words = merged
    added = [{"content": s, "id": len(vocab) + 8 + i} for i, s in enumerate(ADDED)]  # a gap of unused ids, as real files have
    return {"model": {"type": "BPE", "vocab": vocab, "merges": merges}, "added_tokens": added}


def main():
    ref = sys.argv[1]
    tj = train()
    with open(os.path.join(HERE, "tokenizer_synthetic.json"), "w", encoding="utf-8") as f:
        json.dump(tj, f, ensure_ascii=True)
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "abacus")
        srcs = sorted(os.path.join(ref, "src", n) for n in os.listdir(os.path.join(ref, "src")) if n.endswith(".c"))
        subprocess.run(["cc", "-O2", "-march=native", "-std=c11", "-D_GNU_SOURCE", "-pthread", "-o", exe, *srcs, "-lm"],
                       check=True)  # Makefile:13-14
        folder = make_model_folder(tmp, "A")
        with open(os.path.join(folder, "tokenizer.json"), "w", encoding="utf-8") as f:
            json.dump(tj, f, ensure_ascii=True)
        model_bin = os.path.join(tmp, "model.bin")
        subprocess.run([sys.executable, os.path.join(ref, "tools", "export.py"), folder, model_bin], check=True)
        cases = []
        for kind, text in CASES:
            out = subprocess.run([exe, model_bin, "--tokenize", text], check=True, capture_output=True, text=True).stdout
            cases.append({"kind": kind, "text": text, "ids": [int(t) for t in out.split()]})
    with open(os.path.join(HERE, "tokenizer_abacus.json"), "w", encoding="utf-8") as f:
        json.dump({"vocab_size": len(tj["model"]["vocab"]), "merges": len(tj["model"]["merges"]), "cases": cases}, f,
                  ensure_ascii=True, indent=0)
    print(len(tj["model"]["vocab"]), "pieces,", len(tj["model"]["merges"]), "merges,", len(cases), "cases")


if __name__ == "__main__":
    main()
