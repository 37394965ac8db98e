"""The tokenizer and the command line's option parsing (CPU), and the command line itself (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from abacus_b200.cli import Options, UsageError, parse
from abacus_b200.tokenizer import Tokenizer, _byte_decoder, next_word
from helpers import ROOT, make_model_folder


def words(text):
    out, i = [], 0
    while i < len(text):
        j = next_word(text, i)
        out.append(text[i:j])
        i = j
    return out


def test_pre_tokenizer_follows_the_qwen_rules():
    """The alternatives of the regex quoted at src/tokenizer.c:61-62, in order."""
    assert words("Hello, world!") == ["Hello", ",", " world", "!"]
    assert words("It's 2026 and I'm") == ["It", "'s", " ", "2", "0", "2", "6", " and", " I", "'m"]
    assert words("a   b") == ["a", "  ", " b"]  # \s+(?!\S) leaves the last space to the word
    assert words("x\n\n\ny") == ["x", "\n\n\n", "y"]
    assert words("tabs\tand\r\nnew") == ["tabs", "\tand", "\r\n", "new"]
    assert words("I'VE we'd've") == ["I", "'VE", " we", "'d", "'ve"]
    assert words("f(x):\n    return") == ["f", "(x", "):\n", "   ", " return"]
    assert words("Café 中文") == ["Café", " 中文"]
    assert words("trailing  ") == ["trailing", "  "]


def tiny_tokenizer(tmp_path):
    enc = {b: ch for ch, b in _byte_decoder().items()}
    vocab = {enc[b]: b for b in range(256)}
    merges = []

    def add(a, b):
        vocab[a + b] = len(vocab)
        merges.append(f"{a} {b}")

    sp = enc[ord(" ")]
    add("l", "l"), add("h", "e"), add("he", "ll"), add("hell", "o"), add(sp, "w"), add("o", "r")
    added = [{"content": "<|endoftext|>", "id": 300}, {"content": "<|im_start|>", "id": 301},
             {"content": "<|im_end|>", "id": 302}]
    path = tmp_path / "tokenizer.json"
    path.write_text(json.dumps({"model": {"vocab": vocab, "merges": merges}, "added_tokens": added}))
    return Tokenizer.from_file(str(path)), vocab


def test_bpe_merges_lowest_rank_first_and_matches_added_tokens(tmp_path):
    tok, vocab = tiny_tokenizer(tmp_path)
    enc = {b: ch for ch, b in _byte_decoder().items()}
    assert tok.encode("hello") == [vocab["hello"]]
    assert tok.encode("hello world") == [vocab["hello"], vocab[enc[32] + "w"], vocab["or"], ord("l"), ord("d")]
    ids = tok.encode("<|im_start|>hello<|im_end|>\n")
    assert ids == [301, vocab["hello"], 302, ord("\n")]
    assert tok.decode(ids) == "hello\n" and tok.decode(ids, skip_special=False) == "<|im_start|>hello<|im_end|>\n"
    assert sorted(tok.stop_ids()) == [300, 302] and tok.is_special(301) and not tok.is_special(5)
    text = "Café → 中文 🙂 it's\t2 b"
    assert tok.decode(tok.encode(text)) == text  # bytes go in, the same bytes come out


def test_token_ids_are_abacus_own(tmp_path):
    """abacus's check begins with identical token ids (tools/check.py:56-61). tests/golden/tokenizer_abacus.json holds
    what abacus's `--tokenize` (src/main.c:146-149) gives with a synthetic vocabulary of real merges
    (tests/golden/make_tokenizer_golden.py): plain ASCII, contractions in both cases, digits, runs of blanks, tabs and
    newlines, code, CJK, accents, Cyrillic and Greek, emoji and symbols, the chat template with its added tokens, an
    added token cut short. Two more cases are ones where this tokenizer follows Unicode's categories and abacus's C
    code its coarse classes (src/tokenizer.c:73-88): digits that are not ASCII are digits here (one to a word, as
    \\p{N} says) and letters there, and a combining accent is no letter here and one there. There the ids differ on
    purpose, and the words say how."""
    golden_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    tok = Tokenizer.from_file(os.path.join(golden_dir, "tokenizer_synthetic.json"))
    with open(os.path.join(golden_dir, "tokenizer_abacus.json")) as f:
        golden = json.load(f)
    assert golden["merges"] >= 150 and len(golden["cases"]) >= 19
    kinds = set()
    for case in golden["cases"]:
        kinds.add(case["kind"])
        ids = tok.encode(case["text"])
        assert tok.decode(ids, skip_special=False) == case["text"]
        if case["kind"] == "unicode":
            assert ids != case["ids"], case["text"]
        else:
            assert ids == case["ids"], case["text"]
    assert kinds == {"ascii", "beyond", "added", "unicode"}
    assert words("\u0663\u0664 apples") == ["\u0663", "\u0664", " apples"]  # \p{N}: one digit a word
    assert words("e\u0301te") == ["e", "\u0301te"]  # the accent is no letter: it ends a word and leads the next


def test_options_keep_abacus_names_and_defaults():
    o = parse(["model"])
    assert (o.steps, o.temp, o.raw, o.prompt, o.top_k) == (512, 0.7, False, "Why is the ocean salty?", 20)  # src/main.c:109-112
    o = parse(["m", "-p", "hi", "-n", "7", "--temp", "0", "--seed", "3", "--raw", "--fp32", "--top-k", "5"])
    assert (o.prompt, o.steps, o.temp, o.seed, o.raw, o.fp32, o.top_k) == ("hi", 7, 0.0, 3, True, True, 5)
    o = parse(["m", "--ids", "1 2 3", "--dump-logits", "f.bin", "--from", "2", "--chunk", "1"])
    assert (o.ids, o.dump, o.start, o.chunk) == ([1, 2, 3], "f.bin", 2, 1)
    o = parse(["m", "--bench", "128", "64", "--batch", "4"])
    assert (o.pp, o.tg, o.batch) == (128, 64, 4)
    for bad in ([], ["-p", "x"], ["m", "--nonsense"], ["m", "-n"], ["m", "--q4"]):
        with pytest.raises(UsageError):
            parse(bad)


@pytest.mark.gpu
def test_command_line_ids_dump_and_info(tmp_path):
    """--info, --ids (greedy ids, as tools/check.py:66-68 uses it) and --dump-logits with --from/--chunk
    (tools/check.py:70-75) against the plain implementation, in true 32-bit."""
    from plain import qwen3_plain as plain
    from helpers import assert_logits
    folder = make_model_folder(tmp_path, "A")
    cfg, w = plain.load(folder)
    exe = [sys.executable, os.path.join(ROOT, "bin", "abacus"), folder, "--fp32"]
    run = lambda *a: subprocess.run([*exe, *a], check=True, capture_output=True, text=True).stdout
    assert run("--info").strip() == "qwen3 dim=64 hidden=128 layers=2 heads=4/2 head_dim=16 vocab=256 weights=f32 kernels=sm_100a"
    ids = [int(t) for t in np.random.default_rng(3).integers(0, 256, 21)]
    text = " ".join(map(str, ids))
    assert [int(t) for t in run("--ids", text, "-n", "9").split()] == plain.generate(cfg, w, ids, 9)
    want = plain.forward(cfg, w, ids)
    for chunk in ("0", "1", "5"):
        path = str(tmp_path / f"dump{chunk}.f32")
        run("--ids", text, "--dump-logits", path, "--from", "12", "--chunk", chunk)
        got = np.fromfile(path, dtype="<f4").reshape(-1, 256)
        assert_logits(got, want[11:], "float32", f"chunk {chunk}")  # positions >= from - 1 (src/main.c:93-96)
