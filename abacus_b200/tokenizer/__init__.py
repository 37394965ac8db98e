"""Byte-level BPE as Qwen uses it, read straight from a tokenizer.json.

The algorithm is abacus's (src/tokenizer.c): text is cut at added tokens, which are matched
literally (src/tokenizer.c:153-172); the stretches between are split into words by the Qwen
pre-tokenizer rules, followed alternative by alternative (src/tokenizer.c:93-128); a word starts
as single bytes and adjacent pairs are merged, lowest rank first, until no merge applies
(src/tokenizer.c:137-151). abacus reads a digest of tokenizer.json that tools/export.py:54-69
writes into its model file; here the JSON itself is read: model.vocab (pieces in GPT-2's
byte-to-unicode alphabet, tools/export.py:15-25), model.merges ("a b" strings or pairs) and
added_tokens.

Letters and digits are Unicode's (categories L* and N*), where abacus's C code is exact for ASCII
and coarse beyond it (src/tokenizer.c:73-88).
"""
import json
import unicodedata


def _byte_decoder():
    """Printable character -> byte: the inverse of GPT-2's bytes_to_unicode (tools/export.py:15-25)."""
    bs = [*range(ord("!"), ord("~") + 1), *range(ord("¡"), ord("¬") + 1), *range(ord("®"), ord("ÿ") + 1)]
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {chr(c): b for b, c in zip(bs, cs)}


def _is_letter(ch):
    return unicodedata.category(ch).startswith("L")


def _is_digit(ch):
    return unicodedata.category(ch).startswith("N")


def _is_space(ch):
    return ch.isspace()


def _is_other(ch):
    return not (_is_letter(ch) or _is_digit(ch) or _is_space(ch))


def next_word(s, i):
    """End of the word of `s` that starts at i, by the alternatives of
    (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|\\s+(?!\\S)|\\s+
    in order (src/tokenizer.c:93-128)."""
    n = len(s)
    ch = s[i]
    if ch == "'" and i + 1 < n:
        a = s[i + 1].lower()
        b = s[i + 2].lower() if i + 2 < n else ""
        if a in "stmd":
            return i + 2
        if a + b in ("re", "ve", "ll"):
            return i + 3
    j = i
    if not _is_letter(ch) and not _is_digit(ch) and ch not in "\r\n" and i + 1 < n and _is_letter(s[i + 1]):
        j = i + 1
    if _is_letter(s[j]):
        while j < n and _is_letter(s[j]):
            j += 1
        return j
    if _is_digit(ch):
        return i + 1
    j = i + 1 if (ch == " " and i + 1 < n and _is_other(s[i + 1])) else i
    if _is_other(s[j]):
        while j < n and _is_other(s[j]):
            j += 1
        while j < n and s[j] in "\r\n":
            j += 1
        return j
    end = i
    while end < n and _is_space(s[end]):
        end += 1
    for e in range(end - 1, i - 1, -1):  # \s*[\r\n]+ : up to the last newline of the run
        if s[e] in "\r\n":
            return e + 1
    if end < n and end - i > 1:  # \s+(?!\S) : the last space goes with the word that follows
        return end - 1
    return end


class Tokenizer:
    def __init__(self, vocab, merges, added):
        dec = _byte_decoder()
        n_tokens = max([*vocab.values(), *added.values(), -1]) + 1
        self.pieces = [b""] * n_tokens
        for s, i in vocab.items():
            self.pieces[i] = bytes(dec[ch] for ch in s)
        for s, i in added.items():
            self.pieces[i] = s.encode()
        self.added = sorted(added.items(), key=lambda kv: kv[1])  # matched in id order (src/tokenizer.c:153-159)
        self.added_ids = {i for _, i in self.added}
        self.byte_token = {}
        for i, p in enumerate(self.pieces):
            if len(p) == 1 and i not in self.added_ids:
                self.byte_token[p[0]] = i
        self.ranks = {}
        for rank, m in enumerate(merges):
            a, b = m.split(" ") if isinstance(m, str) else m
            if a in vocab and b in vocab and a + b in vocab:
                self.ranks[(vocab[a], vocab[b])] = (rank, vocab[a + b])

    @classmethod
    def from_file(cls, path):
        with open(path, encoding="utf-8") as f:
            tj = json.load(f)
        added = {t["content"]: t["id"] for t in tj.get("added_tokens", [])}
        return cls(tj["model"]["vocab"], tj["model"].get("merges", []), added)

    def stop_ids(self):
        """<|im_end|> and <|endoftext|>, abacus's eos and bos (tools/export.py:88, src/main.c:176)."""
        return [i for s, i in self.added if s in ("<|im_end|>", "<|endoftext|>")]

    def is_special(self, token):
        return token in self.added_ids

    def _match_added(self, text, i):
        for s, tid in self.added:
            if text.startswith(s, i):
                return s, tid
        return None

    def _bpe(self, word):
        out = [self.byte_token[b] for b in word]
        while len(out) > 1:
            best, best_rank, merged = -1, None, None
            for i in range(len(out) - 1):
                hit = self.ranks.get((out[i], out[i + 1]))
                if hit is not None and (best_rank is None or hit[0] < best_rank):
                    best, best_rank, merged = i, hit[0], hit[1]
            if best < 0:
                break
            out[best:best + 2] = [merged]
        return out

    def encode(self, text):
        ids, i, n = [], 0, len(text)
        while i < n:
            hit = self._match_added(text, i)
            if hit:
                ids.append(hit[1])
                i += len(hit[0])
                continue
            stop = i + 1  # the word ends before the next added token (src/tokenizer.c:174-176)
            while stop < n and not self._match_added(text, stop):
                stop += 1
            end = next_word(text[:stop], i)
            ids.extend(self._bpe(text[i:end].encode("utf-8")))
            i = end
        return ids

    def decode(self, ids, skip_special=True):
        """Bytes of the pieces, special tokens left out as abacus's chat loop does (src/main.c:177-180)."""
        data = b"".join(self.pieces[t] for t in ids if 0 <= t < len(self.pieces) and not (skip_special and self.is_special(t)))
        return data.decode("utf-8", errors="replace")
