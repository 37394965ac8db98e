"""The command line, in abacus's own manner (src/main.c:9-23, 104-189).

    abacus MODEL [options]

MODEL is a folder with config.json, *.safetensors and, for text, tokenizer.json (abacus takes the
model.bin its converter makes of such a folder). Options keep abacus's names and meanings; -t and
--q4 have nothing to do here (GPU; no quantized weights) and say so. New: --fp32, --top-k, --batch.
"""
import json
import sys
import time

USAGE = """usage: abacus MODEL [options]
  -p TEXT          prompt, wrapped in the chat template (default: a question)
  -n N             tokens to generate (default 512)
  --temp T         sampling temperature, 0 = greedy (default 0.7)
  --seed S         sampling seed
  --raw            continue the prompt as plain text, no chat template
  --bench PP TG    time a PP-token prefill and a TG-token decode, print JSON
  --tokenize TEXT  print token ids
  --ids "1 2 3"    start from token ids; prints N greedy token ids
  --dump-logits F  with --ids: write float32 logits for positions >= --from K - 1,
                   feeding the ids in chunks of --chunk C (default: all at once)
  --info           print the model shape and weight format
  --fp32           run everything in true 32-bit floating point (default: bfloat16)
  --top-k K        sample among the K most likely tokens (default 20, at most 64; 0: all tokens)
  --batch B        with --bench: B sequences at once (default 1)
  -t N, --q4       abacus's CPU threads and 4-bit weights: not built here
"""


class Options:
    def __init__(self):
        self.model = None
        self.prompt = "Why is the ocean salty?"  # src/main.c:109
        self.steps, self.temp, self.seed = 512, 0.7, int(time.time())  # src/main.c:110-112
        self.raw = self.info = self.fp32 = False
        self.pp = self.tg = 0
        self.text = self.ids = self.dump = None
        self.start, self.chunk, self.top_k, self.batch = 1, 0, 20, 1


class UsageError(Exception):
    pass


def parse(argv):
    """argv without the program name -> Options (the hand-rolled loop of src/main.c:113-134)."""
    if not argv or argv[0].startswith("-"):
        raise UsageError(USAGE)
    o = Options()
    o.model = argv[0]
    i = 1
    while i < len(argv):
        a = argv[i]
        more = i + 1 < len(argv)

        def value():
            nonlocal i
            i += 1
            return argv[i]

        if a == "-p" and more:
            o.prompt = value()
        elif a == "-n" and more:
            o.steps = int(value())
        elif a == "-t" and more:
            value()
            print("abacus: -t is ignored (the work runs on the GPU)", file=sys.stderr)
        elif a == "--temp" and more:
            o.temp = float(value())
        elif a == "--seed" and more:
            o.seed = int(value())
        elif a == "--raw":
            o.raw = True
        elif a == "--q4":
            raise UsageError("abacus: --q4: quantized weights are not built\n")
        elif a == "--bench" and i + 2 < len(argv):
            o.pp, o.tg = int(value()), int(value())
        elif a == "--tokenize" and more:
            o.text = value()
        elif a == "--ids" and more:
            o.ids = [int(t) for t in value().split()]
        elif a == "--dump-logits" and more:
            o.dump = value()
        elif a == "--from" and more:
            o.start = int(value())
        elif a == "--chunk" and more:
            o.chunk = int(value())
        elif a == "--info":
            o.info = True
        elif a == "--fp32":
            o.fp32 = True
        elif a == "--top-k" and more:
            o.top_k = int(value())
        elif a == "--batch" and more:
            o.batch = int(value())
        else:
            raise UsageError(USAGE)
        i += 1
    return o


def info_line(model):
    """abacus's --info line (src/main.c:143-145): the architecture says what it is called and which sizes it shows;
    tools/check.py:52-53 keys its rule on the weights= word."""
    import torch
    from .config.registry import get_architecture
    weights = "f32" if model.ctx.dtype == torch.float32 else "bf16"
    return f"{get_architecture(model.spec.architecture).info(model.spec)} weights={weights} kernels=sm_100a"


def dump_logits(lm, ids, start, chunk, path):
    """Teacher forcing (src/main.c:85-102): run the ids in chunks and write the logits that predict ids[start..]."""
    engine = lm.engine
    slot = engine.open()
    n = len(ids)
    chunk = chunk if chunk > 0 else n
    with open(path, "wb") as f:
        for pos in range(0, n, chunk):
            part = ids[pos:pos + chunk]
            first = max(pos, start - 1)
            want = list(range(first - pos, len(part))) if first < pos + len(part) else []
            logits = engine.step([(slot, part, want)])
            if want:
                f.write(logits.cpu().numpy().astype("<f4").tobytes())
    engine.close(slot)


def bench(lm, pp, tg, batch):
    """abacus's --bench (src/main.c:65-82): its token pattern, a warm-up, a timed prefill, timed greedy steps.
    abacus restarts at position 0 for the decode; here the decode follows the prompt."""
    import torch
    from .sampling import Sampler
    engine, vocab = lm.engine, lm.model.spec.vocab
    tokens = [(1000 + 37 * i % 50000) % vocab for i in range(max(pp, 16))]
    warm = engine.open()
    engine.step([(warm, tokens[:16], [15])])
    engine.close(warm)
    slots = [engine.open() for _ in range(batch)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    logits = engine.step([(s, tokens[:pp], [pp - 1]) for s in slots])
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    sampler = Sampler(lm.model.ctx.device, temperature=0.0)
    for _ in range(tg):
        nxt = sampler.sample(logits, None).tolist()
        logits = engine.step([(s, [t], [0]) for s, t in zip(slots, nxt)])
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    for s in slots:
        engine.close(s)
    return {"prefill_tok_s": round(batch * pp / (t1 - t0), 3), "decode_tok_s": round(batch * tg / (t2 - t1), 3),
            "pp": pp, "tg": tg, "batch": batch}


def main(argv=None):
    try:
        o = parse(sys.argv[1:] if argv is None else argv)
    except UsageError as e:
        sys.stderr.write(str(e))
        return 1
    from .api import LM
    need = max(o.pp + o.tg + 64, 4096) * max(o.batch, 1) if (o.pp or o.tg) else None
    lm = LM(o.model, dtype="float32" if o.fp32 else "bfloat16", max_tokens=need)
    if o.info:
        print(info_line(lm.model))
    elif o.text is not None:
        if lm.tokenizer is None:
            sys.stderr.write("abacus: this model folder has no tokenizer.json\n")
            return 1
        print(" ".join(str(t) for t in lm.tokenizer.encode(o.text)))
    elif o.pp > 0 or o.tg > 0:
        print(json.dumps(bench(lm, o.pp, o.tg, o.batch)))
    elif o.ids is not None:
        if o.dump:
            dump_logits(lm, o.ids, o.start, o.chunk, o.dump)
        else:  # src/main.c:152-164: greedy ids, no stop token
            out = lm.generate([o.ids], max_new_tokens=o.steps, temperature=0.0, stop_tokens=[])[0]
            print(" ".join(str(t) for t in out))
    else:
        if lm.tokenizer is None:
            sys.stderr.write("abacus: this model folder has no tokenizer.json; use --ids\n")
            return 1
        ids = lm.encode(o.prompt, raw=o.raw)
        out = sys.stdout.buffer if hasattr(sys.stdout, "buffer") else None

        def show(request, token):  # each piece as it comes, special tokens left out (src/main.c:177-180)
            if not lm.tokenizer.is_special(token):
                piece = lm.tokenizer.pieces[token] if 0 <= token < len(lm.tokenizer.pieces) else b""
                if out is not None:
                    out.write(piece)
                    out.flush()
                else:
                    sys.stdout.write(piece.decode("utf-8", errors="replace"))
                    sys.stdout.flush()

        t0 = time.perf_counter()
        req = lm.generate([ids], max_new_tokens=o.steps, temperature=o.temp, top_k=o.top_k, seed=o.seed,
                          return_requests=True, on_token=show)[0]
        t1 = time.perf_counter()
        first = lm.last_stats.get("t_first_token", t1) - t0
        rest = max(t1 - t0 - first, 1e-9)
        sys.stderr.write(f"\n\nprompt {len(ids)} tokens, {len(ids) / max(first, 1e-9):.1f} tok/s | "
                         f"generated {len(req.output)} tokens, {len(req.output) / rest:.1f} tok/s\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
