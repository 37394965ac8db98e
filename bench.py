#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-0.6B shape on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the whole batch. The default run has the layer sizes of the
Qwen3-0.6B checkpoint (28 layers, width 1024, 16/8 heads of 128, MLP 3072, vocabulary 151936,
tied head) with random bfloat16 weights, a batch of 8 sequences with 2,048-token prompts in a
cache sized for a context of 4,096, and times K decode steps after W warm-up steps with CUDA
events. It prints ONE JSON line: `value` is decoded tokens per second on the device-driven loop
(captured graph, sampled token fed back on the device), `e2e` the same through the Python entry
point's generation loop with host tokens in and out every step, `prefill` a 2,048-token prompt,
`roofline` the bytes a decode step must read over its time, `points` batch 1 and 64.
More than one GPU is not built: the line says so and the exit code is 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE = dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
             num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=40960,
             rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
CONTEXT, PROMPT, PREFILL_TOKENS = 4096, 2048, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS, source="fallback")


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.startswith("Active")})
        top = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(top) if top else None,
                "reasons": reasons, "samples": len(mhz)}


def build_model(layers=None):
    import torch
    from abacus_b200.config import Qwen3Config, get_architecture
    from abacus_b200.models import Model
    from abacus_b200.weights import random_tensors
    raw = dict(SHAPE, architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    if layers:
        raw["num_hidden_layers"] = layers
    config = Qwen3Config.from_dict(raw)
    arch = get_architecture(config.architecture)
    spec = config.to_spec()
    expected, _ = arch.tensor_names(spec, None)
    tensors = random_tensors(expected, seed=2, std=0.02)
    return Model(spec, arch.layout(spec), tensors, torch.bfloat16, torch.device("cuda", 0)), config


def kv_bytes_per_token(model):
    total = 0
    for need in model.cache_needs():
        if need is not None and need.n_kv_heads:
            total += 2 * need.n_kv_heads * need.head_dim * 2
    return total


def prompts_for(batch, vocab, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(0, vocab, PROMPT)] for _ in range(batch)]


def device_decode(model, batch, steps, warmup, with_clocks=False):
    """Tokens per second of `steps` decode steps of `batch` sequences after their prompts, the host only
    launching: the graph of the step, then the sampler, which writes the next tokens where the graph reads
    them. Returns (tokens/s, ms per step, launches in the timed region, mean context, clocks)."""
    import torch
    from abacus_b200.engine import Engine
    from abacus_b200.kernels import ops
    from abacus_b200.sampling import Sampler
    engine = Engine(model, max_tokens=batch * CONTEXT, max_slots=max(batch, 1), max_context=CONTEXT)
    sampler = Sampler(model.ctx.device, temperature=0.0)
    slots = [engine.open() for _ in range(batch)]
    prompts = prompts_for(batch, model.spec.vocab, 10 + batch)
    logits = engine.step([(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = sampler.sample(logits, None).tolist()
    logits = engine.step([(s, [t], [0]) for s, t in zip(slots, first)])  # captures the graph
    graph = engine.graphs.get(engine.plan([(s, [0], [0]) for s in slots]))
    tokens = graph.batch.tokens[:batch]
    sampler.sample(logits, None, out=tokens)

    def one_step():
        for s in slots:
            engine.cache.reserve(s, engine.cache.length[s] + 1)
            engine.cache.advance(s, 1)
        lg = graph.replay_advanced()
        sampler.sample(lg, None, out=tokens)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    clocks = Clocks()
    if with_clocks:
        clocks.start()
        time.sleep(0.2)
    before = ops.LAUNCHES
    context0 = engine.cache.length[slots[0]]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    launches = (ops.LAUNCHES - before) + steps * graph.n_kernels
    clock_info = clocks.stop() if with_clocks else None
    engine.check_status()
    mean_context = context0 + (steps + 1) / 2.0
    for s in slots:
        engine.close(s)
    del engine
    torch.cuda.empty_cache()
    return batch * steps / (ms / 1e3), ms / steps, launches, mean_context, clock_info


def e2e_decode(model, batch, steps):
    """The same decode through the generation loop of the Python entry point: every step the host sends
    that step's tokens and indices from pinned memory and reads the sampled tokens back."""
    import torch
    from abacus_b200.engine import Engine
    from abacus_b200.engine.generate import Generator
    from abacus_b200.sampling import Sampler
    engine = Engine(model, max_tokens=batch * CONTEXT, max_slots=max(batch, 1), max_context=CONTEXT)
    gen = Generator(engine, Sampler(model.ctx.device, temperature=0.0), stop_tokens=())
    prompts = prompts_for(batch, model.spec.vocab, 10 + batch)
    gen.generate(prompts, 4)  # warm-up: kernels, graph capture
    gen = Generator(engine, Sampler(model.ctx.device, temperature=0.0), stop_tokens=())
    requests = gen.generate(prompts, steps + 1)
    assert all(len(r.output) == steps + 1 for r in requests)
    seconds = gen.stats["t_end"] - gen.stats["t_first_token"]
    h2d = engine.last_batch._host.numel() * 4
    del engine
    torch.cuda.empty_cache()
    return batch * steps / seconds, h2d, batch * 4


def prefill(model, repeats=3):
    """One 2,048-token prompt in one step; median time of `repeats`, and the step's FLOPs."""
    import torch
    from abacus_b200.engine import Engine
    engine = Engine(model, max_tokens=CONTEXT, max_slots=1, max_context=CONTEXT)
    prompt = prompts_for(1, model.spec.vocab, 99)[0][:PREFILL_TOKENS]
    times, untimed = [], 2  # the first run loads the kernels, the second captures the step's graph
    for i in range(repeats + untimed):
        slot = engine.open()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([(slot, prompt, [len(prompt) - 1])])
        end.record()
        torch.cuda.synchronize()
        if i >= untimed:
            times.append(start.elapsed_time(end))
        engine.close(slot)
    engine.check_status()
    ms = statistics.median(times)
    spec, t = model.spec, PREFILL_TOKENS
    linear = 0
    for e in spec.schedule:
        m, f = spec.layers[e.layer].mixer, spec.layers[e.layer].ffn
        linear += m.hidden * (m.n_heads + 2 * m.n_kv_heads) * m.head_dim + m.n_heads * m.head_dim * m.hidden
        linear += 3 * f.hidden * f.inter
    attn = sum(4 * spec.layers[e.layer].mixer.head_dim * spec.layers[e.layer].mixer.n_heads * (t * (t + 1) // 2)
               for e in spec.schedule)
    flops = 2 * t * linear + attn + 2 * spec.hidden * spec.vocab
    return ms, flops


def timeline(model, batch):
    """The launches of one decode step and of one 2,048-token prefill with the time each took inside its step
    (from the records of abacus_b200/kernels/trace.py; the libraries must be built with ABACUS_TRACE=1)."""
    import torch
    from abacus_b200.engine import Engine
    from abacus_b200.kernels import trace

    def show(title, rows):
        print(title)
        for i, row in enumerate(rows):
            # a launch's release comes when the launch before it is complete: the gap is that launch's time
            took = rows[i + 1]["after_previous_us"] if i + 1 < len(rows) else float("nan")
            print(f"  {row['module']:22s} grid {row['grid']:6d} x {row['block']:4d}  waited {row['waited_us']:6.2f} us"
                  f"  took {took:7.2f} us")

    device_decode(model, batch, 4, 3)
    torch.cuda.synchronize()
    trace.read()
    device_decode(model, batch, 2, 0)
    rows = trace.timeline(trace.read())
    per_step = len(rows) // 3 if len(rows) >= 3 else len(rows)  # the prompts' step and two decode steps were recorded
    show(f"decode step, batch {batch} (kernels without a dependency wait are not recorded)", rows[-per_step:])
    engine = Engine(model, max_tokens=CONTEXT, max_slots=1, max_context=CONTEXT)
    prompt = prompts_for(1, model.spec.vocab, 99)[0][:PREFILL_TOKENS]
    for i in range(3):
        slot = engine.open()
        engine.step([(slot, prompt, [len(prompt) - 1])])
        torch.cuda.synchronize()
        engine.close(slot)
        if i == 1:
            trace.read()
    show(f"prefill of {PREFILL_TOKENS} tokens", trace.timeline(trace.read()))
    return 0


def run_ours(args):
    import torch
    from abacus_b200.kernels import build_all
    build_all(verbose=False)
    torch.cuda.set_device(0)
    pk = peaks()
    model, config = build_model(args.layers)
    full_layers = SHAPE["num_hidden_layers"]
    weight_bytes = model.weight_bytes_read_per_step()
    kv_token = kv_bytes_per_token(model)

    if args.only == "timeline":  # with ABACUS_TRACE=1: what each launch of a decode step and of a prefill took, as they ran
        return timeline(model, args.batch)
    if args.only == "prefill":  # for profiling: the prefill step alone
        pre_ms, pre_flops = prefill(model, repeats=1)
        print(json.dumps({"prefill_ms": round(pre_ms, 3), "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0
    tok_s, ms_step, launches, mean_ctx, clocks = device_decode(model, args.batch, args.steps, args.warmup, True)
    bytes_step = weight_bytes + args.batch * mean_ctx * kv_token
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    if args.only == "decode":  # for profiling: the decode loop alone
        print(json.dumps({"value": round(tok_s, 1), "ms_per_step": round(ms_step, 4), "batch": args.batch,
                          "hbm_frac": round(achieved / pk["hbm_gbs"], 4), "gpu_launches": launches}))
        return 0
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(device_decode(model, b, min(args.steps, 128), args.warmup)[0], 1)
    e2e, h2d, d2h = e2e_decode(model, args.batch, min(args.steps, 128))
    pre_ms, pre_flops = prefill(model)
    line = {
        "metric": "decode tokens/s (Qwen3-0.6B shape, batch 8, 2048-token prompts)", "value": round(tok_s, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "Qwen3-0.6B shape, random weights seed 2", "global_batch": args.batch, "seq_len": CONTEXT,
                   "prompt_tokens": PROMPT, "layers": len(model.spec.schedule), "layers_of_config": full_layers,
                   "hidden": SHAPE["hidden_size"], "heads": SHAPE["num_attention_heads"],
                   "kv_heads": SHAPE["num_key_value_heads"], "head_dim": SHAPE["head_dim"],
                   "intermediate": SHAPE["intermediate_size"], "vocab": SHAPE["vocab_size"], "tied_head": True,
                   "parallelism": "single GPU", "l2": "a step reads more than the 126 MB L2 (weights 1.2 GB + cache)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    """abacus itself: its C engine built from an unmodified copy of its sources under baseline/_ref and run
    through its own command line (--bench PP TG, src/main.c:65-82) on a model its own converter made from the
    same shape with random weights. It is a CPU engine with int8 weights that decodes one sequence at a time."""
    src = os.path.join(ROOT, "baseline", "_ref", "abacus_src")

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if not os.path.isdir(os.path.join(src, "src")):
        return unavailable("pip installs only metadata (the package has no modules; the engine is a C program) "
                           "and no copy of its sources is under baseline/_ref/abacus_src")
    try:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from abacus_b200.config import Qwen3Config
        from abacus_b200.weights import write_random_model
        with tempfile.TemporaryDirectory() as tmp:
            exe = os.path.join(tmp, "abacus")
            files = sorted(os.path.join(src, "src", n) for n in os.listdir(os.path.join(src, "src")) if n.endswith(".c"))
            subprocess.run(["cc", "-O3", "-march=native", "-std=c11", "-D_GNU_SOURCE", "-pthread", "-o", exe, *files,
                            "-lm"], check=True, capture_output=True)
            raw = dict(SHAPE, architectures=["Qwen3ForCausalLM"], model_type="qwen3")
            folder = write_random_model(os.path.join(tmp, "model"), Qwen3Config.from_dict(raw), seed=2)
            vocab = SHAPE["vocab_size"]
            with open(os.path.join(folder, "tokenizer.json"), "w") as f:
                json.dump({"model": {"vocab": {}, "merges": []},
                           "added_tokens": [{"content": "<|endoftext|>", "id": vocab - 2},
                                            {"content": "<|im_end|>", "id": vocab - 1}]}, f)
            model_bin = os.path.join(tmp, "model.bin")
            subprocess.run([sys.executable, os.path.join(src, "tools", "export.py"), folder, model_bin], check=True,
                           capture_output=True)
            t0 = time.time()
            out = subprocess.run([exe, model_bin, "--bench", str(PROMPT), str(args.steps)], check=True,
                                 capture_output=True, text=True, timeout=1500).stdout
            res = json.loads(out.strip().splitlines()[-1])
    except (subprocess.CalledProcessError, subprocess.TimeoutExpired, OSError, ValueError) as e:
        return unavailable(f"building or running abacus failed: {type(e).__name__}: {str(e)[:200]}")
    tok_s = res["decode_tok_s"]
    print(json.dumps({
        "metric": "decode tokens/s (Qwen3-0.6B shape, batch 8, 2048-token prompts)", "value": round(tok_s, 2),
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": 1, "ms_per_step": round(1e3 / tok_s, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 weights on the CPU",
        "data": "synthetic", "impl": "reference",
        "config": {"model": "Qwen3-0.6B shape, random weights seed 2", "global_batch": 1, "seq_len": CONTEXT,
                   "threads": res.get("threads"), "note": "abacus decodes one sequence at a time on the CPU (a batch of 8 "
                   "is 8 runs at this rate); its --bench decodes from position 0 (src/main.c:74-78)"},
        "prefill": {"value": round(res["prefill_tok_s"], 2), "tokens": PROMPT}, "wall_s": round(time.time() - t0, 1)}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "timeline"],
                    help="run one part (for profiling); timeline needs ABACUS_TRACE=1")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not built (no multi-GPU path)")
        return 2
    args.warmup = max(args.warmup, 3)
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
