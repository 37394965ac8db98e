#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3 shapes on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 0.6b|4b|8b]

One "step" is one decode step of the whole batch. The default run has the layer sizes of the
Qwen3-0.6B checkpoint (28 layers, width 1024, 16/8 heads of 128, MLP 3072, vocabulary 151936,
tied head) with random bfloat16 weights, a batch of 8 sequences with 2,048-token prompts in a
cache sized for a context of 4,096, and times K decode steps after W warm-up steps with CUDA
events. It prints ONE JSON line: `value` is decoded tokens per second on the device-driven loop
(captured graph, sampled token fed back on the device), `e2e` the same through the Python entry
point's generation loop with host tokens in and out every step, `prefill` a 2,048-token prompt,
`roofline` the bytes a decode step must read over its time, `points` batch 1 and 64 and the two
larger workloads: the Qwen3-4B shape (16 prompts of 64 to 2,048 tokens, then 128 decode steps, context
4,096) and the Qwen3-8B shape (untied head; 32 prompts of 128 to 4,096 tokens, then 128 decode steps,
context 8,192), each with decode tokens/s and its fraction of the HBM peak from the contexts the steps
really had, and the ragged prompts' step with its fraction of the tensor peak. --config 4b or 8b makes
that workload the line's own (value, roofline, prefill) instead.
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

COMMON = dict(head_dim=128, vocab_size=151936, max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6)
# layer sizes of the three checkpoints; workload: (sequences, shortest prompt, longest prompt, decode steps, context, seed)
CONFIGS = {
    "0.6b": dict(shape=dict(COMMON, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                            num_key_value_heads=8, tie_word_embeddings=True),
                 name="Qwen3-0.6B", seed=2, workload=(8, 2048, 2048, 256, 4096)),
    "4b": dict(shape=dict(COMMON, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32,
                          num_key_value_heads=8, tie_word_embeddings=True),
               name="Qwen3-4B", seed=3, workload=(16, 64, 2048, 128, 4096)),
    "8b": dict(shape=dict(COMMON, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                          num_key_value_heads=8, tie_word_embeddings=False),
               name="Qwen3-8B", seed=4, workload=(32, 128, 4096, 128, 8192)),
}
SHAPE = CONFIGS["0.6b"]["shape"]
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


def build_model(name="0.6b", layers=None):
    """The model of configuration `name` with random weights, filled on the device (csrc/utility.cu)."""
    import torch
    from abacus_b200.config import Qwen3Config, get_architecture
    from abacus_b200.models import Model
    from abacus_b200.weights import random_tensors
    c = CONFIGS[name]
    raw = dict(c["shape"], architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    if layers:
        raw["num_hidden_layers"] = layers
    config = Qwen3Config.from_dict(raw)
    arch = get_architecture(config.architecture)
    spec = config.to_spec()
    expected, _ = arch.tensor_names(spec, None)
    device = torch.device("cuda", 0)
    tensors = random_tensors(expected, seed=c["seed"], std=0.02, device=device)
    model = Model(spec, arch.layout(spec), tensors, torch.bfloat16, device)
    del tensors
    torch.cuda.empty_cache()
    return model, config


def kv_bytes_per_token(model):
    total = 0
    for need in model.cache_needs():
        if need is not None and need.n_kv_heads:
            total += 2 * need.n_kv_heads * need.head_dim * 2
    return total


def prompts_for(batch, vocab, seed, shortest=PROMPT, longest=PROMPT):
    """`batch` prompts of seeded uniform token ids, their lengths seeded uniform in [shortest, longest]."""
    import numpy as np
    rng = np.random.default_rng(seed)
    lengths = [int(n) for n in rng.integers(shortest, longest + 1, batch)]
    return [[int(t) for t in rng.integers(0, vocab, n)] for n in lengths]


def device_decode(model, prompts, steps, warmup, context=CONTEXT, with_clocks=False):
    """Tokens per second of `steps` decode steps after the prompts, the host only launching: the graph of the
    step, then the sampler, which writes the next tokens where the graph reads them. Returns a dict: tokens/s,
    ms per step, launches in the timed region, the mean over the timed steps of the tokens all sequences hold
    together (what the step reads of the cache), and the clocks."""
    import torch
    from abacus_b200.engine import Engine
    from abacus_b200.kernels import ops
    from abacus_b200.sampling import Sampler
    batch = len(prompts)
    engine = Engine(model, max_tokens=batch * context, max_slots=max(batch, 1), max_context=context)
    sampler = Sampler(model.ctx.device, temperature=0.0)
    slots = [engine.open() for _ in range(batch)]
    logits = engine.step([(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = sampler.sample(logits, None).tolist()
    # The graph of the loop's step: captured for a bound on the positions that holds to the loop's end, so that no
    # row outgrows it on the way (a decode graph's grid is sized for its bound).
    from abacus_b200.engine import Sequence
    seqs = engine.plan([(s, [t], [0]) for s, t in zip(slots, first)])
    last = max(len(p) for p in prompts) + warmup + steps + 2
    graph = engine.graphs.get([Sequence(q.slot, q.tokens, last - 1, q.want) for q in seqs])
    logits = graph.run(seqs)
    for s in slots:
        engine.cache.advance(s, 1)
    tokens = graph.batch.tokens[:batch]
    sampler.sample(logits, None, out=tokens)

    def one_step():
        engine.cache.reserve_all([(s, engine.cache.length[s] + 1) for s in slots])
        for s in slots:
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
    held0 = sum(engine.cache.length[s] for s in slots)  # the first timed step reads this many cached tokens, and its own
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
    for s in slots:
        engine.close(s)
    del engine, graph
    torch.cuda.empty_cache()
    return {"tok_s": batch * steps / (ms / 1e3), "ms_step": ms / steps, "launches": launches,
            "mean_tokens_held": held0 + batch * (steps + 1) / 2.0, "clocks": clock_info}


def decode_roofline(model, run, pk):
    """(bytes a step must read, achieved GB/s, fraction of the HBM peak): every weight once and the cache of the
    live requests at the contexts the timed steps really had."""
    bytes_step = model.weight_bytes_read_per_step() + run["mean_tokens_held"] * kv_bytes_per_token(model)
    achieved = bytes_step / (run["ms_step"] / 1e3) / 1e9
    return bytes_step, achieved, achieved / pk["hbm_gbs"]


def e2e_decode(model, prompts, steps, context=CONTEXT):
    """The same decode through the generation loop of the Python entry point: every step the host sends
    that step's tokens and indices from pinned memory and reads the sampled tokens back."""
    import torch
    from abacus_b200.engine import Engine
    from abacus_b200.engine.generate import Generator
    from abacus_b200.sampling import Sampler
    batch = len(prompts)
    engine = Engine(model, max_tokens=batch * context, max_slots=max(batch, 1), max_context=context)
    gen = Generator(engine, Sampler(model.ctx.device, temperature=0.0), stop_tokens=())
    gen.generate(prompts, 4)  # warm-up: kernels, graph capture
    gen = Generator(engine, Sampler(model.ctx.device, temperature=0.0), stop_tokens=())
    requests = gen.generate(prompts, steps + 1)
    assert all(len(r.output) == steps + 1 for r in requests)
    seconds = gen.stats["t_end"] - gen.stats["t_first_token"]
    h2d = engine.last_batch._host.numel() * 4
    del engine
    torch.cuda.empty_cache()
    return batch * steps / seconds, h2d, batch * 4


def prefill_flops(spec, lengths):
    """FLOPs of one step that brings whole prompts of these lengths: the linear layers on every token, causal
    attention within each prompt, the output matrix on one row per prompt."""
    t = sum(lengths)
    linear = 0
    for e in spec.schedule:
        m, f = spec.layers[e.layer].mixer, spec.layers[e.layer].ffn
        linear += m.hidden * (m.n_heads + 2 * m.n_kv_heads) * m.head_dim + m.n_heads * m.head_dim * m.hidden
        linear += 3 * f.hidden * f.inter
    attn = sum(4 * spec.layers[e.layer].mixer.head_dim * spec.layers[e.layer].mixer.n_heads * (n * (n + 1) // 2)
               for e in spec.schedule for n in lengths)
    return 2 * t * linear + attn + 2 * spec.hidden * spec.vocab * len(lengths)


def prefill(model, prompts=None, context=CONTEXT, repeats=3):
    """One step that brings the prompts whole (by default one 2,048-token prompt); median time of `repeats`, and
    the step's FLOPs."""
    import torch
    from abacus_b200.engine import Engine
    if prompts is None:
        prompts = [prompts_for(1, model.spec.vocab, 99)[0][:PREFILL_TOKENS]]
    engine = Engine(model, max_tokens=len(prompts) * context, max_slots=len(prompts), max_context=context)
    times, untimed = [], 2  # the first run loads the kernels, the second captures the step's graph
    for i in range(repeats + untimed):
        slots = [engine.open() for _ in prompts]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        end.record()
        torch.cuda.synchronize()
        if i >= untimed:
            times.append(start.elapsed_time(end))
        for s in slots:
            engine.close(s)
    engine.check_status()
    del engine
    torch.cuda.empty_cache()
    return statistics.median(times), prefill_flops(model.spec, [len(p) for p in prompts])


def workload(name, pk, steps=None, warmup=3, layers=None, with_clocks=False):
    """Configuration `name` as written: its ragged prompts in one step, then its decode steps on the device-driven
    loop. Returns (model, numbers)."""
    c = CONFIGS[name]
    n_seqs, shortest, longest, n_steps, context = c["workload"]
    model, _ = build_model(name, layers)
    prompts = prompts_for(n_seqs, model.spec.vocab, 10 + c["seed"], shortest, longest)
    run = device_decode(model, prompts, steps or n_steps, warmup, context, with_clocks)
    _, achieved, frac = decode_roofline(model, run, pk)
    pre_ms, pre_flops = prefill(model, prompts, context)
    tokens = sum(len(p) for p in prompts)
    return model, {"decode_tok_s": run["tok_s"], "ms_step": run["ms_step"], "hbm_gbs": achieved, "hbm_frac": frac,
                   "prefill_tok_s": tokens / (pre_ms / 1e3), "prefill_ms": pre_ms, "prefill_tokens": tokens,
                   "prefill_frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "launches": run["launches"],
                   "clocks": run["clocks"], "mean_context": run["mean_tokens_held"] / n_seqs, "run": run,
                   "prompts": prompts}


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

    prompts = prompts_for(batch, model.spec.vocab, 10 + batch)
    device_decode(model, prompts, 4, 3)
    torch.cuda.synchronize()
    trace.read()
    device_decode(model, prompts, 2, 0)
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


def large_points(name, pk, points):
    """The workload of configuration `name` (4b or 8b) into `points`, flat."""
    import torch
    model, w = workload(name, pk)
    points[f"{name}_decode"] = round(w["decode_tok_s"], 1)
    points[f"{name}_decode_ms_per_step"] = round(w["ms_step"], 4)
    points[f"{name}_decode_hbm_frac"] = round(w["hbm_frac"], 4)
    points[f"{name}_decode_mean_context"] = round(w["mean_context"], 1)
    points[f"{name}_prefill"] = round(w["prefill_tok_s"], 1)
    points[f"{name}_prefill_tokens"] = w["prefill_tokens"]
    points[f"{name}_prefill_ms"] = round(w["prefill_ms"], 3)
    points[f"{name}_prefill_frac"] = round(w["prefill_frac"], 4)
    del model
    torch.cuda.empty_cache()


def run_ours(args):
    import torch
    from abacus_b200.kernels import build_all
    build_all(verbose=False)
    torch.cuda.set_device(0)
    pk = peaks()
    name = args.config
    c = CONFIGS[name]
    shape = c["shape"]
    n_seqs, shortest, longest, _, context = c["workload"]
    model, config = build_model(name, args.layers)
    if name == "0.6b":
        n_seqs = args.batch
    prompts = prompts_for(n_seqs, model.spec.vocab, 10 + (n_seqs if name == "0.6b" else c["seed"]), shortest, longest)

    if args.only == "timeline":  # with ABACUS_TRACE=1: what each launch of a decode step and of a prefill took, as they ran
        return timeline(model, args.batch)
    if args.only == "prefill":  # for profiling: the prefill step alone (--ragged: the configuration's own prompts)
        pre_ms, pre_flops = prefill(model, prompts if args.ragged else None, context, repeats=1)
        print(json.dumps({"prefill_ms": round(pre_ms, 3), "tokens": sum(len(q) for q in prompts) if args.ragged else PREFILL_TOKENS,
                          "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0
    run = device_decode(model, prompts, args.steps, args.warmup, context, True)
    _, achieved, frac = decode_roofline(model, run, pk)
    if args.only == "decode":  # for profiling: the decode loop alone
        print(json.dumps({"value": round(run["tok_s"], 1), "ms_per_step": round(run["ms_step"], 4), "batch": n_seqs,
                          "hbm_frac": round(frac, 4), "gpu_launches": run["launches"]}))
        return 0
    points = {}
    for b in (1, 64):
        if name == "0.6b" or b == 1:
            few = prompts_for(b, model.spec.vocab, 10 + b)
            points[f"decode_b{b}"] = round(device_decode(model, few, min(args.steps, 128), args.warmup, CONTEXT)["tok_s"], 1)
    e2e, h2d, d2h = e2e_decode(model, prompts, min(args.steps, 128), context)
    pre_ms, pre_flops = prefill(model)
    if name != "0.6b":  # the configuration's own prompts in one step
        rag_ms, rag_flops = prefill(model, prompts, context)
        tokens = sum(len(q) for q in prompts)
        points.update({"ragged_prefill": round(tokens / (rag_ms / 1e3), 1), "ragged_prefill_tokens": tokens,
                       "ragged_prefill_ms": round(rag_ms, 3),
                       "ragged_prefill_frac": round(rag_flops / (rag_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)})
    weight_gb = model.weight_bytes_read_per_step() / 1e9
    layers_run = len(model.spec.schedule)
    del model
    torch.cuda.empty_cache()
    if name == "0.6b" and not args.skip_large and not args.layers:
        for other in ("4b", "8b"):
            large_points(other, pk, points)
    what = (f"batch {n_seqs}, 2048-token prompts" if name == "0.6b" else
            f"{n_seqs} prompts of {shortest} to {longest} tokens")
    line = {
        "metric": f"decode tokens/s ({c['name']} shape, {what})", "value": round(run["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(run["ms_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"{c['name']} shape, random weights seed {c['seed']}", "global_batch": n_seqs, "seq_len": context,
                   "prompt_tokens": PROMPT if name == "0.6b" else round(sum(len(q) for q in prompts) / n_seqs, 1),
                   "layers": layers_run, "layers_of_config": shape["num_hidden_layers"],
                   "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"],
                   "kv_heads": shape["num_key_value_heads"], "head_dim": shape["head_dim"],
                   "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
                   "tied_head": shape["tie_word_embeddings"], "parallelism": "single GPU",
                   "l2": f"a step reads more than the 126 MB L2 (weights {weight_gb:.1f} GB + cache)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": run["launches"],
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(frac, 4)},
        "points": points,
        "clocks": run["clocks"],
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
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 / tok_s, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 weights on the CPU",
        "data": "synthetic", "impl": "reference",
        "config": {"model": "Qwen3-0.6B shape, random weights seed 2", "global_batch": 1, "seq_len": CONTEXT,
                   "threads": res.get("threads"), "note": "abacus decodes one sequence at a time on the CPU (a batch of 8 "
                   "is 8 runs at this rate); its --bench decodes from position 0 after one warm-up call of 16 tokens, whatever "
                   "--warmup says (src/main.c:70-78)"},
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
    ap.add_argument("--config", default="0.6b", choices=sorted(CONFIGS), help="whose workload the line reports")
    ap.add_argument("--skip-large", action="store_true", help="leave the 4b and 8b workloads out of `points`")
    ap.add_argument("--ragged", action="store_true", help="with --only prefill: the configuration's own prompts")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not built (no multi-GPU path)")
        return 2
    args.warmup = max(args.warmup, 3)
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
