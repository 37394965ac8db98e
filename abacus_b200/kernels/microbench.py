"""Times one kernel alone, at a given size, with CUDA events.

    python -m abacus_b200.kernels.microbench gemm --m 8 --n 4096 --k 1024 [--out f32] [--iters 20]
    python -m abacus_b200.kernels.microbench decode_attention --batch 8 --context 2176 --heads 16 --kv-heads 8
    python -m abacus_b200.kernels.microbench prefill_attention --tokens 2048 --heads 16 --kv-heads 8
    python -m abacus_b200.kernels.microbench qkv_prep --tokens 2048 --heads 16 --kv-heads 8
    python -m abacus_b200.kernels.microbench argmax --rows 8 --vocab 151936
    python -m abacus_b200.kernels.microbench add_rmsnorm --rows 8 --width 1024

Between timed launches a buffer larger than the L2 cache is written, so every launch reads its
operands from HBM. Prints one JSON line: the median time, and the rate of the bytes (or FLOPs)
the operation must move at least. This is also the command to put under ncu for one kernel.
"""
import argparse
import json
import statistics
import sys

import torch


def timed(fn, iters, flush=True):
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if scrub is not None:
            scrub.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    return statistics.median(times), min(times)


def timed_graph(fns, replays=5):
    """Median time per launch of a captured graph that runs every function of `fns` once, back to
    back, with no host in between. Give each function operands of its own, together larger than
    the L2 cache, and every launch reads from HBM as in a real step."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in fns:
            f()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / len(fns))
    return statistics.median(times), min(times)


def timed_graph_flushed(fn, repeats=5):
    """Time of one launch of `fn` that finds nothing of its operands in the L2 cache, without the host's
    launch latency: a captured graph alternates a write of 256 MB with the launch; the same graph
    without the launches is timed too and subtracted."""
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn()
    torch.cuda.synchronize()

    def graph_of(with_fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(repeats):
                scrub.zero_()
                if with_fn:
                    fn()
        return g

    both, alone = graph_of(True), graph_of(False)
    results = []
    for g in (both, alone):
        g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / repeats)
        results.append(statistics.median(times))
    return results[0] - results[1], results[0] - results[1]


def bench_gemm(args):
    from . import ops
    dt = torch.float32 if args.out == "f32" else torch.bfloat16
    x = torch.randn(args.m, args.k, device="cuda").to(torch.bfloat16)
    copies = max(2, min(64, (160 << 20) // (args.n * args.k * 2) + 1))  # weights that together exceed the L2
    ws = [torch.randn(args.n, args.k, device="cuda").to(torch.bfloat16) for _ in range(copies)]
    out = torch.empty(args.m, args.n, dtype=dt, device="cuda")
    if args.rows_kernel:
        us, best = timed_graph([lambda w=w: ops.gemm_rows(x, w, out) for w in ws])
    elif args.with_norm:  # alternate with a small kernel, as in a model step
        xs, wn = torch.randn(args.m, args.k, device="cuda"), torch.ones(args.k, device="cuda")
        fns = []
        for w in ws:
            fns.append(lambda w=w: ops.gemm_tc(x, w, out, tile_n=args.tile_n, swap=args.swap, splits=args.splits,
                                                   persistent=args.persistent))
            fns.append(lambda: ops.add_rmsnorm(xs, None, wn, x, 1e-6))
        us, best = timed_graph(fns)
        us, best = 2 * us, 2 * best  # per pair
    else:
        us, best = timed_graph([lambda w=w: ops.gemm_tc(x, w, out, tile_n=args.tile_n, swap=args.swap,
                                                        splits=args.splits, persistent=args.persistent) for w in ws])
    nbytes = (args.m * args.k + args.n * args.k) * 2 + out.numel() * out.element_size()
    flops = 2.0 * args.m * args.n * args.k
    return {"kernel": "gemm_tc", "m": args.m, "n": args.n, "k": args.k, "us": round(us, 2), "best_us": round(best, 2),
            "GB/s": round(nbytes / us / 1e3, 1), "TFLOP/s": round(flops / us / 1e6, 2)}


def _attention_setup(batch, context, heads, kv_heads, head_dim, new_tokens):
    from ..cache import CacheNeed, SequenceCache
    from ..engine.batch import Sequence, StepBatch
    cache = SequenceCache([CacheNeed(kv_heads, head_dim)], [None], batch * (context + 64), torch.bfloat16, "cuda",
                          max_context=context + 64)
    kv = cache.views[0].kv
    kv.k.normal_()
    kv.v.normal_()
    seqs = []
    for _ in range(batch):
        slot = cache.open_slot()
        cache.reserve(slot, context)
        seqs.append(Sequence(slot, [0] * new_tokens, context - new_tokens, []))
    rows = batch * new_tokens
    from ..parts.attention_plan import AttentionLists, AttentionStepPlan
    plan = AttentionStepPlan(heads)
    b = StepBatch(rows, batch, 0, "cuda", plans=[plan]).fill(seqs)
    b.lists = AttentionLists(b.plan[plan.name])
    qkv = torch.randn(rows, (heads + 2 * kv_heads) * head_dim, device="cuda").to(torch.bfloat16)
    out = torch.empty(rows, heads * head_dim, dtype=torch.bfloat16, device="cuda")
    return cache, kv, b, qkv, out


def bench_decode_attention(args):
    from . import ops
    from ..parts import Workspace
    cache, kv, b, qkv, out = _attention_setup(args.batch, args.context, args.heads, args.kv_heads, args.head_dim, 1)
    ws = Workspace(torch.device("cuda", 0))
    scale = args.head_dim ** -0.5
    prepare = None
    if args.prepares:  # the kernel norms and rotates q and k and writes the new key and value itself
        hd = args.head_dim
        qn, kn = torch.ones(hd, device="cuda"), torch.ones(hd, device="cuda")
        pos = torch.arange(args.context + 64, device="cuda", dtype=torch.float32)[:, None]
        inv = 1.0 / (1e6 ** (torch.arange(0, hd, 2, device="cuda", dtype=torch.float32) / hd))
        prepare = dict(q_norm=qn, k_norm=kn, eps=1e-6, cos=torch.cos(pos * inv).contiguous(), sin=torch.sin(pos * inv).contiguous(), keep=True)
    fn = lambda: ops.attention_decode(qkv, out, args.heads, args.kv_heads, args.head_dim, scale, None, b, kv, ws,
                                      simt=args.simt, prepare=prepare)
    us, best = timed_graph_flushed(fn)
    nbytes = args.batch * args.context * args.kv_heads * args.head_dim * 2 * 2
    return {"kernel": "attention_decode", "batch": args.batch, "context": args.context, "us": round(us, 2),
            "best_us": round(best, 2), "GB/s": round(nbytes / us / 1e3, 1)}


def bench_prefill_attention(args):
    from . import ops
    from ..parts import Workspace
    cache, kv, b, qkv, out = _attention_setup(args.batch, args.tokens, args.heads, args.kv_heads, args.head_dim,
                                              args.tokens)
    ws = Workspace(torch.device("cuda", 0))
    scale = args.head_dim ** -0.5
    ops.qkv_prep(qkv, args.heads, args.kv_heads, args.head_dim, b, None, None, 0.0, None, None, 0, False, kv)
    fn = lambda: ops.attention(qkv, out, args.heads, args.kv_heads, args.head_dim, scale, None, b, kv, ws=ws, lists=b.lists)
    us, best = timed_graph_flushed(fn)
    flops = args.batch * 4.0 * args.head_dim * args.heads * args.tokens * (args.tokens + 1) / 2
    return {"kernel": "attention (prefill)", "batch": args.batch, "tokens": args.tokens, "us": round(us, 2),
            "best_us": round(best, 2), "TFLOP/s": round(flops / us / 1e6, 2)}


def bench_qkv_prep(args):
    """q/k norm, rotation and the cache write of the `tokens` rows of one prompt step (batch sequences)."""
    from . import ops
    heads, kv_heads, hd = args.heads, args.kv_heads, args.head_dim
    cache, kv, b, qkv, out = _attention_setup(args.batch, args.tokens, heads, kv_heads, hd, args.tokens)
    qn, kn = torch.ones(hd, device="cuda"), torch.ones(hd, device="cuda")
    pos = torch.arange(args.tokens + 64, device="cuda", dtype=torch.float32)[:, None]
    inv = 1.0 / (1e6 ** (torch.arange(0, hd, 2, device="cuda", dtype=torch.float32) / hd))
    cos, sin = torch.cos(pos * inv).contiguous(), torch.sin(pos * inv).contiguous()
    us, best = timed_graph([lambda: ops.qkv_prep(qkv, heads, kv_heads, hd, b, qn, kn, 1e-6, cos, sin, hd, False, kv)])
    rows = args.batch * args.tokens
    nbytes = rows * hd * 2 * (2 * (heads + kv_heads) + heads + 2 * kv_heads)  # rows read, q and k written, k and v kept
    return {"kernel": "qkv_prep", "rows": rows, "us": round(us, 2), "best_us": round(best, 2),
            "GB/s": round(nbytes / us / 1e3, 1)}


def bench_qkv_product(args):
    """The q/k/v product of one prompt step of `tokens` rows (batch sequences) against a matrix of --k columns, with the
    preparation of its heads in the epilogue (or, with --separate, as the product and the preparation kernel after it)."""
    from . import ops
    heads, kv_heads, hd = args.heads, args.kv_heads, args.head_dim
    cache, kv, b, qkv, out = _attention_setup(args.batch, args.tokens, heads, kv_heads, hd, args.tokens)
    rows, width = args.batch * args.tokens, (heads + 2 * kv_heads) * hd
    x = torch.randn(rows, args.k, device="cuda").to(torch.bfloat16)
    copies = max(2, min(16, (160 << 20) // (width * args.k * 2) + 1))
    ws = [(torch.randn(width, args.k, device="cuda") / args.k ** 0.5).to(torch.bfloat16) for _ in range(copies)]
    qn, kn = torch.ones(hd, device="cuda"), torch.ones(hd, device="cuda")
    pos = torch.arange(args.tokens + 64, device="cuda", dtype=torch.float32)[:, None]
    inv = 1.0 / (1e6 ** (torch.arange(0, hd, 2, device="cuda", dtype=torch.float32) / hd))
    cos, sin = torch.cos(pos * inv).contiguous(), torch.sin(pos * inv).contiguous()
    if args.separate:
        fns = []
        for w in ws:
            fns += [lambda w=w: ops.gemm_tc(x, w, qkv), lambda: ops.qkv_prep(qkv, heads, kv_heads, hd, b, qn, kn, 1e-6, cos, sin, hd, False, kv)]
        us, best = timed_graph(fns)
        us, best = 2 * us, 2 * best
    else:
        assert ops.gemm_tc_qkv_takes(x, ws[0], qkv, rows, heads, kv_heads, hd, kv, qn, kn, cos, sin, hd, False)
        us, best = timed_graph([lambda w=w: ops.gemm_tc_qkv(x, w, qkv, heads, kv_heads, b, qn, kn, 1e-6, cos, sin, kv) for w in ws])
    return {"kernel": "q/k/v product" + (" + qkv_prep" if args.separate else " that prepares"), "rows": rows, "n": width, "k": args.k,
            "us": round(us, 2), "best_us": round(best, 2), "TFLOP/s": round(2.0 * rows * width * args.k / us / 1e6, 2)}


def bench_argmax(args):
    from . import ops
    copies = max(2, (160 << 20) // (args.rows * args.vocab * 4) + 1)
    logits = [torch.randn(args.rows, args.vocab, device="cuda") for _ in range(copies)]
    out = torch.empty(args.rows, dtype=torch.int32, device="cuda")
    us, best = timed_graph([lambda l=l: ops.argmax(l, out) for l in logits])
    logits = logits[0]
    return {"kernel": "argmax", "rows": args.rows, "vocab": args.vocab, "us": round(us, 2), "best_us": round(best, 2),
            "GB/s": round(logits.numel() * 4 / us / 1e3, 1)}


def bench_add_rmsnorm(args):
    from . import ops
    x, y = torch.randn(args.rows, args.width, device="cuda"), torch.randn(args.rows, args.width, device="cuda")
    w = torch.ones(args.width, device="cuda")
    out = torch.empty(args.rows, args.width, dtype=torch.bfloat16, device="cuda")
    us, best = timed_graph([lambda: ops.add_rmsnorm(x, y, w, out, 1e-6)] * 50)
    return {"kernel": "add_rmsnorm", "rows": args.rows, "width": args.width, "us": round(us, 2), "best_us": round(best, 2),
            "GB/s": round(args.rows * args.width * 14 / us / 1e3, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm", "decode_attention", "prefill_attention", "qkv_prep", "qkv_product", "argmax", "add_rmsnorm"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--out", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--swap", type=int, default=-1)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--persistent", type=int, default=-1, help="gemm: 1 / 0 pins the persistent kernel on / off")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2176)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--rows-kernel", action="store_true", help="gemm: the weight-streaming kernel for m <= 16")
    ap.add_argument("--separate", action="store_true", help="qkv_product: the product and the preparation as two kernels")
    ap.add_argument("--prepares", action="store_true", help="decode_attention: q, k and v are prepared in the attention kernel")
    ap.add_argument("--simt", action="store_true", help="decode_attention: the CUDA-core kernel")
    ap.add_argument("--with-norm", action="store_true", help="gemm: alternate with an add_rmsnorm, as a model step does")
    args = ap.parse_args(argv)
    if args.kernel in ("prefill_attention", "qkv_prep") and "--batch" not in (argv or sys.argv):
        args.batch = 1
    fn = {"gemm": bench_gemm, "decode_attention": bench_decode_attention, "prefill_attention": bench_prefill_attention,
          "qkv_prep": bench_qkv_prep, "qkv_product": bench_qkv_product, "argmax": bench_argmax, "add_rmsnorm": bench_add_rmsnorm}[args.kernel]
    print(json.dumps(fn(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
