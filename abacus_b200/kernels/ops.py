"""Python faces of the CUDA kernels: they check their arguments and launch on torch's current stream.

Every function here runs a hand-written kernel from csrc/; none has a CPU or
library fallback. Tensors must live on the GPU and be contiguous where a kernel
assumes it; a kernel that does not take a size raises KernelRefused with the
reason instead of computing something else.
"""
import ctypes

import torch

from . import guards
from .build import load_module

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


class KernelRefused(KernelError):
    """The sizes or types given are outside what the kernel is built for."""


def _dt(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {t.dtype} is neither float32 nor bfloat16")


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    # torch's current stream as a raw handle (the public torch.cuda.current_stream() builds a Stream object
    # for it and takes fifty times as long: a few microseconds on every launch)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("a kernel was given a tensor that is not on the GPU; there is no CPU path")


LAUNCHES = 0  # kernels launched through this module (a captured graph's replays are not counted here)


def _check(lib, rc, what, kernels=1):
    global LAUNCHES
    if rc == 0:
        LAUNCHES += kernels
        return
    if rc < 0:
        raise KernelRefused(lib.abk_last_error().decode())
    raise KernelError(f"{what}: CUDA error {rc} at launch")


_i, _ll, _f = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def fill_normal(out, key, mean, amplitude, first=0):
    """out.flat[i] = mean + amplitude * z(key, first + i), z a unit normal that depends on (key, index) alone
    (csrc/utility.cu; weights/random_init.py holds the host twin). out float32 or bfloat16, contiguous."""
    _need_cuda(out)
    lib = load_module("utility")
    assert out.is_contiguous()
    _check(lib, lib.abk_fill_normal(_p(out), _i(_dt(out)), _ll(out.numel()), _ll(first), ctypes.c_ulonglong(key),
                                    _f(mean), _f(amplitude), _stream()), "fill_normal")


def embed(tokens, table, x, status):
    """x[t] = float(table[tokens[t]]) (src/model.c:290-291). tokens int32 [T], x float32 [T, d]."""
    _need_cuda(tokens, table, x, status)
    lib = load_module("elementwise")
    n, d = x.shape
    assert tokens.dtype == torch.int32 and x.dtype == torch.float32 and tokens.numel() >= n
    assert table.is_contiguous() and x.is_contiguous() and table.shape[1] == d
    _check(lib, lib.abk_embed(_p(tokens), _p(table), _i(_dt(table)), _p(x), _i(n), _i(d), _i(table.shape[0]),
                              _p(status), _stream()), "embed")


def add_rmsnorm(x, y, weight, out, eps, rows=None, n_rows=None):
    """x += y (if given); out = weight * x / sqrt(mean(x^2) + eps) (src/model.c:238-244).

    rows (int32) picks the rows of x that are normed into out[0:len(rows)]; x is then left unchanged.
    """
    _need_cuda(x, y, weight, out, rows)
    lib = load_module("elementwise")
    d = x.shape[-1]
    n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == d
    assert y is None or (y.dtype == torch.float32 and y.shape == x.shape and y.is_contiguous())
    assert x.is_contiguous() and out.is_contiguous() and out.shape[-1] == d and out.shape[0] >= n
    _check(lib, lib.abk_add_rmsnorm(_p(x), _p(y), _p(weight), _p(out), _i(_dt(out)), _p(rows), _i(n), _i(d),
                                    _f(eps), _stream()), "add_rmsnorm")


def swiglu(gate_up, act, block=None):
    """act = silu(gate) * up (src/model.c:274-282). A row of gate_up holds gate and up in turns of `block`
    columns (gate of features [0, block), up of the same, gate of the next block, ...); by default all gates
    and then all ups."""
    _need_cuda(gate_up, act)
    lib = load_module("elementwise")
    n, two_i = gate_up.shape
    assert act.shape == (n, two_i // 2) and act.dtype == gate_up.dtype
    assert gate_up.is_contiguous() and act.is_contiguous()
    _check(lib, lib.abk_swiglu(_p(gate_up), _p(act), _i(_dt(act)), _i(n), _i(two_i // 2), _i(block or two_i // 2),
                               _stream()), "swiglu")


def qkv_prep(qkv, n_heads, n_kv_heads, head_dim, batch, q_norm, k_norm, eps, cos, sin, rotary_dim, interleaved,
             cache, q_only=False):
    """Per-head norm of q and k, rotary encoding, and the cache write of k and v (src/model.c:247-259).

    qkv [T, (Hq + 2 Hkv) * hd] is changed in place. batch: engine.batch.StepBatch. cache: a
    cache.LayerKV or None (nothing written). q_only: only the q heads are prepared.
    """
    _need_cuda(qkv, q_norm, k_norm, cos, sin)
    lib = load_module("elementwise")
    n = batch.n_rows
    assert qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim and qkv.shape[0] >= n
    if cos is not None:
        assert cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[1] == rotary_dim // 2
        if batch.max_position >= cos.shape[0]:
            raise KernelError(f"position {batch.max_position} is beyond the rotary table of {cos.shape[0]} positions")
    if cache is not None:
        assert cache.k.dtype == qkv.dtype and cache.k.shape[1:] == (n_kv_heads, cache.tokens_per_page, head_dim)
    _check(lib, lib.abk_qkv_prep(
        _p(qkv), _i(_dt(qkv)), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(1 if q_only else 0),
        _p(batch.token_seq),
        _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_len_after), _p(q_norm), _p(k_norm), _f(eps or 0.0),
        _p(cos), _p(sin), _i(rotary_dim), _i(1 if interleaved else 0),
        _p(cache.k if cache is not None else None), _p(cache.v if cache is not None else None),
        _p(cache.page_table if cache is not None else None), _i(cache.table_width if cache is not None else 0),
        _i(cache.ring_pages if cache is not None else 0), _i(cache.tokens_per_page if cache is not None else 1),
        _stream()), "qkv_prep")


def advance_decode(batch):
    """Every row of a decode step one position on, on the device (engine.batch.StepBatch.advance_on_device)."""
    lib = load_module("elementwise")
    _check(lib, lib.abk_advance_decode(_p(batch.token_seq), _p(batch.token_pos), _i(batch.n_rows), _p(batch.seq_pos0),
                                       _p(batch.seq_len_after), _i(batch.n_seqs), _stream()), "advance_decode")


def attention_generic(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, from_step=False):
    """Causal grouped-query attention of every token of the step (src/model.c:197-211).

    q is read from qkv's q columns. Keys and values come from `cache` (a cache.LayerView), or, with
    from_step, from this step's own rows of qkv (only right when every sequence starts at position 0).
    """
    _need_cuda(qkv, out)
    lib = load_module("attention_generic")
    n = batch.n_rows
    row = (n_heads + 2 * n_kv_heads) * head_dim
    assert qkv.is_contiguous() and qkv.shape[1] == row and out.is_contiguous() and out.dtype == qkv.dtype
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n and qkv.shape[0] >= n
    esize = qkv.element_size()
    k_step = ctypes.c_void_p(qkv.data_ptr() + n_heads * head_dim * esize) if from_step else ctypes.c_void_p(0)
    v_step = ctypes.c_void_p(qkv.data_ptr() + (n_heads + n_kv_heads) * head_dim * esize) if from_step else ctypes.c_void_p(0)
    if not from_step:
        assert cache is not None and cache.k.dtype == qkv.dtype
    _check(lib, lib.abk_attention_generic(
        _p(qkv), _ll(row), _p(out), _i(_dt(qkv)), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale),
        _i(window or 0), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_start),
        _p(batch.seq_pos0), _p(cache.k if cache is not None else None), _p(cache.v if cache is not None else None),
        _p(cache.page_table if cache is not None else None), _i(cache.table_width if cache is not None else 0),
        _i(cache.ring_pages if cache is not None else 0), _i(cache.tokens_per_page if cache is not None else 1),
        k_step, v_step, _ll(row), _stream()), "attention")


def gemm_simt(x, w, out, m=None):
    """out[:m] = x[:m] . w^T on the CUDA cores in float32, any sizes (src/model.c:299 and the like)."""
    _need_cuda(x, w, out)
    lib = load_module("gemm_simt")
    m = x.shape[0] if m is None else m
    n, k = w.shape
    assert x.shape[1] == k and out.shape[1] == n and x.shape[0] >= m and out.shape[0] >= m
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib, lib.abk_gemm_simt(_p(x), _i(_dt(x)), _p(w), _i(_dt(w)), _p(out), _i(_dt(out)), _i(m), _i(n), _i(k),
                                  _ll(x.stride(0)), _ll(w.stride(0)), _ll(out.stride(0)), _stream()), "gemm_simt")


def gemm_rows_takes(x, w, out, m):
    """Whether the weight-streaming kernel for a handful of rows takes this product."""
    k = w.shape[1]
    return (m <= 64 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 32 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1)


def gemm_rows(x, w, out, m=None):
    """out[:m] = x[:m] . w^T for m <= 16 rows: the weights stream once through warp-level tensor-core
    products, no scratch memory (src/model.c:299 and the like)."""
    _need_cuda(x, w, out)
    lib = load_module("gemm_rows")
    m = x.shape[0] if m is None else m
    n, k = w.shape
    assert x.shape[1] == k and out.shape[1] == n and x.shape[0] >= m and out.shape[0] >= m
    _check(lib, lib.abk_gemm_rows(_p(x), _p(w), _p(out), _i(_dt(out)), _i(m), _i(n), _i(k), _ll(x.stride(0)),
                                  _ll(w.stride(0)), _ll(out.stride(0)), _stream()), "gemm_rows")


def gemm_rows_swiglu(x, w_gate_up, act, m=None, block=None):
    """act[:m] = silu(x . gate^T) * (x . up^T) for m <= 64 rows, w_gate_up [2 I, K] holding gate and up rows in
    turns of `block` rows (by default all gates, then all ups): the feed-forward's first product and its
    activation in one kernel (src/model.c:307-308)."""
    _need_cuda(x, w_gate_up, act)
    lib = load_module("gemm_rows")
    m = x.shape[0] if m is None else m
    two_i, k = w_gate_up.shape
    assert x.shape[1] == k and act.shape[1] == two_i // 2 and act.dtype == torch.bfloat16 and act.stride(1) == 1
    _check(lib, lib.abk_gemm_rows_swiglu(_p(x), _p(w_gate_up), _p(act), _i(m), _i(two_i // 2), _i(k), _ll(x.stride(0)),
                                         _ll(w_gate_up.stride(0)), _ll(act.stride(0)), _i(block or two_i // 2), _stream()),
           "gemm_rows_swiglu")


def gemm_tc_swiglu_takes(x, w_gate_up, act, m, block):
    """Whether the tensor-core product with the activation in its epilogue takes this: many rows, gate and up
    rows in turns of 128."""
    return (block == 128 and m > 256 and act.dtype == torch.bfloat16 and w_gate_up.shape[0] % 256 == 0
            and act.stride(0) % 8 == 0 and act.data_ptr() % 16 == 0 and gemm_tc_takes(x, w_gate_up, act))


def gemm_tc_swiglu(x, w_gate_up, act, m=None):
    """act[:m] = silu(x . gate^T) * (x . up^T) on the tcgen05 tensor cores for more than 256 rows, w_gate_up
    [2 I, K] holding gate and up rows in turns of 128: the activation runs in the product's epilogue, under the
    next tile's multiplication (src/model.c:307-308)."""
    _need_cuda(x, w_gate_up, act)
    lib = load_module("gemm_tc")
    m = x.shape[0] if m is None else m
    two_i, k = w_gate_up.shape
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and act.dtype == torch.bfloat16
    assert x.shape[1] == k and act.shape[1] == two_i // 2 and x.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1
    _check(lib, lib.abk_gemm_tc_swiglu(_p(x), _p(w_gate_up), _p(act), _i(m), _i(two_i // 2), _i(k), _ll(x.stride(0)),
                                       _ll(w_gate_up.stride(0)), _ll(act.stride(0)), _p(_Scratch.of(x.device).status),
                                       _stream()), "gemm_tc_swiglu")


def gemm_tc_qkv_takes(x, w_qkv, qkv, m, n_heads, n_kv_heads, head_dim, cache, q_norm, k_norm, cos, sin, rotary_dim, interleaved):
    """Whether the q/k/v product of a step takes the preparation of its heads (per-head norm, rotation, keys and values
    into the cache) into its epilogue: many rows, heads of 128, the rotation over the whole head in halves (or none),
    a cache that keeps every page."""
    tensors = [t for t in (q_norm, k_norm, cos, sin, cache.k, cache.v) if t is not None]
    return (m > 256 and head_dim == 128 and qkv.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
            and cache.ring_pages == 0 and w_qkv.shape[0] == (n_heads + 2 * n_kv_heads) * 128 == qkv.shape[1]
            and (cos is None or (rotary_dim == head_dim and not interleaved))
            and all(t.data_ptr() % 16 == 0 for t in tensors) and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0
            and all(t is None or t.dtype == torch.float32 for t in (q_norm, k_norm, cos, sin))
            and gemm_tc_takes(x, w_qkv, qkv))


def gemm_tc_qkv(x, w_qkv, qkv, n_heads, n_kv_heads, batch, q_norm, k_norm, eps, cos, sin, cache, m=None):
    """The q columns of qkv[:m] = the prepared q heads of x . w_qkv^T, and the prepared k and the v heads of every token
    that belongs to a sequence into the cache (cache.LayerKV): the q/k/v product of a prompt on the tcgen05 tensor
    cores with what stands between it and attention in its epilogue (src/model.c:299, 247-259). The k and v columns of
    qkv are not written."""
    _need_cuda(x, w_qkv, qkv)
    lib = load_module("gemm_tc")
    m = x.shape[0] if m is None else m
    assert x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16
    assert x.shape[1] == w_qkv.shape[1] and x.stride(1) == 1 and w_qkv.stride(1) == 1 and qkv.stride(1) == 1
    assert cache.k.shape[1:] == (n_kv_heads, cache.tokens_per_page, 128) and cache.k.is_contiguous() and cache.v.is_contiguous()
    if cos is not None and batch.max_position >= cos.shape[0]:
        raise KernelError(f"position {batch.max_position} is beyond the rotary table of {cos.shape[0]} positions")
    _check(lib, lib.abk_gemm_tc_qkv(
        _p(x), _p(w_qkv), _p(qkv), _i(m), _i(n_heads), _i(n_kv_heads), _i(x.shape[1]), _ll(x.stride(0)), _ll(w_qkv.stride(0)),
        _ll(qkv.stride(0)), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(q_norm), _p(k_norm), _f(eps or 0.0),
        _p(cos), _p(sin), _p(cache.k), _p(cache.v), _p(cache.page_table), _i(cache.table_width), _i(cache.tokens_per_page),
        _p(_Scratch.of(x.device).status), _stream()), "gemm_tc_qkv")


def argmax(logits, out, n_rows=None):
    """out[r] = index of the first maximum of logits[r] (src/main.c:31-36)."""
    _need_cuda(logits, out)
    lib = load_module("sampling")
    n = logits.shape[0] if n_rows is None else n_rows
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32 and out.numel() >= n
    sc = _Scratch.of(logits.device)
    if n > sc.argmax_rows:
        raise KernelRefused(f"argmax: {n} rows are more than the scratch of {sc.argmax_rows} rows")
    _check(lib, lib.abk_argmax(_p(logits), _ll(logits.stride(0)), _i(n), _i(logits.shape[1]), _p(out),
                               _p(sc.argmax_part), _p(sc.argmax_tickets), _stream()), "argmax")


def sample_topk(logits, temperature, top_k, rng_state, out, n_rows=None, rng_index=None):
    """Draw from the top_k logits at a temperature (src/main.c:39-56).

    rng_state int64 holds xorshift64 states; row r uses and advances rng_state[rng_index[r]]
    (rng_state[r] without rng_index).
    """
    _need_cuda(logits, rng_state, out, rng_index)
    lib = load_module("sampling")
    n = logits.shape[0] if n_rows is None else n_rows
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert rng_state.dtype == torch.int64 and out.numel() >= n
    assert rng_index is None or (rng_index.dtype == torch.int32 and rng_index.numel() >= n)
    assert rng_index is not None or rng_state.numel() >= n
    sc = _Scratch.of(logits.device)
    if n > sc.sample_rows:
        raise KernelRefused(f"sample_topk: {n} rows are more than the scratch of {sc.sample_rows} rows")
    _check(lib, lib.abk_sample_topk(_p(logits), _ll(logits.stride(0)), _i(n), _i(logits.shape[1]), _f(temperature),
                                    _i(top_k), _p(rng_state), _p(rng_index), _p(out), _p(sc.sample_part),
                                    _p(sc.sample_tickets), _stream()), "sample_topk")


def sample_all(logits, temperature, rng_state, out, n_rows=None, rng_index=None):
    """Draw from the whole vocabulary at a temperature (top_k = 0): p_j = exp((l_j - l_max) / temperature) over all j,
    walked in index order with abacus's generator (src/main.c:49-55 without the cut to 20 of src/main.c:41)."""
    _need_cuda(logits, rng_state, out, rng_index)
    lib = load_module("sampling")
    lib.abk_sample_all_scratch_bytes.restype = ctypes.c_longlong
    n = logits.shape[0] if n_rows is None else n_rows
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32 and out.numel() >= n
    assert rng_state.dtype == torch.int64
    assert rng_index is None or (rng_index.dtype == torch.int32 and rng_index.numel() >= n)
    assert rng_index is not None or rng_state.numel() >= n
    sc = _Scratch.of(logits.device)
    top = sc.grown("sample_all_top", n, torch.int32)
    sums = sc.grown("sample_all_sums", lib.abk_sample_all_scratch_bytes(_i(n), _i(logits.shape[1])), torch.uint8)
    argmax(logits, top, n)
    _check(lib, lib.abk_sample_all(_p(logits), _ll(logits.stride(0)), _i(n), _i(logits.shape[1]), _f(temperature), _p(top),
                                   _p(rng_state), _p(rng_index), _p(out), _p(sums), _stream()), "sample_all", kernels=2)


def attention(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, from_step=False, ws=None, lists=None,
              prepare=None):
    """Attention of a step: picks the kernel for the phase and sizes; every case the faster kernels
    do not take goes to the general one. lists: the step's tiles and work list for the prefill kernels
    (parts/attention_plan.py: AttentionLists); without them a step of several tokens runs on the general kernel.
    prepare: see attention_decode (only where attention_decode_prepares() said yes for this step)."""
    if (batch.is_decode and not from_step and ws is not None and qkv.dtype == torch.bfloat16
            and attention_decode_takes(n_heads, n_kv_heads, head_dim, cache)):
        attention_decode(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, prepare=prepare)
        return
    assert prepare is None, "q, k and v must be prepared before any kernel but decode attention's"
    if (not batch.is_decode and not from_step and not window and qkv.dtype == torch.bfloat16 and lists is not None
          and attention_prefill_takes(head_dim, cache)):
        attention_prefill(qkv, out, n_heads, n_kv_heads, head_dim, scale, batch, cache, lists)
    else:
        attention_generic(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, from_step=from_step)


PREFILL_ON_MMA = False  # True: head size 128 too runs on the warp-level kernel (for comparison)


def attention_prefill_takes(head_dim, cache):
    return head_dim in (64, 128) and cache.tokens_per_page == 64 and cache.ring_pages == 0


def attention_prefill(qkv, out, n_heads, n_kv_heads, head_dim, scale, batch, cache, lists):
    """Causal attention of whole prompts (or any several tokens per sequence) against the paged bfloat16
    cache, on the tensor cores (src/model.c:197-211). No window. lists: the step's tiles of query rows and the
    work list of the kernel that halves long tiles (parts/attention_plan.py)."""
    _need_cuda(qkv, out)
    n = batch.n_rows
    row = (n_heads + 2 * n_kv_heads) * head_dim
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
    assert qkv.is_contiguous() and qkv.shape[1] == row and out.is_contiguous() and out.shape[1] == n_heads * head_dim
    assert cache.k.is_contiguous() and cache.v.is_contiguous()
    pool_rows = cache.k.shape[0] * cache.k.shape[1] * cache.k.shape[2]
    if head_dim == 128 and not PREFILL_ON_MMA:  # tcgen05: tiles of 128 query rows, scores and output in tensor memory
        lib = load_module("attention_tc")
        work = lists.work  # what each CTA does: whole tiles, long tiles twice
        sc = _Scratch.of(qkv.device)
        room = sc.attention_halves_pairs // n_heads
        if lists.n_halved > room:
            raise KernelRefused(f"attention_prefill_tc: the step halves {lists.n_halved} tiles, its scratch memory holds "
                                f"{room} for {n_heads} heads (the lists were made for another number of heads)")
        _check(lib, lib.abk_attention_prefill_tc(
            _p(qkv), _ll(row), _i(n), _p(out), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _p(work),
            _i(work.shape[0]), _i(room), _p(sc.attention_halves), _p(sc.attention_halves_tickets), _p(cache.k), _p(cache.v), _ll(pool_rows), _p(cache.page_table), _i(cache.table_width),
            _i(cache.tokens_per_page), _p(kernel_status(qkv.device)), _stream()), "attention_prefill_tc")
        return
    lib = load_module("attention_mma")
    tiles = lists.tiles(64)
    _check(lib, lib.abk_attention_prefill(
        _p(qkv), _ll(row), _i(n), _p(out), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _p(tiles),
        _i(tiles.shape[0]), _p(batch.seq_start), _p(batch.seq_pos0), _p(batch.seq_len_after), _p(batch.seq_slot),
        _p(cache.k), _p(cache.v), _ll(pool_rows), _p(cache.page_table), _i(cache.table_width),
        _i(cache.tokens_per_page), _p(kernel_status(qkv.device)), _stream()), "attention_prefill")


def attention_decode_prepares(qkv, n_heads, n_kv_heads, head_dim, cache, q_norm, k_norm, cos, sin, rotary_dim, interleaved):
    """Whether decode attention takes the q/k/v preparation (per-head norm, rotation, the new token's key and value
    into the cache) into its own kernel: on the tensor-core kernel, with the rotation over the whole head in halves
    (or none), and everything 16-byte aligned."""
    tensors = [t for t in (qkv, q_norm, k_norm, cos, sin, cache.k, cache.v) if t is not None]
    return (qkv.dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads // n_kv_heads <= 16
            and attention_decode_takes(n_heads, n_kv_heads, head_dim, cache)
            and (cos is None or (rotary_dim == head_dim and not interleaved))
            and all(t.data_ptr() % 16 == 0 for t in tensors) and qkv.stride(0) % 8 == 0
            and all(t is None or t.dtype == torch.float32 for t in (q_norm, k_norm, cos, sin)))


def _attention_decode_mma(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, max_positions,
                          prepare=None):
    lib = load_module("attention_decode_ring")
    n = batch.n_rows
    row = (n_heads + 2 * n_kv_heads) * head_dim
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
    assert qkv.is_contiguous() and qkv.shape[1] == row and out.is_contiguous() and out.shape[1] == n_heads * head_dim
    max_positions = max_positions or getattr(batch, "position_bound", None) or batch.max_len_after
    if batch.max_len_after > max_positions:
        raise KernelError(f"a row at position {batch.max_len_after - 1} is beyond the bound {max_positions}")
    pool_rows = cache.k.shape[0] * cache.k.shape[1] * cache.k.shape[2]
    if prepare is not None:
        cos = prepare["cos"]
        if cos is not None and batch.max_position >= cos.shape[0]:
            raise KernelError(f"position {batch.max_position} is beyond the rotary table of {cos.shape[0]} positions")
        _check(lib, lib.abk_attention_decode_ring_prepare(
            _p(qkv), _ll(row), _p(out), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _i(window or 0),
            _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(cache.k), _p(cache.v), _ll(pool_rows),
            _p(cache.page_table), _i(cache.table_width), _i(cache.ring_pages), _i(cache.tokens_per_page),
            _i(max_positions), _p(prepare["q_norm"]), _p(prepare["k_norm"]), _f(prepare["eps"] or 0.0), _p(cos),
            _p(prepare["sin"]), _i(1 if prepare["keep"] else 0), _p(kernel_status(qkv.device)), _stream()),
            "attention_decode_mma")
        return
    _check(lib, lib.abk_attention_decode_ring(
        _p(qkv), _ll(row), _p(out), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _i(window or 0),
        _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(cache.k), _p(cache.v), _ll(pool_rows),
        _p(cache.page_table), _i(cache.table_width), _i(cache.ring_pages), _i(cache.tokens_per_page),
        _i(max_positions), _p(kernel_status(qkv.device)), _stream()), "attention_decode_mma")


def attention_decode_takes(n_heads, n_kv_heads, head_dim, cache):
    group = n_heads // n_kv_heads
    smem = 4 * 64 * head_dim * 2 + 4 * group * (head_dim + 2) * 4 + 64
    return head_dim in (64, 128, 256) and cache.tokens_per_page == 64 and smem <= 200 * 1024


def attention_decode(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws, max_positions=None,
                     simt=False, prepare=None):
    """One new token per row against the paged bfloat16 cache, split along the keys (src/model.c:197-211).

    Head sizes 64 and 128 with groups of up to 16 query heads run on the tensor cores (mma.sync);
    head size 256, larger groups, or simt=True, on the CUDA cores.
    max_positions bounds every row's position + 1 (it sizes the grid and the scratch); by default
    the step's own maximum. A captured graph passes the bound it was captured for.
    prepare: dict(q_norm, k_norm, eps, cos, sin, keep) where attention_decode_prepares() says so: qkv is as the
    product left it, and the kernel norms and rotates q and k and (keep) writes the new key and value to the cache
    itself (src/model.c:247-259).
    """
    _need_cuda(qkv, out)
    if not simt and head_dim in (64, 128) and n_heads // n_kv_heads <= 16:
        return _attention_decode_mma(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, batch, cache, ws,
                                     max_positions, prepare)
    assert prepare is None, "only the tensor-core kernel prepares q, k and v itself"
    lib = load_module("attention_decode")
    lib.abk_attention_decode_scratch_floats.restype = ctypes.c_longlong
    n = batch.n_rows
    row = (n_heads + 2 * n_kv_heads) * head_dim
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
    assert qkv.is_contiguous() and qkv.shape[1] == row and out.is_contiguous() and out.shape[1] == n_heads * head_dim
    max_positions = max_positions or getattr(batch, "position_bound", None) or batch.max_len_after
    if batch.max_len_after > max_positions:
        raise KernelError(f"a row at position {batch.max_len_after - 1} is beyond the bound {max_positions}")
    chunks = -(-max_positions // 128)
    floats = lib.abk_attention_decode_scratch_floats(_i(n), _i(n_heads), _i(head_dim), _i(chunks))
    scratch = ws.get("attention_partials", (floats,), torch.float32)
    _check(lib, lib.abk_attention_decode(
        _p(qkv), _ll(row), _p(out), _i(n), _i(n_heads), _i(n_kv_heads), _i(head_dim), _f(scale), _i(window or 0),
        _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(cache.k), _p(cache.v), _p(cache.page_table),
        _i(cache.table_width), _i(cache.ring_pages), _i(cache.tokens_per_page), _i(max_positions), _p(scratch),
        _p(_attention_tickets(qkv.device, n * n_kv_heads)), _p(kernel_status(qkv.device)), _stream()),
        "attention_decode")


class _Scratch:
    """Per-device scratch of the kernels that need some: split-K partial tiles and their tickets,
    attention partials, and the status words a kernel sets when one of its bounded waits runs out."""
    _of_device = {}

    def __init__(self, device):
        self.device = device
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.argmax_rows = 4096
        self._made = {}

    def grown(self, name, count, dtype):
        """A buffer of at least `count` elements that is kept and only ever replaced by a larger one."""
        have = self._made.get(name)
        if have is None or have.numel() < count or have.dtype != dtype:
            have = self._made[name] = guards.empty(max(int(count), 1), dtype, self.device, what=f"scratch {name}")
        return have

    def _lazy(self, name, make):
        # each kernel's scratch is made at that kernel's first use, so that a model loads
        # (and compiles) only the kernel libraries it runs
        if name not in self._made:
            self._made[name] = make()
        return self._made[name]

    @property
    def gemm_floats(self):
        def make():
            lib = load_module("gemm_tc")
            lib.abk_gemm_tc_scratch_floats.restype = ctypes.c_longlong
            return guards.empty(lib.abk_gemm_tc_scratch_floats(), torch.float32, self.device, what="scratch of split K")
        return self._lazy("gemm_floats", make)

    @property
    def gemm_tickets(self):
        return self._lazy("gemm_tickets", lambda: guards.zeros(load_module("gemm_tc").abk_gemm_tc_scratch_tickets(),
                                                               torch.int32, self.device, what="tickets of split K"))

    @property
    def argmax_part(self):
        return self._lazy("argmax_part", lambda: guards.empty(
            self.argmax_rows * load_module("sampling").abk_argmax_slices() * 2, torch.float32, self.device, what="scratch of argmax"))

    sample_rows = 1024

    @property
    def sample_part(self):
        def make():
            lib = load_module("sampling")
            lib.abk_sample_topk_scratch_bytes.restype = ctypes.c_longlong
            return guards.empty(lib.abk_sample_topk_scratch_bytes(_i(self.sample_rows)), torch.uint8, self.device,
                                what="scratch of sampling")
        return self._lazy("sample_part", make)

    @property
    def sample_tickets(self):
        return self._lazy("sample_tickets", lambda: guards.zeros(self.sample_rows, torch.int32, self.device, what="tickets of sampling"))

    @property
    def argmax_tickets(self):
        return self._lazy("argmax_tickets", lambda: guards.zeros(self.argmax_rows, torch.int32, self.device, what="tickets of argmax"))

    attention_halves_pairs = 384  # (tile, head) pairs the prefill attention may halve in one launch (parts/attention_plan.py)

    @property
    def attention_halves(self):
        def make():
            lib = load_module("attention_tc")
            lib.abk_attention_prefill_tc_scratch_floats.restype = ctypes.c_longlong
            floats = lib.abk_attention_prefill_tc_scratch_floats(_i(self.attention_halves_pairs), _i(1))
            return guards.empty(floats, torch.float32, self.device, what="scratch of halved attention tiles")
        return self._lazy("attention_halves", make)

    @property
    def attention_halves_tickets(self):
        return self._lazy("attention_halves_tickets",
                          lambda: guards.zeros(2 * self.attention_halves_pairs, torch.int32, self.device,
                                               what="tickets of halved attention tiles"))

    @property
    def attention_tickets(self):
        return self._lazy("attention_tickets", lambda: guards.zeros(1 << 18, torch.int32, self.device, what="tickets of decode attention"))

    @classmethod
    def of(cls, device):
        key = (device.type, device.index)
        if key not in cls._of_device:
            cls._of_device[key] = cls(device)
        return cls._of_device[key]


def _attention_tickets(device, n):
    sc = _Scratch.of(device)
    if n > sc.attention_tickets.numel():
        raise KernelRefused(f"attention_decode: {n} (row, kv head) pairs are more than its {sc.attention_tickets.numel()} tickets")
    return sc.attention_tickets


def set_wait_limit_ns(ns, modules=("utility",)):
    """The limit of the bounded waits (on barriers, on another CTA's flag) of the named kernel libraries on the current
    device: a wait that has not been satisfied after `ns` nanoseconds gives up, the kernel sets its status word and
    returns. The libraries start at a quarter of a second."""
    for module in modules:
        lib = load_module(module)
        rc = lib.abk_set_wait_limit_ns(ctypes.c_ulonglong(int(ns)))
        if rc:
            raise KernelError(f"set_wait_limit_ns({module}): CUDA error {rc}")


def wait_that_runs_out(status, bit=4, word=1):
    """Launches the kernel whose one wait nothing can satisfy (csrc/utility.cu): after the utility library's limit it
    sets `bit` in status[word] and returns. For walking the way from a wait that ran out to the host's exception."""
    _need_cuda(status)
    lib = load_module("utility")
    assert status.dtype == torch.int32 and status.numel() > word
    _check(lib, lib.abk_wait_that_runs_out(ctypes.c_void_p(status.data_ptr() + 4 * word), _i(bit), _stream()),
           "wait_that_runs_out")


def kernel_status(device):
    """Status words of the device's kernels: all zero unless a kernel gave up on a wait."""
    return _Scratch.of(device).status


def gemm_tc_takes(x, w, out):
    """Whether the tensor-core kernel takes this product (else the CUDA-core kernel runs it):
    bfloat16 operands, K and both row pitches multiples of 8, 16-byte aligned."""
    k = w.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1)


def gemm_tc(x, w, out, m=None, tile_n=0, swap=-1, splits=0, persistent=-1):
    """out[:m] = x[:m] . w^T in bfloat16 on the tcgen05 tensor cores, float32 accumulation.

    tile_n, swap, splits and persistent pin the tile configuration (tests); 0 / -1 / 0 / -1 let the
    kernel choose.
    """
    _need_cuda(x, w, out)
    lib = load_module("gemm_tc")
    sc = _Scratch.of(x.device)
    m = x.shape[0] if m is None else m
    n, k = w.shape
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.shape[1] == k and out.shape[1] == n and x.shape[0] >= m and out.shape[0] >= m
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib, lib.abk_gemm_tc(_p(x), _p(w), _p(out), _i(_dt(out)), _i(m), _i(n), _i(k), _ll(x.stride(0)),
                                _ll(w.stride(0)), _ll(out.stride(0)), _p(sc.gemm_floats), _p(sc.gemm_tickets),
                                _p(sc.status), _i(tile_n), _i(swap), _i(splits), _i(persistent), _stream()), "gemm_tc")
