"""abk_attention_decode_noalloc, called through its exported C symbol.

This is the entry point for callers that cannot allocate device memory themselves (a process
whose whole GPU memory belongs to its own pool, a loop that cannot afford cudaMalloc's
synchronisation, a plugin inside someone else's process): its scratch is an array inside the
library. The test gives it inputs and an output it made itself, like such a caller would, and
checks the result on two calls in a row that share the built-in array: against plain attention
over the keys and values gathered from the pages (an oracle that shares nothing with the kernel:
windows, both page sizes' edges, the padding rows and the second call are all held to it), and,
bit for bit, against abk_attention_decode, which takes its scratch as an argument. The file's name
makes pytest collect it last.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HQ, HKV, HD = 16, 8, 128


def _setup(lengths, seed):
    """A paged cache holding random keys and values for sequences of the given lengths, and one decode
    row per sequence."""
    from abacus_b200.cache import CacheNeed, SequenceCache
    from abacus_b200.engine.batch import Sequence, StepBatch
    g = torch.Generator(device="cuda").manual_seed(seed)
    cache = SequenceCache([CacheNeed(HKV, HD)], [None], 64 * 40, torch.bfloat16, "cuda", max_context=1024)
    kv = cache.views[0].kv
    kv.k.copy_(torch.randn(kv.k.shape, generator=g, device="cuda"))
    kv.v.copy_(torch.randn(kv.v.shape, generator=g, device="cuda"))
    seqs = []
    for n in lengths:
        slot = cache.open_slot()
        cache.reserve(slot, n)
        seqs.append(Sequence(slot, [0], n - 1, []))
    batch = StepBatch(len(lengths) + 2, len(lengths), 0, "cuda").fill(seqs)  # two padding rows
    qkv = torch.randn(batch.n_rows, (HQ + 2 * HKV) * HD, generator=g, device="cuda").to(torch.bfloat16)
    return cache, kv, batch, qkv


def _call_noalloc(lib, qkv, out, batch, kv, window, max_positions, status):
    i, ll, f, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, lambda t: ctypes.c_void_p(t.data_ptr())
    return lib.abk_attention_decode_noalloc(
        p(qkv), ll(qkv.shape[1]), p(out), i(batch.n_rows), i(HQ), i(HKV), i(HD), f(HD ** -0.5), i(window),
        p(batch.token_seq), p(batch.token_pos), p(batch.seq_slot), p(kv.k), p(kv.v), p(kv.page_table),
        i(kv.table_width), i(kv.ring_pages), i(kv.tokens_per_page), i(max_positions), p(status),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _plain_attention(qkv, lengths, kv, window):
    """What plain attention gives for each sequence's last position, from the keys and values its pages hold
    (sequence i sits in slot i: slots are handed out lowest first)."""
    from plain import qwen3_plain as plain
    k_pool, v_pool = kv.k.float().cpu().numpy(), kv.v.float().cpu().numpy()  # [pages, kv heads, 64, hd]
    table = kv.page_table.cpu().numpy()
    rows = []
    for i, n in enumerate(lengths):
        pages = table[i, :-(-n // 64)]
        k = np.concatenate([k_pool[p] for p in pages], axis=1)[:, :n].transpose(1, 0, 2)  # [n, kv heads, hd]
        v = np.concatenate([v_pool[p] for p in pages], axis=1)[:, :n].transpose(1, 0, 2)
        q = np.zeros((n, HQ, HD), dtype=np.float32)  # only the last position's query is the row's
        q[-1] = qkv[i, :HQ * HD].float().cpu().numpy().reshape(HQ, HD)
        rows.append(plain.attention(q, k, v, window or None, rnd=plain.bf16_round)[-1].reshape(-1))
    return np.stack(rows)


def test_noalloc_entry_point_matches_the_one_with_a_scratch_argument():
    from abacus_b200.kernels import load_module, ops
    from abacus_b200.parts import Workspace
    lib = load_module("attention_decode_static")
    assert hasattr(lib, "abk_attention_decode_noalloc")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ws = Workspace(torch.device("cuda", 0))
    # two calls in a row on the same built-in array, of different shapes: the second must not see the first
    for call, (lengths, window) in enumerate([([700, 1, 130, 257, 64], 0), ([65, 512, 383], 200)]):
        cache, kv, batch, qkv = _setup(lengths, seed=call)
        want = torch.full((batch.n_rows, HQ * HD), 3.0, dtype=torch.bfloat16, device="cuda")
        ops.attention_decode(qkv, want, HQ, HKV, HD, HD ** -0.5, window or None, batch, kv, ws, simt=True)
        got = torch.full((batch.n_rows, HQ * HD), 5.0, dtype=torch.bfloat16, device="cuda")
        rc = _call_noalloc(lib, qkv, got, batch, kv, window, batch.max_len_after, status)
        assert rc == 0, lib.abk_last_error().decode()
        torch.cuda.synchronize()
        # against plain attention, at the tolerance of the kernel tests: one bfloat16 rounding of the result
        np.testing.assert_allclose(got[:len(lengths)].float().cpu().numpy(), _plain_attention(qkv, lengths, kv, window),
                                   rtol=2 ** -7, atol=2 ** -7, err_msg=f"call {call}")
        # and the same bits as the entry point that is given its scratch: same kernels, same order of summation
        assert torch.equal(got, want), f"call {call}"
        assert float(got[len(lengths):].float().abs().sum()) == 0.0  # padding rows
    assert status.tolist() == [0, 0, 0, 0]


def test_a_row_beyond_the_bound_is_reported_not_computed():
    """max_positions sizes the grid; a row at or beyond it has no CTA for its last chunks. The kernel says so in the
    status word, writes zeros for that row and leaves the tickets at zero, so that the next call finds them as it must."""
    from abacus_b200.kernels import load_module
    lib = load_module("attention_decode_static")
    lengths = [300, 40]
    cache, kv, batch, qkv = _setup(lengths, seed=4)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.full((batch.n_rows, HQ * HD), 5.0, dtype=torch.bfloat16, device="cuda")
    assert _call_noalloc(lib, qkv, out, batch, kv, 0, 256, status) == 0  # the first row is at position 299
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 2, 0]
    assert float(out[0].float().abs().sum()) == 0.0
    np.testing.assert_allclose(out[1:2].float().cpu().numpy(), _plain_attention(qkv, lengths, kv, 0)[1:2], rtol=2 ** -7, atol=2 ** -7)
    status.zero_()
    assert _call_noalloc(lib, qkv, out, batch, kv, 0, 320, status) == 0  # with the right bound all is well
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    np.testing.assert_allclose(out[:2].float().cpu().numpy(), _plain_attention(qkv, lengths, kv, 0), rtol=2 ** -7, atol=2 ** -7)


def test_noalloc_entry_point_refuses_what_its_array_cannot_hold():
    from abacus_b200.kernels import load_module
    lib = load_module("attention_decode_static")
    cache, kv, batch, qkv = _setup([100, 5], seed=9)
    out = torch.zeros(batch.n_rows, HQ * HD, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = _call_noalloc(lib, qkv, out, batch, kv, 0, 1 << 20, status)  # a bound of a million positions
    assert rc == -1 and "floats of scratch" in lib.abk_last_error().decode()
    assert float(out.float().abs().sum()) == 0.0  # nothing ran
