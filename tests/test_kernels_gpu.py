"""Each kernel alone against its plain reference, at sizes the engine's tiny models do not use."""
import numpy as np
import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from abacus_b200.kernels import ops
    return ops


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def bf(a):
    return plain.bf16_round(np.asarray(a, dtype=np.float32))


def close(got, want, dtype):
    got = got.float().cpu().numpy()
    if dtype == torch.float32:
        np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-6)
    else:  # one bfloat16 rounding of the result: 2^-8 relative, plus float32 noise
        np.testing.assert_allclose(got, want, rtol=2 ** -7, atol=1e-6)


def test_random_fill_is_the_same_bits_on_the_device_and_on_the_host(ops):
    """The counter-based normal fill (csrc/utility.cu) against its numpy twin, for matrices and norm weights, both
    dtypes, a slice that starts in the middle of a tensor, and a tensor too long for one pass of the grid."""
    from abacus_b200.weights import random_init as ri
    for name, shape in [("a.weight", (37, 129)), ("b.norm", (515,)), ("c", (1100, 1000))]:
        for scales in (None, {"norm": 2.5, "a.": 4.0}):
            host = ri.random_tensor(name, shape, seed=9, std=0.02, norm_std=0.1, scales=scales)
            device = ri.random_tensor(name, shape, seed=9, std=0.02, norm_std=0.1, scales=scales, device="cuda")
            assert device.dtype == torch.bfloat16 and torch.equal(device.cpu().view(torch.int16), host.view(torch.int16))
    key = ri.tensor_key(3, "model.layers.0.mlp.down_proj.weight")
    out = torch.empty(5000, dtype=torch.float32, device="cuda")
    ops.fill_normal(out, key, 1.0, 0.37, first=123457)
    assert np.array_equal(out.cpu().numpy(), ri.normal_values(key, 123457, 5000, 1.0, 0.37))
    z = ri.unit_normal(key, 0, 1 << 18)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1.0) < 0.01 and float(np.abs(z).max()) <= 6.0
    assert ri.tensor_key(3, "a") != ri.tensor_key(4, "a") != ri.tensor_key(4, "b")


def test_guard_words_show_a_store_outside_a_buffer(ops):
    """A buffer made by kernels/guards.py has 256 bytes of a pattern on either side. Overwriting one of them (here with
    a plain copy into the allocation's own guard: nothing outside it is touched) is found by the check, and named."""
    from abacus_b200.kernels import guards
    t = guards.zeros((3, 50), torch.float32, "cuda", what="a test buffer")
    assert t.shape == (3, 50) and float(t.abs().sum()) == 0.0 and guards.check()[0] == 0
    whole = t.guarded_allocation
    after = guards.GUARD_BYTES + 768  # 600 bytes of data, rounded up to 768: the guard behind starts here
    saved = whole[after:after + 8].clone()
    whole[after + 4:after + 8] = 0  # what a kernel that stored one float too far would have done
    damaged, where = guards.check()
    assert damaged == 1 and where == ["a test buffer"]
    with pytest.raises(RuntimeError, match="a test buffer"):
        guards.assert_intact()
    whole[after:after + 8] = saved
    assert guards.check()[0] == 0


def test_embed(ops):
    rng = np.random.default_rng(0)
    table = bf(rng.standard_normal((1000, 72)))
    tokens = rng.integers(0, 1000, 33)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for tdtype in (torch.bfloat16, torch.float32):
        x = torch.empty(33, 72, device="cuda")
        ops.embed(dev(tokens, torch.int32), dev(table, tdtype), x, status)
        np.testing.assert_array_equal(x.cpu().numpy(), plain.embed(tokens, table))
    assert status.tolist() == [0, 0, 0, 0]
    ops.embed(dev([5, 1000, 7], torch.int32), dev(table), torch.empty(3, 72, device="cuda"), status)
    assert status[0].item() == 1  # a token outside the vocabulary is reported, not read


@pytest.mark.parametrize("d", [200, 72, 1030, 4096])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(ops, d, out_dtype):
    rng = np.random.default_rng(d)
    x, y = rng.standard_normal((7, d)).astype(np.float32), rng.standard_normal((7, d)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    eps = 3e-5
    xd, out = dev(x), torch.empty(7, d, dtype=out_dtype, device="cuda")
    ops.add_rmsnorm(xd, dev(y), dev(w), out, eps)
    np.testing.assert_array_equal(xd.cpu().numpy(), x + y)  # the residual stream is updated
    close(out, plain.rmsnorm(x + y, w, eps), out_dtype)
    xd = dev(x)
    ops.add_rmsnorm(xd, None, dev(w), out, eps)
    close(out, plain.rmsnorm(x, w, eps), out_dtype)
    rows = [6, 0, 3, 3]
    xd, out = dev(x), torch.empty(4, d, dtype=out_dtype, device="cuda")
    ops.add_rmsnorm(xd, dev(y), dev(w), out, eps, rows=dev(rows, torch.int32))
    close(out, plain.rmsnorm((x + y)[rows], w, eps), out_dtype)
    np.testing.assert_array_equal(xd.cpu().numpy(), x)  # with rows, x is left alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(ops, dtype):
    rng = np.random.default_rng(1)
    gu = (3 * rng.standard_normal((9, 2 * 100))).astype(np.float32)
    if dtype == torch.bfloat16:
        gu = bf(gu)
    act = torch.empty(9, 100, dtype=dtype, device="cuda")
    ops.swiglu(dev(gu, dtype), act)
    close(act, plain.swiglu(gu), dtype)
    # gate and up in turns of 20 columns instead of all gates and then all ups
    turns = np.concatenate([np.concatenate([gu[:, b:b + 20], gu[:, 100 + b:100 + b + 20]], -1) for b in range(0, 100, 20)], -1)
    ops.swiglu(dev(turns, dtype), act, block=20)
    close(act, plain.swiglu(gu), dtype)


@pytest.mark.parametrize("m, n, k", [(5, 37, 50), (1, 389, 96), (130, 70, 33), (64, 64, 16), (3, 1, 7)])
def test_gemm_simt(ops, m, n, k):
    rng = np.random.default_rng(m * n + k)
    x, w = rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((n, k)).astype(np.float32)
    out = torch.empty(m, n, device="cuda")
    ops.gemm_simt(dev(x), dev(w), out)
    np.testing.assert_allclose(out.cpu().numpy(), plain.linear(x, w), rtol=1e-5, atol=1e-5)
    xb, wb = bf(x), bf(w)
    for odt in (torch.float32, torch.bfloat16):
        out = torch.empty(m, n, dtype=odt, device="cuda")
        ops.gemm_simt(dev(xb, torch.bfloat16), dev(wb, torch.bfloat16), out)
        close(out, plain.linear(xb, wb), odt) if odt == torch.bfloat16 else np.testing.assert_allclose(
            out.cpu().numpy(), plain.linear(xb, wb), rtol=1e-5, atol=1e-5)


def test_gemm_simt_rows_do_not_depend_on_the_batch(ops):
    """The float32 product sums over k in one fixed order: a row alone equals the row in a batch, bit for bit."""
    rng = np.random.default_rng(5)
    x, w = rng.standard_normal((77, 300)).astype(np.float32), rng.standard_normal((101, 300)).astype(np.float32)
    whole = torch.empty(77, 101, device="cuda")
    ops.gemm_simt(dev(x), dev(w), whole)
    for r in (0, 63, 64, 76):
        one = torch.empty(1, 101, device="cuda")
        ops.gemm_simt(dev(x[r:r + 1]), dev(w), one)
        assert torch.equal(one[0], whole[r])


def test_argmax_takes_the_first_maximum(ops):
    rng = np.random.default_rng(2)
    logits = rng.standard_normal((6, 5003)).astype(np.float32)
    logits[1, 4000] = logits[1, 77] = 9.0
    logits[2, 5002] = 10.0
    logits[3, :] = 0.5
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.argmax(dev(logits), out)
    assert out.tolist() == [plain.argmax(r) for r in logits]
    assert out[1].item() == 77 and out[2].item() == 5002 and out[3].item() == 0


@pytest.mark.parametrize("temp, top_k", [(0.8, 20), (1.7, 5), (0.3, 64)])
def test_sample_topk_draws_what_the_plain_sampler_draws(ops, temp, top_k):
    rng = np.random.default_rng(3)
    vocab, rows = 2311, 16
    logits = (2 * rng.standard_normal((rows, vocab))).astype(np.float32)
    logits[4, 100] = logits[4, 50] = logits[4].max() + 1  # a tie at the top
    logits[5, :] = 1.0  # all equal: the first top_k indices
    states = [int(s) for s in rng.integers(1, 2 ** 62, rows)]
    st = dev(states, torch.int64)
    index = dev(list(range(rows))[::-1], torch.int32)  # row r uses state rows-1-r
    ld, out = dev(logits), torch.empty(rows, dtype=torch.int32, device="cuda")
    want_states = list(states)
    for step in range(5):
        ops.sample_topk(ld, temp, top_k, st, out, rng_index=index)
        got = out.tolist()
        for r in range(rows):
            tok, want_states[rows - 1 - r] = plain.sample(logits[r], temp, want_states[rows - 1 - r], top_k)
            assert got[r] == tok, (step, r)
    assert [v % (1 << 64) for v in st.tolist()] == want_states  # int64 bit patterns of uint64 states
    with pytest.raises(ops.KernelRefused):
        ops.sample_topk(ld, temp, 65, st, out)
    with pytest.raises(ops.KernelRefused):
        ops.sample_topk(ld, 0.0, 5, st, out)


@pytest.mark.parametrize("vocab, temp", [(2311, 0.8), (70001, 1.3), (151936, 0.6), (1024, 2.0), (5, 1.0)])
def test_sampling_from_the_whole_vocabulary(ops, vocab, temp):
    """top_k = 0: every token can be drawn. The same tokens as the plain sampler, row by row and draw by draw; rows with
    ties, with all logits equal, with -inf entries; and over many draws from a short row, every token with its share."""
    rng = np.random.default_rng(vocab)
    rows = 12
    logits = (2 * rng.standard_normal((rows, vocab))).astype(np.float32)
    logits[1, :] = 0.25                                   # all equal: uniform over the vocabulary
    logits[2, vocab // 2:] = np.float32(-np.inf)          # half of the tokens impossible
    logits[3, [0, vocab - 1]] = logits[3].max() + 3.0     # a tie at the top, first and last token
    states = [int(s) for s in rng.integers(1, 2 ** 62, rows)]
    st, want_states = dev(states, torch.int64), list(states)
    index = dev(list(range(rows))[::-1], torch.int32)
    ld, out = dev(logits), torch.empty(rows, dtype=torch.int32, device="cuda")
    for step in range(6):
        ops.sample_all(ld, temp, st, out, rng_index=index)
        got = out.tolist()
        for r in range(rows):
            tok, want_states[rows - 1 - r] = plain.sample(logits[r], temp, want_states[rows - 1 - r], top_k=0)
            assert got[r] == tok, (step, r)
        assert got[2] < vocab // 2 or vocab < 4
    assert [v % (1 << 64) for v in st.tolist()] == want_states
    if vocab == 5:  # the shares: 4,000 draws from five tokens
        flat = dev(np.tile(np.array([[0.0, 1.0, -1.0, 0.5, 0.0]], dtype=np.float32), (1000, 1)))
        st = dev([int(s) for s in rng.integers(1, 2 ** 62, 1000)], torch.int64)
        out, counts = torch.empty(1000, dtype=torch.int32, device="cuda"), np.zeros(5)
        for _ in range(4):
            ops.sample_all(flat, 1.0, st, out)
            counts += np.bincount(out.cpu().numpy(), minlength=5)
        p = np.exp([0.0, 1.0, -1.0, 0.5, 0.0])
        assert np.abs(counts / 4000 - p / p.sum()).max() < 0.03


def test_a_zero_seed_draws_like_any_other():
    """xorshift64 cannot leave state 0, so the sampler never starts a request there: with seed 0 and a temperature the
    first request's draws from a flat row are not all the first token (which a dead stream would give)."""
    from abacus_b200.sampling import Sampler
    sampler = Sampler(torch.device("cuda", 0), temperature=1.0, top_k=20, seed=0)
    states = sampler.states([0, 1])
    assert 0 not in states.tolist()
    flat = torch.zeros(2, 500, device="cuda")
    drawn = [sampler.sample(flat, states).tolist() for _ in range(12)]
    assert len({d[0] for d in drawn}) > 3 and len({d[1] for d in drawn}) > 3


@pytest.mark.parametrize("top_k", [20, 64])
def test_sample_topk_on_a_large_vocabulary(ops, top_k):
    """Slices of more than a thousand logits take the two-pass way (a bound from the threads' maxima, then the
    candidates above it): random rows, the top spread over slices or crowded into one, ties across slices, and
    rows with so many equal logits at the top that the candidates overflow and the slice is searched one by one."""
    rng = np.random.default_rng(5)
    vocab, rows, temp = 70001, 7, 0.8
    logits = (2 * rng.standard_normal((rows, vocab))).astype(np.float32)
    logits[1, 30000:30100] += 9.0                       # the whole top in one slice
    logits[2, [5, 2200, 40000, 69999]] = 11.0           # equal maxima in four slices
    logits[3, :] = -2.5                                 # all equal: the first top_k indices, by the slow way
    logits[4, 1000:4000] = 7.0                          # three thousand equal maxima: overflow in two slices
    logits[5, :] = np.float32(-np.inf)
    logits[5, 123], logits[5, 60000] = 0.5, 0.25        # fewer finite logits than top_k
    states = [int(s) for s in rng.integers(1, 2 ** 62, rows)]
    st, want_states = dev(states, torch.int64), list(states)
    ld, out = dev(logits), torch.empty(rows, dtype=torch.int32, device="cuda")
    for step in range(4):
        ops.sample_topk(ld, temp, top_k, st, out)
        got = out.tolist()
        for r in range(rows):
            tok, want_states[r] = plain.sample(logits[r], temp, want_states[r], top_k)
            assert got[r] == tok, (step, r)
    from abacus_b200.kernels.ops import _Scratch
    assert int(_Scratch.of(torch.device("cuda", 0)).sample_tickets.abs().sum()) == 0


# ------------------------------------------------------------------ q/k/v preparation and attention

class Harness:
    """A cache and steps for one attention layer, without a model around it."""

    def __init__(self, hq, hkv, hd, dtype, window=None, max_tokens=64 * 24):
        from abacus_b200.cache import CacheNeed, SequenceCache
        self.hq, self.hkv, self.hd, self.dtype, self.window = hq, hkv, hd, dtype, window
        self.cache = SequenceCache([CacheNeed(hkv, hd, window)], [None], max_tokens, dtype, "cuda", max_context=1024)

    def step(self, ops, seqs, qkv, q_norm, k_norm, eps, cos, sin, rotary_dim, interleaved, scale, from_step=False,
             general=True, simt=False, prepares=False):
        """seqs: [(slot, n_new)]; qkv float32 numpy [rows, (hq + 2 hkv) * hd]. Returns attention output.
        general=False lets ops.attention pick the kernel for the phase, as the model does; simt=True sends a decode
        step to the CUDA-core decode kernel whatever the head size; prepares=True leaves the preparation of q, k and v
        to the decode attention kernel."""
        from abacus_b200.engine.batch import Sequence, StepBatch
        ss = []
        for slot, n in seqs:
            ss.append(Sequence(slot, [0] * n, self.cache.length[slot], []))
            self.cache.reserve(slot, self.cache.length[slot] + n)
        rows = sum(n for _, n in seqs)
        from abacus_b200.parts.attention_plan import AttentionLists, AttentionStepPlan
        plan = AttentionStepPlan(self.hq)
        batch = self.last_batch = StepBatch(rows + 3, len(seqs) + 1, 0, "cuda", plans=[plan]).fill(ss)  # three padding rows at the end
        lists = self.last_lists = AttentionLists(batch.plan[plan.name])
        pad = np.full((3, qkv.shape[1]), 7.0, dtype=np.float32)
        q = dev(np.concatenate([qkv, pad]), self.dtype)
        kv = self.cache.views[0].kv
        prepare = None
        if prepares:
            assert ops.attention_decode_prepares(q, self.hq, self.hkv, self.hd, kv, q_norm, k_norm, cos, sin, rotary_dim, interleaved)
            prepare = dict(q_norm=q_norm, k_norm=k_norm, eps=eps, cos=cos, sin=sin, keep=True)
        else:
            ops.qkv_prep(q, self.hq, self.hkv, self.hd, batch, q_norm, k_norm, eps, cos, sin, rotary_dim, interleaved, kv)
        out = torch.full((rows + 3, self.hq * self.hd), 5.0, dtype=self.dtype, device="cuda")
        if general:
            ops.attention_generic(q, out, self.hq, self.hkv, self.hd, scale, self.window, batch, kv, from_step=from_step)
        elif simt:
            from abacus_b200.parts import Workspace
            self.ws = getattr(self, "ws", None) or Workspace(torch.device("cuda", 0))
            ops.attention_decode(q, out, self.hq, self.hkv, self.hd, scale, self.window, batch, kv, self.ws, simt=True)
        else:
            from abacus_b200.parts import Workspace
            self.ws = getattr(self, "ws", None) or Workspace(torch.device("cuda", 0))
            ops.attention(q, out, self.hq, self.hkv, self.hd, scale, self.window, batch, kv, from_step=from_step,
                          ws=self.ws, lists=lists, prepare=prepare)
        for slot, n in seqs:
            self.cache.advance(slot, n)
        if general or all(n == 1 for _, n in seqs):
            assert float(out[rows:].float().abs().sum()) == 0.0  # padding rows give zeros and disturb nothing
        # (the prefill kernel works on the sequences' own rows only and leaves padding rows as they were)
        return q[:rows].float().cpu().numpy(), out[:rows].float().cpu().numpy()


def plain_prep(qkv, hq, hkv, hd, qn, kn, eps, cos, sin, rotary_dim, interleaved, pos0):
    n = qkv.shape[0]
    q = qkv[:, :hq * hd].reshape(n, hq, hd)
    k = qkv[:, hq * hd:(hq + hkv) * hd].reshape(n, hkv, hd)
    v = qkv[:, (hq + hkv) * hd:].reshape(n, hkv, hd)
    if qn is not None:
        q, k = plain.rmsnorm(q, qn, eps), plain.rmsnorm(k, kn, eps)

    def rot(x):
        if cos is None:
            return x
        c, s = cos[pos0:pos0 + n], sin[pos0:pos0 + n]
        part = x[..., :rotary_dim]
        if interleaved:  # pairs (2i, 2i+1): bring them to the half layout, rotate, and back
            half = np.concatenate([part[..., 0::2], part[..., 1::2]], axis=-1)
            r = plain.rope(half, c, s)
            back = np.empty_like(part)
            back[..., 0::2], back[..., 1::2] = r[..., :rotary_dim // 2], r[..., rotary_dim // 2:]
            part = back
        else:
            part = plain.rope(part, c, s)
        return np.concatenate([part, x[..., rotary_dim:]], axis=-1)

    return rot(q), rot(k), v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq, hkv, hd, rotary_dim, interleaved, norm, window", [
    (6, 2, 48, 48, False, True, None),
    (3, 3, 16, 16, True, False, None),
    (8, 1, 80, 32, False, True, None),     # one kv head for all, partial rotation
    (4, 2, 128, 128, False, True, 70),     # a window across page boundaries
    (2, 1, 256, 64, True, True, 5),
])
def test_qkv_prep_and_attention(ops, dtype, hq, hkv, hd, rotary_dim, interleaved, norm, window):
    """Two sequences, one prefilled in two chunks and then decoded, the other whole: every cut reads
    the paged cache (and, windowed, its ring) and must equal attention over the whole sequence."""
    rng = np.random.default_rng(hq * 1000 + hd)
    eps, scale = 2e-5, 0.37 / np.sqrt(hd)
    qn = (1 + 0.3 * rng.standard_normal(hd)).astype(np.float32) * 3 if norm else None
    kn = (1 + 0.3 * rng.standard_normal(hd)).astype(np.float32) * 3 if norm else None
    cos, sin = plain.rope_table(400, rotary_dim, 1234.5)
    width = (hq + 2 * hkv) * hd
    lens = {"a": 150, "b": 93}
    data = {k: rng.standard_normal((n, width)).astype(np.float32) * (1.0 if norm else 2.0) for k, n in lens.items()}
    if dtype == torch.bfloat16:
        data = {k: bf(v) for k, v in data.items()}
    want = {}
    # plain.attention uses 1/sqrt(hd); fold our own scale in by scaling q beforehand
    for key, qkv in data.items():
        q, k, v = plain_prep(qkv, hq, hkv, hd, qn, kn, eps, cos, sin, rotary_dim, interleaved, 0)
        if dtype == torch.bfloat16:
            q, k = bf(q), bf(k)
        want[key] = (q, plain.attention((q * np.float32(scale * np.sqrt(hd))).astype(np.float32), k, v, window,
                                        rnd=bf if dtype == torch.bfloat16 else None).reshape(lens[key], hq * hd))
    h = Harness(hq, hkv, hd, dtype, window)
    sa, sb = h.cache.open_slot(), h.cache.open_slot()
    args = (dev(qn) if norm else None, dev(kn) if norm else None, eps, dev(cos), dev(sin), rotary_dim, interleaved,
            scale)
    tol = dict(rtol=2e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=2 ** -6, atol=2 ** -7)
    got_a, got_b = [], []
    # step 1: the first 70 tokens of a and all of b (windowed layers read this step's own rows)
    q, o = h.step(ops, [(sa, 70), (sb, 93)], np.concatenate([data["a"][:70], data["b"]]), *args,
                  from_step=window is not None)
    np.testing.assert_allclose(q[:70, :hq * hd].reshape(70, hq, hd), want["a"][0][:70], **tol)
    got_a.append(o[:70]), got_b.append(o[70:])
    if window is None:
        # step 2: 50 more tokens of a, at positions 70..119, reading the cache for the first 70
        _, o = h.step(ops, [(sa, 50)], data["a"][70:120], *args)
        got_a.append(o)
        first = 120
    else:
        first = 70
    # then a token by token, in a batch with nothing else
    for i in range(first, 150):
        _, o = h.step(ops, [(sa, 1)], data["a"][i:i + 1], *args)
        got_a.append(o)
    np.testing.assert_allclose(np.concatenate(got_a), want["a"][1], **tol)
    np.testing.assert_allclose(np.concatenate(got_b), want["b"][1], **tol)


@pytest.mark.parametrize("hq, hkv, hd", [(6, 2, 64), (16, 8, 128), (3, 1, 256), (40, 4, 128)])
def test_qkv_prep_of_a_long_prompt_step(ops, hq, hkv, hd):
    """A step of more tokens than one-token CTAs fit the GPU at a time goes to the kernel that takes several tokens
    a CTA (40 + 8 heads: more than it holds in flight per token): the rows and the cache come out bit for bit as
    from two steps that are short enough for the one-token kernel, and as the plain formulas give them."""
    rng = np.random.default_rng(hq + hd)
    eps, width, lens = 1e-6, (hq + 2 * hkv) * hd, (700, 333)
    qn, kn = [(1 + 0.3 * rng.standard_normal(hd)).astype(np.float32) for _ in range(2)]
    cos, sin = plain.rope_table(800, hd, 1e6)
    data = [bf(rng.standard_normal((n, width))) for n in lens]
    args = (dev(qn), dev(kn), eps, dev(cos), dev(sin), hd, False, hd ** -0.5)
    one, two = Harness(hq, hkv, hd, torch.bfloat16), Harness(hq, hkv, hd, torch.bfloat16)
    slots = [(h.cache.open_slot(), h.cache.open_slot()) for h in (one, two)]
    q1, _ = one.step(ops, [(slots[0][0], lens[0]), (slots[0][1], lens[1])], np.concatenate(data), *args)
    q2 = np.concatenate([two.step(ops, [(slots[1][i], lens[i])], data[i], *args)[0] for i in range(2)])
    assert np.array_equal(q1, q2)
    kv1, kv2 = one.cache.views[0].kv, two.cache.views[0].kv
    assert torch.equal(kv1.page_table, kv2.page_table)
    assert torch.equal(kv1.k, kv2.k) and torch.equal(kv1.v, kv2.v) and float(kv1.k.float().abs().sum()) > 0
    # for an entry that reads another entry's cache only q is prepared: k and v stay as they came, nothing is kept
    rows = sum(lens)
    again = dev(np.concatenate(data + [np.full((3, width), 7.0, dtype=np.float32)]), torch.bfloat16)
    before = kv1.k.clone()
    ops.qkv_prep(again, hq, hkv, hd, one.last_batch, *args[:5], hd, False, None, q_only=True)
    again = again[:rows].float().cpu().numpy()
    assert np.array_equal(again[:, :hq * hd], q1[:, :hq * hd]) and np.array_equal(again[:, hq * hd:], np.concatenate(data)[:, hq * hd:])
    assert torch.equal(kv1.k, before)
    at = 0
    for n, qkv in zip(lens, data):
        q, k, v = plain_prep(qkv, hq, hkv, hd, qn, kn, eps, cos, sin, hd, False, 0)
        got = q1[at:at + n]
        np.testing.assert_allclose(got[:, :hq * hd].reshape(n, hq, hd), q, rtol=2 ** -7, atol=2 ** -8)
        np.testing.assert_allclose(got[:, hq * hd:(hq + hkv) * hd].reshape(n, hkv, hd), k, rtol=2 ** -7, atol=2 ** -8)
        assert np.array_equal(got[:, (hq + hkv) * hd:].reshape(n, hkv, hd), v)
        at += n


def test_attention_finds_one_far_key(ops):
    """Among 600 keys with scores near zero, one key 500 places back scores high: the output must be its value."""
    hq, hkv, hd, n = 2, 1, 64, 600
    rng = np.random.default_rng(9)
    qkv = 0.01 * rng.standard_normal((n, (hq + 2) * hd)).astype(np.float32)
    needle = 99
    qkv[needle, hq * hd:(hq + 1) * hd] = 3.0  # its key
    qkv[needle, (hq + 1) * hd:] = np.arange(hd)  # its value
    qkv[n - 1, :hq * hd] = 3.0  # the last token's queries point at it
    h = Harness(hq, hkv, hd, torch.float32)
    slot = h.cache.open_slot()
    h.step(ops, [(slot, n - 1)], qkv[:n - 1], None, None, 0.0, None, None, 0, False, 1.0)
    _, o = h.step(ops, [(slot, 1)], qkv[n - 1:], None, None, 0.0, None, None, 0, False, 1.0)
    np.testing.assert_allclose(o.reshape(hq, hd), np.tile(np.arange(hd, dtype=np.float32), (hq, 1)), atol=1e-3)


def test_refusals_are_errors_not_results(ops):
    from abacus_b200.engine.batch import Sequence, StepBatch
    batch = StepBatch(1, 1, 0, "cuda").fill([Sequence(0, [0], 0, [])])
    qkv = torch.zeros(1, 3 * 260, device="cuda")
    with pytest.raises(ops.KernelRefused, match="head_dim"):
        ops.qkv_prep(qkv, 1, 1, 260, batch, None, None, 0.0, None, None, 0, False, None)
    with pytest.raises(ops.KernelError, match="not on the GPU"):
        ops.swiglu(torch.zeros(2, 4), torch.zeros(2, 2))


# ------------------------------------------------------------------ tensor-core matrix product

def product_tolerance(want, k, out_dtype):
    """Absolute bound on a bfloat16 product's distance from the exact result. Stored as bfloat16: one rounding of the
    largest result. Stored as float32: the tensor cores add each instruction's 16 products to the float32 accumulator
    and cut off what does not fit (measured: the error grows with K in a straight line and leans towards zero,
    2.4e-4 at K = 1,024 and 7.6e-3 at K = 12,288 on results of up to 150 and 550), so at most one unit in the last place
    of the largest result for every instruction along K, and two for the final roundings."""
    top = np.abs(want).max()
    return 2 ** -8 * top if out_dtype == torch.bfloat16 else (k / 16 + 2) * 2 ** -24 * top


def _gemm_case(ops, m, n, k, out_dtype, rng, **pin):
    x, w = bf(rng.standard_normal((m, k))), bf(rng.standard_normal((n, k)))
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    ops.gemm_tc(dev(x, torch.bfloat16), dev(w, torch.bfloat16), out, **pin)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all(), (m, n, k, pin)
    np.testing.assert_allclose(got, want, rtol=0 if out_dtype == torch.float32 else 2 ** -8, atol=product_tolerance(want, k, out_dtype),
                               err_msg=str((m, n, k, pin)))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tc_every_tile_configuration(ops, out_dtype):
    """Each column tile, both operand orders, with and without split K, on sizes that leave ragged
    edges in every direction (M, N no tile multiples; K not a multiple of 64)."""
    rng = np.random.default_rng(21)
    for tile_n in (16, 32, 64, 128, 256):
        for swap in (0, 1):
            for splits in (1, 3):
                m = min(tile_n, 37) if swap else 150
                _gemm_case(ops, m, 389 if swap else 264, 328, out_dtype, rng, tile_n=tile_n, swap=swap, splits=splits)
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tc_persistent_kernel(ops, out_dtype):
    """The kernel for many rows: both column tiles; fewer tiles than SMs, and so many that a CTA walks over
    several and both accumulators come round again (165 and 330 tiles); ragged edges in M, N and K; a K
    shorter than the ring of stages."""
    rng = np.random.default_rng(23)
    for tile_n, (m, n, k) in [(256, (300, 520, 72)), (128, (300, 520, 72)), (256, (1300, 3600, 136)),
                              (128, (1300, 3600, 136)), (256, (2048, 1024, 1032)), (128, (257, 128, 8))]:
        _gemm_case(ops, m, n, k, out_dtype, rng, tile_n=tile_n, persistent=1)
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tc_pairs_of_ctas(ops, out_dtype):
    """The kernel in which two CTAs of a cluster share a tile of 256 rows (tcgen05.mma.cta_group::2, every CTA loading
    its own halves): fewer tiles than pairs of SMs and so many that a pair walks several and both accumulators come
    round; ragged edges in M, N and K, among them a last tile of rows that only the leader's half reaches and a last
    tile of columns that only the leader's half of the weights reaches; a K shorter than the ring of stages and one
    far longer."""
    rng = np.random.default_rng(29)
    for m, n, k in [(300, 520, 72), (1300, 3600, 136), (2048, 1024, 1032), (257, 256, 8), (120, 100, 64), (2048, 4096, 1024),
                    (600, 2560, 9728)]:
        _gemm_case(ops, m, n, k, out_dtype, rng, persistent=2)
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("hq, hkv, k, lens, norm, rotated", [
    (16, 8, 1024, [2048], True, True),                  # pairs of CTAs, every tile full
    (3, 1, 72, [300], True, True),                      # the persistent kernel; a last column tile of one head; a ragged K
    (5, 2, 136, [700, 1, 64, 65, 470], True, True),     # pairs (9 heads: a last column tile of one head), ragged prompts
    (4, 4, 264, [257, 130], False, True), (2, 1, 64, [400], True, False), (32, 8, 2560, [513, 300], True, True)])
def test_gemm_tc_qkv_prepares_in_its_epilogue(ops, hq, hkv, k, lens, norm, rotated):
    """The q/k/v product of a prompt step with the preparation of its heads in the epilogue, against the product and the
    preparation's own kernel after it: the same bits in the q columns and in the cache. The second sequence starts at
    position 37 (a continuation: its keys go to the middle of a page); three padding rows follow the last sequence."""
    from abacus_b200.cache import CacheNeed, SequenceCache
    from abacus_b200.engine.batch import Sequence, StepBatch
    rng = np.random.default_rng(hq * 10 + k)
    hd, rows = 128, sum(lens)
    width = (hq + 2 * hkv) * hd
    x = dev(bf(rng.standard_normal((rows + 3, k))), torch.bfloat16)
    w = dev(bf(rng.standard_normal((width, k)) / np.sqrt(k)), torch.bfloat16)
    qn = dev(1.0 + 0.3 * rng.standard_normal(hd), torch.float32) if norm else None
    kn = dev(1.0 + 0.3 * rng.standard_normal(hd), torch.float32) if norm else None
    angles = rng.uniform(0, 6.28, (4096, hd // 2))
    cos = dev(np.cos(angles), torch.float32) if rotated else None
    sin = dev(np.sin(angles), torch.float32) if rotated else None
    results = []
    for fused in (False, True):
        cache = SequenceCache([CacheNeed(hkv, hd, None)], [None], 64 * 64, torch.bfloat16, "cuda", max_context=4096)
        seqs = []
        for i, n in enumerate(lens):
            slot = cache.open_slot()
            if i == 1:
                cache.reserve(slot, 37), cache.advance(slot, 37)
            seqs.append(Sequence(slot, [0] * n, cache.length[slot], []))
            cache.reserve(slot, cache.length[slot] + n)
        batch = StepBatch(rows + 3, len(lens) + 1, 0, "cuda", plans=[]).fill(seqs)
        kv = cache.views[0].kv
        qkv = torch.full((rows + 3, width), 3.0, dtype=torch.bfloat16, device="cuda")
        if fused:
            assert ops.gemm_tc_qkv_takes(x, w, qkv, rows + 3, hq, hkv, hd, kv, qn, kn, cos, sin, hd if rotated else 0, False)
            ops.gemm_tc_qkv(x, w, qkv, hq, hkv, batch, qn, kn, 1e-5, cos, sin, kv)
        else:
            ops.gemm_tc(x, w, qkv)
            ops.qkv_prep(qkv, hq, hkv, hd, batch, qn, kn, 1e-5, cos, sin, hd if rotated else 0, False, kv)
        results.append((qkv[:rows, :hq * hd].clone(), kv.k.clone(), kv.v.clone(), kv.page_table.clone()))
    (q_a, k_a, v_a, t_a), (q_b, k_b, v_b, t_b) = results
    assert torch.equal(t_a, t_b)
    assert torch.equal(q_a, q_b)
    assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
    assert float(k_a.float().abs().sum()) > 0 and float(q_a.float().abs().max()) > 0.1
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]
    small = torch.empty(200, width, dtype=torch.bfloat16, device="cuda")
    assert not ops.gemm_tc_qkv_takes(x[:200], w, small, 200, hq, hkv, hd, kv, qn, kn, cos, sin, hd if rotated else 0, False)


@pytest.mark.parametrize("m, n, k", [(1, 128, 64), (1, 1024, 2048), (8, 4096, 1024), (64, 1000, 72), (65, 192, 96),
                                      (300, 389, 96), (2048, 1024, 1024), (5, 151936, 128), (130, 70, 8), (1500, 4096, 264),
                                      # the down projections of the 4B and 8B shapes: K beyond the persistent kernel's 4,096
                                      (1100, 2560, 9728), (300, 4096, 12288), (40, 2560, 9728), (17, 4096, 12288)])
def test_gemm_tc_chosen_configuration(ops, m, n, k):
    rng = np.random.default_rng(m + n + k)
    _gemm_case(ops, m, n, k, torch.float32, rng)
    _gemm_case(ops, m, n, k, torch.bfloat16, rng)
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]


def test_gemm_tc_split_k_is_deterministic_and_leaves_its_tickets_at_zero(ops):
    rng = np.random.default_rng(22)
    x, w = dev(bf(rng.standard_normal((8, 3072))), torch.bfloat16), dev(bf(rng.standard_normal((1024, 3072))), torch.bfloat16)
    outs = []
    for _ in range(4):
        out = torch.empty(8, 1024, device="cuda")
        ops.gemm_tc(x, w, out)
        outs.append(out)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    from abacus_b200.kernels.ops import _Scratch
    assert int(_Scratch.of(torch.device("cuda", 0)).gemm_tickets.abs().sum()) == 0


def test_gemm_tc_refuses_what_tma_cannot_address(ops):
    x, w = torch.zeros(4, 20, dtype=torch.bfloat16, device="cuda"), torch.zeros(16, 20, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(4, 16, device="cuda")
    assert not ops.gemm_tc_takes(x, w, out)  # K = 20 is no multiple of 8: the linear layer uses the CUDA-core kernel
    with pytest.raises(ops.KernelRefused, match="multiples of 8"):
        ops.gemm_tc(x, w, out)


@pytest.mark.parametrize("hq, hkv, hd, window, simt", [
    (16, 8, 128, None, False), (6, 2, 64, None, False), (4, 4, 256, None, False), (8, 1, 64, None, False),
    (4, 2, 128, 200, False), (3, 1, 128, 64, False), (10, 2, 64, 129, False),
    # the CUDA-core kernel at the head sizes the tensor-core one usually takes, with and without windows
    (16, 8, 128, None, True), (6, 2, 64, 64, True), (4, 2, 128, 129, True), (3, 1, 64, 200, True), (4, 4, 256, 200, True)])
def test_decode_attention_split_along_the_keys(ops, hq, hkv, hd, window, simt):
    """Rows of very different lengths (1 key to 700: up to six chunks of 128, chunk and page edges
    included) decoded in one step by the kernel the model uses for decode (or, with simt, by the
    CUDA-core decode kernel), against plain attention."""
    rng = np.random.default_rng(hq * 100 + hd + (window or 0))
    lens = [1, 64, 65, 128, 129, 257, 700, 383]
    width = (hq + 2 * hkv) * hd
    scale = 1.0 / np.sqrt(hd)
    h = Harness(hq, hkv, hd, torch.bfloat16, window, max_tokens=64 * 40)
    assert ops.attention_decode_takes(hq, hkv, hd, h.cache.views[0].kv)
    data = [bf(rng.standard_normal((n, width)) * 1.5) for n in lens]
    slots = [h.cache.open_slot() for _ in lens]
    none = (None, None, 0.0, None, None, 0, False, scale)
    # fill the caches with everything but the last token of each (the general kernel runs these steps)
    for slot, d in zip(slots, data):
        if len(d) > 1:
            h.step(ops, [(slot, len(d) - 1)], d[:-1], *none, from_step=window is not None)
    # the decode step: one row per sequence, plus the harness's padding rows
    _, got = h.step(ops, [(slot, 1) for slot in slots], np.concatenate([d[-1:] for d in data]), *none, general=False,
                    simt=simt)
    for i, d in enumerate(data):
        n = len(d)
        q = d[:, :hq * hd].reshape(n, hq, hd)
        k = d[:, hq * hd:(hq + hkv) * hd].reshape(n, hkv, hd)
        v = d[:, (hq + hkv) * hd:].reshape(n, hkv, hd)
        want = plain.attention(q, k, v, window, rnd=bf)[-1].reshape(hq * hd)
        np.testing.assert_allclose(got[i], want, rtol=2 ** -7, atol=2 ** -7, err_msg=f"row {i} of length {n}")
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("hq, hkv, hd, window, norm, rotated", [
    (16, 8, 128, None, True, True), (6, 2, 64, None, True, True), (32, 8, 128, None, True, True), (4, 4, 128, None, False, True),
    (3, 1, 64, None, True, False), (8, 1, 64, 129, False, False), (4, 2, 128, 200, True, True), (16, 1, 128, 64, True, True)])
def test_decode_attention_prepares_its_heads(ops, hq, hkv, hd, window, norm, rotated):
    """Decode attention that norms and rotates q and k and writes the new key and value to the cache itself, against
    the preparation's own kernel followed by attention: the same bits in the output and in the cache, over three decode
    steps in a row (the later ones read what the earlier ones wrote). The rows' lengths put the new token into every
    quarter of a page, at a page's first and last place, and into a sequence's very first place."""
    rng = np.random.default_rng(hq * 100 + hd + (window or 0))
    lens = [1, 2, 16, 17, 33, 50, 64, 65, 127, 128, 129, 257, 700, 383]
    width = (hq + 2 * hkv) * hd
    scale = 1.0 / np.sqrt(hd)
    qn = dev(1.0 + 0.3 * rng.standard_normal(hd), torch.float32) if norm else None
    kn = dev(1.0 + 0.3 * rng.standard_normal(hd), torch.float32) if norm else None
    angles = rng.uniform(0, 6.28, (1024, hd // 2))
    cos = dev(np.cos(angles), torch.float32) if rotated else None
    sin = dev(np.sin(angles), torch.float32) if rotated else None
    prep = (qn, kn, 1e-5, cos, sin, hd if rotated else 0, False, scale)
    data = [bf(rng.standard_normal((n + 2, width)) * 1.5) for n in lens]
    results = []
    for prepares in (False, True):
        h = Harness(hq, hkv, hd, torch.bfloat16, window, max_tokens=64 * 60)
        slots = [h.cache.open_slot() for _ in lens]
        for slot, d, n in zip(slots, data, lens):
            if n > 1:
                h.step(ops, [(slot, n - 1)], d[:n - 1], *prep, from_step=window is not None)
        outs = []
        for t in range(3):
            rows = np.concatenate([d[n - 1 + t:n + t] for d, n in zip(data, lens)])
            outs.append(h.step(ops, [(slot, 1) for slot in slots], rows, *prep, general=False, prepares=prepares)[1])
        kv = h.cache.views[0].kv
        results.append((np.stack(outs), kv.k.clone(), kv.v.clone(), kv.page_table.clone()))
    (out_a, k_a, v_a, table_a), (out_b, k_b, v_b, table_b) = results
    assert torch.equal(table_a, table_b)
    assert np.array_equal(out_a, out_b)
    assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
    assert np.isfinite(out_a).all() and np.abs(out_a).max() > 0.1
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("hq, hkv, hd", [(16, 8, 128), (6, 2, 64), (4, 4, 128), (5, 1, 64)])
def test_prefill_attention_on_the_tensor_cores(ops, hq, hkv, hd):
    """Prompts of unequal lengths in one step (1 token to 330: page and tile edges included), and a prompt
    given in two parts, the second reading the first from the cache: the kernel the model uses for
    prefill against plain attention."""
    rng = np.random.default_rng(hq * 10 + hd)
    lens = [1, 63, 64, 65, 330, 130, 128]
    width = (hq + 2 * hkv) * hd
    scale = 1.0 / np.sqrt(hd)
    h = Harness(hq, hkv, hd, torch.bfloat16, None, max_tokens=64 * 40)
    assert ops.attention_prefill_takes(hd, h.cache.views[0].kv)
    data = [bf(rng.standard_normal((n, width)) * 1.5) for n in lens]
    slots = [h.cache.open_slot() for _ in lens]
    none = (None, None, 0.0, None, None, 0, False, scale)
    cut = 70  # of the fifth prompt: 70 tokens now, the other 260 in a second step
    first = [d if i != 4 else d[:cut] for i, d in enumerate(data)]
    _, got1 = h.step(ops, [(s, len(d)) for s, d in zip(slots, first)], np.concatenate(first), *none, general=False)
    _, got2 = h.step(ops, [(slots[4], lens[4] - cut)], data[4][cut:], *none, general=False)
    at = 0
    for i, d in enumerate(data):
        n = len(d)
        q = d[:, :hq * hd].reshape(n, hq, hd)
        k = d[:, hq * hd:(hq + hkv) * hd].reshape(n, hkv, hd)
        v = d[:, (hq + hkv) * hd:].reshape(n, hkv, hd)
        want = plain.attention(q, k, v, rnd=bf).reshape(n, hq * hd)
        m = len(first[i])
        got = got1[at:at + m] if i != 4 else np.concatenate([got1[at:at + m], got2])
        at += m
        np.testing.assert_allclose(got, want, rtol=2 ** -6, atol=2 ** -6, err_msg=f"prompt {i} of length {n}")
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]


def test_prefill_attention_halves_long_tiles(ops):
    """Tiles that see eight pages of keys or more stand twice in the kernel's work list, each CTA with half of
    the pages; the one that is through first leaves its partial result for the other. A prompt of 700 tokens and
    one given as 500 and then 300 (its second part's tiles see 9 to 13 pages): against plain attention, twice
    with the same bits whoever came second, and the tickets back at zero."""
    from abacus_b200.kernels.ops import _Scratch
    rng = np.random.default_rng(77)
    hq, hkv, hd = 4, 2, 128
    width, scale = (hq + 2 * hkv) * hd, 1.0 / np.sqrt(hd)
    none = (None, None, 0.0, None, None, 0, False, scale)
    runs = []
    for run in range(2):
        h = Harness(hq, hkv, hd, torch.bfloat16, None, max_tokens=64 * 40)
        data = [bf(np.random.default_rng(78 + i).standard_normal((n, width)) * 1.5) for i, n in enumerate((700, 800, 200))]
        slots = [h.cache.open_slot() for _ in data]
        first = [data[0], data[1][:500], data[2]]
        _, got1 = h.step(ops, [(s, len(d)) for s, d in zip(slots, first)], np.concatenate(first), *none, general=False)
        assert h.last_lists.n_halved == 4  # the tiles from row 384 on of the prompts of 700 and of 500 tokens
        _, got2 = h.step(ops, [(slots[1], 300)], data[1][500:], *none, general=False)
        assert h.last_lists.n_halved == 3
        got = [got1[:700], np.concatenate([got1[700:1200], got2]), got1[1200:]]
        runs.append(got)
        if run == 0:
            for i, (d, g) in enumerate(zip(data, got)):
                n = len(d)
                q = d[:, :hq * hd].reshape(n, hq, hd)
                k = d[:, hq * hd:(hq + hkv) * hd].reshape(n, hkv, hd)
                v = d[:, (hq + hkv) * hd:].reshape(n, hkv, hd)
                np.testing.assert_allclose(g, plain.attention(q, k, v, rnd=bf).reshape(n, hq * hd), rtol=2 ** -6, atol=2 ** -6,
                                           err_msg=f"prompt {i}")
    for a, b in zip(*runs):
        np.testing.assert_array_equal(a, b)
    assert int(_Scratch.of(torch.device("cuda", 0)).attention_halves_tickets.abs().sum()) == 0
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("m, n, k", [(1, 16, 32), (8, 4096, 1024), (3, 1000, 96), (9, 389, 160), (16, 1024, 3072),
                                      (5, 24, 2048), (17, 520, 64), (33, 72, 1024), (64, 6144, 1024), (50, 1024, 3072),
                                      (16, 2560, 9728), (8, 4096, 12288), (16, 6144, 4096), (3, 2560, 4096)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_rows(ops, m, n, k, out_dtype):
    """The weight-streaming product for a handful of rows, at sizes that leave partial tiles of 16
    features and of 8 tokens, and K with fewer blocks than warps."""
    rng = np.random.default_rng(m * 7 + n + k)
    x, w = bf(rng.standard_normal((m, k))), bf(rng.standard_normal((n, k)))
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    assert ops.gemm_rows_takes(xd, wd, out, m)
    ops.gemm_rows(xd, wd, out)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=0 if out_dtype == torch.float32 else 2 ** -8,
                               atol=product_tolerance(want, k, out_dtype))
    with pytest.raises(ops.KernelRefused):
        ops.gemm_rows(dev(bf(rng.standard_normal((65, k))), torch.bfloat16), wd, torch.empty(65, n, device="cuda"))


@pytest.mark.parametrize("m, inter, k", [(1, 8, 32), (8, 3072, 1024), (5, 100, 96), (16, 272, 192), (11, 40, 2048),
                                         (64, 3072, 1024), (29, 104, 96), (16, 9728, 2560), (8, 12288, 4096)])
def test_gemm_rows_with_swiglu(ops, m, inter, k):
    """The feed-forward's first product and its activation in one kernel, against product then swiglu."""
    rng = np.random.default_rng(m + inter + k)
    x, w = bf(rng.standard_normal((m, k))), bf(0.3 * rng.standard_normal((2 * inter, k)))
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_rows_swiglu(dev(x, torch.bfloat16), dev(w, torch.bfloat16), act)
    want = plain.swiglu(plain.linear(x, w))
    np.testing.assert_allclose(act.float().cpu().numpy(), want, rtol=2 ** -7, atol=2 ** -7 * np.abs(want).max())
    if inter % 8 == 0:  # the same weights with gate and up rows in turns of 8
        turns = np.concatenate([np.concatenate([w[b:b + 8], w[inter + b:inter + b + 8]]) for b in range(0, inter, 8)])
        again = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.gemm_rows_swiglu(dev(x, torch.bfloat16), dev(turns, torch.bfloat16), again, block=8)
        assert torch.equal(again, act)


def _in_turns(w, inter, block):
    return np.concatenate([np.concatenate([w[b:b + block], w[inter + b:inter + b + block]]) for b in range(0, inter, block)])


@pytest.mark.parametrize("m, inter, k", [(300, 128, 72), (1300, 2304, 136), (2048, 3072, 1024), (257, 384, 8),
                                         (700, 9728, 2560), (520, 12288, 4096)])
def test_gemm_tc_with_swiglu(ops, m, inter, k):
    """The tensor-core product of many rows with the activation in its epilogue (gate and up rows in turns of
    128): against product then swiglu, and the same bits as the rows kernel gives for the first of the rows
    where both round gate and up to bfloat16 before the activation."""
    rng = np.random.default_rng(m + inter + k)
    x, w = bf(rng.standard_normal((m, k))), bf(0.3 * rng.standard_normal((2 * inter, k)))
    xd, wd = dev(x, torch.bfloat16), dev(_in_turns(w, inter, 128), torch.bfloat16)
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.gemm_tc_swiglu_takes(xd, wd, act, m, 128) and not ops.gemm_tc_swiglu_takes(xd, wd, act, 256, 128)
    ops.gemm_tc_swiglu(xd, wd, act)
    want = plain.swiglu(plain.linear(x, w))
    np.testing.assert_allclose(act.float().cpu().numpy(), want, rtol=2 ** -7, atol=2 ** -7 * np.abs(want).max())
    assert ops.kernel_status(torch.device("cuda", 0)).tolist() == [0, 0, 0, 0]
