"""Plain, slow implementation of the Qwen3 dense decoder, for comparison only.

Whole sequences, no cache, one function for each part, numpy float32 only. It
shares no code with the package under test: it has its own safetensors reader,
its own rotation table and its own sampler. Every function cites the lines of
mottopanikeiku/abacus whose formula it restates.

abacus's engine itself is int8 in its linear layers (src/matmul.c), so it can
anchor this file only at quantisation-noise level; tests/golden/ holds that
comparison. Everything else here rests on the formulas cited below.

`rnd` (optional) is applied where a reduced-precision engine stores a tensor,
so that a bfloat16 engine can be compared more tightly than against pure
float32 math. With rnd=None everything is float32.
"""
import json
import struct

import numpy as np

F32 = np.float32
P_ROUNDED = True  # with rnd: the probabilities are a stored tensor too (see attention)


# ----------------------------------------------------------------- file reading

def read_safetensors(path):
    """name -> float32 array (BF16 widened exactly) or int array.

    Container format as tools/export.py:28-38 reads it: 8-byte little-endian
    header length, JSON header, data_offsets relative to the end of the header.
    """
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = raw[8 + n + a:8 + n + b]
        if info["dtype"] == "BF16":  # src/abacus.h:39-44: bf16 is the top half of a float32
            arr = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(F32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4").copy()
        elif info["dtype"] == "I32":
            arr = np.frombuffer(buf, dtype="<i4").copy()
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        out[name] = arr.reshape(info["shape"])
    return out


def read_config(path):
    """The keys tools/export.py:76-88 reads, with its defaults."""
    c = json.loads(open(path).read())
    theta = c.get("rope_theta") or c["rope_parameters"]["rope_theta"]  # tools/export.py:83
    hd = c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"]  # tools/export.py:82
    layer_types = c.get("layer_types") or ["full_attention"] * c["num_hidden_layers"]
    return dict(
        dim=c["hidden_size"], inter=c["intermediate_size"], n_layers=c["num_hidden_layers"],
        n_heads=c["num_attention_heads"], n_kv_heads=c["num_key_value_heads"], head_dim=hd,
        vocab=c["vocab_size"], theta=float(theta), eps=float(c["rms_norm_eps"]),
        tied=bool(c.get("tie_word_embeddings", False)),  # tools/export.py:81
        windows=[c.get("sliding_window") if t == "sliding_attention" else None for t in layer_types],
    )


def bf16_round(a):
    """Round float32 to the nearest bfloat16 (ties to even), as tools/export.py:49-51 does."""
    u = np.ascontiguousarray(a, dtype=F32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(F32).reshape(np.shape(a))


# ----------------------------------------------------------------- the parts

def embed(tokens, table):
    """x[i,:] = float(embed[token_i,:]), no scale (src/model.c:290-291)."""
    return table[np.asarray(tokens)].astype(F32)


def rmsnorm(x, w, eps):
    """out = w * (x * 1/sqrt(mean(x^2) + eps)), all float32 (src/model.c:164-169)."""
    x = x.astype(F32)
    ss = np.sum(x * x, axis=-1, keepdims=True, dtype=F32)
    scale = F32(1.0) / np.sqrt(ss / F32(x.shape[-1]) + F32(eps), dtype=F32)
    return (w.astype(F32) * (x * scale)).astype(F32)


def linear(x, w):
    """out = x . w^T, weights [out, in] row-major, no bias (src/model.c:299,302,307,309,324)."""
    return (x.astype(F32) @ w.astype(F32).T).astype(F32)


def rope_table(n_pos, head_dim, theta):
    """cos/sin of pos * theta^(-2i/head_dim) in float32 (src/model.c:116-124)."""
    half = head_dim // 2
    i = np.arange(half, dtype=F32)
    inv = F32(1.0) / np.power(F32(theta), (F32(2.0) * i) / F32(head_dim), dtype=F32)
    angle = (np.arange(n_pos, dtype=F32)[:, None] * inv[None, :]).astype(F32)
    return np.cos(angle, dtype=F32), np.sin(angle, dtype=F32)


def rope(x, cos, sin):
    """Rotate pairs (i, i + head_dim/2) of every head (src/model.c:173-181).

    x: [tokens, heads, head_dim]; cos, sin: [tokens, head_dim/2].
    """
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1).astype(F32)


def softmax(x):
    """exp(x - max) / sum (src/model.c:183-192)."""
    e = np.exp(x - np.max(x), dtype=F32)
    return (e / np.sum(e, dtype=F32)).astype(F32)


def attention(q, k, v, window=None, rnd=None):
    """Causal attention of one sequence (src/model.c:197-211).

    q: [n, Hq, hd]; k, v: [n, Hkv, hd]. Query head h reads kv head h // (Hq/Hkv)
    (src/model.c:200); scores are scaled by 1/sqrt(hd) (src/model.c:202-204);
    token i reads keys 0..i (the loop bound of src/model.c:203 is the mask).
    abacus has no window; with `window` = W token i reads keys max(0, i-W+1)..i,
    which is what config.json's sliding_window means.
    rnd: where a reduced-precision engine stores the probabilities for the second product (tensor cores take
    them as bfloat16). Such an engine meets a row's keys tile by tile and cannot know the row's maximum when it
    rounds the first; so that the rounded value does not depend on the tiling, the exponentials are taken against
    the maximum rounded up to a whole power of two: p = 2^(s log2(e) - ceil(max s log2(e))), in (1/2, 1] at the
    maximum. p is rounded before it multiplies the values, and the row's sum is taken of the unrounded values.
    abacus keeps everything in float32 against the maximum itself (src/model.c:183-192, 206-210): rnd=None.
    """
    n, hq, hd = q.shape
    group = hq // k.shape[1]
    scale = F32(1.0) / np.sqrt(F32(hd))
    out = np.zeros((n, hq, hd), dtype=F32)
    for i in range(n):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(hq):
            g = h // group
            scores = (k[lo:i + 1, g, :] @ q[i, h, :]).astype(F32) * scale
            if rnd is None:
                out[i, h, :] = softmax(scores) @ v[lo:i + 1, g, :]
            else:
                t = scores * F32(1.4426950408889634)
                e = np.exp2(t - np.ceil(np.max(t)), dtype=F32)
                out[i, h, :] = (rnd(e) @ v[lo:i + 1, g, :]) / np.sum(e, dtype=F32)
    return out


def swiglu(gate_up):
    """silu(gate) * up with rows laid out [gate | up] (src/model.c:274-282)."""
    inter = gate_up.shape[-1] // 2
    g, u = gate_up[..., :inter], gate_up[..., inter:]
    with np.errstate(over="ignore"):  # exp(-g) may be inf for a very negative gate: g / inf is the 0 that is meant
        return (g / (F32(1.0) + np.exp(-g, dtype=F32)) * u).astype(F32)


# ----------------------------------------------------------------- the model

def layer_weights(w, l):
    p = f"model.layers.{l}."
    return dict(
        attn_norm=w[p + "input_layernorm.weight"],
        wq=w[p + "self_attn.q_proj.weight"], wk=w[p + "self_attn.k_proj.weight"],
        wv=w[p + "self_attn.v_proj.weight"], wo=w[p + "self_attn.o_proj.weight"],
        q_norm=w[p + "self_attn.q_norm.weight"], k_norm=w[p + "self_attn.k_norm.weight"],
        ffn_norm=w[p + "post_attention_layernorm.weight"],
        w_gate=w[p + "mlp.gate_proj.weight"], w_up=w[p + "mlp.up_proj.weight"],
        w_down=w[p + "mlp.down_proj.weight"],
    )  # names: tools/export.py:90-99


def forward(cfg, w, tokens, rnd=None, schedule=None):
    """Logits [n, vocab] of one whole sequence (src/model.c:286-313, 322-325).

    schedule: list of (layer, source) pairs, the order layers run in. `source`
    is None when the layer uses its own keys and values, or the index of an
    earlier schedule entry whose keys and values it reads instead of making
    its own. Default: every layer once, in order, each with its own.
    """
    r = (lambda a: a) if rnd is None else rnd
    n = len(tokens)
    hq, hkv, hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    cos, sin = rope_table(n, hd, cfg["theta"])
    if schedule is None:
        schedule = [(l, None) for l in range(cfg["n_layers"])]
    x = embed(tokens, w["model.embed_tokens.weight"])
    kept = []
    for l, source in schedule:
        L = layer_weights(w, l)
        xn = r(rmsnorm(x, L["attn_norm"], cfg["eps"]))  # src/model.c:297-298
        q = r(linear(xn, L["wq"])).reshape(n, hq, hd)  # src/model.c:299
        q = r(rope(rmsnorm(q, L["q_norm"], cfg["eps"]), cos, sin))  # src/model.c:251-255
        if source is None:
            k = r(linear(xn, L["wk"])).reshape(n, hkv, hd)
            v = r(linear(xn, L["wv"])).reshape(n, hkv, hd)
            k = r(rope(rmsnorm(k, L["k_norm"], cfg["eps"]), cos, sin))
        else:
            k, v = kept[source]
        kept.append((k, v))
        att = r(attention(q, k, v, cfg["windows"][l], rnd=rnd if P_ROUNDED else None).reshape(n, hq * hd))  # :301
        x = x + linear(att, L["wo"])  # src/model.c:302, 305
        xn = r(rmsnorm(x, L["ffn_norm"], cfg["eps"]))  # src/model.c:306
        gate_up = r(np.concatenate([linear(xn, L["w_gate"]), linear(xn, L["w_up"])], axis=-1))  # :307
        act = r(swiglu(gate_up))  # src/model.c:308
        x = x + linear(act, L["w_down"])  # src/model.c:309, next add_norm
    xn = r(rmsnorm(x, w["model.norm.weight"], cfg["eps"]))  # src/model.c:311-312
    head = w["model.embed_tokens.weight"] if cfg["tied"] or "lm_head.weight" not in w else w["lm_head.weight"]
    return linear(xn, head)  # src/model.c:102-103, 322-325


def forward64(cfg, w, tokens, schedule=None):
    """The same formulas evaluated in float64: what float32 results scatter around. The distance
    between forward() and this is the rounding noise of float32 for that input."""
    global F32
    keep, F32 = F32, np.float64
    try:
        return forward(cfg, {k: v.astype(np.float64) for k, v in w.items()}, tokens, schedule=schedule)
    finally:
        F32 = keep


def load(folder):
    cfg = read_config(f"{folder}/config.json")
    return cfg, read_safetensors(f"{folder}/model.safetensors")


# ----------------------------------------------------------------- sampling

def argmax(x):
    """First maximum wins (src/main.c:31-36)."""
    best = 0
    for i in range(1, len(x)):
        if x[i] > x[best]:
            best = i
    return best


def xorshift64(state):
    """src/main.c:52."""
    m = (1 << 64) - 1
    state ^= (state << 13) & m
    state ^= state >> 7
    state ^= (state << 17) & m
    return state


def sample(logits, temp, state, top_k=20):
    """Top-20 sampling at a temperature; returns (token, new state) (src/main.c:39-56).

    top_k = 0 is this library's own: no cut to the most likely tokens (src/main.c:41), the same probabilities
    exp((l_j - l_max) / temp) over the whole vocabulary, the same generator, and the walk of src/main.c:53-55 in
    index order, since there is no sorted short list; sums in float64."""
    if temp <= 0.0:
        return argmax(logits), state
    if top_k == 0:
        x = np.asarray(logits, dtype=F32)
        p = np.exp((x - x[argmax(x)]) * F32(F32(1.0) / F32(temp)), dtype=F32).astype(np.float64)
        run = np.cumsum(p)
        state = xorshift64(state)
        r = float(state >> 40) / float(1 << 24) * run[-1]
        hit = np.flatnonzero(run >= r)
        return (int(hit[0]) if len(hit) else len(x) - 1), state
    top = []
    for i in range(len(logits)):
        if len(top) == top_k and logits[i] <= logits[top[-1]]:
            continue
        if len(top) < top_k:
            top.append(i)
        j = len(top) - 1
        while j > 0 and logits[top[j - 1]] < logits[i]:
            top[j] = top[j - 1]
            j -= 1
        top[j] = i
    p, total = [], F32(0.0)
    for j in top:
        pj = np.exp((F32(logits[j]) - F32(logits[top[0]])) / F32(temp), dtype=F32)
        p.append(pj)
        total = F32(total + pj)
    state = xorshift64(state)
    rr = F32(F32(state >> 40) / F32(1 << 24) * total)
    for j, pj in zip(top, p):
        rr = F32(rr - pj)
        if rr <= 0.0:
            return j, state
    return top[-1], state


def generate(cfg, w, prompt, steps, temp=0.0, seed=0, stop=(), rnd=None):
    """Whole forward pass for every new token, no cache (tools/reference.py:67-71);
    stops before a stop token is kept (src/main.c:174-182)."""
    seq, out, state = list(prompt), [], seed
    for _ in range(steps):
        token, state = sample(forward(cfg, w, seq, rnd=rnd)[-1], temp, state)
        if token in stop:
            break
        out.append(int(token))
        seq.append(int(token))
    return out
