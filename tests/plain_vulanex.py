"""Vulanex, written plainly from its equations: float64 numpy, one function per mechanism, token by token where
the design is a recurrence.  It shares no code with the library; the tests compare the library with it.

A model is a config (a dict as config.json holds it) and a dict name -> numpy array of weights.  `forward` runs a whole
sequence and returns the logits at every position and, if asked, the residual stream after every layer.
"""
import math

import numpy as np


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, w, b, eps):
    mu = np.mean(x, axis=-1, keepdims=True)
    var = np.mean((x - mu) ** 2, axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every position: the last row for a sequence's first token."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embed(tokens, table, bigram, cfg):
    bg = cfg["embedding"]["bigram"]
    rows = bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    return table[np.asarray(tokens)] + bigram[np.asarray(rows)]


def input_conv(h, w):
    """h + conv(h): conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start.  h [T, C], w [C, taps]."""
    T, taps = h.shape[0], w.shape[1]
    out = h.copy()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def softmax_rows(scores, seen, extra=None):
    """Softmax over the seen entries of each row; `extra` [rows] joins the denominator only."""
    out = np.zeros_like(scores)
    for i in range(scores.shape[0]):
        idx = np.nonzero(seen[i])[0]
        if idx.size == 0:
            continue
        s = scores[i, idx]
        m = s.max() if extra is None else max(s.max(), extra[i])
        e = np.exp(s - m)
        den = e.sum() + (0.0 if extra is None else math.exp(extra[i] - m))
        out[i, idx] = e / den
    return out


def query_temperature(T, coef, every):
    p = np.arange(T)
    return 1.0 + coef * np.log(np.floor((p + 1) / every) + 1.0)


def attention_keys_as_values(h, W, m):
    """Causal softmax attention without rotation whose values are the keys, queries scaled by position."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W["q"].T).reshape(T, H, d)
    k = (h @ W["k"].T).reshape(T, G, d)
    q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    seen = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, d))
    for hh in range(H):
        g = hh // (H // G)
        p = softmax_rows((q[:, hh] @ k[:, g].T) * m["scale"], seen)
        out[:, hh] = p @ k[:, g]
    return out.reshape(T, H * d) @ W["o"].T


def rotary_table(rot):
    """Angular frequency of each pair and the multiplier of cosine and sine."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        def dim_of(t):
            return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(dim_of(sc["fast"])), 0)
        hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
        ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(sc["factor"]) + 1.0
    return f, mult


def rotate_half(x, rot):
    """x [T, heads, d]: dimension i pairs with i + dims/2 among the first dims."""
    f, mult = rotary_table(rot)
    dims = rot["dims"]
    half = dims // 2
    T = x.shape[0]
    a = np.arange(T)[:, None] * f[None, :]
    c, s = (np.cos(a) * mult)[:, None, :], (np.sin(a) * mult)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def pooled_window_attention(h, W, m, eps):
    """Softmax attention behind a sliding window, with one mean key and value for each block of tokens that lies wholly
    before the window, and a sink per head in the denominator."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, P = m["mask"]["size"], m["mask"]["pool"]
    q = (h @ W["q"].T).reshape(T, H, d)
    k = (h @ W["k"].T).reshape(T, G, d)
    v = (h @ W["v"].T).reshape(T, G, dv)
    q = rms_unit(q, eps) * W["q.norm"]
    k = rms_unit(k, eps) * W["k.norm"]
    q, k = rotate_half(q, m["rot"]), rotate_half(k, m["rot"])
    nb = T // P
    kb = k[:nb * P].reshape(nb, P, G, d).mean(axis=1) if nb else np.zeros((0, G, d))
    vb = v[:nb * P].reshape(nb, P, G, dv).mean(axis=1) if nb else np.zeros((0, G, dv))
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    seen_tok = (i - j >= 0) & (i - j < size)
    b = np.arange(nb)[None, :]
    seen_blk = (b * P + P - 1) <= (i - size)
    seen = np.concatenate([seen_tok, seen_blk], axis=1)
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        keys = np.concatenate([k[:, g], kb[:, g]], axis=0)
        vals = np.concatenate([v[:, g], vb[:, g]], axis=0)
        p = softmax_rows((q[:, hh] @ keys.T) * m["scale"], seen, extra=np.full(T, float(W["sink"][hh])))
        out[:, hh] = p @ vals
    return out.reshape(T, H * dv) @ W["o"].T


def delta_rule(h, W, m, eps, state=None):
    """Generalized delta rule: S <- diag(w) S - (a u)(u^T S) + k v^T, both terms reading the old state; o = S^T r."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ W["r"].T).reshape(T, H, d)
    k = (h @ W["k"].T).reshape(T, H, d)
    v = (h @ W["v"].T).reshape(T, H, d)
    w = np.exp(-math.exp(-0.5) * sigmoid(np.tanh(h @ W["w1"].T) @ W["w2"].T + W["w0"])).reshape(T, H, d)
    a = sigmoid(h @ W["a"].T + W["a.b"]).reshape(T, H, d)
    u = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    S = np.zeros((H, d, d)) if state is None else state
    o = np.zeros((T, H, d))
    for t in range(T):
        for hh in range(H):
            old = S[hh]
            S[hh] = w[t, hh][:, None] * old - np.outer(a[t, hh] * u[t, hh], u[t, hh] @ old) + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ r[t, hh]
    o = rms_unit(o, eps).reshape(T, H * d) * W["norm"] * sigmoid(h @ W["g"].T)
    return o @ W["o"].T


def parallel_mixer(h, W, m, eps):
    left = {n[len("left."):]: x for n, x in W.items() if n.startswith("left.") and n != "left.out"}
    right = {n[len("right."):]: x for n, x in W.items() if n.startswith("right.") and n != "right.out"}
    yl = pooled_window_attention(h, left, m["left"], eps)
    yr = delta_rule(h, right, m["right"], eps)
    return 0.5 * (rms_unit(yl, eps) * W["left.out"] + rms_unit(yr, eps) * W["right.out"])


def feed_forward(h, W):
    return (gelu_tanh(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def sub(weights, prefix):
    return {n[len(prefix):]: x for n, x in weights.items() if n.startswith(prefix)}


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence; layers_out (a list) receives the stream after every layer."""
    W = {n: np.asarray(x, dtype=np.float64) for n, x in weights.items()}
    eps = cfg["norm"]["eps"]
    x = embed(tokens, W["embed"], W["bigram"], cfg)
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = input_conv(layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps), W[p + "canon1"])
        mix = sub(W, p + "mix.")
        if L["type"] == "attention":
            x = x + attention_keys_as_values(h, mix, L["mixer"])
        elif L["type"] == "parallel":
            x = x + parallel_mixer(h, mix, L["mixer"], eps)
        else:
            raise ValueError("no mixer of type %r" % L["type"])
        if L.get("mlp"):
            h = input_conv(layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps), W[p + "canon2"])
            x = x + feed_forward(h, sub(W, p + "mlp."))
        if layers_out is not None:
            layers_out.append(x.copy())
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return (x @ W["embed"].T) * cfg["logit_scale"]


def load(model_dir):
    """config.json and every tensor of model.safetensors (BF16, F32 or I32) as float64 / int arrays."""
    import json
    import os
    import struct
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    path = os.path.join(model_dir, "model.safetensors")
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        meta = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        a, b = m["data_offsets"]
        raw = np.frombuffer(blob[a:b], dtype=np.uint8)
        if m["dtype"] == "BF16":
            x = (raw.view("<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif m["dtype"] == "F32":
            x = raw.view("<f4").astype(np.float64)
        elif m["dtype"] == "I32":
            x = raw.view("<i4")
        else:
            raise ValueError("tensor %s: dtype %s" % (name, m["dtype"]))
        out[name] = x.reshape(m["shape"])
    return cfg, out


def greedy(cfg, weights, prompt, n):
    """The n tokens that follow `prompt` when the largest logit is taken every time (the first of equal ones)."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(forward(cfg, weights, toks)[-1])))
    return toks[len(prompt):]
