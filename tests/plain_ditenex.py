"""Plain, slow statement of the Ditenex decoder: whole sequences, float64, no cache, no
batching, no kernels; one function per mechanism.  It shares no code with the package
under test (own reader of config.json and of the safetensors file).

Notation: X is [T, width] (the residual stream of one sequence), h a sublayer's input.
Weights are [out, in] and act as h @ W.T.

The design, in this file's words:
  X = embed[tokens] + pos[0 .. T-1]
  a layer:  X += m * rms(mixer(shift(rms(X, norm1))), norm1b)
            X += m * rms(ff(rms(X, norm2)), norm2b)             (if the layer has a feed-forward)
  shift(h)[t] = h[t] + (h[t-1] - h[t]) * s   (h[-1] = 0)
  mixer: softmax attention inside a sliding window, grouped key/value heads, biased projections, no rotation;
         a penalty slope_h * distance on every score; the heads' scores mixed by a matrix before the softmax;
         values blended with the values of the first blending layer; a sigmoid gate on the heads' results
  ff:    dense with a two-sided quadratic/exponential activation, or routed experts (sigmoid scores, a choice bias,
         groups of neighbouring experts) plus an expert that every token uses
  logits = rms(X, final.norm) @ embed.T
"""
import json
import math
import os
import struct

import numpy as np

F64 = np.float64


def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[lo:hi]
        shape = tuple(info["shape"])
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(F64)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(F64)
        elif info["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError("dtype %s" % info["dtype"])
        out[name] = arr.reshape(shape)
    return out


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---------------------------------------------------------------------------
# small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rms(x, w, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def token_shift(h, s):
    before = np.zeros_like(h)
    before[1:] = h[:-1]
    return h + (before - h) * s


def two_sided_activation(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    pos = softplus(p) * z * z + 0.5 * z
    zn = np.minimum(z, 0.0)
    neg = (0.5 + softplus(q)) * (np.expm1(zn) - zn) + 0.5 * z
    return np.where(z > 0, pos, neg)


def distance_slopes(heads):
    return np.array([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)


# ---------------------------------------------------------------------------
# the mixer
def values_of(h, W, p):
    return h @ W[p + "v"].T + W[p + "v.b"]


def attention(h, m, W, p, v):
    """h [T, width]; v [T, G * vdim] are the values this layer uses (blended already, if it blends)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window = m["mask"]["size"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, d)
    v = v.reshape(T, G, dv)
    per = H // G
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    dist = (i - j).astype(F64)
    slopes = distance_slopes(H)
    raw = np.empty((H, T, T), dtype=F64)
    for a in range(H):
        raw[a] = (q[:, a] @ k[:, a // per].T) * m["scale"] - slopes[a] * dist
    mixed = np.einsum("ab,bij->aij", W[p + "talk"], raw)
    seen = (dist >= 0) & (dist < window)
    out = np.empty((T, H, dv), dtype=F64)
    for a in range(H):
        s = np.where(seen, mixed[a], -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        e = np.exp(s)
        out[:, a] = (e / e.sum(axis=1, keepdims=True)) @ v[:, a // per]
    gate = sigmoid(h @ W[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ W[p + "o"].T


# ---------------------------------------------------------------------------
# feed-forwards
def dense_ff(h, W, p):
    a = W[p + "act"]
    return two_sided_activation(h @ W[p + "up"].T, a[0], a[1]) @ W[p + "down"].T


def gated_expert(h, W, p):
    z = h @ W[p + "gate"].T
    return (z * sigmoid(z) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def choose_experts(h, mlp, W, p):
    """Per token: ids of the chosen experts and their weights."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    s = sigmoid(h @ W[p + "router"].T)                       # [T, E]
    choice = s + W[p + "correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    n_groups, keep = groups["count"], groups["keep"]
    size = E // n_groups
    ids = np.empty((h.shape[0], top), dtype=np.int64)
    weights = np.empty((h.shape[0], top), dtype=F64)
    for t in range(h.shape[0]):
        c = choice[t].copy()
        if n_groups > 1:
            gscore = np.array([np.sort(c[g * size:(g + 1) * size])[-2:].sum() for g in range(n_groups)])
            kept = np.argsort(-gscore, kind="stable")[:keep]
            allowed = np.zeros(E, dtype=bool)
            for g in kept:
                allowed[g * size:(g + 1) * size] = True
            c = np.where(allowed, c, -np.inf)
        best = np.argsort(-c, kind="stable")[:top]
        ids[t] = best
        weights[t] = s[t, best] * r["scale"]
    return ids, weights


def routed_ff(h, mlp, W, p):
    ids, weights = choose_experts(h, mlp, W, p)
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]), dtype=F64)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], weights[t]):
            out[t] += w * gated_expert(h[t:t + 1], W, "%se%d." % (p, e))[0]
    if mlp.get("shared"):
        out += gated_expert(h, W, p + "shared.")
    return out


# ---------------------------------------------------------------------------
# the model
def first_blending_layer(cfg):
    for i, L in enumerate(cfg["layers"]):
        if L["mixer"].get("v_mix"):
            return i
    return -1


def forward(cfg, W, tokens, streams=None):
    """Logits [T, vocab] of one sequence; `streams`, if a list, receives X after every layer."""
    tokens = np.asarray(tokens)
    T = len(tokens)
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    X = W["embed"][tokens] + W["pos"][:T]
    first = first_blending_layer(cfg)
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = L["mixer"]
        h = token_shift(rms(X, W[p + "norm1"], eps), W[p + "shift"])
        v = values_of(h, W, p + "mix.")
        if m.get("v_mix"):
            if i == first:
                v_first = v
            else:
                lam = float(W[p + "mix.vmix"])
                v = (1.0 - lam) * v + lam * v_first
        X = X + mult * rms(attention(h, m, W, p + "mix.", v), W[p + "norm1b"], eps)
        mlp = L.get("mlp")
        if mlp:
            h2 = rms(X, W[p + "norm2"], eps)
            y = dense_ff(h2, W, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h2, mlp, W, p + "mlp.")
            X = X + mult * rms(y, W[p + "norm2b"], eps)
        if streams is not None:
            streams.append(X.copy())
    return rms(X, W["final.norm"], eps) @ W["embed"].T


def greedy(cfg, W, prompt, n_new):
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(np.argmax(forward(cfg, W, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
