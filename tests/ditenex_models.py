"""Small Ditenex configurations of the tests' own and weights drawn so that faults show.

N(0, 0.02) everywhere would hide faults: a flat softmax does not care which keys it sees, a mixing matrix near zero
mixes nothing, a router that barely prefers anybody hides a wrong choice.  So: queries and keys give scores of a few
units, the mixing matrix is the identity plus a dense part, shifts lie between 0 and 1, the routers' logits and the
choice biases are of the size of the scores' differences (negative ones among them).

`standout` rewrites a folder's tensors so that one token's key outweighs every other in every head of one layer:
whether that token is in sight decides the result, so a window that is one token off, or a far key that is lost,
changes the logits by as much as they vary at all.
"""
import json
import os

import numpy as np

import harness


def att(heads, kv, dim, vdim, window, scale, v_mix=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale, groups=None, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(width, vocab, layers, mult, eps=1e-5, max_positions=1024):
    return {"architecture": "Ditenex", "vocab": vocab, "width": width, "max_positions": max_positions, "residual_mult": mult,
            "norm": {"eps": eps}, "layers": [{"type": "attention", "mixer": m, "mlp": f} for m, f in layers]}


CONFIGS = {
    # the first blending layer is not the first layer; a layer without feed-forward; windows below, across and above a page
    "P": config(96, 300, [(att(4, 2, 16, 24, 20, 0.3), dense(40)),
                          (att(6, 3, 16, 8, 33, 0.25, True), moe(6, 2, 24, 2.5, (3, 2), 40)),
                          (att(3, 3, 8, 8, 70, 0.4, True), None),
                          (att(2, 1, 32, 24, 130, 0.2, True), dense(56))], 0.7, eps=3e-6),
    # values that are 1 or equal: one head, keys as wide as values, windows of 1, 2 and 3 tokens, one expert chosen,
    # no groups, no expert for everybody, a multiplier of 1, a flag that says false
    "Q": config(64, 200, [(att(1, 1, 16, 16, 1, 0.25, True), moe(2, 1, 16, 1.0)),
                          (att(1, 1, 16, 16, 2, 0.25, True), None),
                          (att(2, 2, 8, 8, 3, 1.0, False), dense(16))], 1.0),
    # sizes that the tensor-core products like; prompts of several pages; sixteen experts in four groups
    "R": config(128, 512, [(att(8, 4, 32, 64, 100, 0.18, True), moe(16, 4, 64, 1.5, (4, 2), 128)),
                           (att(8, 2, 32, 128, 64, 0.18, True), dense(256)),
                           (att(4, 4, 64, 64, 300, 0.125, True), moe(8, 2, 32, 1.0, (2, 1))),
                           (att(16, 4, 16, 64, 129, 0.25, True), dense(128))], 0.5),
    # sizes that nothing divides; every expert chosen; as many kept experts as choices
    "S": config(100, 333, [(att(5, 5, 10, 12, 7, 0.4, True), moe(9, 3, 22, 0.8, (3, 1), 30)),
                           (att(10, 5, 6, 12, 65, 0.5, True), dense(50)),
                           (att(3, 1, 24, 40, 63, 0.2), moe(5, 5, 10, 2.0, None, 6))], 0.3, eps=1e-6),
    # a width that is a multiple of 4 only; groups of single experts; ten heads on one key head
    "T": config(52, 97, [(att(10, 1, 10, 7, 17, 0.4), dense(22)),
                         (att(5, 5, 6, 5, 64, 0.5, True), None),
                         (att(1, 1, 6, 25, 128, 0.3, True), moe(4, 2, 10, 1.3, (4, 2)))], 1.6),
    # heads as large as real models have them
    "U": config(256, 200, [(att(2, 1, 128, 128, 200, 0.088, True), dense(64)),
                           (att(4, 2, 256, 64, 96, 0.0625, True), moe(4, 2, 64, 1.0, (2, 2), 64))], 0.5),
    # single mechanisms
    "attention_only": config(64, 100, [(att(4, 2, 16, 24, 20, 0.3), None)], 0.8),
    "blend_only": config(64, 100, [(att(2, 2, 16, 12, 9, 0.3, True), None), (att(4, 1, 8, 24, 30, 0.4, True), None)], 0.8),
    "dense_only": config(64, 100, [(att(1, 1, 8, 8, 1, 0.3), dense(48))], 0.8),
    "experts_only": config(64, 100, [(att(1, 1, 8, 8, 1, 0.3), moe(8, 3, 16, 1.7, (4, 2), 24))], 0.8),
    # one wide window (a key hundreds of tokens back), one narrow one
    "far": config(64, 120, [(att(4, 2, 16, 16, 400, 0.25, True), dense(32)), (att(2, 1, 16, 32, 50, 0.25, True), None)], 0.6),
    # head counts between the powers of two, up to 32, with keys and values in eights (the tensor cores' prompt kernels pad them)
    "V": config(160, 250, [(att(12, 4, 16, 40, 45, 0.25, True), dense(72)),
                           (att(20, 5, 8, 32, 70, 0.35, True), moe(6, 2, 24, 1.2, (3, 2), 16)),
                           (att(32, 8, 8, 8, 64, 0.35), None)], 0.9),
}
SEEDS = {name: 170 + i for i, name in enumerate(CONFIGS)}


def tensors_of(cfg, rng, clear_routing=False):
    """Every tensor of the design by name, float32.  clear_routing: the routers barely depend on the token and the choice
    biases are far apart, so that rounding cannot change a choice (what a comparison in bfloat16 needs)."""
    w = cfg["width"]
    out = {}

    def normal(shape, std=0.02, mean=0.0):
        return (rng.standard_normal(shape) * std + mean).astype(np.float32)

    out["embed"] = normal((cfg["vocab"], w), 1.0)
    out["pos"] = normal((cfg["max_positions"], w), 0.3)
    out["final.norm"] = normal((w,), 0.1, 1.0)
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = L["mixer"]
        H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        for n in ("norm1", "norm1b"):
            out[p + n] = normal((w,), 0.1, 1.0)
        out[p + "shift"] = normal((w,), 0.3, 0.5)
        # the mixer's input has entries of about 1: q and k entries of size a, scores a^2 sqrt(dim) scale = about 3
        a = (3.0 / (np.sqrt(d) * m["scale"])) ** 0.5
        out[p + "mix.q"] = normal((H * d, w), a / np.sqrt(w))
        out[p + "mix.q.b"] = normal((H * d,), 0.3 * a)
        out[p + "mix.k"] = normal((G * d, w), a / np.sqrt(w))
        out[p + "mix.k.b"] = normal((G * d,), 0.3 * a)
        out[p + "mix.v"] = normal((G * vd, w), 1.0 / np.sqrt(w))
        out[p + "mix.v.b"] = normal((G * vd,), 0.3)
        out[p + "mix.vmix"] = np.float32(0.2 + 0.1 * i) * np.ones((), dtype=np.float32)
        out[p + "mix.talk"] = (np.eye(H) + rng.standard_normal((H, H)) * 0.3 / np.sqrt(H)).astype(np.float32)
        out[p + "mix.g"] = normal((H * vd, w), 1.0 / np.sqrt(w))
        out[p + "mix.o"] = normal((w, H * vd), 1.0 / np.sqrt(H * vd))
        mlp = L.get("mlp")
        if not mlp:
            continue
        for n in ("norm2", "norm2b"):
            out[p + n] = normal((w,), 0.1, 1.0)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            out[p + "mlp.up"] = normal((ff, w), 1.0 / np.sqrt(w))
            out[p + "mlp.down"] = normal((w, ff), 1.0 / np.sqrt(ff))
            out[p + "mlp.act"] = np.array([0.3 - 0.2 * i, -0.4 + 0.3 * i], dtype=np.float32)
            continue
        r = mlp["router"]
        E, ff = r["experts"], mlp["expert"]["ff"]
        names = ["e%d." % e for e in range(E)]
        inner = [ff] * E
        if mlp.get("shared"):
            names.append("shared.")
            inner.append(mlp["shared"]["ff"])
        for n, f in zip(names, inner):
            out[p + "mlp." + n + "gate"] = normal((f, w), 1.0 / np.sqrt(w))
            out[p + "mlp." + n + "up"] = normal((f, w), 1.0 / np.sqrt(w))
            out[p + "mlp." + n + "down"] = normal((w, f), 1.0 / np.sqrt(f))
        if not clear_routing:
            out[p + "mlp.router"] = normal((E, w), 1.5 / np.sqrt(w))
            out[p + "mlp.correction"] = normal((E,), 0.25)
            continue
        out[p + "mlp.router"] = normal((E, w), 0.05 / np.sqrt(w))
        groups = (r.get("groups") or {"count": 1})["count"]
        size = E // groups
        while True:                                   # biases 0.4 apart, and the groups' sums of two clearly apart as well
            c = (rng.permutation(E) * 0.4 + rng.uniform(0.0, 0.1, E) - 0.2 * E).astype(np.float32)
            sums = sorted(np.sort(c[g * size:(g + 1) * size])[-2:].sum() for g in range(groups))
            if groups == 1 or min(b - a for a, b in zip(sums, sums[1:])) > 0.2:
                break
        out[p + "mlp.correction"] = c
    return out


def bf16_round(x):
    return harness.bf16_bytes_to_f32(harness.f32_to_bf16_bytes(x)).reshape(np.shape(x))


def standout(cfg, t, layer, token, gain=12.0):
    """Changes layer `layer` of the tensors `t` in place: the key of `token` gets a large part along one direction per key
    head, and every query a fixed part along the same direction, so that the score of a query against that token's key
    is about `gain` above the others'.  The token's value is made large too."""
    p = "l%d." % layer
    m = cfg["layers"][layer]["mixer"]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = cfg["width"]
    if layer == 0:
        x = t["embed"][token].astype(np.float64)          # positions are a small part of the first layer's input
        h = x / np.sqrt((x * x).mean() + cfg["norm"]["eps"]) * t[p + "norm1"]
        h = h * (1.0 - t[p + "shift"])                     # what the shift leaves of the token's own row
    else:
        raise ValueError("standout is built for the first layer")
    rng = np.random.default_rng(5)
    direction = rng.standard_normal(d)
    direction /= np.linalg.norm(direction)
    amount = np.sqrt(gain / m["scale"])
    k = t[p + "mix.k"].astype(np.float64)
    for g in range(G):
        k[g * d:(g + 1) * d] += amount * np.outer(direction, h) / (h @ h)
    t[p + "mix.k"] = k.astype(np.float32)
    qb = t[p + "mix.q.b"].astype(np.float64)
    for a in range(H):
        qb[a * d:(a + 1) * d] += amount * direction
    t[p + "mix.q.b"] = qb.astype(np.float32)
    v = t[p + "mix.v"].astype(np.float64)
    v += 3.0 * np.outer(rng.standard_normal(G * vd), h) / (h @ h)
    t[p + "mix.v"] = v.astype(np.float32)
    return t


def write_folder(path, cfg, tensors):
    from friday_inference_engine_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      [(n, "BF16", list(x.shape), harness.f32_to_bf16_bytes(x)) for n, x in tensors.items()])
    return path
