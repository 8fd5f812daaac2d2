"""Vulanex through the engine against the plain implementation (tests/plain_vulanex.py), on small configurations of
the tests' own with weights drawn here: each mechanism alone, whole prompts, decoding token by token, prompts cut into
portions down to two tokens, batches of unequal requests, slots and pages used again, keys far away, at page borders and
just inside and just outside the window, pooled blocks that are just seen or not yet, the first tokens of a sequence, long
decoding, and greedy generation through Engine.generate.

Weights N(0, 0.02) everywhere would hide faults (a flat softmax, a sink that weighs nothing, states that forget at once), so
the folders are written with queries and keys scaled up, sinks of the size of the scores, decays that remember, taps and
biases that matter.  Where even that would hide a fault (one key at a window's edge, one pooled block among many) a test
plants a standout: a token whose key and value are large and a later token whose query asks for exactly that key, so that
the logits change by far more than the bound when the key is seen or not.

float32 must agree with the plain implementation to summation order; bfloat16 within bounds relative to the logits' spread.
"""
import json
import os

import numpy as np
import pytest

import harness
import plain_vulanex as plain
import tiny_configs
from friday_inference_engine_b200 import Engine
from friday_inference_engine_b200.weights import write_safetensors

pytestmark = pytest.mark.gpu
DTYPES = [pytest.param("float32", id="f32"), pytest.param("bfloat16", id="bf16")]


def attention(heads, kv, dim, scale=None, coef=0.5, every=16):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale or dim ** -0.5,
                                           "q_temp": {"coef": coef, "every": every}}}


def parallel(heads, kv, dim, vdim, size, pool, rot_dims, rheads, rdim, base=10000.0, scaling=None, scale=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "mask": {"size": size, "pool": pool}, "rot": rot}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": rheads, "dim": rdim}}}


def config(width, vocab, layers, ffs, taps=3, buckets=101, muls=(31, 5), eps=1e-5, logit_scale=1.0):
    c = {"architecture": "Vulanex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "logit_scale": logit_scale,
         "embedding": {"bigram": {"buckets": buckets, "mul_prev": muls[0], "mul_cur": muls[1]}}, "layers": []}
    for L, ff in zip(layers, ffs):
        c["layers"].append(dict(L, mlp={"kind": "dense", "ff": ff} if ff else None))
    return c


# name -> (config, rank of the decay's two-step projection per parallel layer)
CONFIGS = {
    # both kinds of layer; a window that is no multiple of the block, which is no divisor of a page; part of a head rotated
    "P": (config(96, 300, [attention(4, 2, 16, every=8), parallel(4, 2, 16, 24, 40, 12, 8, 3, 16, 10000.0, (8.0, 64, 16.0, 2.0)),
                           attention(6, 3, 16, 0.2, 0.25, 5), parallel(2, 1, 32, 16, 21, 5, 32, 2, 24)],
                 [40, 56, None, 24], taps=4, buckets=97, muls=(13, 3), eps=3e-6, logit_scale=1.5), {1: 6, 3: 4}),
    # one head everywhere; a block of one token; a window of one; two taps; a single bucket
    "Q": (config(64, 200, [parallel(1, 1, 32, 8, 1, 1, 16, 1, 8, 500.0), attention(1, 1, 24, coef=1.0, every=1), parallel(1, 1, 8, 40, 7, 3, 2, 1, 40)],
                 [16, None, 32], taps=2, buckets=1, muls=(1, 0)), {0: 3, 2: 2}),
    # sizes that the tensor-core kernels like; prompts of several pages; a window of two pages and a block of a quarter page
    "R": (config(128, 512, [parallel(4, 2, 32, 64, 128, 16, 32, 4, 32, 20000.0, (4.0, 256, 32.0, 1.0), 0.11), attention(4, 2, 64, 0.1, 0.4, 48),
                            parallel(4, 4, 64, 32, 96, 32, 16, 2, 64), attention(2, 2, 32)],
                 [128, 64, 128, None], taps=3, buckets=251, muls=(61, 9), logit_scale=1.25), {0: 16, 2: 8}),
    # sizes that fit no tile: a width that is no multiple of 8, odd head sizes and counts, a block larger than the window,
    # a block larger than a page, one tap (no convolution history), eight taps elsewhere
    "S": (config(100, 333, [parallel(6, 2, 24, 40, 10, 30, 6, 3, 20, 777.0, (2.0, 100, 8.0, 0.5)), attention(5, 5, 10, coef=0.1, every=3),
                            parallel(3, 1, 40, 24, 50, 70, 40, 5, 12)],
                 [56, 6, 30], taps=1, buckets=50, muls=(7, 11), logit_scale=0.5), {0: 6, 2: 10}),
    "T": (config(52, 97, [attention(5, 1, 6), parallel(5, 5, 10, 12, 33, 4, 10, 4, 10, 300.0, (3.0, 50, 4.0, 0.25), 0.4), attention(2, 2, 14)],
                 [10, 22, None], taps=8, buckets=23, muls=(0, 1), logit_scale=1.7), {1: 3}),
    # heads as large as real models have them
    "U": (config(256, 200, [parallel(2, 1, 128, 128, 64, 16, 64, 2, 128, 10000.0, (4.0, 128, 32.0, 1.0)), attention(2, 1, 128, 0.05)],
                 [64, None], taps=3), {0: 16}),
    # single mechanisms
    "attention_only": (config(64, 100, [attention(4, 2, 16, every=4)], [None]), {}),
    "parallel_only": (config(64, 100, [parallel(4, 2, 16, 12, 20, 6, 16, 2, 16, 10000.0, (4.0, 32, 8.0, 1.0))], [None]), {0: 5}),
    "mlp_conv": (config(64, 100, [attention(1, 1, 16)], [48], taps=5, logit_scale=2.0), {}),
}
SEEDS = {name: 170 + i for i, name in enumerate(CONFIGS)}


def tensors_of(cfg, ranks, rng):
    """Every tensor of the design by name, float32, shaped so that faults show."""
    w, taps = cfg["width"], cfg["canon"]["taps"]
    out = {}

    def normal(shape, std=0.02, mean=0.0):
        return (rng.standard_normal(shape) * std + mean).astype(np.float32)

    def thin(n):                     # keeps scores a few units whatever the sizes
        return min(1.0, (96.0 / n) ** 0.5)

    out["embed"] = normal((cfg["vocab"], w), 0.3)
    out["bigram"] = normal((cfg["embedding"]["bigram"]["buckets"] + 1, w), 0.3)
    out["final.norm"] = normal((w,), 0.1, 1.0)
    out["final.norm.b"] = normal((w,), 0.1)
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = L["mixer"]
        out[p + "norm1"] = normal((w,), 0.1, 1.0)
        out[p + "norm1.b"] = normal((w,), 0.2)
        out[p + "canon1"] = normal((w, taps), 0.3)
        if L["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            # scores of a few units at the largest query multiplier: peaked, but not so that rounding a key moves the softmax
            out[p + "mix.q"] = normal((H * d, w), 0.12 * thin(w) * min(1.0, (32.0 / d) ** 0.5))
            out[p + "mix.k"] = normal((G * d, w), 0.12 * thin(w))
            out[p + "mix.o"] = normal((w, H * d), 0.1)
        else:
            l, r = m["left"], m["right"]
            H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            out[p + "mix.left.q"] = normal((H * d, w), 0.3)
            out[p + "mix.left.k"] = normal((G * d, w), 0.3)
            out[p + "mix.left.v"] = normal((G * dv, w), 0.3)
            # normed heads have a root mean square of one: weights of this size make scores of a few units
            out[p + "mix.left.q.norm"] = normal((d,), 0.3, 1.2 * (16.0 / d) ** 0.25)
            out[p + "mix.left.k.norm"] = normal((d,), 0.3, 1.2 * (16.0 / d) ** 0.25)
            out[p + "mix.left.sink"] = normal((H,), 1.5, 1.0)
            out[p + "mix.left.o"] = normal((w, H * dv), 0.1)
            out[p + "mix.left.out"] = normal((w,), 0.2, 1.0)
            out[p + "mix.right.out"] = normal((w,), 0.2, 1.0)
            RH, rd, rank = r["heads"], r["dim"], ranks[i]
            for n in ("r", "k", "v", "g"):
                out[p + "mix.right." + n] = normal((RH * rd, w), 0.2)
            out[p + "mix.right.a"] = normal((RH * rd, w), 0.2)
            out[p + "mix.right.a.b"] = normal((RH * rd,), 1.0)
            out[p + "mix.right.w1"] = normal((rank, w), 0.3)
            out[p + "mix.right.w2"] = normal((RH * rd, rank), 0.5)
            out[p + "mix.right.w0"] = normal((RH * rd,), 1.0, -2.0)        # decays near one: the state remembers
            out[p + "mix.right.norm"] = normal((RH * rd,), 0.1, 1.0)
            out[p + "mix.right.o"] = normal((w, RH * rd), 0.1)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            out[p + "norm2"] = normal((w,), 0.1, 1.0)
            out[p + "norm2.b"] = normal((w,), 0.2)
            out[p + "canon2"] = normal((w, taps), 0.3)
            out[p + "mlp.gate"] = normal((ff, w), 0.15)
            out[p + "mlp.up"] = normal((ff, w), 0.15)
            out[p + "mlp.down"] = normal((w, ff), 0.1)
    return out


def write_folder(path, cfg, tensors):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      [(n, "BF16", list(x.shape), harness.f32_to_bf16_bytes(x)) for n, x in tensors.items()])
    return path


_made = {}


def model(root, name):
    key = (str(root), name)
    if key not in _made:
        cfg, ranks = CONFIGS[name]
        d = write_folder(os.path.join(str(root), "vulanex_" + name), cfg, tensors_of(cfg, ranks, np.random.default_rng(SEEDS[name])))
        _made[key] = (d,) + plain.load(d)
    return _made[key]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("vulanex")


def engine(root, name, dtype, **kw):
    d, cfg, t = model(root, name)
    kw.setdefault("max_ctx", 1024)
    kw.setdefault("max_batch", 6)
    return Engine(model_path=d, dtype=dtype, **kw), cfg, t


_plain = {}


def plain_logits(root, name, prompt):
    key = (str(root), name, tuple(prompt))
    if key not in _plain:
        _, cfg, t = model(root, name)
        _plain[key] = plain.forward(cfg, t, prompt)
    return _plain[key]


def compare(got, ref, places, dtype, what):
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == (len(places), ref.shape[1]), what
    assert np.isfinite(got).all(), what
    if dtype == "float32":
        spread = np.sqrt((ref ** 2).mean())
        err = np.abs(got - ref[places]).max()
        assert err <= 1e-4 * max(spread, 1.0), "%s: |engine - plain| = %.3g (spread %.3g)" % (what, err, spread)
        return
    for i in range(len(places)):
        ok, text = harness.bf16_ok(got[i], ref[places[i]], what, harness.BF16_WIDE)
        assert ok, "%s, place %d: %s" % (what, places[i], text)


def agree(got, root, name, prompt, places, dtype, what):
    compare(got, plain_logits(root, name, prompt), places, dtype, what)


def prompts(lengths, vocab, seed):
    return tiny_configs.random_prompts(lengths, vocab, seed)


def nothing_held(eng):
    st = eng.stats()
    return st["slots_held"] == 0 and all(g["pages_held"] == 0 for g in st["groups"])


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention_only", "parallel_only", "mlp_conv"])
def test_each_mechanism_alone(root, name, dtype):
    eng, cfg, _ = engine(root, name, dtype)
    for n, p in zip([1, 2, 40, 90], prompts([1, 2, 40, 90], cfg["vocab"], 3)):
        s = eng.alloc_slot()
        got = eng.step([s], [p], [list(range(n))], to="host")
        eng.free_slot(s)
        agree(got, root, name, p, list(range(n)), dtype, "%s alone, %d tokens" % (name, n))
    eng.check()
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n", [("P", 150), ("Q", 70), ("R", 300), ("S", 200), ("T", 130), ("U", 100)])
def test_whole_prompt(root, name, n, dtype):
    eng, cfg, _ = engine(root, name, dtype)
    (p,) = prompts([n], cfg["vocab"], 5)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [list(range(n))], to="host")
    eng.free_slot(s)
    agree(got, root, name, p, list(range(n)), dtype, "%s whole %d" % (name, n))
    assert nothing_held(eng)


def test_faults_would_show(root):
    """What the comparisons above would see: the plain implementation with one mechanism changed a little differs from itself
    by far more than the float32 bound."""
    _, cfg, t = model(root, "P")
    (p,) = prompts([150], cfg["vocab"], 5)
    ref = plain.forward(cfg, t, p)
    bound = 100 * 1e-4 * max(np.sqrt((ref ** 2).mean()), 1.0)

    def changed(**kw):
        c = json.loads(json.dumps(cfg))
        for path, v in kw.items():
            node, keys = c, path.split("__")
            for k in keys[:-1]:
                node = node[int(k)] if k.isdigit() else node[k]
            node[keys[-1]] = v
        return np.abs(plain.forward(c, t, p) - ref).max()

    no_sink = dict(t)
    no_sink["l1.mix.left.sink"] = t["l1.mix.left.sink"] - 30.0
    assert np.abs(plain.forward(cfg, no_sink, p) - ref).max() > bound
    assert changed(layers__1__mixer__left__mask__size=41) > bound          # a window one token longer
    assert changed(layers__1__mixer__left__mask__pool=11) > bound          # other blocks
    assert changed(layers__0__mixer__q_temp__every=9) > bound
    assert changed(embedding__bigram__mul_prev=14) > bound
    assert changed(canon__taps=4) == 0.0
    forgetful = dict(t)
    forgetful["l1.mix.right.w0"] = t["l1.mix.right.w0"] + 3.0
    assert np.abs(plain.forward(cfg, forgetful, p) - ref).max() > bound
    late = plain.forward(cfg, t, p[100:])              # keys, blocks, state and history lost
    assert np.abs(late[-1] - ref[-1]).max() > bound


# ---- a standout key: one token whose key and value are large, asked for by a later token
def standout_model(root, name, window, pool, dim=16, vdim=16):
    """One parallel layer whose left attention copies: token id 1 is marked along channel 0 of the stream, token id 2 asks
    along channel 1; the last key dimension (not rotated) reads channel 0, the last query dimension channel 1, the other
    dimensions read ordinary channels, so that after the heads' norms only the marked key is large where the asking query is;
    the marked token's value is large in every channel."""
    key = (str(root), name)
    if key in _made:
        return _made[key]
    cfg = config(32, 40, [parallel(1, 1, dim, vdim, window, pool, 2, 1, 8, 10000.0, None, 1.0)], [None], taps=1, buckets=7, muls=(0, 0))
    rng = np.random.default_rng(5)
    t = tensors_of(cfg, {0: 2}, rng)
    w = cfg["width"]
    t["embed"] = (rng.standard_normal((40, w)) * 0.3).astype(np.float32)
    t["embed"][:, :2] = 0.0
    t["embed"][1, 0] = 3.0           # the marked token
    t["embed"][2, 1] = 3.0           # the asking token
    t["bigram"][:] = 0.0
    t["l0.norm1"][:] = 1.0
    t["l0.norm1.b"][:] = 0.0
    t["l0.canon1"][:] = 0.0
    q = np.zeros((dim, w), np.float32)
    k = np.zeros((dim, w), np.float32)
    for j in range(dim - 1):         # ordinary channels fill the other dimensions
        q[j, 2 + j] = 1.0
        k[j, 2 + dim + (j % (w - 2 - dim))] = 1.0
    q[dim - 1, 1] = 1.0
    k[dim - 1, 0] = 1.0
    v = (rng.standard_normal((vdim, w)) * 0.05).astype(np.float32)
    v[:, 0] = 2.0
    t["l0.mix.left.q"], t["l0.mix.left.k"], t["l0.mix.left.v"] = q, k, v
    t["l0.mix.left.q.norm"][:] = 1.5
    t["l0.mix.left.k.norm"][:] = 1.5
    t["l0.mix.left.sink"][:] = 0.0
    t["l0.mix.left.out"][:] = 3.0            # what the attention adds outweighs the token's own row
    t["l0.mix.right.out"][:] = 0.05
    d = write_folder(os.path.join(str(root), "vulanex_" + name), cfg, t)
    _made[key] = (d,) + plain.load(d)
    return _made[key]


def standout_prompt(n, marked_at, asking_at, seed):
    rng = np.random.default_rng(seed)
    p = rng.integers(3, 40, size=n).tolist()
    p[marked_at] = 1
    for a in asking_at:
        p[a] = 2
    return p


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode", ["whole", "decode", "portions"])
def test_window_edges_with_a_standout_key(root, mode, dtype):
    """The marked token just inside the window, just outside it and in no block yet, in a block that has just come into
    sight, and far back among many blocks: the asking tokens' logits differ widely between these cases, and the engine follows
    the plain implementation in each, in prompts, in decoding and in portions."""
    window, pool = 37, 6
    d, cfg, t = standout_model(root, "standout", window, pool)
    eng = Engine(model_path=d, dtype=dtype, max_ctx=512, max_batch=2)
    n, ask = 200, 150
    asking = [ask, ask + 1, n - 1]
    at_second = {}
    # seen from position 151: the window is 115 .. 151, the blocks end at 114 - 37 ... : position 114 is in nobody's sight
    for marked in [149, 115, 114, 113, 108, 107, 20, 0]:
        p = standout_prompt(n, marked, asking, 17)
        ref = plain.forward(cfg, t, p)
        s = eng.alloc_slot()
        if mode == "whole":
            got = eng.step([s], [p], [asking], to="host")
        elif mode == "decode":
            eng.step([s], [p[:ask - 3]], [[]], to="host")
            rows = [eng.step([s], [[tok]], [[0]], to="host") for tok in p[ask - 3:]]
            got = np.concatenate([rows[3], rows[4], rows[-1]])
        else:
            at, rows = 0, {}
            for c in [2, 61, 3, 64, 17, 2, 2, 30, 19]:
                out = eng.step([s], [p[at:at + c]], [list(range(c))], to="host")
                for i in range(c):
                    rows[at + i] = out[i:i + 1]
                at += c
            assert at == n
            got = np.concatenate([rows[a] for a in asking])
        eng.free_slot(s)
        compare(got, ref, asking, dtype, "marked token at %d, %s" % (marked, mode))
        at_second[marked] = ref[ask + 1]
    # the cases really differ at position 151: first key of the window against the token that nothing shows, and that against
    # the last token of the youngest block in sight
    spread = np.sqrt((at_second[115] ** 2).mean())
    assert np.abs(at_second[115] - at_second[114]).max() > 0.2 * spread
    assert np.abs(at_second[113] - at_second[114]).max() > 0.05 * spread
    assert np.abs(at_second[20] - at_second[114]).max() > 0.05 * spread


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R", "S", "T", "U"])
def test_prompt_then_token_by_token(root, name, dtype):
    """The last tokens one by one, across page borders of 64 and while the window and the blocks move on: states, the
    convolutions' histories, the previous token, the cached keys and the blocks' sums go from step to step."""
    eng, cfg, _ = engine(root, name, dtype)
    n, tail = (330, 150) if name == "R" else (120, 60)
    (p,) = prompts([n], cfg["vocab"], 6)
    s = eng.alloc_slot()
    got = [eng.step([s], [p[:n - tail]], [[n - tail - 1]], to="host")]
    for i in range(n - tail, n):
        got.append(eng.step([s], [[p[i]]], [[0]], to="host"))
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(n - tail - 1, n)), dtype, "%s decode" % name)
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "S"])
def test_all_tokens_one_by_one(root, name, dtype):
    """From the very first token: states start at zero, the rows before the first are zero, the first token takes the pair
    table's last row."""
    eng, cfg, _ = engine(root, name, dtype)
    (p,) = prompts([90], cfg["vocab"], 7)
    s = eng.alloc_slot()
    got = [eng.step([s], [[tok]], [[0]], to="host") for tok in p]
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(90)), dtype, "%s one by one" % name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,cuts", [("P", [2, 3, 7, 64, 65, 9, 1, 1, 2]), ("R", [64, 2, 128, 100, 6]), ("Q", [1, 2, 30, 37, 3]),
                                       ("S", [5, 64, 3, 70, 2, 2]), ("T", [3, 2, 40, 1, 5, 66, 2])])
def test_portions(root, name, cuts, dtype):
    """A prompt cut into steps of several sizes, down to two tokens (and one): portions shorter than the convolution keep
    part of the history that was there, and blocks are finished by later portions than began them."""
    eng, cfg, _ = engine(root, name, dtype)
    n = sum(cuts)
    (p,) = prompts([n], cfg["vocab"], 8)
    s = eng.alloc_slot()
    got, at = [], 0
    for c in cuts:
        got.append(eng.step([s], [p[at:at + c]], [list(range(c))], to="host"))
        at += c
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(n)), dtype, "%s portions %s" % (name, cuts))


@pytest.mark.parametrize("dtype", DTYPES)
def test_passes_of_the_step_function(root, dtype):
    """A prompt longer than the step function's pass: state, histories, blocks and cache go from pass to pass."""
    eng, cfg, _ = engine(root, "R", dtype, prefill_chunk=64)
    (p,) = prompts([300], cfg["vocab"], 9)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [list(range(300))], to="host")
    eng.free_slot(s)
    agree(got, root, "R", p, list(range(300)), dtype, "R in passes of 64")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R"])
def test_batch_of_unequal_requests(root, name, dtype):
    """Requests of different lengths in one batch (one of a single token), then decoded together; the shorter ones end
    earlier.  Every request must come out as it does alone."""
    eng, cfg, _ = engine(root, name, dtype)
    lengths = [1, 70, 131, 40] if name == "P" else [1, 200, 90]
    tail = 20
    ps = prompts([n + tail for n in lengths], cfg["vocab"], 10)
    slots = [eng.alloc_slot() for _ in ps]
    got = {i: [] for i in range(len(ps))}
    first = eng.step(slots, [p[:n] for p, n in zip(ps, lengths)], [[n - 1] for n in lengths], to="host")
    for i in range(len(ps)):
        got[i].append(first[i:i + 1])
    live = list(range(len(ps)))
    for k in range(tail):
        if k == 7:
            eng.free_slot(slots[live.pop(0)])               # the first request ends early
        out = eng.step([slots[i] for i in live], [[ps[i][lengths[i] + k]] for i in live], [[0]] * len(live), to="host")
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
    for i in live:
        eng.free_slot(slots[i])
    for i, p in enumerate(ps):
        n = lengths[i]
        places = list(range(n - 1, n - 1 + len(got[i])))
        agree(np.concatenate(got[i]), root, name, p, places, dtype, "%s request %d of a batch" % (name, i))
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(root, dtype):
    """A slot that held a long request is given to a short one: states, histories, the previous token and the blocks' sums
    start anew, stale pages are not read."""
    eng, cfg, _ = engine(root, "P", dtype, max_batch=2, max_ctx=256, max_tokens=512)
    a, b, c = prompts([200, 30, 90], cfg["vocab"], 11)
    for p in (a, b, c, b):
        s = eng.alloc_slot()
        got = eng.step([s], [p], [list(range(len(p)))], to="host")
        eng.free_slot(s)
        agree(got, root, "P", p, list(range(len(p))), dtype, "P in a slot used before (%d tokens)" % len(p))
    s1, s2 = eng.alloc_slot(), eng.alloc_slot()
    g1 = eng.step([s1, s2], [c[:50], b], [[49], [len(b) - 1]], to="host")
    g2 = eng.step([s1], [c[50:]], [list(range(40))], to="host")
    eng.free_slot(s1)
    eng.free_slot(s2)
    agree(np.concatenate([g1[:1], g2]), root, "P", c, [49] + list(range(50, 90)), dtype, "P cut in two, in a used slot")
    agree(g1[1:], root, "P", b, [len(b) - 1], dtype, "P beside it")
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(root, dtype):
    """Hundreds of single-token steps: the states run on, the window passes over decoded tokens, blocks fill up and come
    into sight, pages of the window go back."""
    eng, cfg, _ = engine(root, "R", dtype)
    (p,) = prompts([10 + 400], cfg["vocab"], 12)
    s = eng.alloc_slot()
    eng.step([s], [p[:10]], [[]], to="host")
    got = [eng.step([s], [[tok]], [[0]], to="host") for tok in p[10:]]
    eng.free_slot(s)
    agree(np.concatenate(got), root, "R", p, list(range(10, 410)), dtype, "R long decoding")


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation(root, name):
    """Engine.generate (the library's scheduler, its decoder with captured steps, its sampler) chooses the tokens that the
    plain implementation chooses."""
    eng, cfg, t = engine(root, name, "float32", max_batch=3)
    ps = prompts([5, 23, 64, 9], cfg["vocab"], 13)
    out = eng.generate(ps, max_new_tokens=12, temperature=0.0, ignore_eos=True)
    for p, g in zip(ps, out):
        want = plain.greedy(cfg, t, p, 12)
        for i, (a, b) in enumerate(zip(g.tokens, want)):
            if a != b:
                lg = plain.forward(cfg, t, p + want[:i])[-1]
                top2 = np.sort(lg)[-2:]
                assert top2[1] - top2[0] < 1e-4, "%s: token %d is %d, plain chooses %d" % (name, i, a, b)
                break
    assert nothing_held(eng)


def test_bf16_generation_runs_and_repeats(root):
    eng, cfg, _ = engine(root, "R", "bfloat16", max_batch=4)
    ps = prompts([5, 23, 64, 9], cfg["vocab"], 14)
    a = eng.generate(ps, max_new_tokens=20, temperature=0.0, ignore_eos=True)
    b = eng.generate(ps, max_new_tokens=20, temperature=0.0, ignore_eos=True)
    assert [g.tokens for g in a] == [g.tokens for g in b]
    assert all(len(g.tokens) == 20 for g in a)
    assert nothing_held(eng)
