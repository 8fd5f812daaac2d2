"""Vulanex without a GPU: its configuration, what its layers ask of the cache, the tensors it declares, the cache's books
for rows that stand for blocks of positions, and the plain implementation's own mechanisms against hand-made cases."""
import copy
import math

import numpy as np
import pytest

from friday_inference_engine_b200 import ConfigError, describe_model, read_config
from friday_inference_engine_b200.cache import PAGE, CacheBook, CacheError, kv_request, several, state_request

import plain_vulanex as plain

ATT = {"heads": 6, "kv_heads": 3, "dim": 16, "vdim": 16, "scale": 0.2, "q_temp": {"coef": 0.25, "every": 5}}
LEFT = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "mask": {"size": 40, "pool": 12},
        "rot": {"base": 10000.0, "dims": 8, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}}}
RIGHT = {"heads": 3, "dim": 20}
MLP = {"kind": "dense", "ff": 40}
CFG = {"architecture": "Vulanex", "vocab": 50, "width": 32, "logit_scale": 1.5, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
       "embedding": {"bigram": {"buckets": 97, "mul_prev": 13, "mul_cur": 3}},
       "layers": [{"type": "attention", "mixer": ATT, "mlp": MLP}, {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT}, "mlp": None},
                  {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT}, "mlp": MLP}]}


def test_the_name_selects_the_design():
    assert read_config(CFG)["architecture"] == "Vulanex"
    d = describe_model(CFG)
    assert d["architecture"] == "Vulanex"
    assert [c["layer"] for c in d["program"]] == [0, 1, 2] and [c["cache"] for c in d["program"]] == [0, 1, 2]


def test_cache_requests():
    reqs = describe_model(CFG)["cache_requests"]
    hist = {"kind": "state", "shape": [3 * 32], "dtype": "float32"}
    # keys only (the values are the keys), then the two convolutions' histories
    keys = {"kind": "kv", "n_kv_heads": 3, "head_dim": 16, "window": 0, "v_head_dim": 16, "keep_first": 0, "keys_only": True}
    assert reqs["0"] == {"kind": "several", "parts": [keys, hist, hist]}
    tokens = {"kind": "kv", "n_kv_heads": 2, "head_dim": 16, "window": 40, "v_head_dim": 24, "keep_first": 0}
    blocks = {"kind": "kv", "n_kv_heads": 2, "head_dim": 16, "window": 0, "v_head_dim": 24, "keep_first": 0, "every": 12, "store_f32": True}
    state = {"kind": "state", "shape": [3 * 20 * 20], "dtype": "float32"}
    assert reqs["1"] == {"kind": "several", "parts": [tokens, blocks, state, hist]}          # no feed-forward: one history
    assert reqs["2"] == {"kind": "several", "parts": [tokens, blocks, state, hist, hist]}
    # the previous token of the pair table, one integer per sequence
    (embed,) = [v for k, v in reqs.items() if k not in ("0", "1", "2")]
    assert embed == {"kind": "state", "shape": [1], "dtype": "int32"}


def test_declared_tensors():
    d = describe_model(CFG)
    shapes = {p["name"]: p["shape"] for p in d["params"]}
    assert shapes["embed"] == [50, 32] and shapes["bigram"] == [98, 32] and "head" not in shapes
    assert shapes["final.norm"] == [32] and shapes["final.norm.b"] == [32]
    assert shapes["l0.norm1.b"] == [32] and shapes["l0.canon1"] == [32, 4] and shapes["l0.canon2"] == [32, 4]
    assert shapes["l0.mix.q"] == [96, 32] and shapes["l0.mix.k"] == [48, 32] and shapes["l0.mix.o"] == [32, 96] and "l0.mix.v" not in shapes
    assert shapes["l1.mix.left.q"] == [64, 32] and shapes["l1.mix.left.k"] == [32, 32] and shapes["l1.mix.left.v"] == [48, 32]
    assert shapes["l1.mix.left.q.norm"] == [16] and shapes["l1.mix.left.sink"] == [4] and shapes["l1.mix.left.o"] == [32, 96]
    assert shapes["l1.mix.left.out"] == [32] and shapes["l1.mix.right.out"] == [32]
    for n in ("r", "k", "v", "g", "a"):
        assert shapes["l1.mix.right." + n] == [60, 32]
    assert shapes["l1.mix.right.a.b"] == [60] and shapes["l1.mix.right.w0"] == [60] and shapes["l1.mix.right.norm"] == [60]
    assert shapes["l1.mix.right.w1"] == [-1, 32] and shapes["l1.mix.right.w2"] == [60, -1] and shapes["l1.mix.right.o"] == [32, 60]
    assert "l1.norm2" not in shapes and "l1.canon2" in d["ignorable"] and "l1.mlp.gate" not in shapes
    assert shapes["l2.mlp.gate"] == [40, 32] and shapes["l2.mlp.down"] == [32, 40]


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.pop("logit_scale"), "logit_scale"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["canon"].update(taps=9), "taps"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
    (lambda c: c["embedding"]["bigram"].update(mul_cur=-1), "mul_cur"),
    (lambda c: c["layers"][0].update(type="mamba"), "mamba"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "moe"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "share"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][1]["mixer"]["left"]["mask"].pop("pool"), "pool"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=3), "dims"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].update(factor=0), "factor"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
])
def test_bad_config_names_the_key(change, word):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        read_config(cfg)
    assert word in str(e.value)


# ---- the cache's books for rows that stand for blocks of positions
def test_rows_for_blocks_take_pages_by_blocks():
    P = 5
    book = CacheBook({0: several(kv_request(1, 8, window=70), kv_request(1, 8, every=P, store_f32=True), state_request([4]))},
                     16 * PAGE, 8 * PAGE, max_slots=2)
    info = book.info()
    tokens, blocks = info["groups"]
    assert tokens["window"] == 70 and blocks["window"] == 0
    assert blocks["n_pages"] == (16 + P - 1) // P + 2                  # a fifth of the tokens' pages, and one begun page per sequence
    s = book.alloc_slot()
    held = []
    for step in [3, 61, 1, 200, 55, 1, 1, 90]:
        book.reserve([s], [step])
        book.commit([s], [step])
        info = book.info()
        n = info["lens"][s]
        # blocks: a page for every 64 blocks begun, never given back while the sequence lives
        assert info["groups"][1]["pages_held"] == ((n + P - 1) // P + PAGE - 1) // PAGE
        # tokens: the pages from the window's first position to the last token
        first = max(0, n - 70 + 1) // PAGE
        assert info["groups"][0]["pages_held"] == (n + PAGE - 1) // PAGE - first
        held.append(n)
    book.free_slot(s)
    info = book.info()
    assert all(g["pages_held"] == 0 for g in info["groups"]) and info["slots_held"] == 0


def test_rows_for_blocks_have_no_window():
    with pytest.raises(CacheError):
        CacheBook({0: kv_request(1, 8, window=16, every=4)}, 4 * PAGE, 2 * PAGE, max_slots=1)


# ---- the plain implementation's mechanisms against cases worked by hand
def test_plain_pair_rows_and_convolution():
    assert plain.bigram_rows([4, 9, 2], 7, 3, 5) == [7, (4 * 3 + 9 * 5) % 7, (9 * 3 + 2 * 5) % 7]
    h = np.arange(8, dtype=np.float64).reshape(4, 2)
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]])
    y = plain.input_conv(h, w)
    # the last tap is the present row's, and the row itself is added
    assert y[0].tolist() == [0.0, 1.0 + 2.0] and y[1].tolist() == [2 + 200.0, 3 + 6.0]
    assert y[3].tolist() == [6 + 1 * 2 + 10 * 4 + 100 * 6, 7 + 14.0]
    ln = plain.layer_norm(np.array([[1.0, 3.0]]), np.array([2.0, 2.0]), np.array([0.5, 0.5]), 0.0)
    assert np.allclose(ln, [[-1.5, 2.5]])


def test_plain_query_multiplier_and_rotation_table():
    m = plain.query_temperature(9, 0.5, 4)
    assert np.allclose(m[:3], 1.0) and np.isclose(m[3], 1.0 + 0.5 * math.log(2.0)) and np.isclose(m[7], 1.0 + 0.5 * math.log(3.0))
    f, mult = plain.rotary_table({"base": 100.0, "dims": 4})
    assert np.allclose(f, [1.0, 0.1]) and mult == 1.0
    f, mult = plain.rotary_table({"base": 100.0, "dims": 4, "scaling": {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0}})
    assert np.isclose(mult, 0.1 * math.log(4.0) + 1.0)
    assert np.isclose(f[0], 1.0) and 0.1 / 4.0 <= f[1] < 0.1              # the short wavelength stays, the long one is stretched
    x = np.zeros((3, 1, 6))
    x[:, 0, 0] = 1.0                                                        # pairs (0, 2) and (1, 3); 4 and 5 pass unchanged
    x[:, 0, 5] = 7.0
    r = plain.rotate_half(x, {"base": 100.0, "dims": 4})
    assert np.allclose(r[2, 0], [math.cos(2.0), 0.0, math.sin(2.0), 0.0, 0.0, 7.0])


def test_plain_window_blocks_and_sink():
    """One head of size 2 with identity projections: which tokens and blocks a row sees, that a block's key is the mean of
    its keys, and that the sink only joins the denominator."""
    T, size, P = 9, 3, 2
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "mask": {"size": size, "pool": P}, "rot": {"base": 10.0, "dims": 0}}
    eye = np.eye(2)
    W = {"q": eye * 0.0, "k": eye, "v": eye, "o": eye, "q.norm": np.ones(2), "k.norm": np.ones(2), "sink": np.array([-1e9])}
    h = np.arange(2 * T, dtype=np.float64).reshape(T, 2) + 1.0
    out = plain.pooled_window_attention(h, W, m, 1e-9)
    # queries are zero: every seen key weighs the same, so a row's result is the mean of the values it sees
    i = 8                       # sees tokens 6, 7, 8 and the blocks wholly before position 6: (0, 1), (2, 3), (4, 5)
    seen = [h[6], h[7], h[8], h[0:2].mean(0), h[2:4].mean(0), h[4:6].mean(0)]
    assert np.allclose(out[i], np.mean(seen, axis=0))
    i = 4                       # tokens 2, 3, 4; block (0, 1) ends at 1 = i - size: seen; block (2, 3) not
    assert np.allclose(out[i], np.mean([h[2], h[3], h[4], h[0:2].mean(0)], axis=0))
    i = 3                       # tokens 1, 2, 3; block (0, 1) ends at 1 > i - size = 0: token 0 is seen by nobody
    assert np.allclose(out[i], np.mean([h[1], h[2], h[3]], axis=0))
    W["sink"] = np.array([0.0])                    # exp(0) = 1 beside n weights of 1: the result shrinks by n / (n + 1)
    assert np.allclose(plain.pooled_window_attention(h, W, m, 1e-9)[3], np.mean([h[1], h[2], h[3]], axis=0) * 3.0 / 4.0)


def test_plain_delta_rule_decays_removes_and_writes():
    # one head of two channels; projections picked so that k = (1, 0) then (0, 1) then (1, 0), v = r = k
    H = {"heads": 1, "dim": 2}
    eye = np.eye(2)
    big = 50.0
    W = {"r": eye, "k": eye, "v": eye, "g": eye * 0.0, "a": eye * 0.0, "a.b": np.array([big, big]),          # a = 1: full removal
         "w1": np.zeros((1, 2)), "w2": np.zeros((2, 1)), "w0": np.array([-big, -big]),                      # w = exp(0) = 1: no decay
         "norm": np.ones(2), "o": eye}
    h = np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 0.0]])
    S = np.zeros((1, 2, 2))
    plain.delta_rule(h, W, H, 1e-5, state=S)
    # token 3 removes what token 1 wrote along (1, 0) and writes it again: the state is the identity, not 2 at [0, 0]
    assert np.allclose(S[0], np.eye(2), atol=1e-5)
    W["a.b"] = np.array([-big, -big])              # a = 0: nothing is removed, writes add up
    S = np.zeros((1, 2, 2))
    plain.delta_rule(h, W, H, 1e-5, state=S)
    assert np.allclose(S[0], [[2.0, 0.0], [0.0, 1.0]], atol=1e-5)
    W["w0"] = np.array([big, big])                 # w = exp(-exp(-1/2)): every step shrinks what was there
    S = np.zeros((1, 2, 2))
    plain.delta_rule(h, W, H, 1e-5, state=S)
    d = math.exp(-math.exp(-0.5))
    assert np.allclose(S[0], [[d * d + 1.0, 0.0], [0.0, d]], atol=1e-5)
