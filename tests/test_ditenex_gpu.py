"""Ditenex through the engine against the plain implementation (tests/plain_ditenex.py), on small configurations of
the tests' own (tests/ditenex_models.py) with weights drawn here: each mechanism alone, whole prompts, decoding token
by token, prompts cut into portions, batches of unequal requests, slots and pages used again, keys just inside and
just outside the windows and hundreds of tokens back, the first tokens of a sequence, long decoding, and greedy
generation through Engine.generate.

float32 must agree with the plain implementation to summation order.  In bfloat16 a router's close call can go the
other way, and another expert is another function, not a rounding: the bfloat16 runs use folders whose routers are
dominated by choice biases that lie far apart, and are compared with a bound relative to the logits' spread.
"""
import os

import numpy as np
import pytest

import ditenex_models as models
import harness
import plain_ditenex as plain
import tiny_configs
from friday_inference_engine_b200 import Engine

pytestmark = pytest.mark.gpu
DTYPES = [pytest.param("float32", id="f32"), pytest.param("bfloat16", id="bf16")]
STANDOUT_TOKEN = 7

_made = {}


def model(root, name, dtype, standout=False):
    clear = dtype != "float32"
    key = (str(root), name, clear, standout)
    if key not in _made:
        cfg = models.CONFIGS[name]
        t = models.tensors_of(cfg, np.random.default_rng(models.SEEDS[name]), clear_routing=clear)
        if standout:
            models.standout(cfg, t, 0, STANDOUT_TOKEN)
        d = models.write_folder(os.path.join(str(root), "ditenex_%s_%d_%d" % (name, clear, standout)), cfg, t)
        _made[key] = (d,) + plain.load(d)
    return _made[key]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("ditenex")


def engine(root, name, dtype, standout=False, **kw):
    d, cfg, t = model(root, name, dtype, standout)
    kw.setdefault("max_ctx", 1024)
    kw.setdefault("max_batch", 6)
    return Engine(model_path=d, dtype=dtype, **kw), cfg, t


_plain = {}


def plain_logits(root, name, prompt, dtype, standout=False):
    key = (str(root), name, tuple(prompt), dtype != "float32", standout)
    if key not in _plain:
        _, cfg, t = model(root, name, dtype, standout)
        _plain[key] = plain.forward(cfg, t, prompt)
    return _plain[key]


def agree(got, root, name, prompt, places, dtype, what, standout=False):
    ref = plain_logits(root, name, prompt, dtype, standout)
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


def prompts(lengths, vocab, seed, without=None):
    ps = tiny_configs.random_prompts(lengths, vocab, seed)
    if without is not None:
        ps = [[(tok + 1) % vocab if tok == without else tok for tok in p] for p in ps]
    return ps


def nothing_held(eng):
    st = eng.stats()
    return st["slots_held"] == 0 and all(g["pages_held"] == 0 for g in st["groups"])


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention_only", "blend_only", "dense_only", "experts_only"])
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
@pytest.mark.parametrize("name,n", [("P", 200), ("Q", 70), ("R", 400), ("S", 150), ("T", 200), ("U", 260), ("V", 170)])
def test_whole_prompt(root, name, n, dtype):
    eng, cfg, _ = engine(root, name, dtype)
    (p,) = prompts([n], cfg["vocab"], 5)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [list(range(n))], to="host")
    eng.free_slot(s)
    agree(got, root, name, p, list(range(n)), dtype, "%s whole %d" % (name, n))
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R", "S", "T", "U", "V"])
def test_prompt_then_token_by_token(root, name, dtype):
    """The last tokens one by one, across page borders of 64 and with the windows moving over decoded tokens: keys,
    values and the shift's row go from step to step."""
    eng, cfg, _ = engine(root, name, dtype)
    n, tail = (460, 330) if name == "R" else (230, 150)
    (p,) = prompts([n], cfg["vocab"], 6)
    s = eng.alloc_slot()
    got = [eng.step([s], [p[:n - tail]], [[n - tail - 1]], to="host")]
    for i in range(n - tail, n):
        got.append(eng.step([s], [[p[i]]], [[0]], to="host"))
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(n - tail - 1, n)), dtype, "%s decode" % name)
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_all_tokens_one_by_one(root, name, dtype):
    """From the very first token: the row before the first is zero, the first windows are not full."""
    eng, cfg, _ = engine(root, name, dtype)
    (p,) = prompts([80], cfg["vocab"], 7)
    s = eng.alloc_slot()
    got = [eng.step([s], [[tok]], [[0]], to="host") for tok in p]
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(80)), dtype, "%s one by one" % name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,cuts", [("P", [2, 3, 7, 64, 65, 9, 1, 1, 2, 50]), ("R", [64, 2, 128, 100, 6, 130]), ("Q", [1, 2, 30, 37, 3]),
                                       ("S", [5, 64, 3, 70, 2, 2]), ("T", [3, 2, 40, 1, 5, 66, 2, 90])])
def test_portions(root, name, cuts, dtype):
    """A prompt cut into steps of several sizes, down to two tokens (and one): the first row of a portion shifts with the
    last row of the portion before, its queries see the keys that earlier portions left."""
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
    """A prompt longer than the step function's pass: the shift's row, the first layer's values and the cache go from
    pass to pass."""
    eng, cfg, _ = engine(root, "R", dtype, prefill_chunk=64)
    (p,) = prompts([300], cfg["vocab"], 9)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [list(range(300))], to="host")
    eng.free_slot(s)
    agree(got, root, "R", p, list(range(300)), dtype, "R in passes of 64")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R", "S", "V"])
def test_batch_of_unequal_requests(root, name, dtype):
    """Requests of different lengths in one batch (one of a single token), then decoded together; the shorter ones
    end earlier.  Every request must come out as it does alone."""
    eng, cfg, _ = engine(root, name, dtype)
    lengths = [1, 70, 131, 40] if name != "R" else [1, 200, 90]
    tail = 40
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
        if k == 25:
            eng.free_slot(slots[live.pop(1)])               # and one from the middle
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
    """A slot that held a long request is given to a short one: the shift's row starts at zero again, stale pages are
    not read."""
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


# ---------------------------------------------------------------------------------------------
# one key that outweighs all others: in sight or not decides the logits
def standout_prompt(cfg, n, at, seed):
    (p,) = prompts([n], cfg["vocab"], seed, without=STANDOUT_TOKEN)
    p[at] = STANDOUT_TOKEN
    return p


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,at", [("attention_only", 30), ("attention_only", 0), ("attention_only", 63), ("P", 64), ("far", 5), ("far", 127)])
def test_window_edges_in_a_prompt(root, name, at, dtype):
    """The token whose key outweighs all others sits at `at` (a sequence's first token, a page's last or first row); the
    positions around the one where it leaves the first layer's window are asked for, in a whole prompt."""
    eng, cfg, _ = engine(root, name, dtype, True)
    window = cfg["layers"][0]["mixer"]["mask"]["size"]
    n = at + window + 6
    p = standout_prompt(cfg, n, at, 21)
    places = sorted({0, 1, at, at + 1} | set(range(at + window - 4, n)))
    s = eng.alloc_slot()
    got = eng.step([s], [p], [places], to="host")
    eng.free_slot(s)
    agree(got, root, name, p, places, dtype, "%s: the standout token at %d, window %d" % (name, at, window), True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,at,cut", [("attention_only", 30, 40), ("attention_only", 63, 64), ("P", 64, 70), ("far", 127, 130), ("far", 1, 2)])
def test_window_edges_in_decoding(root, name, at, cut, dtype):
    """The same with the positions around the edge decoded one by one after a prompt of `cut` tokens, and once more with
    the prompt's rest in portions of three."""
    eng, cfg, _ = engine(root, name, dtype, True)
    window = cfg["layers"][0]["mixer"]["mask"]["size"]
    n = at + window + 6
    p = standout_prompt(cfg, n, at, 22)
    s = eng.alloc_slot()
    got = [eng.step([s], [p[:cut]], [[cut - 1]], to="host")]
    for i in range(cut, n):
        got.append(eng.step([s], [[p[i]]], [[0]], to="host"))
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(cut - 1, n)), dtype, "%s: decoding past the edge" % name, True)
    s = eng.alloc_slot()
    got = [eng.step([s], [p[:cut]], [[cut - 1]], to="host")]
    for i in range(cut, n, 3):
        got.append(eng.step([s], [p[i:i + 3]], [list(range(len(p[i:i + 3])))], to="host"))
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(cut - 1, n)), dtype, "%s: portions of three past the edge" % name, True)
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(root, dtype):
    """Hundreds of single-token steps: the windows move over decoded tokens, pages behind them go back and come again."""
    eng, cfg, _ = engine(root, "R", dtype, max_batch=1, max_ctx=1024, max_tokens=1024)
    (p,) = prompts([10 + 500], cfg["vocab"], 12)
    s = eng.alloc_slot()
    eng.step([s], [p[:10]], [[]], to="host")
    got = [eng.step([s], [[tok]], [[0]], to="host") for tok in p[10:]]
    eng.free_slot(s)
    agree(np.concatenate(got), root, "R", p, list(range(10, 510)), dtype, "R long decoding")
    assert nothing_held(eng)


@pytest.mark.parametrize("name", ["P", "R", "T"])
def test_greedy_generation(root, name):
    """Engine.generate (the library's scheduler, its decoder with captured steps, its sampler) chooses the tokens
    that the plain implementation chooses."""
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
