"""Mozetar through the serving path (ServingEngine -> SequenceEngine -> tha_hyb_step) against the plain float64 statement of the
design in tests/mozetar_oracle.py.

Every test builds its own small configuration with random weights.  float32 runs are compared tightly (they differ from
float64 by rounding only), bfloat16 runs loosely.  Where random weights would hide a fault (one far key among hundreds, a key
at a border of the block table, a key just inside or just outside the window) the weights are made sharp: the queries of one
token are the keys of another and the score scale is large, so that the query probe puts nearly all its weight on the key
probe wherever that is; seeing it or not moves the output by tens of percent.
"""
import copy
import json
import os
import subprocess

import numpy as np
import pytest

import mozetar_oracle as O
from pkgload import load_pkg

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 6e-2


def rel_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.sqrt(((got - want) ** 2).mean()) / (np.sqrt((want ** 2).mean()) + 1e-12))


# ---- configurations ---------------------------------------------------------------------------------------------------
def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=10, groups=(3, 2)):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def windowed(mlp, heads=4, kv_heads=2, dim=16, vdim=12, conv=3, window=20, rot_dims=8, base=10000.0, scaling=(4.0, 1.0, 4.0, 32), scale=None,
             kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": window},
         "scale": scale if scale is not None else dim ** -0.5}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = {"factor": scaling[0], "low": scaling[1], "high": scaling[2], "original": scaling[3]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def differential(mlp, heads=4, kv_heads=2, dim=16, vdim=12, diff=0.4, q_temp=(0.3, 7), scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale if scale is not None else dim ** -0.5}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def recurrent(mlp, heads=3, dim=10, vdim=14):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def model(layers, width=64, vocab=130, streams=2, canon=3, eps=1e-5):
    c = {"architecture": "Mozetar", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width, "streams": streams}
    if canon:
        c["canon"] = {"taps": canon}
    return c


class Built:
    """A model folder, its oracle view, and engines on demand."""

    def __init__(self, tmp, cfg, seed=0, tweak=None):
        self.serving = load_pkg("serving")
        self.cfg = cfg
        self.w = O.random_weights(cfg, seed)
        if tweak:
            tweak(self.w)
            for k in self.w:
                self.w[k] = O.bf16_round(self.w[k]).astype(np.float64)
        self.folder = str(tmp)
        os.makedirs(self.folder, exist_ok=True)
        self.serving.save_model_folder(self.folder, cfg, {k: np.asarray(v, np.float32) for k, v in self.w.items()})
        self._ref = {}

    def engine(self, dtype="float32", max_tokens=1024, max_seqs=4):
        return self.serving.ServingEngine(self.folder, dtype, max_tokens, max_seqs)

    def ref(self, tokens):
        key = tuple(tokens)
        if key not in self._ref:
            self._ref[key] = O.forward(self.cfg, self.w, list(tokens))
        return self._ref[key]


def general_layers():
    # every mixer and both feed-forwards, sizes that differ between the layers, one layer without a feed-forward, one layer that
    # reads another's cache rows under a window of its own; the windows are shorter than the prompts
    return [windowed(dense(), heads=4, kv_heads=2, dim=16, vdim=12, window=20),
            recurrent(moe()),
            differential(dense(40), heads=4, kv_heads=2, dim=16, vdim=24),
            windowed(moe(experts=4, top=3, groups=None), heads=4, kv_heads=2, dim=16, vdim=12, window=33, kv_from=0),
            recurrent(None, heads=2, dim=12, vdim=8),
            differential(moe(experts=8, top=2, groups=(4, 1)), heads=3, kv_heads=1, dim=8, vdim=20, q_temp=(0.5, 16))]


@pytest.fixture(scope="module")
def general(tmp_path_factory):
    return Built(tmp_path_factory.mktemp("general"), model(general_layers(), streams=3), seed=1)


def tokens_for(built, n, seed):
    return np.random.default_rng(seed).integers(0, built.cfg["vocab"], n).tolist()


def feed(e, rid, toks, cuts, want_all=True):
    """the tokens in portions of the given sizes (the last size repeats); logits of every position"""
    out, at, i = [], 0, 0
    while at < len(toks):
        c = min(cuts[min(i, len(cuts) - 1)], len(toks) - at)
        r = e.step([(rid, toks[at:at + c], list(range(c)) if want_all else [])])
        if want_all:
            out.append(r)
        at += c
        i += 1
    return np.concatenate(out, 0) if want_all else None


# ---- whole prompts, every layer ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompt_every_layer(general, dtype, tol):
    toks = tokens_for(general, 97, 3)
    z, layers = general.ref(toks)
    e = general.engine(dtype)
    logits, taps = e.step([("a", toks, list(range(len(toks))))], taps=True)
    assert taps.shape == layers.shape
    for i in range(len(layers)):
        assert rel_err(taps[i], layers[i]) < tol, f"residual stream after layer {i}"
    assert rel_err(logits, z) < tol


# ---- each mechanism alone -----------------------------------------------------------------------------------------------
def one_layer(tmp, layer, width=48, seed=2, tweak=None, **kw):
    return Built(tmp, model([layer], width=width, vocab=90, **kw), seed, tweak)


def check_all_positions(b, n=70, dtype="float32", tol=F32_TOL, cuts=None):
    toks = tokens_for(b, n, 9)
    z, layers = b.ref(toks)
    e = b.engine(dtype)
    if cuts:
        got = feed(e, "a", toks, cuts)
    else:
        got, taps = e.step([("a", toks, list(range(n)))], taps=True)
        assert rel_err(taps[-1], layers[-1]) < tol
    assert rel_err(got, z) < tol
    return got, z


@pytest.mark.parametrize("rot_dims,scaling", [(8, (4.0, 1.0, 4.0, 32)), (16, None), (0, None), (6, (8.0, 2.0, 16.0, 200))])
def test_windowed_attention_alone(tmp_path, rot_dims, scaling):
    b = one_layer(tmp_path, windowed(None, rot_dims=rot_dims, scaling=scaling, window=9), canon=0)
    check_all_positions(b)
    check_all_positions(b, cuts=[3, 1, 20, 2])
    check_all_positions(b, n=3)                                  # the first tokens: the convolutions read zeros before the start


def test_rotary_frequencies_are_stretched_by_wavelength(tmp_path):
    """with the stretch left out, or applied to every frequency, the logits of a long prompt move by percent"""
    layer = windowed(None, heads=2, kv_heads=1, dim=16, vdim=8, rot_dims=16, base=50.0, scaling=(8.0, 1.0, 4.0, 16), window=300, scale=1.5)
    b = one_layer(tmp_path, layer, canon=0)
    toks = tokens_for(b, 200, 5)
    z, _ = b.ref(toks)
    plain = copy.deepcopy(b.cfg)
    del plain["layers"][0]["mixer"]["rot"]["scaling"]
    assert rel_err(O.forward(plain, b.w, toks)[0], z) > 1e-2
    assert rel_err(feed(b.engine(), "a", toks, [150, 1]), z) < F32_TOL


def test_short_convolutions_of_the_projections(tmp_path):
    """taps far from the identity; portions shorter than the taps, so that a tail is carried over several steps"""
    def tweak(w):
        for n in ("q", "k", "v"):
            w["l0.mix.%s.conv" % n][...] *= 2.0
    b = one_layer(tmp_path, windowed(None, conv=5, window=12), canon=0, tweak=tweak)
    check_all_positions(b, n=40, cuts=[1, 2, 1, 1, 3, 2, 7, 1])
    check_all_positions(b, n=40, cuts=[2])
    no_conv = copy.deepcopy(b.w)
    for n in ("q", "k", "v"):
        no_conv["l0.mix.%s.conv" % n][:, :-1] = 0.0
    toks = tokens_for(b, 40, 9)
    assert rel_err(O.forward(b.cfg, no_conv, toks)[0], b.ref(toks)[0]) > 1e-2


def test_input_convolution_alone(tmp_path):
    """the mixer reads h + conv(h): taps of order one, tails carried through portions of one and two tokens"""
    def tweak(w):
        w["l0.canon1"][...] *= 3.0
    for taps in (1, 2, 4):
        b = one_layer(tmp_path / str(taps), recurrent(None), canon=taps, tweak=tweak)
        check_all_positions(b, n=30)
        check_all_positions(b, n=30, cuts=[1, 2, 1, 5, 2])
        off = copy.deepcopy(b.w)
        off["l0.canon1"][...] = 0.0
        toks = tokens_for(b, 30, 9)
        assert rel_err(O.forward(b.cfg, off, toks)[0], b.ref(toks)[0]) > 1e-2


@pytest.mark.parametrize("q_temp", [None, (0.8, 5), (0.3, 1)])
def test_differential_attention_alone(tmp_path, q_temp):
    def tweak(w):
        w["l0.mix.g"][...] *= 3.0                                # gates far from one half
        w["l0.mix.lq1"][...] *= 3.0                              # lambda far from its constant
    b = one_layer(tmp_path, differential(None, heads=4, kv_heads=2, dim=8, vdim=12, diff=0.35, q_temp=q_temp), canon=0, tweak=tweak)
    got, z = check_all_positions(b)
    check_all_positions(b, cuts=[4, 1, 25, 2])
    check_all_positions(b, n=2)
    toks = tokens_for(b, 70, 9)
    w2 = copy.deepcopy(b.w)                                      # the two maps are not interchangeable
    q = w2["l0.mix.q"].reshape(4, 2, 8, -1)
    q[:] = q[:, ::-1].copy()
    assert rel_err(O.forward(b.cfg, w2, toks)[0], z) > 1e-2
    w3 = copy.deepcopy(b.w)                                      # lambda does enter
    w3["l0.mix.lq1"][...] = 0.0
    assert rel_err(O.forward(b.cfg, w3, toks)[0], z) > 1e-3


def test_recurrence_gate_extremes(tmp_path):
    """gates nearly closed (the state keeps what it has), nearly open (the state is the last value), and a high lower bound"""
    for bias, low in ((7.0, 0.0), (-7.0, 0.0), (0.0, 0.97), (-7.0, 0.5)):
        def tweak(w):
            w["l0.mix.f.b"][...] = bias
            w["l0.mix.lower"][...] = low
        b = one_layer(tmp_path / f"g{bias}_{low}", recurrent(None, heads=2, dim=9, vdim=11), canon=0, tweak=tweak)
        check_all_positions(b, n=60)
        check_all_positions(b, n=60, cuts=[7, 1, 2, 30])


def test_polynorm_feed_forward_alone(tmp_path):
    def tweak(w):
        w["l0.mix.o"][...] = 0.0                                 # the mixer adds nothing
        w["l0.mlp.act"][...] = [1.5, -0.7, 0.4, 0.25]
        w["l0.mlp.up.b"][...] *= 3.0
        w["l0.mlp.down.b"][...] *= 3.0
    b = one_layer(tmp_path, recurrent(dense(40)), tweak=tweak)
    got, z = check_all_positions(b, n=40)
    toks = tokens_for(b, 40, 9)
    for swap in ([-0.7, 1.5, 0.4, 0.25], [1.5, 0.4, -0.7, 0.25], [1.5, -0.7, 0.4, 0.0]):   # no two of the numbers are interchangeable
        w2 = copy.deepcopy(b.w)
        w2["l0.mlp.act"][...] = swap
        assert rel_err(O.forward(b.cfg, w2, toks)[0], z) > 1e-2
    for name in ("up.b", "down.b"):
        w2 = copy.deepcopy(b.w)
        w2["l0.mlp." + name][...] = 0.0
        assert rel_err(O.forward(b.cfg, w2, toks)[0], z) > 1e-2
    check_all_positions(b, n=40, dtype="bfloat16", tol=BF16_TOL)


@pytest.mark.parametrize("experts,top,groups", [(8, 2, (4, 2)), (8, 3, (2, 1)), (6, 6, None), (9, 2, (3, 3)), (5, 1, (1, 1)), (12, 4, (6, 2)),
                                                (80, 3, (40, 2)), (66, 4, (66, 37)), (36, 2, (36, 36))])
def test_mixture_router_groups(tmp_path, experts, top, groups):
    def tweak(w):
        w["l0.mix.o"][...] = 0.0
        w["l0.mlp.router"][...] *= 4.0                           # scores far from even: the kept groups differ from token to token
    b = one_layer(tmp_path, recurrent(moe(experts=experts, top=top, ff=12, groups=groups)), tweak=tweak)
    got, z = check_all_positions(b, n=80)
    if groups and groups[1] < min(top, groups[0]):               # fewer kept groups than picks: the groups do bind
        free = copy.deepcopy(b.cfg)
        del free["layers"][0]["mlp"]["router"]["groups"]
        assert rel_err(O.forward(free, b.w, tokens_for(b, 80, 9))[0], z) > 1e-2


def test_prompt_sized_steps_give_each_expert_its_own_product(tmp_path):
    """a step of more than a thousand rows whose experts get a thousand rows each takes, in bfloat16, one tensor-core product per
    expert over gathered rows; every expert is chosen here, so no choice can flip"""
    b = one_layer(tmp_path, recurrent(moe(experts=2, top=2, ff=64, groups=None), heads=2, dim=16, vdim=16), width=64)
    toks = tokens_for(b, 1100, 3)
    z, _ = b.ref(toks)
    got = b.engine("bfloat16", max_tokens=1152).step([("a", toks, list(range(1100)))])
    assert rel_err(got, z) < BF16_TOL
    assert max(rel_err(got[p], z[p]) for p in range(0, 1100, 7)) < 3 * BF16_TOL
    assert rel_err(feed(b.engine("bfloat16", max_tokens=1152), "a", toks, [500, 1]), z) < BF16_TOL


@pytest.mark.parametrize("streams", [1, 2, 4, 5])
def test_residual_streams(tmp_path, streams):
    """mixing matrices far from the identity and not symmetric: [from, to] and [to, from] differ by tens of percent"""
    def tweak(w):
        rng = np.random.default_rng(8)
        for i in range(2):
            for q in ("hc1", "hc2"):
                w["l%d.%s.mix" % (i, q)][...] = 0.6 * np.eye(streams) + 0.5 * rng.standard_normal((streams, streams)) + 0.7 * np.triu(np.ones((streams, streams)), 1)
                w["l%d.%s.in" % (i, q)][...] = rng.standard_normal(streams)
                w["l%d.%s.out" % (i, q)][...] = rng.standard_normal(streams)
    cfg = model([recurrent(dense(24)), differential(dense(16), heads=2, kv_heads=1, dim=8, vdim=8)], width=40, vocab=70, streams=streams)
    b = Built(tmp_path, cfg, 4, tweak)
    toks = tokens_for(b, 30, 1)
    z, layers = b.ref(toks)
    if streams > 1:
        w2 = copy.deepcopy(b.w)
        w2["l0.hc1.mix"] = w2["l0.hc1.mix"].T.copy()
        assert rel_err(O.forward(b.cfg, w2, toks)[0], z) > 1e-2
    logits, taps = b.engine().step([("a", toks, list(range(30)))], taps=True)
    for i in range(2):
        assert rel_err(taps[i], layers[i]) < F32_TOL
    assert rel_err(logits, z) < F32_TOL
    assert rel_err(feed(b.engine(), "a", toks, [4, 1, 2]), z) < F32_TOL


def test_a_layer_that_reads_another_layers_cache_rows(tmp_path):
    """layer 2 has no keys and values of its own: with rows of its own (or the rows of layer 1) the logits differ by percent;
    its query convolution has more taps than the convolutions of the layer whose rows it reads"""
    cfg = model([windowed(dense(24), window=14), windowed(None, window=30), windowed(dense(24), window=25, conv=5, kv_from=0)], width=48, vocab=90)
    b = Built(tmp_path, cfg, 6)
    toks = tokens_for(b, 80, 2)
    z, layers = b.ref(toks)
    other = copy.deepcopy(cfg)
    other["layers"][2]["mixer"]["kv_from"] = 1
    assert rel_err(O.forward(other, b.w, toks)[0], z) > 1e-2
    logits, taps = b.engine().step([("a", toks, list(range(80)))], taps=True)
    for i in range(3):
        assert rel_err(taps[i], layers[i]) < F32_TOL, f"layer {i}"
    for cuts in ([5, 2, 1, 30], [1], [40, 2]):
        assert rel_err(feed(b.engine(), "a", toks, cuts), z) < F32_TOL
    assert rel_err(feed(b.engine("bfloat16"), "a", toks, [50, 1]), z) < BF16_TOL


# ---- portions, decoding, batches ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cuts", [[1], [2], [3, 5, 2, 7, 1, 16, 2], [40, 1], [64, 2, 2, 33]])
def test_portions_equal_the_whole_prompt(general, cuts):
    toks = tokens_for(general, 110, 11)
    z, _ = general.ref(toks)
    assert rel_err(feed(general.engine(), "a", toks, cuts), z) < F32_TOL


def test_prefill_equals_token_by_token_decoding(general):
    toks = tokens_for(general, 90, 12)
    whole = general.engine().step([("a", toks, list(range(90)))])
    single = feed(general.engine(), "a", toks, [1])
    assert rel_err(single, whole) < 2e-5
    own = O.forward_tokenwise(general.cfg, general.w, toks)[0]
    assert rel_err(single, own) < F32_TOL


def test_portions_bfloat16(general):
    toks = tokens_for(general, 100, 13)
    z, _ = general.ref(toks)
    assert rel_err(feed(general.engine("bfloat16"), "a", toks, [37, 2, 1]), z) < BF16_TOL


def test_long_decoding(general):
    toks = tokens_for(general, 420, 14)
    z, _ = general.ref(toks)
    got = feed(general.engine(), "a", toks, [20, 1])
    assert rel_err(got, z) < F32_TOL
    assert rel_err(got[-1], z[-1]) < 5 * F32_TOL


def test_mixed_batches_equal_each_request_alone(general):
    """Five unequal requests through an engine with three slots and fewer blocks than their sum: portions of some beside
    single tokens of others, requests ending and their slots and blocks going to the next ones."""
    lens = [70, 5, 131, 33, 18]
    reqs = {f"r{i}": tokens_for(general, n, 20 + i) for i, n in enumerate(lens)}
    want = {k: general.ref(v)[0] for k, v in reqs.items()}
    e = general.engine(max_tokens=288, max_seqs=3)
    got = {k: [] for k in reqs}
    at = {k: 0 for k in reqs}
    waiting, live = list(reqs), []
    step = 0
    sizes = [7, 1, 16, 2, 1, 30, 1, 3]
    while waiting or live:
        while waiting and len(live) < 3 and e.free_blocks() * 16 >= len(reqs[waiting[0]]) + 48:
            live.append(waiting.pop(0))
        entries = []
        for j, k in enumerate(live):
            n = min(sizes[(step + j) % len(sizes)], len(reqs[k]) - at[k])
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        out = e.step(entries)
        o = 0
        for k, toks, w in entries:
            got[k].append(out[o:o + len(w)])
            o += len(w)
            at[k] += len(toks)
        for k in [k for k in live if at[k] == len(reqs[k])]:
            e.finish(k)
            live.remove(k)
        step += 1
    for k in reqs:
        assert rel_err(np.concatenate(got[k], 0), want[k]) < F32_TOL, k


def test_a_request_left_out_of_a_step_goes_on_later(general):
    a, b = tokens_for(general, 40, 51), tokens_for(general, 30, 52)
    e = general.engine(max_seqs=2)
    out = [e.step([("a", a[:10], list(range(10))), ("b", b[:7], list(range(7)))])]
    out.append(e.step([("b", b[7:20], list(range(13)))]))        # a waits
    out.append(e.step([("a", a[10:], list(range(30))), ("b", b[20:], list(range(10)))]))
    got_a = np.concatenate([out[0][:10], out[2][:30]])
    got_b = np.concatenate([out[0][10:], out[1], out[2][30:]])
    assert rel_err(got_a, general.ref(a)[0]) < F32_TOL
    assert rel_err(got_b, general.ref(b)[0]) < F32_TOL


def test_a_reused_slot_starts_from_zero_state_and_reused_blocks_hold_nothing(general):
    a, b = tokens_for(general, 80, 31), tokens_for(general, 45, 32)
    e = general.engine(max_tokens=128, max_seqs=1)
    e.step([("a", a, [])])
    e.finish("a")
    got = e.step([("b", b, list(range(45)))])                    # the recurrent state, every convolution tail and the cache start anew
    assert rel_err(got, general.ref(b)[0]) < F32_TOL


def test_pool_exhaustion_is_an_error_not_a_fault(general):
    e = general.engine(max_tokens=64, max_seqs=2)
    with pytest.raises(Exception):
        e.step([("a", tokens_for(general, 100, 1), [])])
    e.finish("a")
    got = e.step([("b", tokens_for(general, 20, 2), [19])])
    assert rel_err(got, general.ref(tokens_for(general, 20, 2))[0][[19]]) < F32_TOL


# ---- sharp attention: far keys, page borders, the edges of the window ----------------------------------------------------
HALF = 32


def sharp_model(tmp, kind, vocab=1024, window=40):
    """One layer whose queries read the upper half of the layer's input and whose keys read the lower half through the same
    matrix, with a large score scale.  The upper half of the embedding of the QUERY probe is the lower half of the embedding
    of the KEY probe, so the query probe puts nearly all its weight on the key probe wherever it can see it -- a different
    token with a different value.  The convolutions pass their input through (the last tap is one, the input convolution
    adds nothing), so that a probe's key is its own."""
    if kind == "windowed":
        layer = windowed(None, heads=2, kv_heads=1, dim=16, vdim=16, scale=2.0, rot_dims=4, window=window, conv=3)
    else:
        layer = differential(None, heads=2, kv_heads=1, dim=64, vdim=16, scale=1.5, diff=0.3, q_temp=(0.2, 64))
    cfg = model([layer], width=2 * HALF, vocab=vocab, streams=2)
    p = "l0.mix."

    def tweak(w):
        w["embed"][vocab - 2, HALF:] = w["embed"][vocab - 1, :HALF]
        w["l0.norm1"][HALF:] = w["l0.norm1"][:HALF]
        w["l0.canon1"][...] = 0.0
        if kind == "windowed":
            for n in ("q", "k", "v"):
                w[p + n + ".conv"][...] = 0.0
                w[p + n + ".conv"][:, -1] = 1.0
            w[p + "k"][:, HALF:] = 0.0
            q = w[p + "q"].reshape(2, 16, 2 * HALF)
            q[:, :, :HALF] = 0.0
            q[:, :, HALF:] = w[p + "k"][None, :, :HALF]
            q[:, :4] *= 0.05                                      # the rotated dimensions carry little
            w[p + "k"][:4] *= 0.05
        else:
            k = w[p + "k"].reshape(1, 2, 64, 2 * HALF)           # 64 channels: one key among hundreds stands out
            k[..., HALF:] = 0.0
            q = w[p + "q"].reshape(2, 2, 64, 2 * HALF)
            q[..., :HALF] = 0.0
            q[:, 0, :, HALF:] = k[0, 0, :, :HALF]                 # the first map is sharp,
            q[:, 1, :, HALF:] = 0.02 * k[0, 1, :, :HALF]          # the second nearly even
            w[p + "g"][...] = 0.0
    return Built(tmp, cfg, 12, tweak)


def distinct_tokens(n, vocab, seed):
    return np.random.default_rng(seed).permutation(vocab - 2)[:n].tolist()   # the last two tokens are the probes


def with_probes(b, n, key_pos, query_pos, seed):
    """distinct tokens with the key probe and the query probe in place; and the same without the key probe"""
    toks = distinct_tokens(n + 1, b.cfg["vocab"], seed)
    spare = toks.pop()
    toks[key_pos], toks[query_pos] = b.cfg["vocab"] - 1, b.cfg["vocab"] - 2
    other = list(toks)
    other[key_pos] = spare
    return toks, other


def check_probe(b, n, key_pos, query_pos, seen, cut_sets, dtype="float32"):
    """the engine agrees with the oracle at the query probe, which does (seen) or does not depend on the key probe"""
    toks, other = with_probes(b, n, key_pos, query_pos, key_pos * 7 + query_pos)
    z, _ = b.ref(toks)
    moved = rel_err(b.ref(other)[0][query_pos], z[query_pos])
    if seen:
        assert moved > 0.1, moved                              # the probe's key does carry the weight
    else:
        assert moved < 1e-9, moved                             # one layer: a key outside the mask changes nothing
    for cuts in cut_sets:
        cuts = [c for c in cuts if c > 0] or [1]
        got = feed(b.engine(dtype), "a", toks, cuts)
        if dtype == "float32":
            assert rel_err(got[query_pos], z[query_pos]) < 10 * F32_TOL, cuts
            assert rel_err(got, z) < F32_TOL, cuts
        else:
            assert rel_err(got[query_pos], z[query_pos]) < BF16_TOL, cuts


@pytest.mark.parametrize("key_pos,query_pos", [(0, 1), (0, 149), (15, 16), (16, 17), (63, 64), (64, 65), (63, 127), (64, 128), (127, 128), (1, 63)])
def test_keys_at_the_borders_of_the_block_table(tmp_path, key_pos, query_pos):
    b = sharp_model(tmp_path, "differential")
    check_probe(b, 150, key_pos, query_pos, True, ([150], [query_pos, 1], [key_pos, 2, 1], [key_pos + 1, 1]))


@pytest.mark.parametrize("dtype,decoded", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_one_far_key_among_hundreds(tmp_path, dtype, decoded):
    b = sharp_model(tmp_path, "differential")
    check_probe(b, 700, 3, 690, True, ([670, 1] if decoded else [300, 400],), dtype)


@pytest.mark.parametrize("query_pos", [41, 64, 95, 130])
def test_keys_just_inside_and_just_outside_the_window(tmp_path, query_pos):
    """window 40: the key at distance 39 is the last one seen, the key at distance 40 the first one lost -- in whole
    prompts, in portions that start at the key, the query or in between, and with the query decoded alone"""
    b = sharp_model(tmp_path, "windowed", window=40)
    for dist, seen in ((39, True), (40, False), (1, True)):
        key_pos = query_pos - dist
        check_probe(b, 140, key_pos, query_pos, seen, ([140], [query_pos, 1], [key_pos, 2, 1], [key_pos + 1, 17, 2], [33, 2]))


def test_window_edges_bfloat16(tmp_path):
    b = sharp_model(tmp_path, "windowed", window=40)
    check_probe(b, 140, 94, 133, True, ([140], [133, 1]), "bfloat16")
    check_probe(b, 140, 93, 133, False, ([140], [133, 1]), "bfloat16")


def test_the_window_of_a_layer_that_reads_another_layers_rows_is_its_own(tmp_path):
    """the giving layer sees 12 tokens, the reading layer 40: a key 30 back moves the reading layer's result only"""
    one = sharp_model(tmp_path / "one", "windowed", window=12)
    cfg = copy.deepcopy(one.cfg)
    cfg["layers"].append(copy.deepcopy(cfg["layers"][0]))
    cfg["layers"][1]["mixer"]["mask"]["size"] = 40
    cfg["layers"][1]["mixer"]["kv_from"] = 0

    def tweak(w):
        for k, v in one.w.items():
            w[k] = v.copy()
            if k.startswith("l0.") and ".mix.k" not in k and ".mix.v" not in k:
                w[k.replace("l0.", "l1.")] = v.copy()
        w["l0.mix.o"][...] = 0.0                                 # the giving layer adds nothing: layer 1 reads what layer 0 read
        w["l0.hc1.mix"][...] = np.eye(2)
    two = Built(tmp_path / "two", cfg, 0, tweak)
    check_probe(two, 140, 100, 130, True, ([140], [130, 1], [101, 2]))
    check_probe(two, 140, 90, 130, False, ([140], [130, 1]))


def test_few_rows_at_a_long_context_with_value_rows_that_are_no_multiple_of_a_warp(tmp_path):
    """Steps of one or two rows behind hundreds of positions are cut along the keys and merged, also for the two maps of a
    differential head whose results leave the attention as 32-bit floats in both number formats."""
    cfg = model([differential(dense(), heads=6, kv_heads=2, dim=32, vdim=40), windowed(None, heads=4, kv_heads=2, dim=16, vdim=72, window=900)],
                width=64, vocab=120)
    b = Built(tmp_path, cfg, 7)
    toks = tokens_for(b, 720, 4)
    z, _ = b.ref(toks)
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        got = feed(b.engine(dtype), "a", toks, [600, 38, 2, 1, 1, 2, 3, 1])
        assert max(rel_err(g, w) for g, w in zip(got[600:], z[600:])) < 3 * tol
        assert rel_err(got, z) < tol


# ---- the tensor-core attention forms of the bfloat16 number format ------------------------------------------------------
@pytest.mark.parametrize("kind", ["windowed", "differential"])
@pytest.mark.parametrize("cuts", [[300], [150, 86, 2, 1], [64, 1]])
def test_tensor_core_attention_bfloat16_every_position(tmp_path, kind, cuts):
    """Heads of 16 .. 128 channels take, in bfloat16, the form that keeps a warp's pairs in registers; it knows the window, the
    value head that two key heads share and the 32-bit result.  Peaked scores and a check of EVERY position by itself."""
    if kind == "windowed":
        layer = windowed(None, heads=6, kv_heads=2, dim=48, vdim=64, rot_dims=24, scale=0.6, window=70)
    else:
        layer = differential(None, heads=4, kv_heads=2, dim=32, vdim=24, scale=0.7, q_temp=(0.3, 50))
    b = Built(tmp_path, model([layer], width=64, vocab=200, streams=1, canon=0), 41)
    n = 300
    toks = tokens_for(b, n, 3)
    _, layers = b.ref(toks)
    base = b.w["embed"][np.asarray(toks)] * b.w["l0.hc1.mix"][0, 0]
    mix = layers[0] - base
    e = b.engine("bfloat16")
    at, got, i = 0, [], 0
    while at < n:
        c = min(cuts[min(i, len(cuts) - 1)], n - at)
        got.append(e.step([("a", toks[at:at + c], [])], taps=True)[1][0])
        at += c
        i += 1
    got = np.concatenate(got, 0) - base
    worst = max(rel_err(got[p], mix[p]) for p in range(n))
    assert worst < 6e-2, worst
    assert rel_err(got, mix) < 2e-2


# ---- other sizes: values that are often equal, or 1 ------------------------------------------------------------------
@pytest.mark.parametrize("case", ["single", "wide_heads", "everything_small", "odd_sizes", "plain", "window_one", "window_beyond", "many_kv_heads",
                                  "recurrent_wide"])
def test_other_sizes(tmp_path, case):
    width, streams, canon, n = 32, 2, 3, 75
    if case == "single":
        layers = [windowed(dense(8), heads=1, kv_heads=1, dim=8, vdim=40, rot_dims=2, conv=1, window=9),
                  differential(moe(experts=1, top=1, ff=16, groups=None), heads=1, kv_heads=1, dim=40, vdim=8),
                  recurrent(dense(16), heads=1, dim=8, vdim=40)]
        width, streams, canon = 24, 1, 1
    elif case == "wide_heads":
        layers = [windowed(dense(40), heads=2, kv_heads=2, dim=72, vdim=70, rot_dims=72, window=30, conv=2),
                  differential(None, heads=2, kv_heads=1, dim=72, vdim=136),
                  recurrent(moe(), heads=2, dim=72, vdim=40)]
        width = 40
    elif case == "everything_small":
        layers = [windowed(dense(1), heads=1, kv_heads=1, dim=2, vdim=1, rot_dims=2, window=2, conv=2),
                  differential(dense(1), heads=1, kv_heads=1, dim=1, vdim=3, q_temp=(1.0, 1)),
                  recurrent(moe(experts=2, top=1, ff=1, groups=(2, 1)), heads=1, dim=1, vdim=2)]
        width, canon = 8, 2
    elif case == "odd_sizes":
        layers = [windowed(dense(11), heads=6, kv_heads=3, dim=7, vdim=5, rot_dims=2, window=13, conv=5),
                  differential(moe(experts=9, top=4, ff=7, groups=(3, 2)), heads=6, kv_heads=3, dim=7, vdim=5, q_temp=(0.2, 3)),
                  recurrent(dense(9), heads=3, dim=11, vdim=7),
                  windowed(None, heads=6, kv_heads=3, dim=7, vdim=5, rot_dims=2, window=21, conv=5, kv_from=0)]
        width, streams, canon = 27, 5, 4
    elif case == "plain":                                     # one stream, no input convolution, no feed-forward anywhere, no rotation
        layers = [windowed(None, rot_dims=0), differential(None, q_temp=None), recurrent(None)]
        streams, canon = 1, 0
    elif case == "window_one":                                # every token sees itself only
        layers = [windowed(dense(), heads=2, kv_heads=1, dim=16, vdim=8, window=1), recurrent(None)]
    elif case == "window_beyond":                             # a window longer than the prompt
        layers = [windowed(dense(), heads=2, kv_heads=1, dim=16, vdim=8, window=500), differential(None)]
    elif case == "many_kv_heads":                             # as many key/value heads as heads; groups of three
        layers = [differential(dense(), heads=3, kv_heads=3, dim=16, vdim=8), windowed(None, heads=6, kv_heads=2, dim=16, vdim=24),
                  differential(None, heads=6, kv_heads=2, dim=16, vdim=8)]
    else:                                                     # more key channels than a warp's lanes, in both register forms
        layers = [recurrent(dense(), heads=2, dim=130, vdim=6), recurrent(None, heads=1, dim=300, vdim=18)]
    b = Built(tmp_path, model(layers, width=width, vocab=61, streams=streams, canon=canon), 5)
    toks = tokens_for(b, n, 2)
    z, layers_ref = b.ref(toks)
    e = b.engine()
    logits, taps = e.step([("a", toks, list(range(n)))], taps=True)
    for i in range(len(layers_ref)):
        assert rel_err(taps[i], layers_ref[i]) < F32_TOL, f"layer {i}"
    assert rel_err(logits, z) < F32_TOL
    assert rel_err(feed(b.engine(), "a", toks, [9, 2, 1]), z) < F32_TOL
    assert rel_err(feed(b.engine("bfloat16"), "a", toks, [40, 1]), z) < 2 * BF16_TOL


# ---- generation through the scheduler ---------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler(general):
    prompts = [tokens_for(general, n, 40 + n) for n in (5, 23, 70, 12, 3, 41)]
    new = [6, 9, 4, 12, 8, 5]
    e = general.engine(max_tokens=384, max_seqs=3)      # fewer slots than requests
    got = e.generate(prompts, new, temperature=0.0, portion=32)
    assert e.free_blocks() > 0 and e.steps_run() > max(new)
    for p, n, g in zip(prompts, new, got):
        assert len(g) == n
        st = O.Stepper(general.cfg, general.w)
        z = st.feed(p)[0][-1]
        for tok in g:
            best = int(np.argmax(z))
            if tok != best:                                # only a near tie may differ
                assert z[best] - z[tok] < 1e-3 * max(1.0, float(np.abs(z).max()))
            z = st.feed([tok])[0][-1]


def test_sampled_generation_is_reproducible_and_independent_of_the_batch(general):
    prompts = [tokens_for(general, n, 60 + n) for n in (9, 30)]
    a = general.engine(max_seqs=2).generate(prompts, [10, 10], temperature=1.0, topp=0.9, seed=7)
    b = general.engine(max_seqs=1).generate(prompts, [10, 10], temperature=1.0, topp=0.9, seed=7, portion=4)
    assert a == b


def test_the_app_serves_a_model_folder(general, tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    app = os.path.join(root, "build", "apps", "llama")
    if not os.path.exists(app):
        pytest.skip("the app is not built")
    prompts = [tokens_for(general, n, 80 + n) for n in (4, 19, 33)]
    (tmp_path / "in.txt").write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    r = subprocess.run([app, general.folder, "-m", "test", "-f", str(tmp_path / "in.txt"), "-o", str(tmp_path / "out.txt"), "-n", "7", "-b", "2",
                        "-d", "f32", "-j", "16"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in line.split()] for line in (tmp_path / "out.txt").read_text().splitlines()]
    want = general.engine(max_seqs=2).generate(prompts, [7, 7, 7], temperature=0.0, portion=16)
    assert got == want


def test_the_trace_replayer_answers_every_step(general, tmp_path):
    """bin/trace_run on a model folder: steps in, logits files out, requests ended and their slot used again"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "build", "apps", "trace_run")
    if not os.path.exists(exe):
        pytest.skip("the program is not built")
    a, b = tokens_for(general, 70, 1), tokens_for(general, 20, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:64], "want": [0, 63]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[64:], "want": [5]}, {"id": "b", "tokens": b[:18], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": b[18:], "want": [0, 1]}], "end": ["b"]}]
    out = tmp_path / "out"
    out.mkdir()
    r = subprocess.run([exe, "--model", general.folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "128", "--max-seqs", "2"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    za, zb = general.ref(a)[0], general.ref(b)[0]
    V = general.cfg["vocab"]
    assert rel_err(np.fromfile(out / "0.f32", np.float32).reshape(-1, V), za[[0, 63]]) < F32_TOL
    assert rel_err(np.fromfile(out / "1.f32", np.float32).reshape(-1, V), za[[69]]) < F32_TOL
    assert rel_err(np.fromfile(out / "2.f32", np.float32).reshape(-1, V), zb[[18, 19]]) < F32_TOL
