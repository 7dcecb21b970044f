"""Bozovik through the serving path (ServingEngine -> SequenceEngine -> tha_hyb_step) against the plain float64 statement
of the design in tests/bozovik_oracle.py.

Every test builds its own small configuration with random weights.  float32 runs are compared tightly (they differ from
float64 by rounding only), bfloat16 runs loosely.  Where random weights would hide a fault (one far key among hundreds,
a key at a border of the block table, a key just inside or just outside a window, a kept first token, a sink) the weights
are made sharp: the queries of one token are the keys of another and the score scale is large, so that the query probe puts
nearly all its weight on the key probe wherever that is; seeing it or not moves the output by tens of percent.
"""
import copy
import json
import os
import subprocess

import numpy as np
import pytest

import bozovik_oracle as O
from pkgload import load_pkg

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 6e-2


def rel_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.sqrt(((got - want) ** 2).mean()) / (np.sqrt((want ** 2).mean()) + 1e-12))


# ---- configurations ---------------------------------------------------------------------------------------------------
def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def attn(heads=4, kv_heads=2, dim=16, vdim=12, scale=None, rot_dims=None, base=10000.0, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot_dims != 0:
        m["rot"] = {"base": base, "dims": rot_dims or dim}
    if mask:
        m["mask"] = {"size": mask[0]}
        if mask[1] is not None:
            m["mask"]["keep_first"] = mask[1]
    return m


def attention(mlp, **kw):
    return {"type": "attention", "mixer": attn(**kw), "mlp": mlp}


def latent(mlp, heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=32, window=20, base=10000.0, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def parallel(mlp, left=None, heads=2, dim=24, left_scale=0.8, right_scale=1.3):
    left = left or attn(heads=2, kv_heads=1, dim=24, vdim=16, rot_dims=8, base=5000.0, mask=(24, 3))
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": heads, "dim": dim}, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def model(layers, width=64, vocab=130, loop=None, side=6, mult=0.8, embed_scale=3.0, eps=1e-5):
    c = {"architecture": "Bozovik", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width, "residual_mult": mult,
         "embedding": {"scale": embed_scale}}
    if side:
        c["token_side"] = {"dim": side}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


class Built:
    """A model folder, its oracle view, and engines on demand."""

    def __init__(self, tmp, cfg, seed=0, tweak=None, decay_rank=5):
        self.serving = load_pkg("serving")
        self.cfg = cfg
        self.w = O.random_weights(cfg, seed, decay_rank=decay_rank)
        if tweak:
            tweak(self.w)
            for k in self.w:
                self.w[k] = O.bf16_round(self.w[k]).astype(np.float64)
        self.folder = str(tmp)
        self.serving.save_model_folder(self.folder, cfg, {k: np.asarray(v, np.float32) for k, v in self.w.items()})
        self._ref = {}

    def engine(self, dtype="float32", max_tokens=1024, max_seqs=4):
        return self.serving.ServingEngine(self.folder, dtype, max_tokens, max_seqs)

    def ref(self, tokens, cfg=None):
        key = (tuple(tokens), json.dumps(cfg, sort_keys=True) if cfg else "")
        if key not in self._ref:
            taps = []
            z = O.forward(cfg or self.cfg, self.w, list(tokens), taps)
            self._ref[key] = (z, np.stack(taps))
        return self._ref[key]


def general_layers():
    # every mixer, sizes that differ between the layers, one layer without a feed-forward; the window of the latent layer
    # and of the left side are shorter than the prompts, the kept first tokens are few
    return [attention(dense(), heads=4, kv_heads=2, dim=16, vdim=12, rot_dims=8),
            latent(dense(40), window=20),
            parallel(None),
            attention(dense(24), heads=3, kv_heads=3, dim=8, vdim=20, base=300.0)]


@pytest.fixture(scope="module")
def general(tmp_path_factory):
    return Built(tmp_path_factory.mktemp("general"), model(general_layers(), loop=(1, 3, 2)), seed=1)


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


# ---- whole prompts, every layer run -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompt_every_layer_run(general, dtype, tol):
    toks = tokens_for(general, 97, 3)
    z, layers = general.ref(toks)
    assert len(layers) == 1 + 2 * 2 + 1                      # the looped pair counts every time
    e = general.engine(dtype)
    logits, taps = e.step([("a", toks, list(range(len(toks))))], taps=True)
    assert taps.shape == layers.shape
    for i in range(len(layers)):
        assert rel_err(taps[i], layers[i]) < tol, f"residual stream after layer run {i}"
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


def test_attention_alone_with_its_head_factors_and_gates(tmp_path):
    def tweak(w):
        w["l0.mix.temp"][...] = [0.3, 2.5, 1.0, 0.05]        # far from one: a factor left out or given to the wrong head shows
        w["l0.mix.g"][...] *= 3.0
    b = one_layer(tmp_path, attention(None, rot_dims=6), side=0, tweak=tweak)
    check_all_positions(b)
    # the first tokens: position 0 sees itself and the sink fixed at zero, so its weight is e^s / (1 + e^s), not 1
    check_all_positions(b, n=3)


def test_latent_attention_alone(tmp_path):
    b = one_layer(tmp_path, latent(None, heads=2, dim=8, rot_dim=4, vdim=6, kv_rank=12, window=9), side=0)
    check_all_positions(b)
    check_all_positions(b, cuts=[3, 1, 20, 2])


@pytest.mark.parametrize("left_scale,right_scale", [(1.0, 0.0), (0.0, 1.0), (0.6, 1.7)])
def test_parallel_mixer_each_side_alone_and_both(tmp_path, left_scale, right_scale):
    b = one_layer(tmp_path, parallel(None, left_scale=left_scale, right_scale=right_scale), side=0)
    check_all_positions(b)
    check_all_positions(b, cuts=[5, 2, 1, 30])


def test_delta_rule_decay_and_removal_extremes(tmp_path):
    # strong removal with slow decay, and fast decay without removal
    for w0, ab in ((-8.0, 6.0), (6.0, -8.0)):
        def tweak(w):
            w["l0.mix.right.w0"][...] = w0
            w["l0.mix.right.a.b"][...] = ab
        b = one_layer(tmp_path / f"d{int(w0)}", parallel(None, left_scale=0.0, right_scale=1.0, heads=3, dim=10), side=0, tweak=tweak)
        check_all_positions(b, n=60)


def test_feed_forward_alone(tmp_path):
    def tweak(w):
        w["l0.mix.o"][...] = 0.0                               # the mixer adds nothing
        w["l0.mlp.act"][...] = [1.5, -0.7]
    b = one_layer(tmp_path, attention(dense(40)), side=0, tweak=tweak)
    got, z = check_all_positions(b, n=40)
    w2 = copy.deepcopy(b.w)
    w2["l0.mlp.act"][...] = [-0.7, 1.5]                        # the two numbers are not interchangeable
    assert rel_err(O.forward(b.cfg, w2, tokens_for(b, 40, 9)), z) > 1e-2


def test_token_side_input_alone(tmp_path):
    def tweak(w):
        w["l0.mix.o"][...] = 0.0
        w["l1.mix.o"][...] = 0.0
    cfg = model([attention(None), attention(None)], width=40, vocab=70, side=5)
    b = Built(tmp_path, cfg, 4, tweak)
    toks = tokens_for(b, 30, 1)
    z, layers = b.ref(toks)
    assert rel_err(layers[0], O.embed(b.cfg, b.w, toks)) > 1e-2   # the side input does move the stream
    logits, taps = b.engine().step([("a", toks, list(range(30)))], taps=True)
    for i in range(2):                                             # layer 1 reads the second column range of the table
        assert rel_err(taps[i], layers[i]) < F32_TOL
    assert rel_err(logits, z) < F32_TOL


def test_loop_adds_the_embedding_and_the_vector_of_the_pass(tmp_path):
    cfg = model([attention(dense(24)), latent(None, window=7), attention(None, heads=2, kv_heads=1)], width=40, vocab=70, loop=(0, 2, 3))
    b = Built(tmp_path, cfg, 6)
    toks = tokens_for(b, 33, 2)
    z, layers = b.ref(toks)
    assert len(layers) == 2 * 3 + 1
    no_step = copy.deepcopy(b.w)
    no_step["loop.step"][...] = 0.0
    assert rel_err(O.forward(b.cfg, no_step, toks), z) > 1e-2
    logits, taps = b.engine().step([("a", toks, list(range(33)))], taps=True)
    for i in range(len(layers)):
        assert rel_err(taps[i], layers[i]) < F32_TOL, f"layer run {i}"
    assert rel_err(feed(b.engine(), "a", toks, [4, 1, 9]), z) < F32_TOL


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
    st = O.Stepper(general.cfg, general.w)
    own = np.concatenate([st.feed([t]) for t in toks])
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


def test_a_reused_slot_starts_from_zero_state_and_reused_blocks_hold_nothing(general):
    a, b = tokens_for(general, 80, 31), tokens_for(general, 45, 32)
    e = general.engine(max_tokens=128, max_seqs=1)
    e.step([("a", a, [])])
    e.finish("a")
    got = e.step([("b", b, list(range(45)))])
    assert rel_err(got, general.ref(b)[0]) < F32_TOL


def test_pool_exhaustion_is_an_error_not_a_fault(general):
    e = general.engine(max_tokens=64, max_seqs=2)
    with pytest.raises(Exception):
        e.step([("a", tokens_for(general, 100, 1), [])])
    e.finish("a")
    got = e.step([("b", tokens_for(general, 20, 2), [19])])
    assert rel_err(got, general.ref(tokens_for(general, 20, 2))[0][[19]]) < F32_TOL


# ---- sharp attention: far keys, page borders, the edges of the windows, the kept first tokens ---------------------------
HALF = 32


def sharp_model(tmp, kind, vocab=1024, window=40, keep_first=5, sink=(1.0, 1.0)):
    """One layer whose queries read the upper half of the layer's input and whose keys read the lower half through the same
    matrix, with a large score scale.  The upper half of the embedding of the QUERY probe is the lower half of the embedding
    of the KEY probe, so the query probe puts nearly all its weight on the key probe wherever it can see it -- a different
    token with a different value."""
    if kind == "attention":
        layer = attention(None, heads=2, kv_heads=1, dim=16, vdim=16, scale=2.0, rot_dims=4)
        p = "l0.mix."
    elif kind == "left":
        layer = parallel(None, left=attn(heads=2, kv_heads=1, dim=16, vdim=16, scale=2.0, rot_dims=4, mask=(window, keep_first)), left_scale=1.0,
                         right_scale=0.0)
        p = "l0.mix.left."
    else:
        layer = latent(None, heads=2, dim=16, rot_dim=4, vdim=16, kv_rank=24, window=window, scale=2.0)
        p = "l0.mix."
    cfg = model([layer], width=2 * HALF, vocab=vocab, side=0, embed_scale=1.0)

    def tweak(w):
        w["embed"][vocab - 2, HALF:] = w["embed"][vocab - 1, :HALF]
        for n in ("l0.norm1", "l0.norm1.b"):
            w[n][HALF:] = w[n][:HALF]
        if kind == "latent":
            w[p + "dkv"][:24, HALF:] = 0.0
            w[p + "dkv"][24:] *= 0.05                            # the rotated part carries little
            w[p + "dkv.norm"][...] = 1.0
            q = w[p + "q"].reshape(2, 20, 2 * HALF)
            uk = w[p + "uk"].reshape(2, 16, 24)
            q[:, :16, :HALF] = 0.0
            q[:, :16, HALF:] = uk @ w[p + "dkv"][:24, :HALF]
            q[:, 16:] *= 0.05
            w[p + "sink"][...] = sink
        else:
            w[p + "k"][:, HALF:] = 0.0
            q = w[p + "q"].reshape(2, 16, 2 * HALF)
            q[:, :, :HALF] = 0.0
            q[:, :, HALF:] = w[p + "k"][None, :, :HALF]
            q[:, :4] *= 0.05                                      # the rotated dimensions carry little
            w[p + "k"][:4] *= 0.05
            w[p + "g"][...] = 0.0
            if kind == "left":
                w[p + "sink"][...] = sink
            else:
                w[p + "temp"][...] = 1.0
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
    b = sharp_model(tmp_path, "attention")
    check_probe(b, 150, key_pos, query_pos, True, ([150], [query_pos, 1], [key_pos, 2, 1], [key_pos + 1, 1]))


@pytest.mark.parametrize("dtype,decoded", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_one_far_key_among_hundreds(tmp_path, dtype, decoded):
    b = sharp_model(tmp_path, "attention")
    check_probe(b, 700, 3, 690, True, ([670, 1] if decoded else [300, 400],), dtype)


@pytest.mark.parametrize("kind", ["left", "latent"])
@pytest.mark.parametrize("query_pos", [41, 64, 95, 130])
def test_keys_just_inside_and_just_outside_the_window(tmp_path, kind, query_pos):
    """window 40: the key at distance 39 is the last one seen, the key at distance 40 the first one lost -- in whole
    prompts, in portions that start at the key, the query or in between, and with the query decoded alone"""
    b = sharp_model(tmp_path, kind, window=40, keep_first=0)
    for dist, seen in ((39, True), (40, False), (1, True)):
        key_pos = query_pos - dist
        check_probe(b, 140, key_pos, query_pos, seen, ([140], [query_pos, 1], [key_pos, 2, 1], [key_pos + 1, 17, 2], [33, 2]))


@pytest.mark.parametrize("query_pos", [60, 133])
def test_the_first_tokens_a_window_keeps(tmp_path, query_pos):
    """window 40 keeping the first 5: keys 0 and 4 are seen from anywhere, key 5 only from inside the window"""
    b = sharp_model(tmp_path, "left", window=40, keep_first=5)
    for key_pos, seen in ((0, True), (4, True), (5, False), (query_pos - 39, True), (query_pos - 40, False)):
        check_probe(b, 140, key_pos, query_pos, seen, ([140], [query_pos, 1], [key_pos + 1, 40, 2], [3, 1]))
    check_probe(b, 140, 5, 44, True, ([140], [44, 1]))        # the same key inside the window


def test_window_edges_bfloat16(tmp_path):
    b = sharp_model(tmp_path, "left", window=40, keep_first=5)
    check_probe(b, 140, 4, 133, True, ([140], [133, 1]), "bfloat16")
    check_probe(b, 140, 93, 133, False, ([140], [133, 1]), "bfloat16")
    b = sharp_model(tmp_path / "lat", "latent", window=40)
    check_probe(b, 140, 94, 133, True, ([140], [133, 1]), "bfloat16")
    check_probe(b, 140, 93, 133, False, ([140], [133, 1]), "bfloat16")


def test_a_sink_takes_its_share(tmp_path):
    """a large sink empties its head; leaving it out would leave the weights summing to one"""
    for kind in ("left", "latent"):
        b = sharp_model(tmp_path / kind, kind, sink=(6.0, -6.0))
        toks = distinct_tokens(50, 1024, 3)
        z, _ = b.ref(toks)
        w2 = copy.deepcopy(b.w)
        w2[("l0.mix.left." if kind == "left" else "l0.mix.") + "sink"][...] = -30.0
        assert rel_err(O.forward(b.cfg, w2, toks), z) > 0.05
        assert rel_err(feed(b.engine(), "a", toks, [20, 1]), z) < F32_TOL


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_few_rows_at_a_long_context_with_value_rows_that_are_no_multiple_of_a_warp(tmp_path, dtype, tol):
    """Steps of one or two rows behind hundreds of positions are cut along the keys into up to sixteen parts and merged; with
    40 or 72 value channels the last group of channels is ragged, and every part's factor must still reach it."""
    cfg = model([attention(dense(), heads=6, kv_heads=2, dim=32, vdim=40, rot_dims=16),
                 parallel(None, left=attn(heads=4, kv_heads=2, dim=16, vdim=72, mask=(900, 2)), heads=1, dim=20)], width=64, vocab=120)
    b = Built(tmp_path, cfg, 7)
    toks = tokens_for(b, 720, 4)
    z, _ = b.ref(toks)
    got = feed(b.engine(dtype), "a", toks, [600, 38, 2, 1, 1, 2, 3, 1])
    assert max(rel_err(g, w) for g, w in zip(got[600:], z[600:])) < 3 * tol
    assert rel_err(got, z) < tol


# ---- the tensor-core attention forms of the bfloat16 number format ------------------------------------------------------
@pytest.mark.parametrize("kind", ["attention", "left", "latent", "wide_latent"])
@pytest.mark.parametrize("cuts", [[300], [150, 86, 2, 1], [64, 1]])
def test_tensor_core_attention_bfloat16_every_position(tmp_path, kind, cuts):
    """Heads of 16 .. 128 channels (multiples of 16 / 8) take, in bfloat16, the form that keeps a warp's pairs in registers;
    a cached latent row wider than 128 channels the form in which a block of warps shares the query rows and the output.
    Both know the window, the kept first tokens, the sink, the head factors and the gates.  Peaked scores and a check of EVERY
    position by itself: a key too many or too few, or a tile of keys lost, is an error of tens of percent there."""
    if kind == "attention":
        layer = attention(None, heads=4, kv_heads=2, dim=32, vdim=24, rot_dims=16, scale=0.7)
    elif kind == "left":
        layer = parallel(None, left=attn(heads=6, kv_heads=2, dim=48, vdim=64, rot_dims=48, scale=0.6, mask=(70, 3)), left_scale=1.0, right_scale=0.0)
    elif kind == "latent":
        layer = latent(None, heads=4, dim=24, rot_dim=16, vdim=16, kv_rank=48, window=70, scale=0.5)
    else:
        layer = latent(None, heads=4, dim=24, rot_dim=32, vdim=16, kv_rank=160, window=70, scale=0.5)
    b = Built(tmp_path, model([layer], width=64, vocab=200, side=0, mult=1.0), 41)
    n = 300
    toks = tokens_for(b, n, 3)
    _, layers = b.ref(toks)
    base = O.embed(b.cfg, b.w, toks)
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
@pytest.mark.parametrize("case", ["single", "wide_heads", "everything_small", "loop_all_twice", "loop_nothing", "loop_once", "odd_sizes", "plain",
                                  "window_one", "window_beyond"])
def test_other_sizes(tmp_path, case):
    width, loop, rank, side, n = 32, None, 5, 4, 75
    if case == "single":
        layers = [attention(dense(8), heads=1, kv_heads=1, dim=8, vdim=40, rot_dims=2),
                  parallel(dense(16), left=attn(heads=1, kv_heads=1, dim=40, vdim=8, mask=(9, 1)), heads=1, dim=40),
                  latent(None, heads=1, dim=8, rot_dim=2, vdim=40, kv_rank=8, window=11)]
        width, rank, side = 24, 1, 1
    elif case == "wide_heads":
        layers = [parallel(dense(40), left=attn(heads=2, kv_heads=2, dim=72, vdim=70, rot_dims=72, mask=(30, 2)), heads=1, dim=72),
                  latent(None, heads=2, dim=72, rot_dim=24, vdim=72, kv_rank=104, window=50),
                  parallel(None, left=attn(heads=4, kv_heads=1, dim=8, vdim=136, rot_dims=0, mask=(64, None)), heads=2, dim=136)]
        width = 40
    elif case == "everything_small":
        layers = [attention(dense(1), heads=1, kv_heads=1, dim=2, vdim=1, rot_dims=2),
                  parallel(dense(1), left=attn(heads=1, kv_heads=1, dim=1, vdim=1, rot_dims=0, mask=(2, 1)), heads=1, dim=1),
                  latent(dense(1), heads=1, dim=1, rot_dim=2, vdim=1, kv_rank=1, window=2)]
        width, rank, side = 8, 2, 1
    elif case == "loop_all_twice":
        layers, loop = [parallel(dense()), latent(dense(24))], (0, 2, 2)
    elif case == "loop_nothing":
        layers, loop = [attention(dense()), latent(None), parallel(None)], (1, 1, 5)
    elif case == "loop_once":
        layers, loop = [attention(dense()), latent(None), parallel(None)], (2, 3, 1)
    elif case == "odd_sizes":
        layers = [attention(dense(11), heads=6, kv_heads=3, dim=7, vdim=5, rot_dims=2),
                  latent(dense(7), heads=3, dim=7, rot_dim=6, vdim=5, kv_rank=19, window=13),
                  parallel(dense(9), left=attn(heads=3, kv_heads=1, dim=11, vdim=7, rot_dims=10, mask=(17, 33)), heads=3, dim=11)]
        width, loop, rank, side = 27, (0, 1, 3), 3, 3
    elif case == "plain":                                     # no loop, no side input, no feed-forward anywhere
        layers, side = [attention(None), parallel(None), latent(None)], 0
    elif case == "window_one":                                # every token sees itself (and the kept first tokens) only
        layers = [parallel(dense(), left=attn(heads=2, kv_heads=1, dim=16, vdim=8, mask=(1, 2))), latent(None, window=1)]
    else:                                                     # windows longer than the prompt, kept tokens beyond it
        layers = [parallel(dense(), left=attn(heads=2, kv_heads=1, dim=16, vdim=8, mask=(500, 300))), latent(None, window=400)]
    b = Built(tmp_path, model(layers, width=width, vocab=61, loop=loop, side=side), 5, decay_rank=rank)
    toks = tokens_for(b, n, 2)
    z, layers_ref = b.ref(toks)
    e = b.engine()
    logits, taps = e.step([("a", toks, list(range(n)))], taps=True)
    for i in range(len(layers_ref)):
        assert rel_err(taps[i], layers_ref[i]) < F32_TOL, f"layer run {i}"
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
        z = st.feed(p)[-1]
        for tok in g:
            best = int(np.argmax(z))
            if tok != best:                                # only a near tie may differ
                assert z[best] - z[tok] < 1e-3 * max(1.0, float(np.abs(z).max()))
            z = st.feed([tok])[-1]


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
