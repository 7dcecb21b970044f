"""Host-side pieces of the layer-program path that need no GPU: exported symbols, the architecture registry and its
error texts, and self-checks of the plain statement of Timerax that the GPU tests compare against."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

import bozovik_oracle as B
import mozetar_oracle as M
import numizen_oracle as N
import timerax_oracle as O
from pkgload import load_pkg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "hip_llama.cpp_b200", "lib")
built = pytest.mark.skipif(not os.path.exists(os.path.join(LIB, "libthablas.so")), reason="libraries are not built")


def _declared(header, pattern):
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", header)).read(), flags=re.S)
    return sorted(set(re.findall(pattern, text)))


@built
def test_every_declared_entry_point_is_exported():
    cuda = C.CDLL(os.path.join(LIB, "libtha_b200.so"))
    for name in _declared("tha_hybrid.h", r"\b(tha_hyb_[a-z0-9_]+)\s*\("):
        assert hasattr(cuda, name), name
    host = C.CDLL(os.path.join(LIB, "libthablas.so"))
    names = _declared("tha_engine.h", r"\b(thaEngine[A-Za-z]+)\s*\(")
    assert "thaEngineStep" in names and "thaEngineGenerate" in names
    for name in names:
        assert hasattr(host, name), name


@built
def test_registry_names_what_it_knows(tmp_path):
    serving = load_pkg("serving")
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(serving.ServingError) as e:
        serving.ServingEngine(str(tmp_path), "float32", 64, 1)
    assert "Nope" in str(e.value) and "Timerax" in str(e.value) and "llama2" in str(e.value) and "Numizen" in str(e.value)
    assert "Bozovik" in str(e.value) and "Mozetar" in str(e.value)


@built
def test_a_config_without_a_needed_key_is_refused_by_name(tmp_path):
    serving = load_pkg("serving")
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Timerax", "vocab": 10, "norm": {"eps": 1e-5}, "layers": []}))
    with pytest.raises(serving.ServingError) as e:
        serving.ServingEngine(str(tmp_path), "float32", 64, 1)
    assert "width" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Timerax", "vocab": 10, "width": 8, "norm": {"eps": 1e-5},
                                                       "layers": [{"type": "spiral", "mixer": {}}]}))
    with pytest.raises(serving.ServingError) as e:
        serving.ServingEngine(str(tmp_path), "float32", 64, 1)
    assert "spiral" in str(e.value)


def test_tensor_shapes_cover_a_config():
    serving = load_pkg("serving")
    cfg = {"architecture": "Timerax", "width": 16, "vocab": 20, "norm": {"eps": 1e-5}, "layers": [
        {"type": "channel_delta", "mixer": {"conv": 3, "dim": 4, "heads": 2, "kv_heads": 1, "vdim": 6, "rank": 5}, "mlp": None}]}
    t = serving.random_timerax_tensors(cfg, 0)
    assert t["l0.mix.q.conv"].shape == (4, 3) and t["l0.mix.a2"].shape == (8, 5) and t["l0.mix.norm"].shape == (6,)
    assert "l0.mlp.router" not in t


# ---- the plain statement checks itself: a recurrence cut in two equals the whole -------------------------------------
def test_plain_matrix_memory_carries_its_state():
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((9, 5)), rng.standard_normal((9, 5)), rng.standard_normal((9, 3))
    ig, fg = rng.standard_normal(9), -np.abs(rng.standard_normal(9))
    whole, _ = O.matrix_memory(q, k, v, ig, fg)
    a, st = O.matrix_memory(q[:4], k[:4], v[:4], ig[:4], fg[:4])
    b, _ = O.matrix_memory(q[4:], k[4:], v[4:], ig[4:], fg[4:], st)
    assert np.allclose(np.concatenate([a, b]), whole, atol=1e-12)


def test_plain_delta_rule_carries_its_state_and_reads_its_own_write():
    rng = np.random.default_rng(1)
    q, k, v = rng.standard_normal((7, 4)), rng.standard_normal((7, 4)), rng.standard_normal((7, 2))
    beta, g = rng.random(7), rng.random((7, 4))
    whole, _ = O.delta_rule(q, k, v, beta, g)
    a, S = O.delta_rule(q[:3], k[:3], v[:3], beta[:3], g[:3])
    b, _ = O.delta_rule(q[3:], k[3:], v[3:], beta[3:], g[3:], S)
    assert np.allclose(np.concatenate([a, b]), whole, atol=1e-12)
    # one token from the zero state: S = k u^T with u = beta v, read out with q
    assert np.allclose(whole[0], beta[0] * v[0] * (k[0] @ q[0]))


def test_plain_convolution_and_rotation():
    x = np.arange(12.0).reshape(6, 2)
    taps = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])      # channel 0: the current token; channel 1: two tokens back
    y = O.causal_conv(x, taps)
    assert np.allclose(y[:, 0], x[:, 0]) and np.allclose(y[2:, 1], x[:-2, 1]) and np.allclose(y[:2, 1], 0.0)
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "fast": 32.0, "original": 8, "slow": 1.0}}
    cos, sin = O.rotary_tables(rot, [0, 3])
    mag = 0.1 * np.log(2.0) + 1.0
    assert np.allclose(cos[0], mag) and np.allclose(sin[0], 0.0) and np.allclose(cos[1] ** 2 + sin[1] ** 2, mag ** 2)
    v = np.random.default_rng(2).standard_normal((2, 1, 6))
    r = O.rotate_interleaved(v, cos, sin)
    assert np.allclose(r[..., 4:], v[..., 4:]) and np.allclose(r[0, 0, :4], v[0, 0, :4] * mag)


def test_plain_attention_sees_its_own_block_only():
    rng = np.random.default_rng(3)
    q, k, v = rng.standard_normal((10, 2, 4)), rng.standard_normal((10, 1, 4)), rng.standard_normal((10, 1, 3))
    o = O.chunked_attention(q, k, v, 0.5, 4)
    assert np.allclose(o[4], np.repeat(v[4], 2, 0)) and np.allclose(o[8], np.repeat(v[8], 2, 0))   # first of a block: itself only
    v2 = v.copy()
    v2[3] += 1.0                                                                                     # the last of block 0
    o2 = O.chunked_attention(q, k, v2, 0.5, 4)
    assert np.allclose(o2[4:], o[4:]) and not np.allclose(o2[3], o[3])


# ---- Numizen: config errors by name, and the plain statement's self-checks -------------------------------------------
def _numizen_cfg(layers, **extra):
    c = {"architecture": "Numizen", "vocab": 40, "width": 16, "norm": {"eps": 1e-5}, "max_positions": 64, "layers": layers}
    c.update(extra)
    return c


@built
def test_numizen_configs_are_refused_by_name(tmp_path):
    serving = load_pkg("serving")
    gla = {"type": "gla", "mixer": {"heads": 1, "dim": 4, "vdim": 4, "tau": 2.0}, "mlp": None}
    for cfg, word in [(_numizen_cfg([{"type": "helix", "mixer": {}, "mlp": None}]), "helix"),
                      (_numizen_cfg([gla], loop={"start": 0, "stop": 3, "times": 2}), "loop"),
                      (_numizen_cfg([dict(gla, mlp={"kind": "sparse"})]), "sparse"),
                      (_numizen_cfg([{"type": "gla", "mixer": {"heads": 1, "dim": 4, "vdim": 4}, "mlp": None}]), "tau")]:
        (tmp_path / "config.json").write_text(json.dumps(cfg))
        with pytest.raises(serving.ServingError) as e:
            serving.ServingEngine(str(tmp_path), "float32", 64, 1)
        assert word in str(e.value), (word, str(e.value))


def _small_numizen():
    lat = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 12},
           "mixer": {"heads": 2, "dim": 4, "rot_dim": 4, "vdim": 6, "q_rank": 8, "kv_rank": 10, "scale": 0.4, "rot": {"base": 100.0, "dims": 2}}}
    gla = {"type": "gla", "mixer": {"heads": 2, "dim": 6, "vdim": 4, "tau": 4.0},
           "mlp": {"kind": "moe", "expert": {"ff": 8}, "shared": {"ff": 6}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}}
    return _numizen_cfg([lat, gla], loop={"start": 0, "stop": 2, "times": 2})


def test_plain_numizen_decoding_equals_the_whole_prompt():
    cfg = _small_numizen()
    W = N.random_weights(cfg, 3, gla_rank=3)
    toks = np.random.default_rng(0).integers(0, 40, 17).tolist()
    taps = []
    whole = N.forward(cfg, W, toks, taps)
    assert len(taps) == 4 and N.layer_runs(cfg) == [0, 1, 0, 1]
    st = N.Stepper(cfg, W)
    parts = np.concatenate([st.feed(toks[:5]), st.feed(toks[5:6]), st.feed(toks[6:])], 0)
    assert np.allclose(parts, whole, atol=1e-9)
    assert np.allclose(N.Stepper(cfg, W).feed(toks[:1]), whole[:1], atol=1e-12)


def test_plain_gated_linear_attention_first_token_and_decay():
    cfg = _small_numizen()
    W = N.random_weights(cfg, 4, gla_rank=3)
    m = cfg["layers"][1]["mixer"]
    h = np.random.default_rng(1).standard_normal((3, 16))
    # one token from the zero state: o = v (k . q) / sqrt(dim) per head, then norm, gate, projection
    p = "l1.mix."
    q = (h[:1] @ W[p + "q"].T).reshape(2, 6) / np.sqrt(6.0)
    k = (h[:1] @ W[p + "k"].T).reshape(2, 6)
    v = (h[:1] @ W[p + "v"].T).reshape(2, 4)
    o = v * (q * k).sum(-1, keepdims=True)
    o = N.rms_unit(o, 1e-5) * W[p + "norm"]
    g = h[:1] @ W[p + "g"].T
    want = (o.reshape(1, 8) * (g * N.sigmoid(g))) @ W[p + "o"].T
    assert np.allclose(N.gla_mixer(h[:1], m, W, p, 1e-5), want, atol=1e-12)
    # a closed gate forgets: with a very negative bias the second token sees its own write only
    W2 = dict(W)
    W2[p + "a2.b"] = np.full_like(W[p + "a2.b"], -200.0)
    both = N.gla_mixer(h[:2], m, W2, p, 1e-5)
    assert np.allclose(both[1:], N.gla_mixer(h[1:2], m, W2, p, 1e-5), atol=1e-9)


def test_plain_router_groups_and_weights():
    f = {"router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}}
    W = {"r.router": np.eye(6), "r.correction": np.array([0.0, 0.0, 0.0, 0.0, 5.0, -5.0])}
    h = np.zeros((1, 6))
    h[0, 0] = 3.0                                     # expert 0 has by far the largest score, but group 2 wins by its correction
    picked, w = N.route(h, f, W, "r.")
    assert sorted(picked[0].tolist()) == [4, 5]      # both of the kept group, although expert 5's choice score is negative
    assert np.allclose(w.sum(), 1.0) and np.allclose(w[0, 0], w[0, 1])   # equal scores s: the correction is not in the weights
    f["router"]["groups"]["keep"] = 3
    picked, _ = N.route(h, f, W, "r.")
    assert sorted(picked[0].tolist()) == [0, 4]


def test_plain_rotation_pairs_neighbours():
    x = np.arange(8.0).reshape(1, 8)
    r = N.rotate(x, [0], 4, 10.0)
    assert np.allclose(r, x)                          # position 0: unchanged
    r = N.rotate(x, [1], 4, 10.0)
    a0, a1 = 1.0, 10.0 ** -0.5                        # f_i = base^(-2i/dims)
    assert np.allclose(r[0, 0], 0 * np.cos(a0) - 1 * np.sin(a0)) and np.allclose(r[0, 1], 1 * np.cos(a0) + 0 * np.sin(a0))
    assert np.allclose(r[0, 2], 2 * np.cos(a1) - 3 * np.sin(a1)) and np.allclose(r[0, 4:], x[0, 4:])


# ---- Bozovik ----------------------------------------------------------------------------------------------------------
def _bozovik_cfg(layers, **extra):
    c = {"architecture": "Bozovik", "width": 16, "vocab": 20, "norm": {"eps": 1e-5}, "residual_mult": 0.9, "embedding": {"scale": 2.0}, "layers": layers}
    c.update(extra)
    return c


@built
def test_bozovik_configs_are_refused_by_name(tmp_path):
    serving = load_pkg("serving")
    att = {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5}, "mlp": None}
    no_scale = {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4}, "mlp": None}
    left = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 0}}
    par = {"type": "parallel", "mixer": {"left": left, "right": {"heads": 1, "dim": 4}, "left_scale": 1.0, "right_scale": 1.0}, "mlp": None}
    for cfg, word in [(_bozovik_cfg([{"type": "helix", "mixer": {}, "mlp": None}]), "helix"),
                      (_bozovik_cfg([att], loop={"start": 0, "stop": 3, "times": 2}), "loop"),
                      (_bozovik_cfg([dict(att, mlp={"kind": "sparse"})]), "sparse"),
                      (_bozovik_cfg([no_scale]), "scale"),
                      (_bozovik_cfg([par]), "window"),
                      ({k: v for k, v in _bozovik_cfg([att]).items() if k != "residual_mult"}, "residual_mult")]:
        (tmp_path / "config.json").write_text(json.dumps(cfg))
        with pytest.raises(serving.ServingError) as e:
            serving.ServingEngine(str(tmp_path), "float32", 64, 1)
        assert word in str(e.value), (word, str(e.value))


def test_bozovik_tensor_shapes_cover_a_config():
    serving = load_pkg("serving")
    lat = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 12},
           "mixer": {"heads": 2, "dim": 4, "rot_dim": 2, "vdim": 6, "kv_rank": 10, "scale": 0.4, "mask": {"size": 5}, "rot": {"base": 100.0, "dims": 2}}}
    left = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "mask": {"size": 3, "keep_first": 1}}
    par = {"type": "parallel", "mixer": {"left": left, "right": {"heads": 3, "dim": 5}, "left_scale": 1.0, "right_scale": 1.0}, "mlp": None}
    cfg = _bozovik_cfg([lat, par], token_side={"dim": 3}, loop={"start": 0, "stop": 1, "times": 4})
    t = serving.random_bozovik_tensors(cfg, 0, decay_rank=7)
    assert t["l0.mix.q"].shape == (12, 16) and t["l0.mix.dkv"].shape == (12, 16) and t["l0.mix.sink"].shape == (2,)
    assert t["l1.mix.left.g"].shape == (2, 16) and t["l1.mix.right.w2"].shape == (15, 7) and t["l1.mix.right.a.b"].shape == (15,)
    assert t["side.embed"].shape == (20, 6) and t["loop.step"].shape == (4, 16) and "l1.mlp.up" not in t and "l1.norm2" not in t
    assert set(t) == set(B.tensor_shapes(cfg, 7))


def test_plain_bozovik_statements_agree():
    assert B.self_check()


def test_plain_bozovik_masks_sinks_and_rotation():
    vis = B.visible([0, 5, 9], 10, window=3, keep_first=2)
    assert vis[0].tolist() == [True] + [False] * 9
    assert vis[1].tolist() == [True, True, False, True, True, True, False, False, False, False]
    assert vis[2].tolist() == [True, True, False, False, False, False, False, True, True, True]
    s = np.zeros((1, 1, 4))
    w = B.sink_softmax(s, np.array([[True, True, False, True]]), np.array([0.0]))
    assert np.allclose(w[0, 0], [0.25, 0.25, 0.0, 0.25])           # the sink takes a quarter and gives nothing back
    x = np.arange(6, dtype=np.float64)[None, :]
    r = B.rotate_half(x, [1], 4, 1.0)                                # pairs (0, 2) and (1, 3); entries 4 and 5 pass
    assert np.allclose(r[0, 4:], [4.0, 5.0])
    assert np.allclose(r[0, 0], 0.0 * np.cos(1.0) - 2.0 * np.sin(1.0)) and np.allclose(r[0, 2], 2.0 * np.cos(1.0) + 0.0 * np.sin(1.0))


def test_plain_delta_rule_removes_along_the_unit_key():
    """one head, a key repeated with full removal and no decay: the second write replaces what the first stored"""
    D = 4
    W = {"r": np.eye(D), "k": np.eye(D), "v": np.eye(D), "g": np.zeros((D, D)), "a": np.zeros((D, D)), "a.b": np.full(D, 40.0),
         "w1": np.zeros((1, D)), "w2": np.zeros((D, 1)), "w0": np.full(D, -40.0), "norm": np.ones(D), "o": np.eye(D)}
    W = {"p." + k: v for k, v in W.items()}
    h = np.array([[2.0, 0, 0, 0], [2.0, 0, 0, 0]])
    st = {}
    B.delta_mixer(h, {"heads": 1, "dim": D}, W, "p.", 1e-6, st)
    # after token 1: S = k v^T (4 at [0, 0]); token 2 removes u u^T S = all of it and writes k v^T again
    assert np.allclose(st["S"][0], np.diag([4.0, 0, 0, 0]), atol=1e-5)


# ---- Mozetar ----------------------------------------------------------------------------------------------------------
def _mozetar_cfg(layers, **extra):
    c = {"architecture": "Mozetar", "width": 16, "vocab": 20, "norm": {"eps": 1e-5}, "streams": 2, "canon": {"taps": 2}, "layers": layers}
    c.update(extra)
    return c


@built
def test_mozetar_configs_are_refused_by_name(tmp_path):
    serving = load_pkg("serving")
    win = {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "conv": 2, "mask": {"size": 3}}, "mlp": None}
    dif = {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5}, "mlp": None}
    for cfg, word in [(_mozetar_cfg([{"type": "helix", "mixer": {}, "mlp": None}]), "helix"),
                      (_mozetar_cfg([dict(win, mlp={"kind": "sparse"})]), "sparse"),
                      (_mozetar_cfg([dif]), "diff"),
                      (_mozetar_cfg([dict(win, mixer=dict(win["mixer"], mask={"size": 0}))]), "window"),
                      (_mozetar_cfg([dict(win, mixer=dict(win["mixer"], kv_from=0))]), "kv_from"),
                      (_mozetar_cfg([win], streams=40), "streams"),
                      (_mozetar_cfg([win], canon={"taps": 0}), "canon"),
                      ({k: v for k, v in _mozetar_cfg([win]).items() if k != "vocab"}, "vocab")]:
        (tmp_path / "config.json").write_text(json.dumps(cfg))
        with pytest.raises(serving.ServingError) as e:
            serving.ServingEngine(str(tmp_path), "float32", 64, 1)
        assert word in str(e.value), (word, str(e.value))


def test_mozetar_tensor_shapes_cover_a_config():
    serving = load_pkg("serving")
    win = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.4, "conv": 3, "mask": {"size": 7}, "rot": {"base": 100.0, "dims": 4}}
    layers = [{"type": "attention_2", "mixer": win, "mlp": {"kind": "dense", "ff": 12}},
              {"type": "hgrn2", "mixer": {"heads": 2, "dim": 3, "vdim": 7}, "mlp": None},
              {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 3, "vdim": 5, "scale": 0.5, "diff": 0.2},
               "mlp": {"kind": "moe", "expert": {"ff": 6}, "router": {"experts": 4, "top": 2}}},
              {"type": "attention_2", "mixer": dict(win, kv_from=0), "mlp": None}]
    cfg = _mozetar_cfg(layers, streams=3)
    t = serving.random_mozetar_tensors(cfg, 0)
    assert t["l0.mix.q"].shape == (24, 16) and t["l0.mix.k.conv"].shape == (12, 3) and t["l0.mix.v.conv"].shape == (10, 3)
    assert t["l0.canon1"].shape == (16, 2) and t["l0.hc2.mix"].shape == (3, 3) and t["l0.mlp.act"].shape == (4,) and t["l0.mlp.up.b"].shape == (12,)
    assert t["l1.mix.lower"].shape == (6,) and t["l1.mix.norm"].shape == (7,) and "l1.hc2.in" not in t and "l1.norm2" not in t
    assert t["l2.mix.q"].shape == (24, 16) and t["l2.mix.k"].shape == (12, 16) and t["l2.mix.v"].shape == (10, 16) and t["l2.mix.g"].shape == (4, 16)
    assert t["l2.mlp.e3.down"].shape == (16, 6) and t["l2.mlp.router"].shape == (4, 16)
    assert "l3.mix.k" not in t and "l3.mix.v.conv" not in t and t["l3.mix.q.conv"].shape == (24, 3)
    assert set(t) == set(M.tensor_shapes(cfg))


def test_plain_mozetar_statements_agree():
    assert M.self_check()


def test_plain_mozetar_convolution_recurrence_and_router():
    # the convolution's last tap multiplies the current input, the first tap the oldest; zeros before the start, then the tail
    w = np.array([[1.0, 10.0, 100.0]])
    y, tail = M.causal_conv(np.array([[1.0], [2.0], [3.0]]), w, np.zeros((2, 1)))
    assert y[:, 0].tolist() == [100.0, 210.0, 321.0] and tail[:, 0].tolist() == [2.0, 3.0]
    y2, _ = M.causal_conv(np.array([[4.0]]), w, tail)
    assert y2[0, 0] == 432.0
    # a closed gate (f = 1) keeps the state and writes nothing; an open gate at bound `lower` keeps that share
    D, E = 2, 2
    W = {"p.q": np.eye(D), "p.f": np.zeros((D, D)), "p.f.b": np.array([40.0, -40.0]), "p.lower": np.array([0.0, 0.25]), "p.v": np.eye(E),
         "p.norm": np.ones(E), "p.o": np.eye(E)}
    st = {"S": np.ones((1, D, E))}
    M.hgrn2_mixer(np.array([[3.0, 5.0]]), {"heads": 1, "dim": D, "vdim": E}, W, "p.", 1e-6, st)
    assert np.allclose(st["S"][0, 0], [1.0, 1.0])                        # f = 1: kept
    assert np.allclose(st["S"][0, 1], [0.25 + 0.75 * 3.0, 0.25 + 0.75 * 5.0])   # f = lower: a quarter kept, three quarters of v written
    # router: the best group only; weights are the chosen scores over their sum
    r = {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}
    ids, wts = M.route(np.array([[1.0]]), r, {"p.router": np.array([[0.0], [3.0], [2.0], [2.5]])}, "p.")
    assert ids[0].tolist() == [1, 0] and np.isclose(wts[0].sum(), 1.0) and wts[0, 0] > wts[0, 1]
    ids, _ = M.route(np.array([[1.0]]), {"experts": 4, "top": 2}, {"p.router": np.array([[0.0], [3.0], [2.0], [2.5]])}, "p.")
    assert ids[0].tolist() == [1, 3]
    # rotation pairs neighbours: entries (0, 1) turn together, entries from `dims` on pass
    x = np.arange(6, dtype=np.float64).reshape(1, 1, 6)
    y = M.rotate_pairs(x, [1], {"dims": 2, "base": 1.0})
    assert np.allclose(y[0, 0, 2:], [2, 3, 4, 5]) and np.isclose(y[0, 0, 0], 0.0 * np.cos(1.0) - 1.0 * np.sin(1.0))
    # PolyNorm: each power is normed by itself, so scaling the input leaves everything but the constant's share unchanged
    z = np.array([[1.0, -2.0, 3.0]])
    assert np.allclose(M.polynorm(z, [0.5, 0.3, 0.2, 0.1], 0.0), M.polynorm(7.0 * z, [0.5, 0.3, 0.2, 0.1], 0.0))
