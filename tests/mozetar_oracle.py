"""Plain float64 statement of the Mozetar design (numpy; one function per mechanism; shares no code with the product).

A model is (cfg, W): cfg the parsed config.json, W a dict name -> float64 array.  Every mechanism takes the rows of ONE
sequence's next portion and the store that sequence carries (cache rows, recurrent state, convolution tails), so
`Stepper.feed` serves whole prompts, portions and single tokens alike; `forward` is a whole prompt in one portion and
`forward_tokenwise` the same prompt one token at a time.

Streams:     n copies X[0..n-1] of the embedding output.  Sublayer q of a layer (1: mixer, 2: feed-forward):
                 u = sum_s in_q[s] X[s];   y = sublayer(rmsnorm_q(u));   X'[t] = sum_s mix_q[s, t] X[s] + out_q[t] y
             The residual stream that is tapped after a layer, and that the final norm reads, is sum_s X[s].
Mixer input: h = rmsnorm_1(u) is replaced by h + causal_conv(h) (per channel, `taps` taps, the tail of h is state).
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


# ---- causal convolution over time, per channel, continuing from a tail --------------------------------------------------
def causal_conv(u, w, tail):
    """u [T, C], w [C, taps], tail [taps - 1, C] (the inputs before u, oldest first).  y_t = sum_j w[:, j] u_(t - taps + 1 + j).
    Returns (y, new tail)."""
    taps = w.shape[1]
    full = np.concatenate([tail, u], axis=0)            # full[t + taps - 1] = u_t
    T = u.shape[0]
    y = np.zeros_like(u)
    for j in range(taps):
        y += w[:, j][None, :] * full[j:j + T]
    return y, full[full.shape[0] - (taps - 1):] if taps > 1 else full[:0]


# ---- rotary: pairs (2i, 2i + 1) on the first `dims` entries, frequencies stretched by wavelength --------------------------
def rotary_frequencies(rot):
    dims = rot["dims"]
    f = float(rot["base"]) ** (-2.0 * np.arange(dims // 2) / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = f.copy()
        for i, fi in enumerate(f):
            wavelength = 2.0 * math.pi / fi
            if wavelength < orig / high:
                continue
            if wavelength > orig / low:
                out[i] = fi / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                out[i] = (1.0 - s) * fi / factor + s * fi
        f = out
    return f


def rotate_pairs(x, pos, rot):
    """x [T, heads, n], pos [T]"""
    dims = rot["dims"]
    ang = np.asarray(pos, dtype=np.float64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def masked_softmax(s, vis):
    s = np.where(vis, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


# ---- mixers -------------------------------------------------------------------------------------------------------------
def diff_attention_mixer(h, m, W, p, eps, store, pos0):
    """Two softmax maps per head over the same values, combined as a1 - lambda a2; causal; no rotation; queries grow with
    the logarithm of their position; one sigmoid gate per head."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = pos0 + np.arange(T)
    q = (h @ W[p + "q"].T).reshape(T, H, 2, D)
    k = (h @ W[p + "k"].T).reshape(T, G, 2, D)
    v = (h @ W[p + "v"].T).reshape(T, G, E)
    qt = m.get("q_temp")
    if qt:
        q = q * (1.0 + qt["coef"] * np.log(np.floor((pos + 1) / qt["every"]) + 1.0))[:, None, None, None]
    store.setdefault("k", []).extend(k)
    store.setdefault("v", []).extend(v)
    K, V = np.array(store["k"]), np.array(store["v"])
    vis = np.arange(K.shape[0])[None, :] <= pos[:, None]
    lam = math.exp(float(np.sum(W[p + "lq1"] * W[p + "lk1"]))) - math.exp(float(np.sum(W[p + "lq2"] * W[p + "lk2"]))) + m["diff"]
    gate = sigmoid(h @ W[p + "g"].T)                     # [T, H]
    out = np.zeros((T, H, E))
    for hh in range(H):
        g = hh // (H // G)
        a = [masked_softmax(q[:, hh, i] @ K[:, g, i].T * m["scale"], vis) @ V[:, g] for i in (0, 1)]
        o = a[0] - lam * a[1]
        out[:, hh] = rms_unit(o, eps) * (1.0 - m["diff"]) * gate[:, hh][:, None]
    return out.reshape(T, H * E) @ W[p + "o"].T


def window_attention_mixer(h, m, W, p, store, donor, pos0):
    """Short convolutions behind the projections, rotary pairs on the first dims of each head, sliding window.  With
    `donor` (another layer's store) the keys and values are that layer's cache rows."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    taps = m["conv"]
    pos = pos0 + np.arange(T)

    def projected(name, channels):
        u = h @ W[p + name].T
        tail = store.get("tail_" + name)
        if tail is None:
            tail = np.zeros((taps - 1, channels))
        y, store["tail_" + name] = causal_conv(u, W[p + name + ".conv"], tail)
        return y

    q = projected("q", H * D).reshape(T, H, D)
    if "rot" in m:
        q = rotate_pairs(q, pos, m["rot"])
    if donor is None:
        k = projected("k", G * D).reshape(T, G, D)
        v = projected("v", G * E).reshape(T, G, E)
        if "rot" in m:
            k = rotate_pairs(k, pos, m["rot"])
        store.setdefault("k", []).extend(k)
        store.setdefault("v", []).extend(v)
        donor = store
    K, V = np.array(donor["k"]), np.array(donor["v"])
    j = np.arange(K.shape[0])[None, :]
    vis = (j <= pos[:, None]) & (pos[:, None] - j < m["mask"]["size"])
    out = np.zeros((T, H, E))
    for hh in range(H):
        g = hh // (H // G)
        out[:, hh] = masked_softmax(q[:, hh] @ K[:, g].T * m["scale"], vis) @ V[:, g]
    return out.reshape(T, H * E) @ W[p + "o"].T


def hgrn2_mixer(h, m, W, p, eps, store):
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T per head, o_t = S_t^T q_t; the forget gate is bounded below."""
    T = h.shape[0]
    H, D, E = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).reshape(T, H, D)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * sigmoid(h @ W[p + "f"].T + W[p + "f.b"])).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, E)
    S = store.get("S")
    if S is None:
        S = np.zeros((H, D, E))
    out = np.zeros((T, H, E))
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hde,hd->he", S, q[t])
    store["S"] = S
    out = rms_unit(out, eps) * W[p + "norm"]
    return out.reshape(T, H * E) @ W[p + "o"].T


# ---- feed-forward ---------------------------------------------------------------------------------------------------------
def polynorm(z, c, eps):
    return c[0] * rms_unit(z, eps) + c[1] * rms_unit(z ** 2, eps) + c[2] * rms_unit(z ** 3, eps) + c[3]


def dense_ff(h, W, p, eps):
    z = h @ W[p + "up"].T + W[p + "up.b"]
    return polynorm(z, W[p + "act"], eps) @ W[p + "down"].T + W[p + "down.b"]


def route(h, r, W, p):
    """-> (experts [T, top], weights [T, top]); softmax over all experts, the choice inside the best groups of neighbours"""
    z = h @ W[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    n, top = r["experts"], r["top"]
    ids = np.zeros((h.shape[0], top), dtype=np.int64)
    wts = np.zeros((h.shape[0], top))
    for t in range(h.shape[0]):
        cand = s[t].copy()
        gr = r.get("groups")
        if gr and gr["count"] > 1:
            per = n // gr["count"]
            best = cand.reshape(gr["count"], per).max(axis=1)
            kept = np.argsort(-best, kind="stable")[:gr["keep"]]
            ok = np.zeros(n, dtype=bool)
            for g in kept:
                ok[g * per:(g + 1) * per] = True
            cand = np.where(ok, cand, -np.inf)
        pick = np.argsort(-cand, kind="stable")[:top]
        ids[t] = pick
        wts[t] = s[t][pick] / (s[t][pick].sum() + 1e-20)
    return ids, wts


def moe_ff(h, f, W, p):
    ids, wts = route(h, f["router"], W, p)
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], wts[t]):
            q = p + "e%d." % e
            out[t] += w * ((silu(h[t] @ W[q + "gate"].T) * (h[t] @ W[q + "up"].T)) @ W[q + "down"].T)
    return out


# ---- the streams ------------------------------------------------------------------------------------------------------------
def streams_read(X, W, p):
    return np.tensordot(W[p + "in"], X, axes=(0, 0))


def streams_write(X, y, W, p):
    return np.tensordot(W[p + "mix"].T, X, axes=(1, 0)) + W[p + "out"][:, None, None] * y[None]


class Stepper:
    """One sequence: feed(tokens) runs its next portion and returns (logits [T, vocab], taps [layers, T, width])."""

    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, W
        self.pos = 0
        self.stores = [dict() for _ in cfg["layers"]]

    def feed(self, tokens):
        cfg, W = self.cfg, self.W
        eps = cfg["norm"]["eps"]
        T = len(tokens)
        x = W["embed"][np.asarray(tokens)]
        n = cfg.get("streams", 1)
        X = np.stack([x] * n)
        taps = []
        for i, L in enumerate(cfg["layers"]):
            pre = "l%d." % i
            st = self.stores[i]
            h = rms_unit(streams_read(X, W, pre + "hc1."), eps) * W[pre + "norm1"]
            if "canon" in cfg:
                ct = cfg["canon"]["taps"]
                tail = st.get("canon")
                if tail is None:
                    tail = np.zeros((ct - 1, h.shape[1]))
                c, st["canon"] = causal_conv(h, W[pre + "canon1"], tail)
                h = h + c
            m, kind = L["mixer"], L["type"]
            if kind == "attention":
                y = diff_attention_mixer(h, m, W, pre + "mix.", eps, st, self.pos)
            elif kind == "attention_2":
                donor = self.stores[m["kv_from"]] if m.get("kv_from") is not None else None
                y = window_attention_mixer(h, m, W, pre + "mix.", st, donor, self.pos)
            elif kind == "hgrn2":
                y = hgrn2_mixer(h, m, W, pre + "mix.", eps, st)
            else:
                raise ValueError(kind)
            X = streams_write(X, y, W, pre + "hc1.")
            f = L.get("mlp")
            if f:
                h = rms_unit(streams_read(X, W, pre + "hc2."), eps) * W[pre + "norm2"]
                y = dense_ff(h, W, pre + "mlp.", eps) if f["kind"] == "dense" else moe_ff(h, f, W, pre + "mlp.")
                X = streams_write(X, y, W, pre + "hc2.")
            taps.append(X.sum(axis=0))
        self.pos += T
        x = rms_unit(X.sum(axis=0), eps) * W["final.norm"]
        return x @ W["head"].T, np.array(taps)


def forward(cfg, W, tokens):
    return Stepper(cfg, W).feed(tokens)


def forward_tokenwise(cfg, W, tokens):
    s = Stepper(cfg, W)
    outs = [s.feed([t]) for t in tokens]
    return np.concatenate([o[0] for o in outs]), np.concatenate([o[1] for o in outs], axis=1)


def bf16_round(a):
    """float64 -> the nearest bfloat16 (ties to even), as float64"""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


# ---- shapes and random weights of a configuration -------------------------------------------------------------------------
def tensor_shapes(cfg):
    Wd, n = cfg["width"], cfg.get("streams", 1)
    out = {"embed": (cfg["vocab"], Wd), "final.norm": (Wd,), "head": (cfg["vocab"], Wd)}
    for i, L in enumerate(cfg["layers"]):
        pre = "l%d." % i
        m, p = L["mixer"], pre + "mix."
        out[pre + "norm1"] = (Wd,)
        if "canon" in cfg:
            out[pre + "canon1"] = (Wd, cfg["canon"]["taps"])
        qs = [1] + ([2] if L.get("mlp") else [])
        for q in qs:
            out[pre + "hc%d.in" % q] = (n,)
            out[pre + "hc%d.out" % q] = (n,)
            out[pre + "hc%d.mix" % q] = (n, n)
        if L["type"] == "attention":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "q": (H * 2 * D, Wd), p + "k": (G * 2 * D, Wd), p + "v": (G * E, Wd), p + "g": (H, Wd), p + "o": (Wd, H * E)})
            for v in ("lq1", "lk1", "lq2", "lk2"):
                out[p + v] = (D,)
        elif L["type"] == "attention_2":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "q": (H * D, Wd), p + "q.conv": (H * D, m["conv"]), p + "o": (Wd, H * E)})
            if m.get("kv_from") is None:
                out.update({p + "k": (G * D, Wd), p + "k.conv": (G * D, m["conv"]), p + "v": (G * E, Wd), p + "v.conv": (G * E, m["conv"])})
        elif L["type"] == "hgrn2":
            H, D, E = m["heads"], m["dim"], m["vdim"]
            out.update({p + "q": (H * D, Wd), p + "f": (H * D, Wd), p + "f.b": (H * D,), p + "lower": (H * D,), p + "v": (H * E, Wd),
                        p + "norm": (E,), p + "o": (Wd, H * E)})
        f = L.get("mlp")
        if f:
            out[pre + "norm2"] = (Wd,)
            q = pre + "mlp."
            if f["kind"] == "dense":
                out.update({q + "up": (f["ff"], Wd), q + "up.b": (f["ff"],), q + "down": (Wd, f["ff"]), q + "down.b": (Wd,), q + "act": (4,)})
            else:
                out[q + "router"] = (f["router"]["experts"], Wd)
                for e in range(f["router"]["experts"]):
                    out.update({q + "e%d.gate" % e: (f["expert"]["ff"], Wd), q + "e%d.up" % e: (f["expert"]["ff"], Wd),
                                q + "e%d.down" % e: (Wd, f["expert"]["ff"])})
    return out


def random_weights(cfg, seed=0):
    """bfloat16-representable float64 values, scaled so that activations stay of order one through the layers"""
    rng = np.random.default_rng(seed)
    n = cfg.get("streams", 1)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith("norm1") or name.endswith("norm2") or name == "final.norm" or name.endswith("mix.norm"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "conv" or leaf == "canon1":
            a = 0.5 * rng.standard_normal(shape)
        elif leaf == "in":
            a = 1.0 / n + 0.2 * rng.standard_normal(shape)
        elif leaf == "out":
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif leaf == "mix":
            a = np.eye(n) + 0.2 * rng.standard_normal(shape)
        elif leaf == "lower":
            a = rng.uniform(0.0, 0.9, shape)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            a = 0.3 * rng.standard_normal(shape)
        elif leaf == "act":
            a = np.array([0.7, 0.4, 0.3, 0.1]) + 0.1 * rng.standard_normal(4)
        elif leaf == "b":
            a = 0.3 * rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif leaf == "router":
            a = 2.0 * rng.standard_normal(shape) / math.sqrt(shape[-1])
        else:
            a = rng.standard_normal(shape) / math.sqrt(shape[-1])
        W[name] = bf16_round(a)
    return W


def self_check():
    """The statements agree with themselves: a whole prompt, the same prompt token by token, and in uneven portions."""
    cfg = {
        "architecture": "Mozetar", "width": 24, "vocab": 40, "streams": 2, "norm": {"eps": 1e-6}, "canon": {"taps": 3},
        "layers": [
            {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "conv": 3, "scale": 0.4, "mask": {"size": 5},
                                              "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}}},
             "mlp": {"kind": "dense", "ff": 20}},
            {"type": "hgrn2", "mixer": {"heads": 2, "dim": 5, "vdim": 7},
             "mlp": {"kind": "moe", "expert": {"ff": 6}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}},
            {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "diff": 0.3, "q_temp": {"coef": 0.4, "every": 3}},
             "mlp": None},
            {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "conv": 3, "scale": 0.4, "mask": {"size": 5}, "kv_from": 0,
                                              "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}}},
             "mlp": {"kind": "dense", "ff": 20}},
        ],
    }
    W = random_weights(cfg, 3)
    toks = list(np.random.default_rng(1).integers(0, 40, 19))
    a, ta = forward(cfg, W, toks)
    b, tb = forward_tokenwise(cfg, W, toks)
    assert np.abs(a - b).max() < 1e-9 and np.abs(ta - tb).max() < 1e-9
    s = Stepper(cfg, W)
    parts, at = [], 0
    for n in (2, 7, 1, 9):
        parts.append(s.feed(toks[at:at + n])[0])
        at += n
    assert np.abs(np.concatenate(parts) - a).max() < 1e-9
    # frequencies: short wavelengths kept, long ones divided by the factor
    f = rotary_frequencies({"dims": 8, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}})
    plain = 10000.0 ** (-2.0 * np.arange(4) / 8)
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 8.0) < 1e-15
    # the forget gate never falls below its bound: a closed gate (f = 1) keeps the state and writes nothing
    return True


if __name__ == "__main__":
    self_check()
    print("ok")
