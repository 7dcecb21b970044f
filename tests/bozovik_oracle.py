"""Plain float64 statement of the Bozovik design (numpy; one function per mechanism; shares no code with the product).

A model is (cfg, W): cfg the parsed config.json, W a dict name -> float64 array.  `forward` runs whole sequences from
position 0; `Stepper` feeds any portion of tokens through explicit caches and recurrent states (one per layer RUN), which
is the second, independent statement that whole prompts are compared with.

Embedding:   x = embed[token] * scale
Layer:       x <- x + m * mixer(LN1 x);  x <- x + m * ff(LN2 x);  x <- x + m * rms(P (gelu(G x) * e_token)) * w
Layer norm:  (x - mean) / sqrt(var + eps) * w + b
Loop:        layers [start, stop) run `times` times with the same weights, every pass with a cache / state of its own;
             before pass t: x += embedding output (t > 0), then x += step[t]
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, W, name, eps):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * W[name] + W[name + ".b"]


def xielu(z, p, q):
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (np.expm1(np.minimum(z, 0.0)) - z) + 0.5 * z
    return np.where(z > 0, pos, neg)


def layer_runs(cfg):
    """[(layer index, pass number or None, first layer of its pass)] in execution order."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, None, False) for i in range(n)]
    a, b, t = lp["start"], lp["stop"], lp["times"]
    out = [(i, None, False) for i in range(a)]
    for p in range(t):
        out += [(i, p, i == a) for i in range(a, b)]
    return out + [(i, None, False) for i in range(b, n)]


# ---- rotary: pairs (i, i + dims/2) on the first `dims` entries ------------------------------------------------------
def rotate_half(x, pos, dims, base):
    """x [..., T, n], pos [T]"""
    out = x.copy()
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(pos, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(ang), np.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ---- softmax with a sink, a window and kept first tokens ------------------------------------------------------------
def visible(qpos, Tk, window=None, keep_first=0):
    """[Tq, Tk] booleans: key j <= query i and (i - j < window or j < keep_first)"""
    i = np.asarray(qpos)[:, None]
    j = np.arange(Tk)[None, :]
    vis = j <= i
    if window is not None:
        vis &= (i - j < window) | (j < keep_first)
    return vis


def sink_softmax(s, vis, sink):
    """s [H, Tq, Tk], sink [H] or None: weights exp(s) / (exp(sink) + sum over visible exp(s))"""
    s = np.where(vis[None], s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink[:, None, None])
    w = np.exp(s - m)
    den = w.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink[:, None, None] - m)
    return w / den


# ---- softmax attention (grouped heads; used alone and as the left side of a parallel mixer) -----------------------
def attention_mixer(h, m, W, p, cache, pos0, kind):
    """kind 'attention': causal, a factor per head on the scores, a sink fixed at zero (a constant 1 in the normalising sum);
    kind 'left': window with kept first tokens, learned sink.  cache: dict with 'k', 'v' of the earlier positions."""
    T = len(h)
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(pos0, pos0 + T)
    q = (h @ W[p + "q"].T).reshape(T, H, D).transpose(1, 0, 2)
    k = (h @ W[p + "k"].T).reshape(T, G, D).transpose(1, 0, 2)
    v = (h @ W[p + "v"].T).reshape(T, G, E).transpose(1, 0, 2)
    if m.get("rot"):
        q = rotate_half(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_half(k, pos, m["rot"]["dims"], m["rot"]["base"])
    if "k" in cache:
        k = np.concatenate([cache["k"], k], axis=1)
        v = np.concatenate([cache["v"], v], axis=1)
    cache["k"], cache["v"] = k, v
    rep = H // G
    kk, vv = np.repeat(k, rep, axis=0), np.repeat(v, rep, axis=0)
    s = q @ kk.transpose(0, 2, 1) * m["scale"]
    if kind == "attention":
        s = s * W[p + "temp"][:, None, None]
        vis = visible(pos, k.shape[1])
        sink = np.zeros(H)
    else:
        vis = visible(pos, k.shape[1], m["mask"]["size"], m["mask"].get("keep_first", 0))
        sink = W[p + "sink"]
    w = sink_softmax(s, vis, sink)
    o = w @ vv                                                    # [H, T, E]
    o = o * sigmoid(h @ W[p + "g"].T).T[:, :, None]               # one gate per head
    return o.transpose(1, 0, 2).reshape(T, H * E) @ W[p + "o"].T


# ---- latent attention ---------------------------------------------------------------------------------------------
def latent_mixer(h, m, W, p, eps, cache, pos0):
    T = len(h)
    H, D, R, E, K = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(pos0, pos0 + T)
    q = (h @ W[p + "q"].T).reshape(T, H, D + R).transpose(1, 0, 2)
    kv = h @ W[p + "dkv"].T
    c = rms_unit(kv[:, :K], eps) * W[p + "dkv.norm"]
    kr = kv[:, K:]
    dims, base = m["rot"]["dims"], m["rot"]["base"]
    q = np.concatenate([q[..., :D], rotate_half(q[..., D:], pos, dims, base)], axis=-1)
    kr = rotate_half(kr, pos, dims, base)
    if "c" in cache:
        c = np.concatenate([cache["c"], c])
        kr = np.concatenate([cache["kr"], kr])
    cache["c"], cache["kr"] = c, kr
    Tk = len(c)
    k = (c @ W[p + "uk"].T).reshape(Tk, H, D).transpose(1, 0, 2)
    v = (c @ W[p + "uv"].T).reshape(Tk, H, E).transpose(1, 0, 2)
    s = (q[..., :D] @ k.transpose(0, 2, 1) + q[..., D:] @ kr.T[None]) * m["scale"]
    w = sink_softmax(s, visible(pos, Tk, m["mask"]["size"], 0), W[p + "sink"])
    return (w @ v).transpose(1, 0, 2).reshape(T, H * E) @ W[p + "o"].T


# ---- generalized delta rule (the right side of a parallel mixer) ----------------------------------------------------
def delta_mixer(h, m, W, p, eps, state):
    """state: dict with 'S' [H, D, D] carried between calls"""
    T = len(h)
    H, D = m["heads"], m["dim"]
    r = (h @ W[p + "r"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, D)
    w = np.exp(-math.exp(-0.5) * sigmoid(np.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, H, D)
    a = sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).reshape(T, H, D)
    u = k / np.sqrt((k * k).sum(axis=-1, keepdims=True) + 1e-6)
    S = state["S"] if "S" in state else np.zeros((H, D, D))
    o = np.zeros((T, H, D))
    for t in range(T):
        uS = np.einsum("hd,hde->he", u[t], S)
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hde,hd->he", S, r[t])
    state["S"] = S
    o = rms_unit(o, eps).reshape(T, H * D) * W[p + "norm"] * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def mixer(h, L, W, pre, eps, store, pos0):
    kind, m, p = L["type"], L["mixer"], pre + "mix."
    if kind == "attention":
        return attention_mixer(h, m, W, p, store, pos0, "attention")
    if kind == "latent_attention":
        return latent_mixer(h, m, W, p, eps, store, pos0)
    if kind == "parallel":
        left = attention_mixer(h, m["left"], W, p + "left.", store.setdefault("left", {}), pos0, "left")
        right = delta_mixer(h, m["right"], W, p + "right.", eps, store.setdefault("right", {}))
        return m["left_scale"] * left + m["right_scale"] * right
    raise ValueError(kind)


def feed_forward(h, W, p):
    act = W[p + "act"]
    return xielu(h @ W[p + "up"].T, act[0], act[1]) @ W[p + "down"].T


def token_side(x, tokens, cfg, W, i, pre, eps):
    dim = cfg["token_side"]["dim"]
    e = W["side.embed"][np.asarray(tokens), i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ W[pre + "side.gate"].T) * e) @ W[pre + "side.proj"].T
    return rms_unit(y, eps) * W[pre + "side.norm"]


class Stepper:
    """Feeds portions of one sequence; keeps a cache / state per layer run."""

    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, W
        self.runs = layer_runs(cfg)
        self.stores = [dict() for _ in self.runs]
        self.pos = 0

    def feed(self, tokens, taps=None):
        """tokens of positions pos .. pos + n - 1 -> logits [n, vocab]; taps (a list) receives x after every layer run"""
        cfg, W = self.cfg, self.W
        eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
        tokens = np.asarray(tokens)
        x0 = W["embed"][tokens] * cfg["embedding"]["scale"]
        x = x0.copy()
        for (i, t, first), store in zip(self.runs, self.stores):
            L, pre = cfg["layers"][i], "l%d." % i
            if first:
                if t > 0:
                    x = x + x0
                x = x + W["loop.step"][t]
            x = x + m * mixer(layer_norm(x, W, pre + "norm1", eps), L, W, pre, eps, store, self.pos)
            if L.get("mlp"):
                x = x + m * feed_forward(layer_norm(x, W, pre + "norm2", eps), W, pre + "mlp.")
            if cfg.get("token_side"):
                x = x + m * token_side(x, tokens, cfg, W, i, pre, eps)
            if taps is not None:
                taps.append(x.copy())
        self.pos += len(tokens)
        return layer_norm(x, W, "final.norm", eps) @ W["head"].T


def forward(cfg, W, tokens, taps=None):
    return Stepper(cfg, W).feed(tokens, taps)


def embed(cfg, W, tokens):
    return W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]


# ---- random models ----------------------------------------------------------------------------------------------------
def bf16_round(a):
    a = np.asarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16 << 16
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def tensor_shapes(cfg, decay_rank=5):
    """name -> shape of every tensor the design needs (the rank of the decay projection is a property of the tensors)"""
    Wd, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, Wd), "head": (V, Wd), "final.norm": (Wd,), "final.norm.b": (Wd,)}
    if cfg.get("loop"):
        s["loop.step"] = (cfg["loop"]["times"], Wd)
    side = cfg.get("token_side")
    if side:
        s["side.embed"] = (V, side["dim"] * len(cfg["layers"]))
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        s[p + "norm1"] = s[p + "norm1.b"] = (Wd,)
        q = p + "mix."
        sides = [(q, m, L["type"])] if L["type"] != "parallel" else [(q + "left.", m["left"], "left")]
        for q2, a, kind in sides:
            if kind == "latent_attention":
                H, D, R, E, K = a["heads"], a["dim"], a["rot_dim"], a["vdim"], a["kv_rank"]
                s[q2 + "q"], s[q2 + "dkv"], s[q2 + "dkv.norm"] = (H * (D + R), Wd), (K + R, Wd), (K,)
                s[q2 + "uk"], s[q2 + "uv"], s[q2 + "sink"], s[q2 + "o"] = (H * D, K), (H * E, K), (H,), (Wd, H * E)
            else:
                H, G, D, E = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
                s[q2 + "q"], s[q2 + "k"], s[q2 + "v"] = (H * D, Wd), (G * D, Wd), (G * E, Wd)
                s[q2 + "g"], s[q2 + "o"] = (H, Wd), (Wd, H * E)
                s[q2 + ("temp" if kind == "attention" else "sink")] = (H,)
        if L["type"] == "parallel":
            r, q2 = m["right"], q + "right."
            HD = r["heads"] * r["dim"]
            for n in ("r", "k", "v", "g", "a"):
                s[q2 + n] = (HD, Wd)
            s[q2 + "a.b"] = s[q2 + "w0"] = s[q2 + "norm"] = (HD,)
            s[q2 + "w1"], s[q2 + "w2"], s[q2 + "o"] = (decay_rank, Wd), (HD, decay_rank), (Wd, HD)
        if L.get("mlp"):
            s[p + "norm2"] = s[p + "norm2.b"] = (Wd,)
            s[p + "mlp.up"], s[p + "mlp.down"], s[p + "mlp.act"] = (L["mlp"]["ff"], Wd), (Wd, L["mlp"]["ff"]), (2,)
        if side:
            s[p + "side.gate"], s[p + "side.proj"], s[p + "side.norm"] = (side["dim"], Wd), (Wd, side["dim"]), (Wd,)
    return s


def random_weights(cfg, seed=0, decay_rank=5):
    """bf16-representable float64 weights, scaled so that activations stay of order one"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        last = name.rsplit(".", 1)[-1]
        if last == "sink":
            a = rng.standard_normal(shape)
        elif last == "temp":
            a = rng.uniform(0.6, 1.5, shape)
        elif last == "act":
            a = 0.5 * rng.standard_normal(shape)
        elif last == "w0":
            a = rng.standard_normal(shape) - 1.0
        elif last == "b":
            a = 0.1 * rng.standard_normal(shape)
        elif name == "loop.step":
            a = 0.3 * rng.standard_normal(shape)
        elif len(shape) == 2 and name not in ("embed", "side.embed"):
            a = rng.standard_normal(shape) / math.sqrt(shape[1])
        elif len(shape) == 2:
            a = rng.standard_normal(shape)
        else:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        W[name] = bf16_round(a).astype(np.float64)
    return W


def self_check():
    """the two statements agree with each other on a small model: whole prompt == portions == token by token"""
    att = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.4, "rot": {"base": 100.0, "dims": 4}}
    left = dict(att, mask={"size": 5, "keep_first": 2})
    lat = {"heads": 2, "dim": 4, "rot_dim": 4, "vdim": 3, "kv_rank": 7, "scale": 0.35, "mask": {"size": 4}, "rot": {"base": 50.0, "dims": 4}}
    cfg = {"architecture": "Bozovik", "width": 20, "vocab": 31, "norm": {"eps": 1e-5}, "residual_mult": 0.8, "embedding": {"scale": 2.0},
           "token_side": {"dim": 3}, "loop": {"start": 1, "stop": 3, "times": 2},
           "layers": [{"type": "attention", "mixer": att, "mlp": {"kind": "dense", "ff": 12}},
                      {"type": "parallel", "mixer": {"left": left, "right": {"heads": 2, "dim": 5}, "left_scale": 0.7, "right_scale": 1.2}, "mlp": None},
                      {"type": "latent_attention", "mixer": lat, "mlp": {"kind": "dense", "ff": 9}}]}
    W = random_weights(cfg, 3)
    toks = np.random.default_rng(1).integers(0, 31, 19).tolist()
    taps = []
    z = forward(cfg, W, toks, taps)
    assert len(taps) == 1 + 2 * 2
    st = Stepper(cfg, W)
    one = np.concatenate([st.feed([t]) for t in toks])
    st = Stepper(cfg, W)
    cut = np.concatenate([st.feed(toks[:7]), st.feed(toks[7:9]), st.feed(toks[9:])])
    assert np.abs(one - z).max() < 1e-9 and np.abs(cut - z).max() < 1e-9
    return True
