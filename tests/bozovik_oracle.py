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
    """kind 'attention': causal, per-head temperature, a constant 1 in the normalising sum;
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
