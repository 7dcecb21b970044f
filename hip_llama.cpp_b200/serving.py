"""Python binding of the layer-program serving path (include/tha_engine.h in lib/libthablas.so), plus the writers of
model folders that tests and benchmarks use.

    eng = ServingEngine(folder, "float32", max_tokens=2048, max_seqs=4)
    logits = eng.step([("a", [5, 17, 3], [0, 2]), ("b", [9], [0])])      # [3, vocab]
    eng.finish("a")
    out = eng.generate([[1, 2, 3], [4, 5]], max_new=[8, 8])              # greedy through the scheduler

Everything that computes runs in the C++ / CUDA libraries; there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
HOST_LIB_PATH = os.path.join(PKG, "lib", "libthablas.so")
DTYPES = {"bfloat16": 0, "bf16": 0, "float32": 1, "f32": 1}

_host = None


def host_lib():
    global _host
    if _host is None:
        if not os.path.exists(HOST_LIB_PATH):
            raise RuntimeError(f"{HOST_LIB_PATH} is missing: run `python hip_llama.cpp_b200/build.py`")
        lib = C.CDLL(HOST_LIB_PATH)
        vp, I = C.c_void_p, C.c_int
        lib.thaEngineOpen.argtypes = [C.c_char_p, I, I, I, C.POINTER(vp)]
        lib.thaEngineOpenError.restype = C.c_char_p
        lib.thaEngineError.restype = C.c_char_p
        lib.thaEngineError.argtypes = [vp]
        lib.thaEngineClose.argtypes = [vp]
        lib.thaEngineClose.restype = None
        for n in ("thaEngineVocab", "thaEngineWidth", "thaEngineLayers"):
            getattr(lib, n).argtypes = [vp]
        lib.thaEngineFreeBlocks.argtypes = [vp]
        lib.thaEngineFreeBlocks.restype = C.c_longlong
        lib.thaEngineSteps.argtypes = [vp]
        lib.thaEngineSteps.restype = C.c_longlong
        lib.thaEngineSlot.argtypes = [vp, C.c_char_p]
        lib.thaEngineStep.argtypes = [vp, I, C.POINTER(C.c_char_p), vp, vp, vp, vp, vp, vp]
        lib.thaEngineFinish.argtypes = [vp, C.c_char_p]
        lib.thaEngineLogits.argtypes = [vp]
        lib.thaEngineLogits.restype = C.POINTER(C.c_float)
        lib.thaEngineWanted.argtypes = [vp]
        lib.thaEngineWanted.restype = C.c_longlong
        lib.thaEngineGenerate.argtypes = [vp, I, vp, vp, vp, C.c_float, C.c_float, C.c_ulonglong, I, vp]
        _host = lib
    return _host


class ServingError(RuntimeError):
    pass


class ServingEngine:
    """A model folder on the current GPU with its block pool and state slots."""

    def __init__(self, folder: str, dtype: str = "bfloat16", max_tokens: int = 4096, max_seqs: int = 4):
        self.lib = host_lib()
        self.h = C.c_void_p()
        st = self.lib.thaEngineOpen(os.fspath(folder).encode(), DTYPES[dtype], max_tokens, max_seqs, C.byref(self.h))
        if st != 0:
            self.h = None
            raise ServingError(self.lib.thaEngineOpenError().decode())
        self.vocab = self.lib.thaEngineVocab(self.h)
        self.width = self.lib.thaEngineWidth(self.h)
        self.layers = self.lib.thaEngineLayers(self.h)

    def close(self):
        if self.h:
            self.lib.thaEngineClose(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def step(self, entries, taps: bool = False, copy: bool = True):
        """entries: [(id, tokens, want), ...].  Returns logits [wanted, vocab] (and the residual stream after every
        layer, [layers, rows, width], with taps=True).  copy=False returns a view of the engine's pinned buffer that the
        next step overwrites."""
        n = len(entries)
        ids = (C.c_char_p * n)(*[e[0].encode() for e in entries])
        counts = np.array([len(e[1]) for e in entries], np.int32)
        tokens = np.array([t for e in entries for t in e[1]], np.int32)
        wc = np.array([len(e[2]) for e in entries], np.int32)
        wants = np.array([w for e in entries for w in e[2]], np.int32)
        nw = int(wc.sum())
        tp = np.zeros((self.layers, int(counts.sum()), self.width), np.float32) if taps else None
        st = self.lib.thaEngineStep(self.h, n, ids, counts.ctypes.data, tokens.ctypes.data, wc.ctypes.data, wants.ctypes.data,
                                    None, tp.ctypes.data if taps else None)
        if st != 0:
            raise ServingError(self.lib.thaEngineError(self.h).decode())
        if nw:
            logits = np.ctypeslib.as_array(self.lib.thaEngineLogits(self.h), shape=(nw, self.vocab))
            if copy:
                logits = logits.copy()
        else:
            logits = np.zeros((0, self.vocab), np.float32)
        return (logits, tp) if taps else logits

    def finish(self, rid: str):
        self.lib.thaEngineFinish(self.h, rid.encode())

    def slot(self, rid: str) -> int:
        return self.lib.thaEngineSlot(self.h, rid.encode())

    def free_blocks(self) -> int:
        return int(self.lib.thaEngineFreeBlocks(self.h))

    def steps_run(self) -> int:
        return int(self.lib.thaEngineSteps(self.h))

    def generate(self, prompts, max_new, temperature: float = 0.0, topp: float = 0.9, seed: int = 1, portion: int = 256):
        lens = np.array([len(p) for p in prompts], np.int32)
        flat = np.array([t for p in prompts for t in p], np.int32)
        mn = np.array(max_new, np.int32)
        out = np.zeros(int(mn.sum()), np.int32)
        st = self.lib.thaEngineGenerate(self.h, len(prompts), lens.ctypes.data, flat.ctypes.data, mn.ctypes.data, temperature, topp, seed,
                                        portion, out.ctypes.data)
        if st != 0:
            raise ServingError(self.lib.thaEngineError(self.h).decode())
        res, at = [], 0
        for k in mn:
            res.append(out[at:at + k].tolist())
            at += k
        return res


# ---- model folders --------------------------------------------------------------------------------------------------
def _to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def save_model_folder(folder: str, config: dict, tensors: dict) -> None:
    """config.json + model.safetensors (every tensor as bfloat16, round to nearest even)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    head, off = {}, 0
    for name, a in tensors.items():
        n = int(np.prod(np.shape(a))) * 2
        head[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for a in tensors.values():
            f.write(_to_bf16_bits(np.asarray(a)).tobytes())


def timerax_tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor a Timerax config asks for."""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = (W,)
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            s[p + "mix.left.q"] = (a["heads"] * a["dim"], W)
            s[p + "mix.left.k"] = (a["kv_heads"] * a["dim"], W)
            s[p + "mix.left.v"] = (a["kv_heads"] * a["vdim"], W)
            s[p + "mix.left.o"] = (W, a["heads"] * a["vdim"])
            s[p + "mix.right.q"] = (r["heads"] * r["dim"], W)
            s[p + "mix.right.k"] = (r["heads"] * r["dim"], W)
            s[p + "mix.right.v"] = (r["heads"] * r["vdim"], W)
            s[p + "mix.right.g"] = (r["heads"] * r["vdim"], W)
            s[p + "mix.right.o"] = (W, r["heads"] * r["vdim"])
            s[p + "mix.right.norm"] = (r["heads"] * r["vdim"],)
            for g in ("i", "f"):
                s[p + f"mix.right.{g}"] = (r["heads"], W)
                s[p + f"mix.right.{g}.b"] = (r["heads"],)
            s[p + "mix.left.out"] = (W,)
            s[p + "mix.right.out"] = (W,)
        else:
            cq, cv, rk = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m.get("rank", max(8, W // 8))
            s[p + "mix.q"], s[p + "mix.k"], s[p + "mix.v"] = (cq, W), (cq, W), (cv, W)
            s[p + "mix.q.conv"], s[p + "mix.k.conv"], s[p + "mix.v.conv"] = (cq, m["conv"]), (cq, m["conv"]), (cv, m["conv"])
            s[p + "mix.b"] = (m["heads"], W)
            s[p + "mix.A_log"] = (m["heads"],)
            s[p + "mix.norm"] = (m["vdim"],)
            s[p + "mix.a1"], s[p + "mix.a2"] = (rk, W), (m["heads"] * m["dim"], rk)
            s[p + "mix.dt_bias"] = (m["heads"] * m["dim"],)
            s[p + "mix.g1"], s[p + "mix.g2"] = (rk, W), (cv, rk)
            s[p + "mix.o"] = (W, cv)
        f = L.get("mlp")
        if f:
            for e in range(f["router"]["experts"]):
                s[p + f"mlp.e{e}.gate"] = (f["expert"]["ff"], W)
                s[p + f"mlp.e{e}.up"] = (f["expert"]["ff"], W)
                s[p + f"mlp.e{e}.down"] = (W, f["expert"]["ff"])
            s[p + "mlp.router"] = (f["router"]["experts"], W)
            if f.get("shared"):
                s[p + "mlp.shared.gate"] = (f["shared"]["ff"], W)
                s[p + "mlp.shared.up"] = (f["shared"]["ff"], W)
                s[p + "mlp.shared.down"] = (W, f["shared"]["ff"])
    return s


def random_timerax_tensors(cfg: dict, seed: int = 0) -> dict:
    """Random weights of a Timerax config: matrices N(0, 1/in), norm weights around zero (layer norms) or around one
    (plain weights), gate biases and decay parameters in the ranges where the recurrences are neither frozen nor
    forgetful.  The "rank" key of a channel_delta mixer (the width of its low-rank projections) is read here only."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in timerax_tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if len(shape) == 2 and not name.endswith(".conv"):
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
            if name == "embed":
                a = rng.standard_normal(shape)
        elif name.endswith(".conv"):
            a = rng.standard_normal(shape) * 0.5
        elif last in ("norm1",) or name == "final.norm":
            a = rng.standard_normal(shape) * 0.1
        elif name.endswith("f.b"):
            a = 3.0 + rng.standard_normal(shape)
        elif name.endswith("i.b"):
            a = rng.standard_normal(shape) * 0.1
        elif last == "A_log":
            a = -1.0 + rng.standard_normal(shape)
        elif last == "dt_bias":
            a = -2.0 + rng.standard_normal(shape)
        else:   # plain weights: .norm, .out
            a = 1.0 + rng.standard_normal(shape) * 0.1
        out[name] = a.astype(np.float32)
    return out


def numizen_tensor_shapes(cfg: dict, decay_rank: int = 64) -> dict:
    """name -> shape of every tensor a Numizen config asks for (decay_rank: rows of the gla mixers' first decay
    projection, a property of the tensors and not of the config)."""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "pos": (cfg["max_positions"], W), "head": (V, W)}

    def norm(n):
        s[n], s[n + ".b"], s[n + ".alpha"] = (W,), (W,), ()

    norm("final.norm")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        norm(p + "norm1")
        norm(p + "norm2")
        s[p + "ls1"] = s[p + "ls2"] = (W,)
        q = p + "mix."
        if L["type"] == "latent_attention":
            H, D, R, E = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            s[q + "dq"], s[q + "dq.norm"], s[q + "uq"] = (m["q_rank"], W), (m["q_rank"],), (H * (D + R), m["q_rank"])
            s[q + "dkv"], s[q + "dkv.norm"] = (m["kv_rank"] + R, W), (m["kv_rank"],)
            s[q + "uk"], s[q + "uv"] = (H * D, m["kv_rank"]), (H * E, m["kv_rank"])
            s[q + "g"], s[q + "o"] = (H * E, W), (W, H * E)
        else:
            H, D, E = m["heads"], m["dim"], m["vdim"]
            s[q + "q"] = s[q + "k"] = (H * D, W)
            s[q + "v"] = s[q + "g"] = (H * E, W)
            s[q + "o"], s[q + "norm"] = (W, H * E), (E,)
            s[q + "a1"], s[q + "a2"], s[q + "a2.b"] = (decay_rank, W), (H * D, decay_rank), (H * D,)
        f = L.get("mlp")
        if not f:
            continue
        q = p + "mlp."
        if f["kind"] == "dense":
            s[q + "gate"] = s[q + "up"] = (f["ff"], W)
            s[q + "down"] = (W, f["ff"])
        else:
            for e in range(f["router"]["experts"]):
                s[q + f"e{e}.up"], s[q + f"e{e}.down"] = (f["expert"]["ff"], W), (W, f["expert"]["ff"])
            s[q + "router"], s[q + "correction"] = (f["router"]["experts"], W), (f["router"]["experts"],)
            if f.get("shared"):
                s[q + "shared.up"], s[q + "shared.down"], s[q + "shared.sg"] = (f["shared"]["ff"], W), (W, f["shared"]["ff"]), (1, W)
    return s


def random_numizen_tensors(cfg: dict, seed: int = 0, decay_rank: int = 64) -> dict:
    """Random weights of a Numizen config: matrices N(0, 1/in), norm weights and layer scales around one, norm scalars
    in (0.5, 1), small router corrections, decay biases where the memory neither freezes nor forgets at once."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in numizen_tensor_shapes(cfg, decay_rank).items():
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            a = np.array(rng.uniform(0.5, 1.0))
        elif name.endswith("a2.b"):
            a = 2.0 + rng.standard_normal(shape)
        elif last == "b":
            a = 0.1 * rng.standard_normal(shape)
        elif last == "correction":
            a = 0.05 * rng.standard_normal(shape)
        elif len(shape) == 2:
            a = rng.standard_normal(shape, dtype=np.float32) * (1.0 if name == "embed" else 0.3 if name == "pos" else 1.0 / np.sqrt(shape[1]))
        else:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        out[name] = np.asarray(a, dtype=np.float32)
    return out


def bozovik_tensor_shapes(cfg: dict, decay_rank: int = 16) -> dict:
    """name -> shape of every tensor a Bozovik config asks for (decay_rank: rows of the delta rule's first decay
    projection, a property of the tensors and not of the config)."""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "head": (V, W)}

    def norm(n):
        s[n], s[n + ".b"] = (W,), (W,)

    def attention(q, m, windowed):
        H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        s[q + "q"], s[q + "k"], s[q + "v"] = (H * D, W), (G * D, W), (G * E, W)
        s[q + "g"], s[q + "o"] = (H, W), (W, H * E)
        s[q + ("sink" if windowed else "temp")] = (H,)

    norm("final.norm")
    lp = cfg.get("loop")
    if lp:
        s["loop.step"] = (lp["times"], W)
    side = cfg.get("token_side")
    if side:
        s["side.embed"] = (V, side["dim"] * len(cfg["layers"]))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        norm(p + "norm1")
        q = p + "mix."
        if L["type"] == "attention":
            attention(q, m, False)
        elif L["type"] == "latent_attention":
            H, D, R, E, K = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            s[q + "q"], s[q + "dkv"], s[q + "dkv.norm"] = (H * (D + R), W), (K + R, W), (K,)
            s[q + "uk"], s[q + "uv"], s[q + "sink"], s[q + "o"] = (H * D, K), (H * E, K), (H,), (W, H * E)
        else:
            attention(q + "left.", m["left"], True)
            r, q = m["right"], q + "right."
            HD = r["heads"] * r["dim"]
            for n in ("r", "k", "v", "g", "a"):
                s[q + n] = (HD, W)
            s[q + "a.b"] = s[q + "w0"] = s[q + "norm"] = (HD,)
            s[q + "w1"], s[q + "w2"], s[q + "o"] = (decay_rank, W), (HD, decay_rank), (W, HD)
        f = L.get("mlp")
        if f:
            norm(p + "norm2")
            s[p + "mlp.up"], s[p + "mlp.down"], s[p + "mlp.act"] = (f["ff"], W), (W, f["ff"]), (2,)
        if side:
            s[p + "side.gate"], s[p + "side.proj"], s[p + "side.norm"] = (side["dim"], W), (W, side["dim"]), (W,)
    return s


def random_bozovik_tensors(cfg: dict, seed: int = 0, decay_rank: int = 16) -> dict:
    """Random weights of a Bozovik config: matrices N(0, 1/in), norm weights around one with small biases, sinks and
    head factors of order one, decay and removal biases where the memory neither freezes nor forgets at once."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in bozovik_tensor_shapes(cfg, decay_rank).items():
        last = name.rsplit(".", 1)[-1]
        if last == "sink":
            a = rng.standard_normal(shape)
        elif last == "temp":
            a = rng.uniform(0.7, 1.4, shape)
        elif last == "act":
            a = rng.standard_normal(shape) * 0.5
        elif last == "w0":
            a = rng.standard_normal(shape) - 1.0
        elif last == "b":
            a = 0.1 * rng.standard_normal(shape)
        elif name == "loop.step":
            a = 0.3 * rng.standard_normal(shape)
        elif len(shape) == 2:
            a = rng.standard_normal(shape, dtype=np.float32) * (1.0 if name in ("embed", "side.embed") else 1.0 / np.sqrt(shape[1]))
        else:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        out[name] = np.asarray(a, dtype=np.float32)
    return out


def mozetar_tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor a Mozetar config asks for."""
    W, V, n = cfg["width"], cfg["vocab"], cfg.get("streams", 1)
    s = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, m, q = f"l{i}.", L["mixer"], f"l{i}.mix."
        s[p + "norm1"] = (W,)
        if "canon" in cfg:
            s[p + "canon1"] = (W, cfg["canon"]["taps"])
        for k in (1, 2) if L.get("mlp") else (1,):
            s[p + f"hc{k}.in"], s[p + f"hc{k}.out"], s[p + f"hc{k}.mix"] = (n,), (n,), (n, n)
        if L["type"] == "attention":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            s[q + "q"], s[q + "k"], s[q + "v"], s[q + "g"], s[q + "o"] = (2 * H * D, W), (2 * G * D, W), (G * E, W), (H, W), (W, H * E)
            for v in ("lq1", "lk1", "lq2", "lk2"):
                s[q + v] = (D,)
        elif L["type"] == "attention_2":
            H, G, D, E, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv", 0)
            s[q + "q"], s[q + "o"] = (H * D, W), (W, H * E)
            if taps:
                s[q + "q.conv"] = (H * D, taps)
            if m.get("kv_from") is None:
                s[q + "k"], s[q + "v"] = (G * D, W), (G * E, W)
                if taps:
                    s[q + "k.conv"], s[q + "v.conv"] = (G * D, taps), (G * E, taps)
        elif L["type"] == "hgrn2":
            H, D, E = m["heads"], m["dim"], m["vdim"]
            s[q + "q"], s[q + "f"], s[q + "v"], s[q + "o"] = (H * D, W), (H * D, W), (H * E, W), (W, H * E)
            s[q + "f.b"], s[q + "lower"], s[q + "norm"] = (H * D,), (H * D,), (E,)
        else:
            raise ValueError(L["type"])
        f = L.get("mlp")
        if f:
            s[p + "norm2"] = (W,)
            q = p + "mlp."
            if f["kind"] == "dense":
                s[q + "up"], s[q + "up.b"], s[q + "down"], s[q + "down.b"], s[q + "act"] = (f["ff"], W), (f["ff"],), (W, f["ff"]), (W,), (4,)
            else:
                s[q + "router"] = (f["router"]["experts"], W)
                for e in range(f["router"]["experts"]):
                    s[q + f"e{e}.gate"], s[q + f"e{e}.up"], s[q + f"e{e}.down"] = (f["expert"]["ff"], W), (f["expert"]["ff"], W), (W, f["expert"]["ff"])
    return s


def random_mozetar_tensors(cfg: dict, seed: int = 0) -> dict:
    """Random weights of a Mozetar config: matrices N(0, 1/in), norm weights around one, stream weights near an even read and an
    identity mixing, forget-gate bounds spread over (0, 0.9), convolution taps of order one half."""
    rng = np.random.default_rng(seed)
    n = cfg.get("streams", 1)
    out = {}
    for name, shape in mozetar_tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("conv", "canon1"):
            a = 0.5 * rng.standard_normal(shape)
        elif last == "in":
            a = 1.0 / n + 0.1 * rng.standard_normal(shape)
        elif last == "out":
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif last == "mix":
            a = np.eye(n) + 0.1 * rng.standard_normal(shape)
        elif last == "lower":
            a = rng.uniform(0.0, 0.9, shape)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            a = 0.3 * rng.standard_normal(shape)
        elif last == "act":
            a = np.array([0.6, 0.3, 0.2, 0.05])
        elif last == "b":
            a = 0.1 * rng.standard_normal(shape)
        elif len(shape) == 2:
            a = rng.standard_normal(shape, dtype=np.float32) * (1.0 if name == "embed" else 1.0 / np.sqrt(shape[1]))
        else:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        out[name] = np.asarray(a, dtype=np.float32)
    return out
