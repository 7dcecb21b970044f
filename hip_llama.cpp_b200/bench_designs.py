"""Throughput of a layer-program design beside the llama2 bf16 path at equal size (bench.py --design timerax), or of
Numizen beside Timerax -- the closest design the framework has: attention + a recurrent mixer + a mixture of experts --
and llama2 at equal size (bench.py --design numizen); or of Bozovik beside Numizen with dense feed-forwards -- the closest
design the framework has: latent attention + a recurrent mixer + a looped segment -- and llama2 at equal size (bench.py
--design bozovik); or of Mozetar beside Numizen -- the closest design the framework has: softmax attention + a gated linear
recurrence + a mixture of experts behind a softmax router with groups -- and llama2 at equal size (bench.py --design mozetar).

Random weights at sizes that resemble a real model's layers; a few layers only, so that building the folder stays
short.  For every size: prompt ingestion (one prompt in one step) and batched decoding (one token per live request per
step, after a prompt each) through ServingEngine.step -- the call a user makes, with the row arrays going up and the
wanted logits coming back inside the timed region -- and the same two workloads through the llama2 bf16 engine with as
many layers, the same width, head count and vocabulary, and a dense feed-forward as wide as the experts a token uses.
With kernels=True the library's per-kernel timeline (THA_TRACE) of one prompt step and one decode step is printed too.
"""
from __future__ import annotations

import json
import os
import shutil
import tempfile
import time

import numpy as np

SIZES = {
    # width, attention heads / kv heads / head size, block of positions, memory heads, delta heads, experts / top / ff, shared ff
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=128, chunk=1024, mheads=4, mdim=64, dheads=8, dkv=4, ddim=64, experts=16, top=2, ff=1024, sff=1024,
                  vocab=32000, layers=4),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, chunk=2048, mheads=4, mdim=128, dheads=16, dkv=8, ddim=128, experts=16, top=4, ff=1024, sff=2048,
                  vocab=32000, layers=4),
}


def timerax_config(s: dict) -> dict:
    rot = {"base": 500000.0, "dims": s["dim"] // 2, "scaling": {"factor": 8.0, "fast": 32.0, "original": 4096, "slow": 1.0}}
    left = {"dim": s["dim"], "heads": s["heads"], "kv_heads": s["kv_heads"], "vdim": s["dim"], "mask": {"size": s["chunk"]}, "rot": rot,
            "scale": s["dim"] ** -0.5}
    right = {"dim": s["mdim"], "heads": s["mheads"], "vdim": s["mdim"], "gate_cap": 15.0}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"], "limit": 7.0}, "router": {"experts": s["experts"], "top": s["top"]},
           "shared": {"ff": s["sff"], "limit": 7.0}}
    par = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}
    dl = {"type": "channel_delta", "mixer": {"conv": 4, "dim": s["ddim"], "heads": s["dheads"], "kv_heads": s["dkv"], "vdim": s["ddim"], "rank": 64},
          "mlp": mlp}
    layers = [dl if i % 4 == 2 else par for i in range(s["layers"])]
    return {"architecture": "Timerax", "layers": layers, "logit_softcap": 30.0, "norm": {"eps": 1e-5}, "vocab": s["vocab"], "width": s["width"]}


# Numizen at the same widths, expert counts and vocabulary.  Layer 0 has a dense feed-forward as wide as the experts a
# token uses, the others the mixture; layer 2 is the gated linear attention.  "w1024" keeps the cached row (latent +
# rotated part) at 128 channels; "w2048" has the full-size latent of 512 + 64.
NUMIZEN = {
    "w1024": dict(heads=8, dim=64, rot_dim=32, vdim=64, q_rank=384, kv_rank=96, gheads=4, gdim=128, gvdim=256, groups=(4, 2)),
    "w2048": dict(heads=16, dim=128, rot_dim=64, vdim=128, q_rank=768, kv_rank=512, gheads=8, gdim=128, gvdim=256, groups=(4, 2)),
}


def numizen_config(s: dict, n: dict, max_positions: int = 8192, dense_everywhere: bool = False) -> dict:
    lat = {"heads": n["heads"], "dim": n["dim"], "rot_dim": n["rot_dim"], "vdim": n["vdim"], "q_rank": n["q_rank"], "kv_rank": n["kv_rank"],
           "scale": (n["dim"] + n["rot_dim"]) ** -0.5, "rot": {"base": 500000.0, "dims": n["rot_dim"]}}
    gl = {"heads": n["gheads"], "dim": n["gdim"], "vdim": n["gvdim"], "tau": 16.0}
    moe = {"kind": "moe", "expert": {"ff": s["ff"]}, "shared": {"ff": s["sff"]},
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": n["groups"][0], "keep": n["groups"][1]}}}
    dense = {"kind": "dense", "ff": s["top"] * s["ff"] + s["sff"]}
    layers = []
    for i in range(s["layers"]):
        mlp = dense if i == 0 or dense_everywhere else moe
        layers.append({"type": "gla", "mixer": gl, "mlp": mlp} if i % 4 == 2 else {"type": "latent_attention", "mixer": lat, "mlp": mlp})
    return {"architecture": "Numizen", "layers": layers, "norm": {"eps": 1e-5}, "vocab": s["vocab"], "width": s["width"],
            "max_positions": max_positions}


# Bozovik at the same widths and vocabulary: softmax attention with grouped heads, latent attention under a sliding window
# ("w1024": cached row 96 + 32; "w2048": the full-size latent of 512 + 64), attention beside a generalized delta rule, and
# attention again; layers 1 and 2 are a looped segment that runs once (so the pass vector is added); an ungated feed-forward
# with as many weights as the gated one of the other arms (1.5 x its hidden size); a per-token side input.
BOZOVIK = {
    "w1024": dict(lheads=8, ldim=64, rot_dim=32, lvdim=64, kv_rank=96, window=1024, keep=4, dheads=8, ddim=64, side=64),
    "w2048": dict(lheads=16, ldim=128, rot_dim=64, lvdim=128, kv_rank=512, window=2048, keep=4, dheads=16, ddim=128, side=128),
}


def bozovik_config(s: dict, n: dict) -> dict:
    rot = {"base": 500000.0, "dims": s["dim"]}
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5, "rot": rot}
    left = dict(att, mask={"size": n["window"], "keep_first": n["keep"]})
    lat = {"heads": n["lheads"], "dim": n["ldim"], "rot_dim": n["rot_dim"], "vdim": n["lvdim"], "kv_rank": n["kv_rank"],
           "scale": (n["ldim"] + n["rot_dim"]) ** -0.5, "mask": {"size": n["window"]}, "rot": {"base": 500000.0, "dims": n["rot_dim"]}}
    mlp = {"kind": "dense", "ff": (s["top"] * s["ff"] + s["sff"]) * 3 // 2}
    par = {"left": left, "right": {"heads": n["dheads"], "dim": n["ddim"]}, "left_scale": 0.7, "right_scale": 0.7}
    kinds = [("attention", att), ("latent_attention", lat), ("parallel", par), ("attention", att)]
    layers = [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": mlp} for i in range(s["layers"])]
    return {"architecture": "Bozovik", "layers": layers, "norm": {"eps": 1e-5}, "vocab": s["vocab"], "width": s["width"], "residual_mult": 0.7,
            "embedding": {"scale": 1.0}, "token_side": {"dim": n["side"]}, "loop": {"start": 1, "stop": min(3, s["layers"]), "times": 1}}


# Mozetar at the same widths, expert sizes and vocabulary: windowed attention with short convolutions (heads of 128, rotary on
# half of a head), the gated linear recurrence with Numizen's linear-attention head sizes, differential attention (two maps of
# 64 channels per head, values of 128), and a windowed layer that reads layer 0's cache rows; three residual streams; a dense
# PolyNorm feed-forward as wide as the experts a token uses in layer 0, the mixture (silu experts, router groups) elsewhere.
MOZETAR = {
    "w1024": dict(window=1024, gheads=4, gdim=128, gvdim=256, ddim=64, groups=(4, 2)),
    "w2048": dict(window=2048, gheads=8, gdim=128, gvdim=256, ddim=64, groups=(4, 2)),
}


def mozetar_config(s: dict, n: dict) -> dict:
    rot = {"base": 500000.0, "dims": s["dim"] // 2, "scaling": {"factor": 16.0, "low": 1.0, "high": 2.0, "original": 4096}}
    win = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "conv": 4, "scale": s["dim"] ** -0.5,
           "mask": {"size": n["window"]}, "rot": rot}
    dif = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": n["ddim"], "vdim": s["dim"], "scale": n["ddim"] ** -0.5, "diff": 0.5,
           "q_temp": {"coef": 0.1, "every": 512}}
    rec = {"heads": n["gheads"], "dim": n["gdim"], "vdim": n["gvdim"]}
    moe = {"kind": "moe", "expert": {"ff": s["ff"]},
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": n["groups"][0], "keep": n["groups"][1]}}}
    dense = {"kind": "dense", "ff": s["top"] * s["ff"] + s["sff"]}
    kinds = [("attention_2", win), ("attention", dif), ("hgrn2", rec), ("attention_2", dict(win, kv_from=0))]
    layers = [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": dense if i == 0 else moe} for i in range(s["layers"])]
    return {"architecture": "Mozetar", "layers": layers, "norm": {"eps": 1e-6}, "canon": {"taps": 3}, "streams": 3, "vocab": s["vocab"],
            "width": s["width"]}


def _time_timerax(serving, folder, prompt_len, batch, ctx, steps, warmup, kernels):
    rng = np.random.default_rng(0)
    out = {}
    eng = serving.ServingEngine(folder, "bfloat16", max_tokens=max(prompt_len + 64, batch * (ctx + steps + warmup + 64)), max_seqs=max(batch, 1))
    vocab = eng.vocab
    # prompt ingestion: a fresh request per repetition
    times = []
    for i in range(warmup + 3):
        toks = rng.integers(0, vocab, prompt_len).tolist()
        t0 = time.perf_counter()
        eng.step([(f"p{i}", toks, [prompt_len - 1])])
        times.append(time.perf_counter() - t0)
        eng.finish(f"p{i}")
    ms = 1e3 * float(np.median(times[warmup:]))
    out["prefill"] = {"tokens": prompt_len, "ms": ms, "tok_s": prompt_len / ms * 1e3}
    if kernels:
        serving.host_lib()   # same process, the CUDA library is loaded: its timeline covers the next step only
        import ctypes as C
        cuda = C.CDLL(os.path.join(os.path.dirname(serving.HOST_LIB_PATH), "libtha_b200.so"))
        cuda.tha_trace_dump(1 << 30)
        eng.step([("pk", rng.integers(0, vocab, prompt_len).tolist(), [prompt_len - 1])])
        print(f"# kernels of one prompt step, {prompt_len} tokens", flush=True)
        cuda.tha_trace_dump(0)
        eng.finish("pk")
    # decoding: `batch` requests with `ctx` tokens each, then single tokens
    ids = [f"d{i}" for i in range(batch)]
    for i in ids:
        eng.step([(i, rng.integers(0, vocab, ctx).tolist(), [])])
    times = []
    for k in range(warmup + steps):
        entries = [(i, [int(rng.integers(0, vocab))], [0]) for i in ids]
        t0 = time.perf_counter()
        eng.step(entries, copy=False)
        times.append(time.perf_counter() - t0)
    ms = 1e3 * float(np.median(times[warmup:]))
    out["decode"] = {"batch": batch, "context": ctx, "ms_per_step": ms, "tok_s": batch / ms * 1e3,
                     "what": "one token per request per step, every request's logits back in pinned host memory"}
    for i in ids:
        eng.finish(i)
    # generation through the scheduler (device sampler, token ids back): two calls that differ in length only
    prompts = [rng.integers(0, vocab, ctx).tolist() for _ in range(batch)]
    t = []
    for new in (2, 2 + steps):
        t0 = time.perf_counter()
        eng.generate(prompts, [new] * batch, temperature=0.0, portion=4096)
        t.append(time.perf_counter() - t0)
    ms = 1e3 * (t[1] - t[0]) / steps
    out["generate"] = {"batch": batch, "context": ctx, "ms_per_step": ms, "tok_s": batch / ms * 1e3,
                       "what": "greedy generation through SequenceEngine.generate, time of %d extra tokens per request" % steps}
    if kernels:
        for i in ids:
            eng.step([(i, rng.integers(0, vocab, ctx).tolist(), [])])
        cuda.tha_trace_dump(1 << 30)
        eng.step([(i, [1], [0]) for i in ids])
        print(f"# kernels of one decode step, {batch} requests at context {ctx}", flush=True)
        cuda.tha_trace_dump(0)
    eng.close()
    return out


def _time_llama(engine_mod, checkpoint_mod, s, prompt_len, batch, ctx, steps, warmup):
    import torch
    hidden = s["top"] * s["ff"] + s["sff"]
    cfg = checkpoint_mod.Config(dim=s["width"], hidden_dim=hidden, n_layers=s["layers"], n_heads=s["heads"], n_kv_heads=s["kv_heads"],
                                vocab_size=s["vocab"], seq_len=max(prompt_len, ctx + 2 * (steps + warmup) + 8))
    dw = engine_mod.DeviceWeightsBF16.random(cfg, seed=1, device="cuda")
    out = {"weights_bytes": dw.nbytes()}
    e = engine_mod.Engine(dw, max(batch, 1), device="cuda", with_att=False)
    rng = np.random.default_rng(0)
    st = torch.cuda.Stream()
    logits = torch.zeros(1, cfg.vocab_size, device="cuda")
    with torch.cuda.stream(st):
        seqs = [(0, 0, rng.integers(3, cfg.vocab_size, size=prompt_len).astype(np.int32))]
        times = []
        for _ in range(warmup + 3):
            st.synchronize()
            t0 = time.perf_counter()
            e.prefill(seqs, logits, None, stream=st)
            logits.cpu()
            st.synchronize()
            times.append(time.perf_counter() - t0)
        ms = 1e3 * float(np.median(times[warmup:]))
        out["prefill"] = {"tokens": prompt_len, "ms": ms, "tok_s": prompt_len / ms * 1e3}
        e.prefill([(b, 0, rng.integers(3, cfg.vocab_size, size=ctx).astype(np.int32)) for b in range(batch)], None, None, stream=st)
        lg = torch.empty(batch, cfg.vocab_size, dtype=torch.float32).pin_memory()
        times = []
        for k in range(warmup + steps):
            tok = rng.integers(3, cfg.vocab_size, size=batch).astype(np.int32)
            pos = np.full(batch, ctx + k, np.int32)
            t0 = time.perf_counter()
            e.forward_batch(tok, pos, lg, stream=st)       # host tokens in, logits back: what the other arm's step does
            times.append(time.perf_counter() - t0)
        ms = 1e3 * float(np.median(times[warmup:]))
        out["decode"] = {"batch": batch, "context": ctx, "ms_per_step": ms, "tok_s": batch / ms * 1e3}
        times = []
        for k in range(warmup + steps):
            tok = rng.integers(3, cfg.vocab_size, size=batch).astype(np.int32)
            pos = np.full(batch, ctx + warmup + steps + k, np.int32)
            t0 = time.perf_counter()
            e.forward_greedy(tok, pos, stream=st)          # host tokens in, greedy token ids back
            times.append(time.perf_counter() - t0)
        ms = 1e3 * float(np.median(times[warmup:]))
        out["generate"] = {"batch": batch, "context": ctx, "ms_per_step": ms, "tok_s": batch / ms * 1e3}
    return out


def _time_folder(serving, folder, *a):
    return _time_timerax(serving, folder, *a)   # the workloads are the same for every layer-program design


def timerax_weight_bytes(cfg: dict, shapes: dict) -> dict:
    total = sum(int(np.prod(sh)) for sh in shapes.values()) * 2
    active = 0
    for name, sh in shapes.items():
        n = int(np.prod(sh)) * 2
        if ".mlp.e" in name:
            li = int(name.split(".")[0][1:])
            r = cfg["layers"][li]["mlp"]["router"]
            n = n * r["top"] / r["experts"]
        active += n
    return {"total": total, "per_token": int(active)}


def run(load_pkg, sizes, prompt_len=4096, batch=64, ctx=512, steps=16, warmup=3, kernels=False, llama=True, design="timerax"):
    serving = load_pkg("serving")
    engine_mod = load_pkg("engine")
    checkpoint_mod = load_pkg("checkpoint")
    results = {}
    for name in sizes:
        s = SIZES[name]
        r = {}
        if design == "mozetar":
            mcfg = mozetar_config(s, MOZETAR[name])
            tmp = tempfile.mkdtemp(prefix="design_bench_")
            try:
                serving.save_model_folder(tmp, mcfg, serving.random_mozetar_tensors(mcfg, 0))
                r["mozetar"] = _time_folder(serving, tmp, prompt_len, batch, ctx, steps, warmup, kernels)
                r["mozetar"]["weights_bytes"] = timerax_weight_bytes(mcfg, serving.mozetar_tensor_shapes(mcfg))
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            if not kernels:
                ncfg = numizen_config(s, NUMIZEN[name], max_positions=max(prompt_len, ctx + steps + warmup) + 64)
                tmp = tempfile.mkdtemp(prefix="design_bench_")
                try:
                    serving.save_model_folder(tmp, ncfg, serving.random_numizen_tensors(ncfg, 0))
                    r["numizen"] = _time_folder(serving, tmp, prompt_len, batch, ctx, steps, warmup, kernels)
                    r["numizen"]["weights_bytes"] = timerax_weight_bytes(ncfg, serving.numizen_tensor_shapes(ncfg))
                finally:
                    shutil.rmtree(tmp, ignore_errors=True)
                if llama:
                    r["llama2_bf16_equal_size"] = _time_llama(engine_mod, checkpoint_mod, s, prompt_len, batch, ctx, steps, warmup)
            results[name] = r
            continue
        if design == "bozovik":
            bcfg = bozovik_config(s, BOZOVIK[name])
            tmp = tempfile.mkdtemp(prefix="design_bench_")
            try:
                serving.save_model_folder(tmp, bcfg, serving.random_bozovik_tensors(bcfg, 0, decay_rank=64))
                r["bozovik"] = _time_folder(serving, tmp, prompt_len, batch, ctx, steps, warmup, kernels)
                r["bozovik"]["weights_bytes"] = timerax_weight_bytes(bcfg, serving.bozovik_tensor_shapes(bcfg, 64))
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            if not kernels:
                ncfg = numizen_config(s, NUMIZEN[name], max_positions=max(prompt_len, ctx + steps + warmup) + 64, dense_everywhere=True)
                tmp = tempfile.mkdtemp(prefix="design_bench_")
                try:
                    serving.save_model_folder(tmp, ncfg, serving.random_numizen_tensors(ncfg, 0))
                    r["numizen_dense"] = _time_folder(serving, tmp, prompt_len, batch, ctx, steps, warmup, kernels)
                    r["numizen_dense"]["weights_bytes"] = timerax_weight_bytes(ncfg, serving.numizen_tensor_shapes(ncfg))
                finally:
                    shutil.rmtree(tmp, ignore_errors=True)
                if llama:
                    r["llama2_bf16_equal_size"] = _time_llama(engine_mod, checkpoint_mod, s, prompt_len, batch, ctx, steps, warmup)
            results[name] = r
            continue
        if design == "numizen":
            ncfg = numizen_config(s, NUMIZEN[name], max_positions=max(prompt_len, ctx + steps + warmup) + 64)
            tmp = tempfile.mkdtemp(prefix="design_bench_")
            try:
                serving.save_model_folder(tmp, ncfg, serving.random_numizen_tensors(ncfg, 0))
                r["numizen"] = _time_folder(serving, tmp, prompt_len, batch, ctx, steps, warmup, kernels)
                r["numizen"]["weights_bytes"] = timerax_weight_bytes(ncfg, serving.numizen_tensor_shapes(ncfg))
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            if kernels:
                results[name] = r
                continue
        cfg = timerax_config(s)
        shapes = serving.timerax_tensor_shapes(cfg)
        tmp = tempfile.mkdtemp(prefix="design_bench_")
        try:
            serving.save_model_folder(tmp, cfg, serving.random_timerax_tensors(cfg, 0))
            r["timerax"] = _time_timerax(serving, tmp, prompt_len, batch, ctx, steps, warmup, kernels)
            r["timerax"]["weights_bytes"] = timerax_weight_bytes(cfg, shapes)
        finally:
            shutil.rmtree(tmp, ignore_errors=True)
        if llama:
            r["llama2_bf16_equal_size"] = _time_llama(engine_mod, checkpoint_mod, s, prompt_len, batch, ctx, steps, warmup)
        results[name] = r
    return results
