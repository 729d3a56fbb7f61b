"""Throughput of the Vasosun design at layer sizes of real models (random weights), beside the closest models of the framework at equal
width and depth: Sopetar (the same sequence engine; window and latent attention, gated feed-forward) and the Llama engine. Prompt tokens
per second of one whole prompt, and decoded tokens per second of 1 and 4 requests stepping together at a context of the prompt's length.
Used by ``bench.py --vasosun``; prints one JSON object per model and size.

Timing and roofline fractions as in ``bench_hybrid`` (CUDA events on the launching stream, 3 warm-ups, medians). The algorithmic work of
a mixture-of-experts layer is that of the experts a token USES (on average top * experts / (experts + identity) of them); where the
implementation computes every expert for every token (small experts, steps of a few tokens) the "executed" fractions show it."""
from __future__ import annotations

import json

import numpy as np

from .bench_hybrid import _time, bench_llama
from .bench_sopetar import bench_sopetar

SIZES = {
    # name: width, layer pattern repeats ([attention, latent, latent over the cache before it, delta] each), prompt length
    "w1024": dict(width=1024, repeats=2, prompt=2048),
    "w2048": dict(width=2048, repeats=2, prompt=2048),
    "w4096": dict(width=4096, repeats=1, prompt=2048),
}
WINDOW = 1024
EXPERTS, IDENTITY, TOP = 8, 2, 3


def vasosun_config(width: int, repeats: int, vocab: int = 32000) -> dict:
    heads = width // 128
    ff = ((8 * width // 3) + 255) // 256 * 256
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // 2}, "router": {"experts": EXPERTS, "identity": IDENTITY, "top": TOP}}
    rot = {"dims": 64, "base": 500000.0, "scaling": {"factor": 4.0, "original": 8192, "fast": 16.0, "slow": 2.0}}
    layers = []
    for r in range(repeats):
        att = {"type": "attention", "mlp": dense,
               "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": WINDOW},
                         "q_temp": {"coef": 0.1, "every": 1024}}}
        lat = {"heads": heads, "dim": 64, "rot_dim": 64, "vdim": 64, "kv_rank": 128, "q_rank": max(128, width // 4), "scale": 128 ** -0.5, "rot": rot}
        layers += [att, {"type": "latent_attention", "mlp": moe, "mixer": lat}, {"type": "latent_attention", "mlp": moe, "mixer": dict(lat, kv_from=4 * r + 1)},
                   {"type": "delta", "mlp": moe, "mixer": {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4}}]
    return {"architecture": "Vasosun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 8191}}, "logit_softcap": 30.0, "layers": layers}


def random_vasosun_weights(cfg: dict, device, seed: int = 0) -> dict:
    """Random bf16 tensors under the design's tensor names, made on the device."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    d, taps = cfg["width"], cfg["canon"]["taps"]

    def mat(n_out, n_in, gain=1.0):
        return (torch.randn(n_out, n_in, generator=g, device=device) * (gain / n_in ** 0.5)).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)

    def one():
        return torch.tensor(1.0, device=device).to(torch.bfloat16)

    w = {"embed": torch.randn(cfg["vocab"], d, generator=g, device=device).to(torch.bfloat16), "head": mat(cfg["vocab"], d), "final.norm": one(),
         "bigram": (0.5 * torch.randn(cfg["embedding"]["bigram"]["buckets"] + 1, d, generator=g, device=device)).to(torch.bfloat16)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            w[p + n] = one()
        for n in ("canon1", "canon2"):
            w[p + n] = (0.3 * torch.randn(d, taps, generator=g, device=device)).to(torch.bfloat16)
        if l["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.o"] = mat(H * dk, d), mat(G * dk, d), mat(G * dv, d), mat(d, H * dv)
            w[p + "mix.r1"], w[p + "mix.r2"] = vec(H, 0.5, 0.1), vec(H, 0.5, 0.1)
        elif l["type"] == "latent_attention":
            H, dn, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.uq"] = mat(Q, d), vec(Q, 1.0), mat(H * (dn + dr), Q)
            if "kv_from" not in m:
                w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(R + dr, d), vec(R, 1.0)
            w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.o"] = mat(H * dn, R), mat(H * dv, R), mat(d, H * dv)
        else:
            H, G, dk, dv, ct = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                w[p + "mix." + n] = mat(rows, d)
                w[p + "mix." + n + ".conv"] = (0.5 * torch.randn(rows, ct, generator=g, device=device)).to(torch.bfloat16)
            w[p + "mix.b"], w[p + "mix.a"], w[p + "mix.g"], w[p + "mix.o"] = mat(H, d), mat(H, d), mat(H * dv, d), mat(d, H * dv)
            w[p + "mix.A_log"], w[p + "mix.dt_bias"], w[p + "mix.norm"] = vec(H, -1.0, 0.5), vec(H), vec(dv, 1.0)
        mlp = l["mlp"]
        if mlp["kind"] == "dense":
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(mlp["ff"], d), mat(mlp["ff"], d), mat(d, mlp["ff"])
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            for e in range(r["experts"]):
                w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(ff, d), mat(d, ff)
            w[p + "mlp.router"], w[p + "mlp.correction"] = mat(r["experts"] + r["identity"], d, 2.0), vec(r["experts"] + r["identity"], 0.0, 0.05)
    return w


def _used_params(cfg: dict, w: dict) -> tuple:
    """(matrix parameters a token uses, all matrix parameters): experts count by the average number a token is routed to."""
    total = used = 0.0
    for n, t in w.items():
        if t.dim() < 2 or n in ("embed", "bigram") or ".conv" in n or "canon" in n:
            continue
        total += t.numel()
        share = 1.0
        if ".mlp.e" in n:
            r = cfg["layers"][int(n[1:n.index(".")])]["mlp"]["router"]
            share = r["top"] / (r["experts"] + r["identity"])
        used += share * t.numel()
    return used, total


def bench_vasosun(name: str, hbm_gbs: float, tflops: float) -> dict:
    import torch

    from .config import BF16, VasosunConfig
    from .layers import ExpertsFeedForward
    from .models.vasosun import VasosunModel
    from .seqengine import SequenceEngine
    from .seqops import Ops
    size = SIZES[name]
    dev = torch.device("cuda")
    cfg = vasosun_config(size["width"], size["repeats"])
    w = random_vasosun_weights(cfg, dev)
    used, total = _used_params(cfg, w)
    ops = Ops(BF16)
    model = VasosunModel(VasosunConfig.from_dict(cfg), w, ops, dev)
    T = size["prompt"]
    eng = SequenceEngine(model, max_tokens=4 * (T + 128), max_seqs=4)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg["vocab"], size=T).astype(np.int32)

    def prefill():
        s = eng.admit()
        eng.run([(s, prompt, [T - 1])])
        eng.release(s)

    l0 = ops.launches
    prefill_ms = _time(prefill, 5)
    out = {"model": f"vasosun-{name}", "width": size["width"], "layers": len(cfg["layers"]), "matrix_params": int(total), "matrix_params_used_per_token": int(used),
           "prompt_len": T, "prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_sec": round(T / prefill_ms * 1e3, 1),
           "prefill_gemm_tflops": round(2.0 * used * T / prefill_ms / 1e9, 1), "prefill_gemm_tflops_executed": round(2.0 * total * T / prefill_ms / 1e9, 1),
           "prefill_launches": (ops.launches - l0) // 8}
    out["prefill_fraction_of_measured_bf16_peak"] = round(out["prefill_gemm_tflops"] / tflops, 3)
    out["prefill_fraction_of_measured_bf16_peak_executed"] = round(out["prefill_gemm_tflops_executed"] / tflops, 3)
    # bytes a decoding step must read per request besides the matrices: cache rows inside the windows (bf16), recurrent state (fp32, read and written)
    state_bytes = 0
    for l in cfg["layers"]:
        m = l["mixer"]
        if l["type"] == "attention":
            state_bytes += 2 * min(T, m["mask"]["size"]) * m["kv_heads"] * (m["dim"] + m["vdim"])
        elif l["type"] == "latent_attention":
            state_bytes += 2 * T * (m["kv_rank"] + m["rot_dim"])
        else:
            state_bytes += 2 * 4 * m["heads"] * m["dim"] * m["vdim"]
    for n in (1, 4):
        slots = [eng.admit() for _ in range(n)]
        eng.run([(s, prompt, []) for s in slots])
        tok = [int(prompt[-1])] * n

        def step():
            eng.run([(s, [t], [0]) for s, t in zip(slots, tok)])

        l0 = ops.launches
        ms = _time(step, 30, warmup=4)
        out[f"decode{n}_ms_per_step"] = round(ms, 4)
        out[f"decode{n}_tokens_per_sec"] = round(n / ms * 1e3, 1)
        # one request reads the experts it uses; four requests together touch most of them
        weights = used if n == 1 else total
        # what the step really streams: only the chosen experts where the expert layers take the indexed form at this batch size
        experts = [sub.body for subs in model.layers for sub in subs if isinstance(sub.body, ExpertsFeedForward)]
        executed = used if (n == 1 and experts and all(f._indexed_pays(n) for f in experts)) else total
        out[f"decode{n}_fraction_of_measured_hbm"] = round((2.0 * weights + n * state_bytes) / (ms * 1e-3) / (hbm_gbs * 1e9), 3)
        out[f"decode{n}_fraction_of_measured_hbm_executed"] = round((2.0 * executed + n * state_bytes) / (ms * 1e-3) / (hbm_gbs * 1e9), 3)
        for s in slots:
            eng.release(s)
    out["graph_replays"] = eng.graph_replays
    return out


def main(sizes, hbm_gbs: float, tflops: float) -> list:
    res = []
    for name in sizes:
        for label, fn in (("vasosun", lambda: bench_vasosun(name, hbm_gbs, tflops)), ("sopetar", lambda: bench_sopetar(name, hbm_gbs, tflops)),
                          ("llama", lambda: bench_llama(name, hbm_gbs, tflops, SIZES[name]))):
            try:
                r = fn()
            except Exception as ex:   # one size that does not fit or run must not hide the others
                r = {"model": f"{label}-{name}", "error": f"{type(ex).__name__}: {ex}"[:300]}
            print(json.dumps(r), flush=True)
            res.append(r)
    return res
