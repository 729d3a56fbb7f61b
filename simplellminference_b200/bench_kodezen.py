"""Throughput of the Kodezen design at layer sizes of real models (random weights), beside the closest model of the framework at equal
width and depth: Vasosun (the same sequence engine; a recurrent mixer walked by the same kernel, window attention, input convolutions
in the seams, a mixture of experts). Prompt tokens per second of one whole prompt, and decoded tokens per second of 1 and 4 requests
stepping together at a context of the prompt's length. Used by ``bench.py --kodezen``; prints one JSON object per model and size.

Timing and roofline fractions as in ``bench_hybrid`` (CUDA events on the launching stream, 3 warm-ups, medians). The algorithmic work of
a mixture-of-experts layer is that of the experts a token USES (``top`` of them); where the implementation computes every expert for
every token (small experts, steps of a few tokens) the "executed" fractions show it."""
from __future__ import annotations

import json

import numpy as np

from .bench_hybrid import _time
from .bench_vasosun import bench_vasosun

SIZES = {
    # name: width, layer pattern repeats ([Mamba-2, Mamba, Mamba-2, attention] each), prompt length
    "w1024": dict(width=1024, repeats=2, prompt=2048),
    "w2048": dict(width=2048, repeats=2, prompt=2048),
    "w4096": dict(width=4096, repeats=1, prompt=2048),
}
WINDOW, KEEP_FIRST = 1024, 4
EXPERTS, TOP = 8, 2


def kodezen_config(width: int, repeats: int, vocab: int = 32000) -> dict:
    heads = width // 128
    dense = {"kind": "dense", "ff": 4 * width}
    moe = {"kind": "moe", "expert": {"ff": ((4 * width // 3) + 127) // 128 * 128}, "router": {"experts": EXPERTS, "top": TOP}}
    ssd = {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 2, "norm_groups": 2, "conv": 4}
    scan = {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}
    att = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "conv": 3,
           "mask": {"size": WINDOW, "keep_first": KEEP_FIRST}, "rot": {"dims": 64, "base": 500000.0}}
    layers = []
    for _ in range(repeats):
        layers += [{"type": "mamba2", "mixer": ssd, "mlp": dense}, {"type": "mamba1", "mixer": scan, "mlp": moe},
                   {"type": "mamba2", "mixer": ssd, "mlp": dense}, {"type": "attention", "mixer": att, "mlp": moe}]
    return {"architecture": "Kodezen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "embedding": {"scale": float(width) ** 0.5}, "layers": layers}


def random_kodezen_weights(cfg: dict, device, seed: int = 0) -> dict:
    """Random bf16 tensors under the design's tensor names, made on the device."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    d, taps = cfg["width"], cfg["canon"]["taps"]

    def mat(n_out, n_in, gain=1.0):
        return (torch.randn(n_out, n_in, generator=g, device=device) * (gain / n_in ** 0.5)).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)

    def taps_of(n, t, std=0.4):
        return (std * torch.randn(n, t, generator=g, device=device)).to(torch.bfloat16)

    w = {"embed": (torch.randn(cfg["vocab"], d, generator=g, device=device) / d ** 0.5).to(torch.bfloat16), "head": mat(cfg["vocab"], d),
         "final.norm": vec(d)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        w[p + "norm1"], w[p + "norm2"], w[p + "canon1"] = vec(d), vec(d), taps_of(d, taps, 0.3)
        if l["type"] == "mamba2":
            H, P, N, G, ct = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * P, H * P + 2 * G * N
            w[p + "mix.in"], w[p + "mix.conv"], w[p + "mix.conv.b"] = mat(inner + ch + H, d), taps_of(ch, ct), vec(ch)
            w[p + "mix.dt_bias"], w[p + "mix.A_log"], w[p + "mix.D"] = vec(H, -2.0, 0.5), vec(H, 0.0, 0.5), vec(H, 1.0)
            w[p + "mix.norm"], w[p + "mix.o"] = vec(inner, 1.0), mat(d, inner)
        elif l["type"] == "mamba1":
            inner, N, R, ct = m["inner"], m["state"], m["dt_rank"], m["conv"]
            w[p + "mix.in"], w[p + "mix.conv"], w[p + "mix.conv.b"] = mat(2 * inner, d), taps_of(inner, ct), vec(inner)
            w[p + "mix.x"], w[p + "mix.dt"], w[p + "mix.dt.b"] = mat(R + 2 * N, inner), mat(inner, R), vec(inner, -2.0, 0.5)
            w[p + "mix.A_log"] = torch.log(torch.arange(1, N + 1, device=device, dtype=torch.float32)).repeat(inner, 1).to(torch.bfloat16)
            w[p + "mix.D"], w[p + "mix.o"] = vec(inner, 1.0), mat(d, inner)
        else:
            H, G, dk, ct = m["heads"], m["kv_heads"], m["dim"], m["conv"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.o"] = mat(H * dk, d), mat(G * dk, d), mat(d, H * dk)
            w[p + "mix.q.conv"], w[p + "mix.k.conv"] = taps_of(H * dk, ct), taps_of(G * dk, ct)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(dk, 1.0), vec(dk, 1.0)
            w[p + "mix.talk"] = (torch.eye(H, device=device) + 0.2 * torch.randn(H, H, generator=g, device=device) / H ** 0.5).to(torch.bfloat16)
        mlp = l["mlp"]
        if mlp["kind"] == "dense":
            w[p + "mlp.up"], w[p + "mlp.up.b"] = mat(mlp["ff"], d), vec(mlp["ff"])
            w[p + "mlp.down"], w[p + "mlp.down.b"] = mat(d, mlp["ff"]), vec(d)
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            for e in range(r["experts"]):
                w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(ff, d), mat(ff, d), mat(d, ff)
            w[p + "mlp.router"] = mat(r["experts"], d, 2.0)
    return w


def _used_params(cfg: dict, w: dict) -> tuple:
    """(matrix parameters a token uses, all matrix parameters): an expert counts by the share of tokens routed to it."""
    total = used = 0.0
    for n, t in w.items():
        if t.dim() < 2 or n == "embed" or ".conv" in n or "canon" in n or n.endswith("A_log") or n.endswith("talk"):
            continue
        total += t.numel()
        share = 1.0
        if ".mlp.e" in n:
            r = cfg["layers"][int(n[1:n.index(".")])]["mlp"]["router"]
            share = r["top"] / r["experts"]
        used += share * t.numel()
    return used, total


def _state_bytes(cfg: dict, T: int) -> int:
    """Bytes a decoding step must move per request besides the matrices: cache rows that are visible (bf16; the keys are the values but
    are cached normed and rotated, so both pools are read), recurrent states (fp32, read and written)."""
    n = 0
    for l in cfg["layers"]:
        m = l["mixer"]
        if l["type"] == "attention":
            n += 2 * min(T, m["mask"]["size"] + m["mask"]["keep_first"]) * m["kv_heads"] * (m["dim"] + m["vdim"])
        elif l["type"] == "mamba2":
            n += 2 * 4 * m["heads"] * m["state"] * m["vdim"]
        else:
            n += 2 * 4 * m["inner"] * m["state"]
    return n


def bench_kodezen(name: str, hbm_gbs: float, tflops: float) -> dict:
    import torch

    from .config import BF16, KodezenConfig
    from .layers import ExpertsFeedForward
    from .models.kodezen import KodezenModel
    from .seqengine import SequenceEngine
    from .seqops import Ops
    size = SIZES[name]
    dev = torch.device("cuda")
    cfg = kodezen_config(size["width"], size["repeats"])
    w = random_kodezen_weights(cfg, dev)
    used, total = _used_params(cfg, w)
    ops = Ops(BF16)
    model = KodezenModel(KodezenConfig.from_dict(cfg), w, ops, dev)
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
    out = {"model": f"kodezen-{name}", "width": size["width"], "layers": len(cfg["layers"]), "matrix_params": int(total), "matrix_params_used_per_token": int(used),
           "prompt_len": T, "prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_sec": round(T / prefill_ms * 1e3, 1),
           "prefill_gemm_tflops": round(2.0 * used * T / prefill_ms / 1e9, 1), "prefill_gemm_tflops_executed": round(2.0 * total * T / prefill_ms / 1e9, 1),
           "prefill_launches": (ops.launches - l0) // 8}
    out["prefill_fraction_of_measured_bf16_peak"] = round(out["prefill_gemm_tflops"] / tflops, 3)
    out["prefill_fraction_of_measured_bf16_peak_executed"] = round(out["prefill_gemm_tflops_executed"] / tflops, 3)
    state_bytes = _state_bytes(cfg, T)
    experts = [l.ff for l in model.layers if isinstance(l.ff, ExpertsFeedForward)]
    for n in (1, 4):
        slots = [eng.admit() for _ in range(n)]
        eng.run([(s, prompt, []) for s in slots])
        tok = [int(prompt[-1])] * n

        def step():
            eng.run([(s, [t], [0]) for s, t in zip(slots, tok)])

        ms = _time(step, 30, warmup=4)
        out[f"decode{n}_ms_per_step"] = round(ms, 4)
        out[f"decode{n}_tokens_per_sec"] = round(n / ms * 1e3, 1)
        # one request reads the experts it uses; four requests together touch most of them
        weights = used if n == 1 else total
        executed = used if (n == 1 and experts and all(f._indexed_pays(n) for f in experts)) else total
        out[f"decode{n}_fraction_of_measured_hbm"] = round((2.0 * weights + n * state_bytes) / (ms * 1e-3) / (hbm_gbs * 1e9), 3)
        out[f"decode{n}_fraction_of_measured_hbm_executed"] = round((2.0 * executed + n * state_bytes) / (ms * 1e-3) / (hbm_gbs * 1e9), 3)
        for s in slots:
            eng.release(s)
    out["graph_replays"] = eng.graph_replays
    return out


def main(sizes, hbm_gbs: float, tflops: float) -> list:
    """A size named ``<size>-alone`` runs Kodezen without the model beside it (for a launch list of one model)."""
    res = []
    for name in sizes:
        alone = name.endswith("-alone")
        name = name[:-len("-alone")] if alone else name
        arms = [("kodezen", lambda: bench_kodezen(name, hbm_gbs, tflops))]
        if not alone:
            arms.append(("vasosun", lambda: bench_vasosun(name, hbm_gbs, tflops)))
        for label, fn in arms:
            try:
                r = fn()
            except Exception as ex:   # one size that does not fit or run must not hide the others
                r = {"model": f"{label}-{name}", "error": f"{type(ex).__name__}: {ex}"[:300]}
            print(json.dumps(r), flush=True)
            res.append(r)
    return res
