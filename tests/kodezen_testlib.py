"""Test helpers for the Kodezen design: small configurations and random weights written as a model folder (config.json +
model.safetensors in bf16), and a stub model that feeds rows to one mechanism through the engine. Nothing here is used by the product
package."""
from __future__ import annotations

import numpy as np

from munazen_testlib import bf16_round, logit_error, to_bf16_bits, write_model  # noqa: F401  (the file format and the measure are the same)


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _mlp(mlp):
    return dense() if mlp == "dense" else mlp


def mamba2_layer(heads=4, vdim=8, state=12, groups=2, norm_groups=2, conv=4, mlp="dense"):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv},
            "mlp": _mlp(mlp)}


def mamba1_layer(inner=40, state=6, dt_rank=5, conv=3, mlp="dense"):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": _mlp(mlp)}


def attention_layer(heads=4, kv_heads=2, dim=16, scale=0.3, size=20, keep_first=3, rot_dims=8, base=1000.0, conv=3, mlp="dense"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "conv": conv}
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep_first}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "attention", "mixer": m, "mlp": _mlp(mlp)}


def make_config(layers, vocab=83, width=48, eps=1e-5, taps=3, scale=3.0):
    return {"architecture": "Kodezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "embedding": {"scale": scale},
            "layers": layers}


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """name -> float32 array of bf16-representable values (so that both storage types hold the same numbers)."""
    rng = np.random.default_rng(seed)
    d, taps = cfg["width"], cfg["canon"]["taps"]
    w = {}

    def mat(n_out, n_in, gain=1.0):
        return bf16_round(rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in))

    def vec(n, mean=0.0, std=0.1):
        return bf16_round(mean + std * rng.standard_normal(n))

    w["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], d)) / cfg["embedding"]["scale"])
    w["head"] = mat(cfg["vocab"], d, 3.0)
    w["final.norm"] = vec(d, -0.2, 0.4)
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"] = vec(d, 0.0, 0.3)
        w[p + "canon1"] = bf16_round(0.4 * rng.standard_normal((d, taps)))
        m = l["mixer"]
        if l["type"] == "mamba2":
            H, P, N, G, ct = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * P, H * P + 2 * G * N
            w[p + "mix.in"] = mat(inner + ch + H, d, 1.5)
            w[p + "mix.conv"], w[p + "mix.conv.b"] = bf16_round(0.6 * rng.standard_normal((ch, ct))), vec(ch, 0.0, 0.2)
            w[p + "mix.dt_bias"], w[p + "mix.A_log"], w[p + "mix.D"] = vec(H, -0.5, 0.8), vec(H, -0.5, 0.8), vec(H, 1.0, 0.3)
            w[p + "mix.norm"] = vec(inner, 1.0, 0.2)
            w[p + "mix.o"] = mat(d, inner)
        elif l["type"] == "mamba1":
            I, N, R, ct = m["inner"], m["state"], m["dt_rank"], m["conv"]
            w[p + "mix.in"] = mat(2 * I, d, 1.5)
            w[p + "mix.conv"], w[p + "mix.conv.b"] = bf16_round(0.6 * rng.standard_normal((I, ct))), vec(I, 0.0, 0.2)
            w[p + "mix.x"] = mat(R + 2 * N, I, 1.5)
            w[p + "mix.dt"], w[p + "mix.dt.b"] = mat(I, R, 1.5), vec(I, -1.0, 1.0)
            w[p + "mix.A_log"] = bf16_round(np.log(np.arange(1, N + 1))[None, :] + 0.3 * rng.standard_normal((I, N)))
            w[p + "mix.D"] = vec(I, 1.0, 0.3)
            w[p + "mix.o"] = mat(d, I)
        else:
            H, G, dk, ct = m["heads"], m["kv_heads"], m["dim"], m["conv"]
            w[p + "mix.q"], w[p + "mix.k"] = mat(H * dk, d, 1.5), mat(G * dk, d, 1.5)
            w[p + "mix.q.conv"], w[p + "mix.k.conv"] = bf16_round(0.6 * rng.standard_normal((H * dk, ct))), bf16_round(0.6 * rng.standard_normal((G * dk, ct)))
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(dk, 1.2, 0.4), vec(dk, 1.2, 0.4)
            w[p + "mix.talk"] = bf16_round(0.5 * np.eye(H) + 0.4 * rng.standard_normal((H, H)))
            w[p + "mix.o"] = mat(d, H * dk)
        mlp = l.get("mlp")
        if mlp:
            w[p + "norm2"] = vec(d, 0.0, 0.3)
            if mlp["kind"] == "dense":
                ff = mlp["ff"]
                w[p + "mlp.up"], w[p + "mlp.up.b"] = mat(ff, d, 2.0), vec(ff, 0.0, 0.3)
                w[p + "mlp.down"], w[p + "mlp.down.b"] = mat(d, ff), vec(d, 0.0, 0.3)
            else:
                r, ff = mlp["router"], mlp["expert"]["ff"]
                for e in range(r["experts"]):
                    w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(ff, d, 2.0), mat(ff, d, 2.0), mat(d, ff, 2.0)
                # scores far enough apart that no choice is a close call
                w[p + "mlp.router"] = mat(r["experts"], d, 4.0)
    return {k: np.asarray(v, dtype=np.float32) for k, v in w.items()}


class Stub:
    """A model that hands the rows it is given to a function of (step, h, states) and keeps what that returns."""

    def __init__(self, specs, fn, ops, dev):
        self.specs, self.fn, self.ops, self.device = specs, fn, ops, dev
        self.h, self.outs = None, None

    def state_specs(self):
        return self.specs

    def forward(self, step, ids, states, rows, n_rows, tap=None):
        self.outs = [o.clone() for o in self.fn(step, self.h, states)]
        return None


def feed(stub, rows, portions, max_tokens=1024, page_len=32, engine=None, slot=None, release=True):
    """rows [T][d] through the stub in portions; returns the concatenated outputs."""
    import torch

    from simplellminference_b200.seqengine import SequenceEngine
    eng = engine or SequenceEngine(stub, max_tokens=max_tokens, page_len=page_len, graphs=False)
    slot, outs, p = eng.admit() if slot is None else slot, None, 0
    for n in portions:
        stub.h = torch.tensor(rows[p:p + n], dtype=torch.float32, device=stub.device).contiguous().view(-1)
        eng.run([(slot, np.zeros(n, np.int32), [])])
        outs = [[] for _ in stub.outs] if outs is None else outs
        for i, o in enumerate(stub.outs):
            outs[i].append(o.cpu().numpy())
        p += n
    if engine is not None and release:
        eng.release(slot)
    return [np.concatenate(o) for o in outs]
