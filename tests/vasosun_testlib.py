"""Test helpers for the Vasosun design: small configurations and random weights written as a model folder (config.json +
model.safetensors in bf16). Nothing here is used by the product package."""
from __future__ import annotations

import numpy as np

from munazen_testlib import bf16_round, logit_error, to_bf16_bits, write_model  # noqa: F401  (the file format and the measure are the same)


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=2, top=3, ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, size=20, coef=0.4, every=7, mlp="dense"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m, "mlp": dense() if mlp == "dense" else mlp}


def latent_layer(heads=3, dim=8, rot_dim=12, vdim=20, kv_rank=40, q_rank=24, scale=0.2, rot_dims=None, base=1000.0, scaling="yarn", kv_from=None,
                 mlp="dense"):
    rot = {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}
    if scaling == "yarn":
        rot["scaling"] = {"factor": 4.0, "original": 24, "fast": 4.0, "slow": 1.0}
    elif scaling:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": dense() if mlp == "dense" else mlp}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=12, conv=3, mlp="dense"):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": dense() if mlp == "dense" else mlp}


def make_config(layers, vocab=83, width=48, eps=1e-5, taps=3, buckets=53, mul_prev=31, mul_cur=7, softcap=12.0):
    return {"architecture": "Vasosun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "logit_softcap": softcap, "layers": layers}


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """name -> float32 array of bf16-representable values (so that both storage types hold the same numbers)."""
    rng = np.random.default_rng(seed)
    d, taps = cfg["width"], cfg["canon"]["taps"]
    w = {}

    def mat(n_out, n_in, gain=1.0):
        return bf16_round(rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in))

    def vec(n, mean=0.0, std=0.1):
        return bf16_round(mean + std * rng.standard_normal(n))

    def one(mean=1.0, std=0.2):
        return bf16_round(np.array(mean + std * rng.standard_normal()))

    w["embed"] = bf16_round(rng.standard_normal((cfg["vocab"], d)))
    w["bigram"] = bf16_round(0.7 * rng.standard_normal((cfg["embedding"]["bigram"]["buckets"] + 1, d)))
    w["head"] = mat(cfg["vocab"], d, 3.0)
    w["final.norm"] = one()
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        for n in ("norm1", "norm1b"):
            w[p + n] = one()
        w[p + "canon1"] = bf16_round(0.4 * rng.standard_normal((d, taps)))
        m = l["mixer"]
        if l["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * dk, d, 1.5), mat(G * dk, d, 1.5), mat(G * dv, d)
            w[p + "mix.r1"], w[p + "mix.r2"] = bf16_round(np.abs(vec(H, 0.6, 0.3))), bf16_round(np.abs(vec(H, 0.5, 0.3)))
            w[p + "mix.o"] = mat(d, H * dv)
        elif l["type"] == "latent_attention":
            H, dn, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.uq"] = mat(Q, d), vec(Q, 1.0, 0.2), mat(H * (dn + dr), Q, 2.0)
            if m.get("kv_from") is None:
                w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(R + dr, d, 2.0), vec(R, 1.0, 0.2)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * dn, R), mat(H * dv, R)
            w[p + "mix.o"] = mat(d, H * dv)
        else:
            H, G, dk, dv, ct = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                w[p + "mix." + n] = mat(rows, d, 1.5)
                w[p + "mix." + n + ".conv"] = bf16_round(0.6 * rng.standard_normal((rows, ct)))
            w[p + "mix.b"], w[p + "mix.a"], w[p + "mix.g"] = mat(H, d, 2.0), mat(H, d, 2.0), mat(H * dv, d)
            w[p + "mix.A_log"], w[p + "mix.dt_bias"] = vec(H, -1.0, 0.8), vec(H, 0.0, 0.5)
            w[p + "mix.norm"] = vec(dv, 1.0, 0.2)
            w[p + "mix.o"] = mat(d, H * dv)
        mlp = l.get("mlp")
        if mlp:
            for n in ("norm2", "norm2b"):
                w[p + n] = one()
            w[p + "canon2"] = bf16_round(0.4 * rng.standard_normal((d, taps)))
            if mlp["kind"] == "dense":
                w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(mlp["ff"], d, 2.0), mat(mlp["ff"], d), mat(d, mlp["ff"])
            else:
                r, ff = mlp["router"], mlp["expert"]["ff"]
                for e in range(r["experts"]):
                    w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(ff, d, 2.0), mat(d, ff, 2.0)
                n_route = r["experts"] + r["identity"]
                # scores far enough apart that no choice is a close call, a correction large enough to change some choices
                w[p + "mlp.router"] = mat(n_route, d, 4.0)
                w[p + "mlp.correction"] = vec(n_route, 0.0, 0.15)
    return {k: np.asarray(v, dtype=np.float32) for k, v in w.items()}
