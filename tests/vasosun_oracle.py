"""Plain float64 restatement of the Vasosun design, one function per mechanism, whole sequences only (no cache, no portions, no
batches). It shares nothing with the package: the tests compare the framework's kernels, cache and scheduler against it.

Notation: x [n][width] is the residual stream of one sequence, W a dictionary name -> float64 array, positions count from 0."""
from __future__ import annotations

import math

import numpy as np


def f64(a):
    return np.asarray(a, dtype=np.float64)


def unit_rms(x, eps):
    x = f64(x)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is ONE number."""
    return unit_rms(x, eps) * float(g)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def softmax(z):
    z = z - z.max(axis=-1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(axis=-1, keepdims=True)


def causal_conv(h, w):
    """out[t][c] = sum_j w[c][j] * h[t - taps + 1 + j][c], zeros before the start; w [channels][taps], the last column is the current token's."""
    h, w = f64(h), f64(w)
    n, taps = h.shape[0], w.shape[1]
    out = np.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < n:
            out[back:] += h[:n - back] * w[:, j]
    return out


def input_conv(h, w):
    """What a sublayer reads: its normed input plus a causal convolution of it."""
    return f64(h) + causal_conv(h, w)


def embed(tokens, table, bigram, buckets, mul_prev, mul_cur):
    """Token embedding plus a hashed embedding of the (previous, current) pair; the first token takes the table's last row."""
    tokens = [int(t) for t in tokens]
    x = f64(table)[tokens].copy()
    for i, t in enumerate(tokens):
        row = buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets
        x[i] += f64(bigram)[row]
    return x


def window_attention(h, W, pre, m):
    """Softmax attention without rotation: queries grow with the logarithm of the position, scores are charged r1 * ln(1 + r2 * distance)
    per head, a query sees the last ``mask.size`` positions (itself included)."""
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).reshape(n, H, dk)
    k = (h @ W[pre + "k"].T).reshape(n, G, dk)
    v = (h @ W[pre + "v"].T).reshape(n, G, dv)
    qt = m.get("q_temp")
    if qt:
        p = np.arange(n)
        q = q * (1.0 + qt["coef"] * np.log(np.floor((p + 1) / qt["every"]) + 1.0))[:, None, None]
    size = (m.get("mask") or {}).get("size") or n + 1
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    dist = (i - j).astype(np.float64)
    sees = (dist >= 0) & (dist < size)
    out = np.zeros((n, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = s - W[pre + "r1"][hh] * np.log1p(W[pre + "r2"][hh] * np.maximum(dist, 0.0))
        s = np.where(sees, s, -np.inf)
        out[:, hh] = softmax(s) @ v[:, g]
    return out.reshape(n, H * dv) @ W[pre + "o"].T


def yarn_table(dims, base, scaling):
    """Angular step of each rotary pair and the factor on cos / sin."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    if not scaling:
        return f, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, rot, first_pos=0):
    """x [n][..][width]: the first rot.dims dimensions turn, pair (2i, 2i+1) by the angle position * f_i."""
    x = f64(x).copy()
    dims = rot["dims"]
    f, mag = yarn_table(dims, rot["base"], rot.get("scaling"))
    n = x.shape[0]
    ang = (np.arange(n) + first_pos)[:, None] * f[None, :]
    shape = (n,) + (1,) * (x.ndim - 2) + (dims // 2,)
    cs, sn = (np.cos(ang) * mag).reshape(shape), (np.sin(ang) * mag).reshape(shape)
    u, v = x[..., 0:dims:2].copy(), x[..., 1:dims:2].copy()
    x[..., 0:dims:2] = u * cs - v * sn
    x[..., 1:dims:2] = v * cs + u * sn
    return x


def latent_kv(h, W, pre, m, eps):
    """What a latent-attention layer caches per token: the normed latent and the rotated key part all heads share."""
    R = m["kv_rank"]
    low = h @ W[pre + "dkv"].T
    c = unit_rms(low[:, :R], eps) * W[pre + "dkv.norm"]
    return c, rotate(low[:, R:], m["rot"])


def latent_attention(h, W, pre, m, eps, kv=None):
    """Causal attention whose keys and values are expanded from a latent; ``kv`` = (latent, rotated key part) of another layer, else its own.
    Returns (output, kv)."""
    n = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = unit_rms(h @ W[pre + "dq"].T, eps) * W[pre + "dq.norm"]
    q = (cq @ W[pre + "uq"].T).reshape(n, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate(q[..., dn:], m["rot"])
    if kv is None:
        kv = latent_kv(h, W, pre, m, eps)
    c, k_rot = kv
    k_plain = (c @ W[pre + "uk"].T).reshape(n, H, dn)
    v = (c @ W[pre + "uv"].T).reshape(n, H, dv)
    sees = np.arange(n)[:, None] >= np.arange(n)[None, :]
    out = np.zeros((n, H, dv))
    for hh in range(H):
        s = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ k_rot.T) * m["scale"]
        out[:, hh] = softmax(np.where(sees, s, -np.inf)) @ v[:, hh]
    return out.reshape(n, H * dv) @ W[pre + "o"].T, kv


def delta_rule(q, k, v, beta, g):
    """One head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q. q, k [n][dk], v [n][dv], beta, g [n]."""
    n, dk = q.shape
    S = np.zeros((dk, v.shape[1]))
    o = np.zeros_like(v)
    for t in range(n):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def delta_mixer(h, W, pre, m, eps):
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def branch(name):
        return silu(causal_conv(h @ W[pre + name].T, W[pre + name + ".conv"]))
    q, k, v = branch("q").reshape(n, G, dk), branch("k").reshape(n, G, dk), branch("v").reshape(n, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[pre + "b"].T)
    g = np.exp(-np.exp(W[pre + "A_log"]) * softplus(h @ W[pre + "a"].T + W[pre + "dt_bias"]))
    gate = silu(h @ W[pre + "g"].T).reshape(n, H, dv)
    out = np.zeros((n, H, dv))
    for hh in range(H):
        kv = hh // (H // G)
        o = delta_rule(q[:, kv], k[:, kv], v[:, hh], beta[:, hh], g[:, hh])
        out[:, hh] = unit_rms(o, eps) * W[pre + "norm"] * gate[:, hh]
    return out.reshape(n, H * dv) @ W[pre + "o"].T


def dense_ff(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(h, W, pre, top):
    """(chosen [n][top], their weights [n][top]): the largest scores + correction are chosen, the weights are the scores themselves."""
    s = softmax(h @ W[pre + "router"].T)
    chosen = np.argsort(-(s + W[pre + "correction"]), axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def moe_ff(h, W, pre, mlp):
    r = mlp["router"]
    E = r["experts"]
    chosen, weight = route(h, W, pre, r["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wgt in zip(chosen[t], weight[t]):
            if e >= E:                       # an identity expert
                out[t] += wgt * h[t]
            else:
                out[t] += wgt * (gelu_erf(h[t] @ W[f"{pre}e{e}.up"].T) @ W[f"{pre}e{e}.down"].T)
    return out


def forward(tokens, W, cfg):
    """tokens of ONE sequence -> (logits [n][vocab], the residual stream after every layer [layers][n][width])."""
    W = {k: f64(v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    big = cfg["embedding"]["bigram"]
    x = embed(tokens, W["embed"], W["bigram"], big["buckets"], big["mul_prev"], big["mul_cur"])
    taps, cached = [], {}
    for i, lc in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = input_conv(scalar_norm(x, W[pre + "norm1"], eps), W[pre + "canon1"])
        m = lc["mixer"]
        if lc["type"] == "attention":
            y = window_attention(h, W, pre + "mix.", m)
        elif lc["type"] == "latent_attention":
            src = m.get("kv_from")
            y, cached[i] = latent_attention(h, W, pre + "mix.", m, eps, None if src is None else cached[src])
        elif lc["type"] == "delta":
            y = delta_mixer(h, W, pre + "mix.", m, eps)
        else:
            raise ValueError(lc["type"])
        x = x + scalar_norm(y, W[pre + "norm1b"], eps)
        mlp = lc.get("mlp")
        if mlp is not None:
            h = input_conv(scalar_norm(x, W[pre + "norm2"], eps), W[pre + "canon2"])
            y = dense_ff(h, W, pre + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, W, pre + "mlp.", mlp)
            x = x + scalar_norm(y, W[pre + "norm2b"], eps)
        taps.append(x.copy())
    logits = scalar_norm(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return logits, np.stack(taps)
