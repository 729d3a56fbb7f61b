"""Plain float64 restatement of the Kodezen design, one function per mechanism, whole sequences only (no cache, no portions, no
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


def offset_norm(x, w, eps):
    """RMS norm whose weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1.0 + f64(w))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def causal_conv(h, w, bias=None):
    """out[t][c] = bias[c] + sum_j w[c][j] * h[t - taps + 1 + j][c], zeros before the start; w [channels][taps], last column = the current token."""
    h, w = f64(h), f64(w)
    n, taps = h.shape[0], w.shape[1]
    out = np.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < n:
            out[back:] += h[:n - back] * w[:, j]
    return out if bias is None else out + f64(bias)


def input_conv(h, w):
    """What a mixer reads: its normed input plus the causal convolution of it."""
    return f64(h) + causal_conv(h, w)


def state_space_duality(h, W, pre, m, eps):
    """Mamba-2: one decay per head and token, state [state][vdim] per head, B and C shared by the heads of a group."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    n = h.shape[0]
    u = f64(h) @ f64(W[pre + "in"]).T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[pre + "conv"], W[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(n, H, P)
    B = xbc[:, inner:inner + G * N].reshape(n, G, N)
    C = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + f64(W[pre + "dt_bias"]))
    rate = np.exp(f64(W[pre + "A_log"]))
    D = f64(W[pre + "D"])
    y = np.zeros((n, H, P))
    for hh in range(H):
        g = hh // (H // G)
        S = np.zeros((N, P))
        for t in range(n):
            S = math.exp(-rate[hh] * dt[t, hh]) * S + dt[t, hh] * np.outer(B[t, g], x[t, hh])
            y[t, hh] = S.T @ C[t, g] + D[hh] * x[t, hh]
    y = y.reshape(n, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(n, parts, inner // parts), eps).reshape(n, inner) * f64(W[pre + "norm"])
    return y @ f64(W[pre + "o"]).T


def selective_scan(h, W, pre, m):
    """Mamba: a state of `state` numbers per channel, step size per channel, B and C shared by all channels."""
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    n = h.shape[0]
    u = f64(h) @ f64(W[pre + "in"]).T
    x, z = u[:, :inner], u[:, inner:]
    x = silu(causal_conv(x, W[pre + "conv"], W[pre + "conv.b"]))
    low = x @ f64(W[pre + "x"]).T
    dt = softplus(low[:, :R] @ f64(W[pre + "dt"]).T + f64(W[pre + "dt.b"]))
    B, C = low[:, R:R + N], low[:, R + N:]
    A = -np.exp(f64(W[pre + "A_log"]))
    D = f64(W[pre + "D"])
    S = np.zeros((inner, N))
    y = np.zeros((n, inner))
    for t in range(n):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return (y * silu(z)) @ f64(W[pre + "o"]).T


def rotate_pairs(x, pos, dims, base):
    """x [n][heads][dim]: the first `dims` dimensions turn, dimension 2i with 2i+1, by pos * base^(-2i/dims)."""
    x = f64(x).copy()
    for i in range(dims // 2):
        a = f64(pos) * base ** (-2.0 * i / dims)
        c, s = np.cos(a)[:, None], np.sin(a)[:, None]
        u, v = x[:, :, 2 * i].copy(), x[:, :, 2 * i + 1].copy()
        x[:, :, 2 * i] = u * c - v * s
        x[:, :, 2 * i + 1] = v * c + u * s
    return x


def visible(n, size, keep_first):
    """mask[i][j]: does position i see position j?"""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    ok = j <= i
    if size:
        ok &= (i - j < size) | (j < keep_first)
    return ok


def talking_attention(h, W, pre, m, eps):
    """Softmax attention whose values are the keys before norm and rotation, whose queries and keys pass a short convolution and a
    per-head RMS norm, and whose weights are mixed over the heads after the softmax."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = causal_conv(f64(h) @ f64(W[pre + "q"]).T, W[pre + "q.conv"])
    k = causal_conv(f64(h) @ f64(W[pre + "k"]).T, W[pre + "k.conv"])
    v = k.reshape(n, G, dk)[:, :, :dv]
    q = unit_rms(q.reshape(n, H, dk), eps) * f64(W[pre + "q.norm"])
    k = unit_rms(k.reshape(n, G, dk), eps) * f64(W[pre + "k.norm"])
    rot = m.get("rot")
    if rot:
        pos = np.arange(n)
        q, k = rotate_pairs(q, pos, rot["dims"], rot["base"]), rotate_pairs(k, pos, rot["dims"], rot["base"])
    mask = m.get("mask") or {}
    see = visible(n, mask.get("size"), mask.get("keep_first") or 0)
    weights = np.zeros((H, n, n))
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh // (H // G)].T) * m["scale"]
        s = np.where(see, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        weights[hh] = e / e.sum(axis=1, keepdims=True)
    mixed = np.einsum("hg,gij->hij", f64(W[pre + "talk"]), weights)
    out = np.zeros((n, H, dv))
    for hh in range(H):
        out[:, hh] = mixed[hh] @ v[:, hh // (H // G)]
    return out.reshape(n, H * dv) @ f64(W[pre + "o"]).T


def dense_ff(h, W, pre):
    z = f64(h) @ f64(W[pre + "up"]).T + f64(W[pre + "up.b"])
    return gelu_erf(z) @ f64(W[pre + "down"]).T + f64(W[pre + "down.b"])


def route(h, W, pre, top):
    """(experts chosen [n][top], their scores): sigmoid of the router's outputs, the largest first, the lower index on a tie."""
    s = sigmoid(f64(h) @ f64(W[pre + "router"]).T)
    order = np.argsort(-s, axis=1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=1)


def experts_ff(h, W, pre, mlp):
    """Every token through its `top` experts; the score multiplies what the expert reads."""
    h = f64(h)
    chosen, score = route(h, W, pre, mlp["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t], score[t]):
            u = s * h[t]
            p = f"{pre}e{int(e)}."
            out[t] += (silu(f64(W[p + "gate"]) @ u) * (f64(W[p + "up"]) @ u)) @ f64(W[p + "down"]).T
    return out


def forward(cfg: dict, W: dict, tokens, layer_outputs: list | None = None):
    """Logits [n][vocab] of one sequence; layer_outputs (if a list) receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = f64(W["embed"])[np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, W[p + "norm1"], eps)
        if p + "canon1" in W:
            h = input_conv(h, W[p + "canon1"])
        m = l["mixer"]
        if l["type"] == "mamba2":
            x = x + state_space_duality(h, W, p + "mix.", m, eps)
        elif l["type"] == "mamba1":
            x = x + selective_scan(h, W, p + "mix.", m)
        elif l["type"] == "attention":
            x = x + talking_attention(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(l["type"])
        mlp = l.get("mlp")
        if mlp:
            h = offset_norm(x, W[p + "norm2"], eps)
            x = x + (dense_ff(h, W, p + "mlp.") if mlp["kind"] == "dense" else experts_ff(h, W, p + "mlp.", mlp))
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return offset_norm(x, W["final.norm"], eps) @ f64(W["head"]).T
