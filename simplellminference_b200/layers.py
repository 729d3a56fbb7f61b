"""Sequence-mixing and feed-forward mechanisms over the ragged-token-batch kernels (seqops.Ops), each with its constants as parameters so
that a model description can combine them: fused input projections, softmax attention with (scaled, partial) rotary positions, rotated
values and a head gate over a paged cache; softmax attention with unit-rms heads, capped scores, distance slopes and a window that keeps
the first positions; latent attention (one cached row per token, absorbed form) with a sink and a head gate; a Griffin-style recurrent block (short causal convolution + real-gated linear recurrent unit);
gated linear attention with a decay per key channel; a PolyNorm feed-forward; a clamped gated feed-forward; softmax attention with a charge on the
logarithm of the distance and a query temperature; the gated delta rule behind short convolutions; a gated (silu) feed-forward and a mixture of
experts with identity experts (softmax or sigmoid scores, plain or gated experts, the score on the expert's output or on its input);
state-space duality (Mamba-2) and the selective scan (Mamba) behind short convolutions; softmax attention whose queries and keys pass a
convolution and a per-head norm, whose values are the keys before the norm, and whose weights are mixed over the heads after the softmax;
a feed-forward with biases and the exact gelu. A mechanism says which per-sequence state it needs
(``state_spec``); the engine's state manager owns that memory and hands it to ``forward`` — no mechanism keeps a cache of its own.

Additive to the reference, whose only model is the Llama forward of source/model/model.cpp:40-140."""
from __future__ import annotations

import math

import torch

from .config import BF16

F32B = 4   # bytes of an activation


def yarn_frequencies(dims: int, base: float, scaling: dict | None):
    """Angular step per position of each of the dims/2 rotary pairs, and the factor on cos / sin. ``scaling`` = {factor, original, fast,
    slow}: pairs that turn more than ``fast`` times over the ``original`` context keep their frequency, those that turn less than ``slow``
    times are slowed down by ``factor``, with a linear ramp over the pair index between the two."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


class FusedLinear:
    """Several projections of the same input as ONE product: weight rows concatenated, one bias vector (zeros where a part has none).
    ``offsets[i]`` is the first output column of part i. ``pad_rows``: rows of zeros are appended until the row count is a multiple of it
    (the tensor-core product takes output widths that are multiples of 4; the consumers of an input product address its columns
    through pointers and the row stride ``N``, so the extra columns cost nothing but their zeros)."""

    def __init__(self, parts, ops, device, pad_rows: int = 1):
        self.ops = ops
        self.K = int(parts[0][0].shape[1])
        self.sizes = [int(w.shape[0]) for w, _ in parts]
        self.offsets = [sum(self.sizes[:i]) for i in range(len(parts))]
        pad = -sum(self.sizes) % max(1, pad_rows)
        if pad:
            parts = list(parts) + [(torch.zeros(pad, self.K, dtype=parts[0][0].dtype, device=parts[0][0].device), None)]
            self.sizes = self.sizes + [pad]
        self.N = sum(self.sizes)
        self.w = torch.cat([w for w, _ in parts], dim=0).contiguous()
        if any(b is not None for _, b in parts):
            self.bias = torch.cat([(b.float() if b is not None else torch.zeros(n, device=device)) for (_, b), n in zip(parts, self.sizes)]).contiguous()
        else:
            self.bias = None

    def __call__(self, step, a_ptr, lda, c_ptr, ldc, alpha=1.0, accumulate=False, a16_ready=False):
        scratch = step.gemm_scratch(self.K, self.N)
        self.ops.linear(a_ptr, lda, self.w, self.K, self.bias, c_ptr, ldc, step.T, self.N, self.K, step.st, alpha=alpha, accumulate=accumulate,
                        scratch=scratch, a16_ready=a16_ready and scratch is not None)

    def operand_rows(self, step):
        """Where a kernel that produces this product's input may leave it as bf16 rows [T][K] (then call with ``a16_ready``), or None when
        the product does not run on the tensor cores in this step."""
        scratch = step.gemm_scratch(self.K, self.N)
        if scratch is None or not self.ops.on_tensor_cores(step.T, self.N, self.K) or self.w.data_ptr() % 16:
            return None
        return scratch


class GatedRotaryAttention:
    """Causal softmax attention over a paged cache: grouped query heads, key width ``dim`` and value width ``vdim``, rotary positions on
    the first ``rot.dims`` dimensions of q and k (scaled frequencies), values rotated by their own position before they are cached and the
    weighted sum turned back by the query's position, one sigmoid gate per head, then the output projection."""

    def __init__(self, cfg, w, pre, ops, device, layout=0):
        self.cfg, self.ops, self.layout = cfg, ops, layout
        self.inputs = [(w[pre + "q"], w.get(pre + "q.b")), (w[pre + "k"], w.get(pre + "k.b")), (w[pre + "v"], w.get(pre + "v.b")), (w[pre + "g"], None)]
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        f, self.magnitude = yarn_frequencies(cfg.rot.dims, cfg.rot.base, cfg.rot.scaling)
        self.freq = torch.tensor(f, dtype=torch.float64, device=device)
        self.vfreq = torch.tensor([cfg.rot.base ** (-2.0 * m / cfg.vdim) for m in range(cfg.vdim // 2)], dtype=torch.float64, device=device)
        self.width = cfg.heads * cfg.vdim

    def state_spec(self):
        return {"pages": [("k", self.cfg.kv_heads, self.cfg.dim), ("v", self.cfg.kv_heads, self.cfg.vdim)], "slots": []}

    def forward(self, step, cols, ld, state, out):
        c, ops = self.cfg, self.ops
        q, k, v, g = cols
        ops.rotary_kv(step.b, q, ld, c.heads, c.dim, k, ld, c.kv_heads, v, ld, c.vdim, self.freq, c.rot.dims // 2, self.magnitude, self.vfreq,
                      self.layout, state["k"], state["v"], step.st)
        ws = step.scratch("attn_ws", step.T * c.heads * step.nsplit * (c.vdim + 2))
        ops.attention(step.b, q, ld, c.heads, c.kv_heads, c.dim, c.vdim, c.scale, state["k"], state["v"], step.nsplit, ws, step.st)
        ops.attention_finish(step.b, ws, step.nsplit, c.heads, c.vdim, self.vfreq, self.layout, g, ld, out, self.width, step.st)


def distance_slopes(heads: int, span: float = 8.0):
    """Charge per position of distance for each head: head h of H gets 2^(-span (h+1) / H) (a geometric ladder down to 2^-span)."""
    return [2.0 ** (-span * (h + 1) / heads) for h in range(heads)]


class CappedWindowAttention:
    """Softmax attention without rotation over a paged cache: every query, key and value head divided by its root mean square (no weight),
    score = cap * tanh(q.k * scale / cap) - slope_h * distance, a sliding window that keeps the first positions of the sequence visible
    at their true distance, grouped query heads. ``share`` = "keep": the values (after the division) are kept for later layers of the
    step; "blend": v <- (1 - lambda) v + lambda * (the kept values of the same token), lambda = the tensor ``vmix``; the blended values
    are what the cache holds."""

    slope_span = 8.0

    def __init__(self, cfg, w, pre, ops, device, eps, share=None):
        self.cfg, self.ops, self.eps, self.share = cfg, ops, eps, share
        self.inputs = [(w[pre + "q"], w.get(pre + "q.b")), (w[pre + "k"], w.get(pre + "k.b")), (w[pre + "v"], w.get(pre + "v.b"))]
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        self.slopes = torch.tensor(distance_slopes(cfg.heads, self.slope_span), dtype=torch.float32, device=device)
        self.lam = float(w[pre + "vmix"].float().item()) if share == "blend" else 0.0
        self.opts = ops.attention_options(cfg.mask.size, cfg.mask.keep_first, cfg.softcap, self.slopes)
        self.width = cfg.heads * cfg.vdim

    def state_spec(self):
        return {"pages": [("k", self.cfg.kv_heads, self.cfg.dim), ("v", self.cfg.kv_heads, self.cfg.vdim)], "slots": []}

    def forward(self, step, cols, ld, state, out):
        c, ops = self.cfg, self.ops
        q, k, v = cols
        kept = step.scratch("v_kept", step.T * c.kv_heads * c.vdim) if self.share else None
        ops.unit_kv(step.b, q, ld, c.heads, c.dim, k, ld, c.kv_heads, v, ld, c.vdim, self.eps, 7, kept, {None: 0, "keep": 1, "blend": 2}[self.share],
                    self.lam, state["k"], state["v"], step.st)
        ws = step.scratch("attn_ws", step.T * c.heads * step.nsplit * (c.vdim + 2))
        ops.attention(step.b, q, ld, c.heads, c.kv_heads, c.dim, c.vdim, c.scale, state["k"], state["v"], step.nsplit, ws, step.st, opts=self.opts)
        ops.attention_finish(step.b, ws, step.nsplit, c.heads, c.vdim, None, 0, None, 0, out, self.width, step.st)


class LatentAttention:
    """Attention over ONE cached row per token: c = RMS norm (weight) of the first kv_rank outputs of the down projection, and the last
    rot_dim outputs rotated by the position, a key part all heads share. Head h's key is (W_uk,h c, rotated part), its value W_uv,h c.
    Computed in the absorbed form, so that nothing but the cached row is read per key: the query of head h becomes (W_uk,h^T q_h, rotated
    q part) against the row itself (one key/value head of width kv_rank + rot_dim whose first kv_rank columns are also the value), and W_uv,h
    is applied to the head's weighted sum of rows. The softmax's denominator holds exp(sink_h) and head h's output is multiplied by
    sigmoid(g_h) when the model has the tensors ``sink`` / ``g``; then the output projection.

    Variants, chosen by the configuration and the tensors present: the queries may go through a latent of their own (``q_rank``:
    q = W_uq RMSnorm(W_dq h), weight ``dq.norm``); the rotation's frequencies may be YaRN-scaled (``rot.scaling``; cos and sin then carry a
    magnitude); with ``kv_from`` the layer has no down projection and attends over the rows another layer cached (its own W_uk / W_uv)."""

    def __init__(self, cfg, w, pre, ops, device, eps):
        self.cfg, self.ops, self.eps = cfg, ops, eps
        H, dn, dr, R = cfg.heads, cfg.dim, cfg.rot_dim, cfg.kv_rank
        self.q_latent = cfg.q_rank is not None
        self.shared = cfg.kv_from is not None
        self.gated = pre + "g" in w
        self.inputs = [(w[pre + "dq"], w.get(pre + "dq.b"))] if self.q_latent else [(w[pre + "q"], w.get(pre + "q.b"))]
        if not self.shared:
            self.inputs.append((w[pre + "dkv"], w.get(pre + "dkv.b")))
            self.norm_w = w[pre + "dkv.norm"].float().contiguous()
        else:
            self.norm_w = None
        if self.gated:
            self.inputs.append((w[pre + "g"], w.get(pre + "g.b")))
        if self.q_latent:
            self.q_norm_w = w[pre + "dq.norm"].float().contiguous()
            self.uq = FusedLinear([(w[pre + "uq"], w.get(pre + "uq.b"))], ops, device)
        self.uk_t = w[pre + "uk"].view(H, dn, R).transpose(1, 2).contiguous()       # [H][R][dn]: rows of W_uk,h^T
        self.uv = w[pre + "uv"].contiguous()                                         # [H * vdim][R]
        self.sink = w[pre + "sink"].float().contiguous() if pre + "sink" in w else None
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        f, self.magnitude = yarn_frequencies(cfg.rot.dims, cfg.rot.base, cfg.rot.scaling)
        self.freq = torch.tensor(f, dtype=torch.float64, device=device)
        self.opts = ops.attention_options(cfg.mask.size, cfg.mask.keep_first, values_in_keys=True)
        self.width = H * cfg.vdim

    def state_spec(self):
        if self.shared:       # no pool of its own: the state manager hands it the named layer's
            return {"pages": [], "slots": [], "borrow": [("row", self.cfg.kv_from, "row")]}
        return {"pages": [("row", 1, self.cfg.kv_rank + self.cfg.rot_dim)], "slots": []}

    def forward(self, step, cols, ld, state, out):
        c, ops, T = self.cfg, self.ops, step.T
        H, dn, dr, R, dv = c.heads, c.dim, c.rot_dim, c.kv_rank, c.vdim
        cols = list(cols)
        q, ldq = cols.pop(0), ld
        low = None if self.shared else cols.pop(0)
        g = cols.pop(0) if self.gated else None
        if self.q_latent:                      # the query's own latent: norm in place, then the up projection of every head
            ops.rmsnorm_rows(q, ld, self.q_norm_w, self.eps, q, ld, T, c.q_rank, step.st)
            qfull = step.scratch("latent_qfull", T * self.uq.N)
            self.uq(step, q, ld, qfull.data_ptr(), self.uq.N)
            q, ldq = qfull.data_ptr(), self.uq.N
        wide = R + dr
        qa = step.scratch("latent_q", T * H * wide)
        ops.latent_kv(step.b, q, ldq, H, dn, dr, low, ld, R, self.norm_w, self.eps, self.freq, c.rot.dims // 2, qa, H * wide, state["row"], step.st,
                      magnitude=self.magnitude)
        ops.linear(q, ldq, self.uk_t, dn, None, qa.data_ptr(), H * wide, T, R, dn, step.st, batch=H, a_bs=dn + dr, w_bs=R * dn, c_bs=wide)
        ws = step.scratch("attn_ws", T * H * step.nsplit * (R + 2))
        ops.attention(step.b, qa.data_ptr(), H * wide, H, 1, wide, R, c.scale, state["row"], None, step.nsplit, ws, step.st, opts=self.opts)
        mixed = step.scratch("latent_o", T * H * R)
        ops.attention_finish(step.b, ws, step.nsplit, H, R, None, 0, g, ld, mixed, H * R, step.st, sink=self.sink)
        ops.linear(mixed.data_ptr(), H * R, self.uv, R, None, out.data_ptr(), self.width, T, dv, R, step.st, batch=H, a_bs=R, w_bs=dv * R, c_bs=dv)


class GatedLinearRecurrence:
    """Griffin's recurrent block: a GELU branch y and a branch u = causal convolution of a projection; per block of channels the gates
    r = sigmoid(A_r u + b_r), i = sigmoid(A_i u + b_i); log a = -``decay_scale`` * r * softplus(lam); S <- a S + sqrt(1 - a^2) (i * u);
    the block returns (S * y) projected. State per sequence: S and the last taps-1 inputs of the convolution, fp32."""

    decay_scale = 8.0

    def __init__(self, cfg, w, pre, ops, device):
        self.cfg, self.ops = cfg, ops
        self.inputs = [(w[pre + "y"], w.get(pre + "y.b")), (w[pre + "x"], w.get(pre + "x.b"))]
        self.conv_w = w[pre + "conv"].float().contiguous()
        self.conv_b = w[pre + "conv.b"].float().contiguous() if pre + "conv.b" in w else None
        self.gates_w = torch.stack([w[pre + "ra"], w[pre + "ri"]]).contiguous()          # [2][blocks][bs][bs]
        self.gates_b = torch.stack([w[pre + "ra.b"].float(), w[pre + "ri.b"].float()]).contiguous()   # [2][blocks][bs]
        self.lam = w[pre + "lam"].float().contiguous()
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        self.width = cfg.width

    def state_spec(self):
        slots = [("S", (self.cfg.width,))]
        if self.cfg.conv > 1:
            slots.append(("tail", (self.cfg.conv - 1, self.cfg.width)))
        return {"pages": [], "slots": slots}

    def forward(self, step, cols, ld, state, out):
        c, ops, T, W = self.cfg, self.ops, step.T, self.cfg.width
        y, x = cols
        u = step.scratch("rg_u", T * W)
        gates = step.scratch("rg_gates", 2 * T * W)          # r logits [T][W], then i logits [T][W]
        tail = state.get("tail")
        ops.conv(step.b, x, ld, W, c.conv, self.conv_w, self.conv_b, tail, u, W, step.st)
        bs = W // c.blocks
        for which in range(2):   # block-diagonal products: one launch per gate, the blocks as its batch
            ops.linear(u.data_ptr(), W, self.gates_w[which], bs, self.gates_b[which], gates.data_ptr() + which * T * W * F32B, W, T, bs, bs, step.st,
                       batch=c.blocks, a_bs=bs, w_bs=bs * bs, bias_bs=bs, c_bs=bs)
        tiles = step.b.n_qtiles
        scan_ws = step.scratch("rg_tiles", 4 * tiles * W) if tiles > step.nseg else None      # (P, Q) per tile and channel, doubles
        ops.rglru_scan(step.b, u, W, gates.data_ptr(), gates.data_ptr() + T * W * F32B, W, y, ld, self.lam, self.decay_scale, W, state["S"],
                       x, ld, c.conv, tail, out, W, scan_ws, step.st)


class GatedLinearAttention:
    """Linear attention with a data-dependent decay per key channel: alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau); per head
    S <- diag(alpha) S + k v^T, o = S^T (q / sqrt(dim)); o is RMS-normed per head (weight shared by the heads), gated by silu(W_g h) and
    projected. State per sequence: S [heads][dim][vdim], fp32."""

    def __init__(self, cfg, w, pre, ops, device, eps):
        self.cfg, self.ops, self.eps = cfg, ops, eps
        self.inputs = [(w[pre + "q"], None), (w[pre + "k"], None), (w[pre + "v"], None), (w[pre + "g"], None), (w[pre + "a1"], None)]
        self.a2 = FusedLinear([(w[pre + "a2"], w.get(pre + "a2.b"))], ops, device)
        self.norm_w = w[pre + "norm"].float().contiguous()
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        self.width = cfg.heads * cfg.vdim

    def state_spec(self):
        return {"pages": [], "slots": [("S", (self.cfg.heads, self.cfg.dim, self.cfg.vdim))]}

    def forward(self, step, cols, ld, state, out):
        c, ops, T = self.cfg, self.ops, step.T
        q, k, v, g, a1 = cols
        z = step.scratch("gla_z", T * c.heads * c.dim)
        self.a2(step, a1, ld, z.data_ptr(), c.heads * c.dim)
        o = step.scratch("gla_o", T * self.width)
        tiles = step.b.n_qtiles
        scan_ws = None
        if tiles > step.nseg:                    # a portion longer than one tile: per tile the decay products and the tile's state
            scan_ws = step.scratch("gla_tiles", (tiles * c.heads * c.dim + 63) // 64 * 64 + tiles * c.heads * c.dim * c.vdim)
        ops.gla_scan(step.b, q, ld, k, ld, v, ld, z.data_ptr(), c.heads * c.dim, c.heads, c.dim, c.vdim, c.dim ** -0.5, c.tau, state["S"], o,
                     self.width, scan_ws, step.st)
        ops.headnorm_gate(o.data_ptr(), self.width, g, ld, self.norm_w, c.heads, c.vdim, self.eps, out, self.width, T, step.st)


class LogDistanceWindowAttention:
    """Softmax attention without rotation over a paged cache: score = (q . k) * scale - r1_h * ln(1 + r2_h * distance) with two numbers
    per head (tensors ``r1`` / ``r2``), a sliding window, grouped query heads, and a query temperature: the query at position p is
    multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)."""

    def __init__(self, cfg, w, pre, ops, device):
        self.cfg, self.ops = cfg, ops
        self.inputs = [(w[pre + "q"], w.get(pre + "q.b")), (w[pre + "k"], w.get(pre + "k.b")), (w[pre + "v"], w.get(pre + "v.b"))]
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        self.logdist = torch.stack([w[pre + "r1"].float(), w[pre + "r2"].float()]).contiguous()      # [2][heads]
        self.opts = ops.attention_options(cfg.mask.size, cfg.mask.keep_first, logdist=self.logdist)
        self.width = cfg.heads * cfg.vdim

    def state_spec(self):
        return {"pages": [("k", self.cfg.kv_heads, self.cfg.dim), ("v", self.cfg.kv_heads, self.cfg.vdim)], "slots": []}

    def forward(self, step, cols, ld, state, out):
        c, ops = self.cfg, self.ops
        q, k, v = cols
        # the cache write of the mixers without rotation, with no head divided by anything; it also applies the query temperature
        ops.unit_kv(step.b, q, ld, c.heads, c.dim, k, ld, c.kv_heads, v, ld, c.vdim, 0.0, 0, None, 0, 0.0, state["k"], state["v"], step.st,
                    q_temp_coef=c.q_temp_coef, q_temp_every=c.q_temp_every)
        ws = step.scratch("attn_ws", step.T * c.heads * step.nsplit * (c.vdim + 2))
        ops.attention(step.b, q, ld, c.heads, c.kv_heads, c.dim, c.vdim, c.scale, state["k"], state["v"], step.nsplit, ws, step.st, opts=self.opts)
        ops.attention_finish(step.b, ws, step.nsplit, c.heads, c.vdim, None, 0, None, 0, out, self.width, step.st)


class GatedDeltaRule:
    """Gated delta rule: q, k (``kv_heads`` heads of ``dim``) and v (``heads`` heads of ``vdim``) each pass a short causal convolution
    (tensors ``<name>.conv``, no bias) and silu; q and k become unit vectors per head (q also times dim^-1/2); per head
    S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q with beta = sigmoid(W_b h) and g = exp(-exp(A_log) softplus(W_a h + dt_bias));
    o is RMS-normed per head (weight ``norm`` shared by the heads), gated by silu(W_g h) and projected. State per sequence: S
    [heads][dim][vdim] and the convolution's last taps-1 inputs (a ring indexed by position), fp32."""

    unit_eps = 1e-6

    def __init__(self, cfg, w, pre, ops, device, eps):
        self.cfg, self.ops, self.eps = cfg, ops, eps
        # q, k, v first and adjacent: one convolution runs over all their channels
        self.inputs = [(w[pre + n], None) for n in ("q", "k", "v", "g", "b", "a")]
        self.conv_w = torch.cat([w[pre + n + ".conv"].float() for n in ("q", "k", "v")], dim=0).contiguous()     # [channels][taps]
        self.channels = int(self.conv_w.shape[0])
        if int(self.conv_w.shape[1]) != cfg.conv:
            raise ValueError(f"{pre}q.conv holds {int(self.conv_w.shape[1])} taps, the configuration says {cfg.conv}")
        self.a_log = w[pre + "A_log"].float().contiguous()
        self.dt_bias = w[pre + "dt_bias"].float().contiguous()
        self.norm_w = w[pre + "norm"].float().contiguous()
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        self.width = cfg.heads * cfg.vdim

    def state_spec(self):
        c = self.cfg
        slots = [("S", (c.heads, c.dim, c.vdim))]
        if c.conv > 1:
            slots.append(("ring", (c.conv - 1, self.channels)))
        return {"pages": [], "slots": slots}

    def forward(self, step, cols, ld, state, out):
        c, ops, T, C = self.cfg, self.ops, step.T, self.channels
        q, k, v, g, bl, al = cols
        u = step.scratch("delta_qkv", T * C)
        ring = state.get("ring")
        ops.conv_ring(step.b, q, ld, C, c.conv, self.conv_w, ring, 1, u, C, step.st)
        nk = c.kv_heads * c.dim
        o = step.scratch("delta_o", T * self.width)
        ops.delta_rule(step.b, u.data_ptr(), C, u.data_ptr() + nk * F32B, C, u.data_ptr() + 2 * nk * F32B, C, bl, ld, al, ld, self.a_log, self.dt_bias,
                       c.heads, c.kv_heads, c.dim, c.vdim, self.unit_eps, c.dim ** -0.5, state["S"], o, self.width, q, ld, C, c.conv, ring, step.st)
        ops.headnorm_gate(o.data_ptr(), self.width, g, ld, self.norm_w, c.heads, c.vdim, self.eps, out, self.width, T, step.st)


class StateSpaceDuality:
    """Mamba-2: ONE input product laid out as [z: inner | x: inner | B: groups * state | C: groups * state | dt: heads], inner = heads * vdim;
    x, B and C pass a causal convolution (tensor ``conv`` [channels][taps] with bias ``conv.b``) and silu; per head (head h reads group
    h / (heads / groups)) dt = softplus(dt + dt_bias), S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; y times silu(z), then RMS-normed
    in ``norm_groups`` equal parts times the weight ``norm``, then the output projection. State per sequence: S [heads][state][vdim] and
    the convolution's last taps-1 inputs (a ring indexed by position), fp32."""

    scan_range = 128     # tokens of a range of the kernel's three-pass form (kSsdRange of csrc/seq_delta.cu)

    def __init__(self, cfg, w, pre, ops, device, eps):
        self.cfg, self.ops, self.eps = cfg, ops, eps
        self.inner = cfg.heads * cfg.vdim
        self.channels = self.inner + 2 * cfg.groups * cfg.state
        if int(w[pre + "in"].shape[0]) != self.inner + self.channels + cfg.heads:
            raise ValueError(f"{pre}in has {int(w[pre + 'in'].shape[0])} rows, the configuration asks for {self.inner + self.channels + cfg.heads}")
        self.inputs = [(w[pre + "in"], None)]
        self.conv_w = w[pre + "conv"].float().contiguous()
        if tuple(self.conv_w.shape) != (self.channels, cfg.conv):
            raise ValueError(f"{pre}conv is {tuple(self.conv_w.shape)}, the configuration says {(self.channels, cfg.conv)}")
        self.conv_b = w[pre + "conv.b"].float().contiguous() if pre + "conv.b" in w else None
        self.a_log = w[pre + "A_log"].float().contiguous()
        self.dt_bias = w[pre + "dt_bias"].float().contiguous()
        self.skip = w[pre + "D"].float().contiguous() if pre + "D" in w else None
        self.norm_w = w[pre + "norm"].float().contiguous()
        if self.inner % cfg.norm_groups:
            raise ValueError(f"{self.inner} channels do not divide into {cfg.norm_groups} norm groups")
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        self.width = self.inner

    def state_spec(self):
        c = self.cfg
        slots = [("S", (c.heads, c.state, c.vdim))]
        if c.conv > 1:
            slots.append(("ring", (c.conv - 1, self.channels)))
        return {"pages": [], "slots": slots}

    def forward(self, step, cols, ld, state, out):
        c, ops, T, C, inner = self.cfg, self.ops, step.T, self.channels, self.inner
        z = cols[0]
        xbc, dt = z + inner * F32B, z + (inner + C) * F32B
        u = step.scratch("ssd_xbc", T * C)
        ring = state.get("ring")
        ops.conv_ring(step.b, xbc, ld, C, c.conv, self.conv_w, ring, 1, u, C, step.st, bias=self.conv_b)
        gn = c.groups * c.state
        y = step.scratch("ssd_y", T * inner)
        # a portion longer than a range of the scan: per range and head its end state from zero and its sum of step sizes (three passes)
        scan_ws = None
        if T - step.nseg + 1 > self.scan_range:
            scan_ws = step.scratch("ssd_ranges", (step.b.n_qtiles // 4 + step.nseg + 1) * c.heads * (c.state * c.vdim + 1))
        ops.ssd_scan(step.b, u.data_ptr(), C, u.data_ptr() + inner * F32B, C, u.data_ptr() + (inner + gn) * F32B, C, dt, ld, self.a_log, self.dt_bias,
                     self.skip, c.heads, c.groups, c.state, c.vdim, state["S"], y, inner, xbc, ld, C, c.conv, ring, step.st, scratch=scan_ws)
        rows16 = self.out.operand_rows(step)       # the output projection on the tensor cores reads bf16 rows: write those, and only those
        ops.headnorm_gate(y.data_ptr(), inner, z, ld, self.norm_w, c.norm_groups, inner // c.norm_groups, self.eps, None if rows16 is not None else out, inner,
                          T, step.st, out16=rows16, gate_first=True, wide_weight=True)
        return rows16 is not None


class SelectiveScan:
    """Mamba: the input product is [x: inner | z: inner]; x passes a causal convolution (``conv`` with bias ``conv.b``) and silu; W_x x is
    [dt: dt_rank | B: state | C: state]; dt = softplus(W_dt dt + bias ``dt.b``) per channel; A = -exp(A_log) [inner][state]; per channel c and
    state n: S[c][n] <- exp(dt_c A[c][n]) S[c][n] + dt_c x_c B_n, y_c = sum_n S[c][n] C_n + D_c x_c; y times silu(z), then the output
    projection. State per sequence: S [inner][state] and the convolution's last taps-1 inputs (a ring indexed by position), fp32."""

    scan_range = 128     # tokens of a range of the kernel's three-pass form (kScanRange of csrc/seq_ssm.cu)

    def __init__(self, cfg, w, pre, ops, device):
        self.cfg, self.ops = cfg, ops
        inner = cfg.inner
        if int(w[pre + "in"].shape[0]) != 2 * inner:
            raise ValueError(f"{pre}in has {int(w[pre + 'in'].shape[0])} rows, the configuration asks for {2 * inner}")
        self.inputs = [(w[pre + "in"], None)]
        self.conv_w = w[pre + "conv"].float().contiguous()
        if tuple(self.conv_w.shape) != (inner, cfg.conv):
            raise ValueError(f"{pre}conv is {tuple(self.conv_w.shape)}, the configuration says {(inner, cfg.conv)}")
        self.conv_b = w[pre + "conv.b"].float().contiguous() if pre + "conv.b" in w else None
        self.low = FusedLinear([(w[pre + "x"], None)], ops, device, pad_rows=4)
        if self.low.sizes[0] != cfg.dt_rank + 2 * cfg.state:
            raise ValueError(f"{pre}x has {self.low.sizes[0]} rows, the configuration asks for {cfg.dt_rank + 2 * cfg.state}")
        self.step = FusedLinear([(w[pre + "dt"], w.get(pre + "dt.b"))], ops, device)
        self.a_log = w[pre + "A_log"].float().contiguous()
        self.skip = w[pre + "D"].float().contiguous()
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        self.width = inner

    def state_spec(self):
        c = self.cfg
        slots = [("S", (c.inner, c.state))]
        if c.conv > 1:
            slots.append(("ring", (c.conv - 1, c.inner)))
        return {"pages": [], "slots": slots}

    def forward(self, step, cols, ld, state, out):
        c, ops, T, inner = self.cfg, self.ops, step.T, self.cfg.inner
        x = cols[0]
        z = x + inner * F32B
        u = step.scratch("scan_x", T * inner)
        ring = state.get("ring")
        ops.conv_ring(step.b, x, ld, inner, c.conv, self.conv_w, ring, 1, u, inner, step.st, bias=self.conv_b)
        L = self.low.N
        low = step.scratch("scan_low", T * L)
        self.low(step, u.data_ptr(), inner, low.data_ptr(), L)
        dtl = step.scratch("scan_dt", T * inner)
        self.step(step, low.data_ptr(), L, dtl.data_ptr(), inner)
        rows16 = self.out.operand_rows(step)
        # a portion longer than a range of the scan: per range its end state from zero and its sum of step sizes (three passes)
        scan_ws = step.scratch("scan_ranges", step.b.n_qtiles * inner * (c.state + 1)) if T - step.nseg + 1 > self.scan_range else None
        ops.selective_scan(step.b, u.data_ptr(), inner, dtl.data_ptr(), inner, low.data_ptr() + c.dt_rank * F32B, L,
                           low.data_ptr() + (c.dt_rank + c.state) * F32B, L, z, ld, self.a_log, self.skip, inner, c.state, state["S"],
                           None if rows16 is not None else out, inner, x, ld, c.conv, ring, step.st, out16=rows16, scratch=scan_ws)
        return rows16 is not None


class TalkingHeadsAttention:
    """Softmax attention over a paged cache with grouped query heads in which: q and k pass a short causal convolution per channel (tensors
    ``q.conv`` / ``k.conv``, no bias) directly after their projections; the VALUES are the keys as they leave that convolution (there is
    no value projection); q and k are then RMS-normed per head (weights ``q.norm`` / ``k.norm`` of the head's width) and rotated on their
    first ``rot.dims`` dimensions (pairs 2i, 2i+1); a sliding window keeps the first positions visible; and after the softmax the heads'
    weights are mixed, weight_h <- sum_g talk[h][g] weight_g, head h applying its mixed weights to the values of its own key/value head.
    Computed without ever forming the weights: the attention kernel returns every query head's weights on EVERY key/value head's values
    (``cross_values``), and the mix is taken over those results. State per sequence: the k and v pools, and the convolution's last
    taps-1 inputs (a ring indexed by position)."""

    def __init__(self, cfg, w, pre, ops, device, eps):
        self.cfg, self.ops, self.eps = cfg, ops, eps
        if cfg.vdim != cfg.dim:
            raise ValueError(f"values that are the keys need vdim = dim, not {cfg.vdim} and {cfg.dim}")
        self.inputs = [(w[pre + "q"], w.get(pre + "q.b")), (w[pre + "k"], w.get(pre + "k.b"))]      # adjacent: one convolution runs over both
        self.nq, self.nk = cfg.heads * cfg.dim, cfg.kv_heads * cfg.dim
        self.channels = self.nq + self.nk
        if cfg.conv > 1:
            self.conv_w = torch.cat([w[pre + "q.conv"].float(), w[pre + "k.conv"].float()], dim=0).contiguous()
            if tuple(self.conv_w.shape) != (self.channels, cfg.conv):
                raise ValueError(f"{pre}q.conv / k.conv hold {tuple(self.conv_w.shape)}, the configuration says {(self.channels, cfg.conv)}")
        else:      # one tap: a weight per channel on the current token, or nothing at all
            self.conv_w = (torch.cat([w[pre + "q.conv"].float(), w[pre + "k.conv"].float()], dim=0).contiguous() if pre + "q.conv" in w
                           else torch.ones(self.channels, 1, device=device))
        self.q_norm = w[pre + "q.norm"].float().contiguous() if pre + "q.norm" in w else None
        self.k_norm = w[pre + "k.norm"].float().contiguous() if pre + "k.norm" in w else None
        self.talk = w[pre + "talk"].float().contiguous() if pre + "talk" in w else torch.eye(cfg.heads, device=device)
        if tuple(self.talk.shape) != (cfg.heads, cfg.heads):
            raise ValueError(f"{pre}talk is {tuple(self.talk.shape)} for {cfg.heads} heads")
        self.n_freq = cfg.rot.dims // 2 if cfg.rot is not None else 0
        self.freq = (torch.tensor([cfg.rot.base ** (-2.0 * i / cfg.rot.dims) for i in range(self.n_freq)], dtype=torch.float64, device=device)
                     if self.n_freq else None)
        self.opts = ops.attention_options(cfg.mask.size, cfg.mask.keep_first, cross_values=True)
        self.out = FusedLinear([(w[pre + "o"], w.get(pre + "o.b"))], ops, device)
        self.width = cfg.heads * cfg.vdim

    def state_spec(self):
        c = self.cfg
        slots = [("ring", (c.conv - 1, self.channels))] if c.conv > 1 else []
        return {"pages": [("k", c.kv_heads, c.dim), ("v", c.kv_heads, c.vdim)], "slots": slots}

    def forward(self, step, cols, ld, state, out):
        c, ops, T, C = self.cfg, self.ops, step.T, self.channels
        H, G, dk, dv = c.heads, c.kv_heads, c.dim, c.vdim
        raw = cols[0]
        ring = state.get("ring")
        u = step.scratch("talk_qk", T * C)
        ops.conv_ring(step.b, raw, ld, C, c.conv, self.conv_w, ring, 0, u, C, step.st)
        if ring is not None:
            ops.ring_store(step.b, raw, ld, C, c.conv, ring, step.st)
        q, k = u.data_ptr(), u.data_ptr() + self.nq * F32B
        ops.normed_rotary_kv(step.b, q, C, H, dk, k, C, G, k, C, dv, self.q_norm, self.k_norm, self.eps, self.freq, self.n_freq, 0, state["k"], state["v"],
                             step.st)
        ws = step.scratch("attn_ws", T * H * G * step.nsplit * (dv + 2))
        ops.attention(step.b, q, C, H, G, dk, dv, c.scale, state["k"], state["v"], step.nsplit, ws, step.st, opts=self.opts)
        cross = step.scratch("talk_cross", T * G * H * dv)
        ops.attention_finish(step.b, ws, step.nsplit, G * H, dv, None, 0, None, 0, cross, G * H * dv, step.st)
        rows16 = self.out.operand_rows(step)
        ops.head_mix(cross, G * H * dv, self.talk, H, G, dv, None if rows16 is not None else out, self.width, T, step.st, out16=rows16)
        return rows16 is not None


class MixerGroup:
    """One or more mechanisms reading the same input: their input projections run as one fused product, each mechanism's result goes
    through its own output projection, and the results are added with the given weights."""

    def __init__(self, members, ops, device):
        self.members = members                       # [(name, mechanism, weight)]
        self.ops = ops
        parts = [p for _, m, _ in members for p in m.inputs]
        self.proj = FusedLinear(parts, ops, device, pad_rows=8)
        self.spans, i = [], 0
        for _, m, _ in members:
            self.spans.append(self.proj.offsets[i:i + len(m.inputs)])
            i += len(m.inputs)

    def state_spec(self):
        spec = {"pages": [], "slots": [], "borrow": []}
        for name, m, _ in self.members:
            s = m.state_spec()
            spec["pages"] += [(f"{name}.{n}", g, wd) for n, g, wd in s["pages"]]
            spec["slots"] += [(f"{name}.{n}", shape) for n, shape in s["slots"]]
            # (own name, layer run that owns the memory, its name there): the member of the same name in that layer's group
            spec["borrow"] += [(f"{name}.{n}", run, f"{name}.{src}") for n, run, src in s.get("borrow", [])]
        return spec

    def forward(self, step, h, state, y, h16_ready=False):
        """h [T][d] -> y [T][d]; ``h16_ready``: the kernel that wrote h also left it in ``self.proj.operand_rows(step)``."""
        T, N = step.T, self.proj.N
        cols = step.scratch("mix_cols", T * N)
        self.proj(step, h.data_ptr(), self.proj.K, cols.data_ptr(), N, a16_ready=h16_ready)
        for i, ((name, m, weight), span) in enumerate(zip(self.members, self.spans)):
            part = step.scratch("mix_part", T * m.width)
            sub = {k[len(name) + 1:]: t for k, t in state.items() if k.startswith(name + ".")}
            # a member whose forward says True has left its result as bf16 operand rows of its output projection
            ready = m.forward(step, [cols.data_ptr() + o * F32B for o in span], N, sub, part)
            m.out(step, part.data_ptr(), m.width, y.data_ptr(), m.out.N, alpha=weight, accumulate=i > 0, a16_ready=ready is True)


class ClampedGluFeedForward:
    """Gated feed-forward with clamped branches: g = min(W_gate h + b, limit), u = clamp(W_up h + b, -limit, limit),
    W_down (g * sigmoid(alpha g) * (u + 1)) + b. It has the interface of a mixer (``inputs`` / ``forward`` / ``out``), so that a
    ``MixerGroup`` runs it beside a mixer on the same normed input: one fused input product, results added."""

    alpha = 1.702

    def __init__(self, cfg, w, pre, ops, device):
        self.cfg, self.ops = cfg, ops
        self.inputs = [(w[pre + "gate"], w.get(pre + "gate.b")), (w[pre + "up"], w.get(pre + "up.b"))]
        self.out = FusedLinear([(w[pre + "down"], w.get(pre + "down.b"))], ops, device)
        self.width = cfg.ff

    def state_spec(self):
        return {"pages": [], "slots": []}

    def forward(self, step, cols, ld, state, out):
        gate, up = cols
        rows16 = self.out.operand_rows(step)       # the down projection on the tensor cores reads bf16 rows: write those, and only those
        self.ops.clamped_glu(gate, ld, up, ld, self.cfg.limit, self.alpha, None if rows16 is not None else out, self.width, step.T, self.width, step.st,
                             out16=rows16)
        return rows16 is not None


class PolyNormFeedForward:
    """Dense feed-forward W_down act(W_up h) with act = a N(z) + b N(z^2) + c N(z^3) + e, N = division of a token's vector by its rms."""

    def __init__(self, w, pre, ops, device, eps):
        self.ops, self.eps = ops, eps
        self.up = FusedLinear([(w[pre + "up"], w.get(pre + "up.b"))], ops, device)
        self.down = FusedLinear([(w[pre + "down"], w.get(pre + "down.b"))], ops, device)
        self.coef = w[pre + "act"].float().contiguous()

    def state_spec(self):
        return {"pages": [], "slots": []}

    def forward(self, step, h, state, y):
        T, n = step.T, self.up.N
        z = step.scratch("ff_z", T * n)
        self.up(step, h.data_ptr(), self.up.K, z.data_ptr(), n)
        self.ops.polynorm(z, n, self.coef, self.eps, z, n, T, n, step.st)
        self.down(step, z.data_ptr(), n, y.data_ptr(), self.down.N)


class GatedFeedForward:
    """W_down (silu(W_gate h) * (W_up h)): gate and up as one fused product, the activation leaves the down projection's bf16 operand rows
    when that product runs on the tensor cores."""

    def __init__(self, cfg, w, pre, ops, device):
        self.ops = ops
        self.up = FusedLinear([(w[pre + "gate"], w.get(pre + "gate.b")), (w[pre + "up"], w.get(pre + "up.b"))], ops, device, pad_rows=8)
        self.down = FusedLinear([(w[pre + "down"], w.get(pre + "down.b"))], ops, device)
        self.ff = cfg.ff

    @property
    def proj(self):
        return self.up

    def forward(self, step, h, y, h16_ready=False):
        T, n = step.T, self.ff
        N = self.up.N                              # 2 * ff, rounded up
        z = step.scratch("ff_z", T * N)
        self.up(step, h.data_ptr(), self.up.K, z.data_ptr(), N, a16_ready=h16_ready)
        rows16 = self.down.operand_rows(step)
        act = step.scratch("ff_act", T * n)        # fp32 rows; not written when the product reads the bf16 rows
        self.ops.gated_act(z.data_ptr(), N, z.data_ptr() + n * F32B, N, None if rows16 is not None else act, n, T, n, step.st, out16=rows16)
        self.down(step, act.data_ptr(), n, y.data_ptr(), self.down.N, a16_ready=rows16 is not None)


class BiasedFeedForward:
    """W_down act(W_up h + b_up) + b_down with act one of the framework's activations (0 = the exact, erf, gelu)."""

    def __init__(self, cfg, w, pre, ops, device, activation=0):
        self.ops, self.activation = ops, activation
        self.up = FusedLinear([(w[pre + "up"], w.get(pre + "up.b"))], ops, device)
        self.down = FusedLinear([(w[pre + "down"], w.get(pre + "down.b"))], ops, device)
        if self.up.N != cfg.ff:
            raise ValueError(f"{pre}up has {self.up.N} rows, the configuration says {cfg.ff}")

    @property
    def proj(self):
        return self.up

    def forward(self, step, h, y, h16_ready=False):
        T, n = step.T, self.up.N
        z = step.scratch("ff_z", T * n)
        self.up(step, h.data_ptr(), self.up.K, z.data_ptr(), n, a16_ready=h16_ready)
        self.ops.act(z.data_ptr(), T * n, self.activation, step.st)
        self.down(step, z.data_ptr(), n, y.data_ptr(), self.down.N)


class ExpertsFeedForward:
    """Mixture of experts W_down,e act(W_up,e h) (tensors ``e<i>.up`` / ``e<i>.down``, no biases): router logits W_router h in fp32,
    scores = softmax over ALL router outputs, the ``top`` largest (score + ``correction``) are chosen, the weights are the chosen scores
    themselves; the last ``identity`` router outputs are experts whose output is h. Computed as two wide products: every expert's up
    projection (and the router) side by side, the activation times the token's weight for that expert (zero if not chosen), and ONE down
    product over the concatenated experts, added to (sum of the chosen identity scores) * h.

    Steps of ``gather_min_tokens`` tokens and more (portions of prompts) take the gathered form instead, which multiplies a token only
    with the experts it uses: the router alone, then a routing kernel that copies every token's input into a buffer per chosen expert,
    per expert an up product, the activation, a down product over the rows in use (their count never leaves the device), and a kernel
    that adds each token's rows times their scores. Steps of one or two tokens (decoding) whose experts are large take the indexed
    form: the router, a routing kernel, and ONE up and ONE down launch in which every (token, choice) pair streams only its own expert's
    matrix, chosen on the device. All forms give the same numbers up to where the score is multiplied in."""

    activation = 0          # the exact (erf) gelu
    GATED, SCALE_INPUT, SIGMOID = 4, 8, 16      # SLLM_MOE_* bits beside the activation
    # The gathered form trades arithmetic for launches (two products per expert): it is taken when the products it saves, at the rate the
    # tensor-core product sustains, outweigh what its launches cost (both measured on B200: small experts are faster computed densely).
    gather_min_tokens = 256
    gather_launch_cost = 35e-6     # seconds per expert product
    gather_product_rate = 7e14     # multiply-adds * 2 per second
    # The indexed form reads (pairs / experts) of the expert bytes at the price of three more launches per layer
    index_launch_cost = 12e-6      # seconds for the three extra launches of a step replayed as a graph
    index_stream_rate = 5e12       # bytes per second the weight-streaming body sustains

    def __init__(self, cfg, w, pre, ops, device, activation=None, gated=False, sigmoid_scores=False, scale_input=False):
        """``gated``: experts W_down (act(W_gate h) * (W_up h)) with tensors ``e<i>.gate`` beside ``up`` / ``down``; ``sigmoid_scores``: the score
        of a router output is its own sigmoid (no softmax over all); ``scale_input``: the score multiplies what the expert reads."""
        self.cfg, self.ops = cfg, ops
        E = cfg.experts
        self.gated, self.scale_input = bool(gated), bool(scale_input)
        act = self.activation if activation is None else activation
        self.mode = act | (self.GATED if gated else 0) | (self.SCALE_INPUT if scale_input else 0) | (self.SIGMOID if sigmoid_scores else 0)
        self.ff_up = (2 if gated else 1) * cfg.ff          # columns of one expert's first product: [gate | up] or up
        self.n_route = E + cfg.identity
        if int(w[pre + "router"].shape[0]) != self.n_route:
            raise ValueError(f"{pre}router has {int(w[pre + 'router'].shape[0])} outputs, the configuration names {self.n_route} experts")
        self.correction = w[pre + "correction"].float().contiguous() if pre + "correction" in w else None
        # experts first, router last: the experts' columns then start at a 16-byte boundary for every ff
        first = [torch.cat([w[f"{pre}e{e}.gate"], w[f"{pre}e{e}.up"]], dim=0) if gated else w[f"{pre}e{e}.up"] for e in range(E)]
        self.up = FusedLinear([(m, None) for m in first] + [(w[pre + "router"], None)], ops, device, pad_rows=8)
        self.down = FusedLinear([(torch.cat([w[f"{pre}e{e}.down"] for e in range(E)], dim=1).contiguous(), None)], ops, device)
        self.wide = E * cfg.ff                     # columns of the activation = rows of the concatenated down matrices
        self.wide_up = E * self.ff_up              # columns of all experts' first products; the router's follow
        # the gathered form: the router as a product of its own, the down matrices one behind the other [E][d][ff]
        self.gathers = cfg.top < self.n_route and E > 0
        if self.gathers:
            self.router = FusedLinear([(w[pre + "router"], None)], ops, device, pad_rows=64)    # wide enough for the tensor-core tiles
            self.down_each = torch.stack([w[f"{pre}e{e}.down"] for e in range(E)]).contiguous()

    @property
    def proj(self):
        return self.up

    def _forward_gathered(self, step, h, y, h16_ready=False):
        c, ops, T, d, st = self.cfg, self.ops, step.T, self.up.K, step.st
        E, top, ff, cap, fu = c.experts, c.top, c.ff, step.T, self.ff_up
        ldl = self.router.N
        logits = step.scratch("moe_logits", T * ldl)
        self.router(step, h.data_ptr(), d, logits.data_ptr(), ldl, a16_ready=h16_ready)     # the bf16 rows left for the up product serve this one
        # counts [E] | expert, row [T][top] each (int32) | score [T][top] | identity sum [T]
        book = step.scratch("moe_book", E + 3 * T * top + T).data_ptr()
        counts, sel_e, sel_pos, sel_w, ident = book, book + 4 * E, book + 4 * (E + T * top), book + 4 * (E + 2 * T * top), book + 4 * (E + 3 * T * top)
        # operands of the tensor-core products are gathered as bf16 rows; shapes its tiles do not take (and the fp32 mode) gather fp32 rows
        tc = (step.gemm_scratch(d, fu) is not None and ops.on_tensor_cores(cap, fu, d) and ops.on_tensor_cores(cap, d, ff)
              and self.up.w.data_ptr() % 16 == 0 and self.down_each.data_ptr() % 16 == 0)
        per = 2 if tc else 1                       # operand elements per float of scratch
        rows = step.scratch("moe_rows", -(-E * cap * d // per)).data_ptr()
        up_out = step.scratch("moe_up", E * cap * fu).data_ptr()
        act = step.scratch("moe_act", -(-E * cap * ff // per)).data_ptr()
        down_out = step.scratch("moe_down", E * cap * d).data_ptr()
        ops.zero(counts, 4 * E, st)
        ops.moe_route(logits.data_ptr(), ldl, self.n_route, E, top, self.correction, h, d, d, counts, cap, sel_e, sel_pos, sel_w, ident,
                      rows if tc else None, None if tc else rows, T, st, mode=self.mode)
        wb = self.up.w.element_size()
        for e in range(E):
            a = rows + e * cap * d * (2 if tc else 4)
            ops.linear(a, d, self.up.w, d, None, up_out + 4 * e * cap * fu, fu, cap, fu, d, st, scratch=a if tc else None, a16_ready=tc, rows_dev=counts + 4 * e,
                       w_ptr=self.up.w.data_ptr() + e * fu * d * wb)
        ops.moe_expert_act(up_out, counts, E, cap, ff, self.mode, act if tc else None, None if tc else act, st)
        for e in range(E):
            a = act + e * cap * ff * (2 if tc else 4)
            ops.linear(a, ff, self.down_each, ff, None, down_out + 4 * e * cap * d, d, cap, d, ff, st, scratch=a if tc else None, a16_ready=tc,
                       rows_dev=counts + 4 * e, w_ptr=self.down_each.data_ptr() + e * d * ff * wb)
        ops.moe_combine(down_out, sel_e, sel_pos, sel_w, top, ident, h, d, cap, d, y, d, T, st)

    def _gathered_pays(self, T: int) -> bool:
        c = self.cfg
        saved = 2.0 * T * (c.ff + self.ff_up) * self.up.K * (c.experts - min(c.top, c.experts)) / self.gather_product_rate
        return self.gathers and T >= self.gather_min_tokens and saved > 2 * c.experts * self.gather_launch_cost

    def _indexed_pays(self, T: int) -> bool:
        c = self.cfg
        pairs = T * c.top
        saved = (c.experts - pairs) * float(c.ff + self.ff_up) * self.up.K * self.up.w.element_size() / self.index_stream_rate
        return self.gathers and T <= 8 and pairs < c.experts and saved > self.index_launch_cost

    def _forward_indexed(self, step, h, y):
        c, ops, T, d, st = self.cfg, self.ops, step.T, self.up.K, step.st
        E, top, ff, fu = c.experts, c.top, c.ff, self.ff_up
        pairs, ldl = T * top, self.router.N
        logits = step.scratch("moe_logits", T * ldl)
        self.router(step, h.data_ptr(), d, logits.data_ptr(), ldl)
        book = step.scratch("moe_book", E + 3 * pairs + T).data_ptr()       # as in the gathered form; the counters stay unused
        sel_e, sel_pos, sel_w, ident = book + 4 * E, book + 4 * (E + pairs), book + 4 * (E + 2 * pairs), book + 4 * (E + 3 * pairs)
        # the products read the token's row as it is; a score on the expert's input is applied to their results (they are linear), so the
        # routing kernel is asked for the plain scores
        ops.moe_route(logits.data_ptr(), ldl, self.n_route, E, top, self.correction, h, d, d, None, T, sel_e, sel_pos, sel_w, ident, None, None, T, st,
                      mode=self.mode & ~self.SCALE_INPUT)
        up_out = step.scratch("moe_up", pairs * fu).data_ptr()
        down_out = step.scratch("moe_down", pairs * d).data_ptr()
        ops.linear_indexed(h.data_ptr(), d, d, top, self.up.w, d, fu * d, sel_e, up_out, fu, fu, pairs, fu, d, st)
        if self.gated or self.scale_input:
            act = step.scratch("moe_act", pairs * ff).data_ptr()
            weights = step.scratch("moe_pair_w", pairs).data_ptr()
            ops.moe_pair_act(up_out, sel_w, pairs, ff, self.mode, act, weights, st)
        else:
            ops.act(up_out, pairs * ff, self.mode & 3, st)
            act, weights = up_out, sel_w
        ops.linear_indexed(act, ff, ff, 1, self.down_each, ff, d * ff, sel_e, down_out, d, d, pairs, d, ff, st)
        # row (t, k) of down_out is pair t * top + k: the combine kernel's (expert, row) address with buffers of 0 rows
        ops.moe_combine(down_out, sel_e, sel_pos, weights, top, ident, h, d, 0, d, y, d, T, st)

    def forward(self, step, h, y, h16_ready=False):
        if self._gathered_pays(step.T):
            return self._forward_gathered(step, h, y, h16_ready)
        if self._indexed_pays(step.T):
            return self._forward_indexed(step, h, y)
        c, T, d, N = self.cfg, step.T, self.up.K, self.up.N
        z = step.scratch("ff_z", T * N)
        self.up(step, h.data_ptr(), d, z.data_ptr(), N, a16_ready=h16_ready)
        rows16 = self.down.operand_rows(step)
        act = step.scratch("ff_act", T * self.wide)   # fp32 rows; not written when the product reads the bf16 rows
        self.ops.moe_act(z.data_ptr() + self.wide_up * F32B, N, self.n_route, c.experts, c.top, self.correction, z.data_ptr(), N, c.ff, self.mode,
                         h, d, d, None if rows16 is not None else act, rows16, y, d, T, step.st)
        self.down(step, act.data_ptr(), self.wide, y.data_ptr(), d, accumulate=True, a16_ready=rows16 is not None)
