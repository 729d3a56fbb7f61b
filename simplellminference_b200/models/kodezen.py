"""Kodezen: a decoder-only model of pre-norm layers, x <- x + mixer(norm1(x)), then x <- x + ff(norm2(x)), whose RMS norms carry a weight
per channel stored as its distance from one and whose mixers read their normed input through a short causal convolution over time
(h + conv(h), per channel). The embedding is scaled by a constant. Mixers: Mamba-2 (state-space duality), Mamba (selective scan), and
softmax attention with convolved, normed, partly rotated queries and keys, the keys as values, a sliding window that keeps the first
positions and heads mixed after the softmax; feed-forwards: dense with biases and the exact gelu, or a mixture of gated (silu) experts
whose sigmoid scores multiply what the experts read.

The class only DESCRIBES the model with the mechanisms of ``layers``; cache, state slots, batching and the step loop belong to
``seqengine.SequenceEngine``. Tensor names: ``embed``, ``l<i>.norm1`` / ``norm2``, ``l<i>.canon1``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``."""
from __future__ import annotations

from ..config import ExpertsConfig
from ..layers import BiasedFeedForward, ExpertsFeedForward, FusedLinear, MixerGroup, SelectiveScan, StateSpaceDuality, TalkingHeadsAttention

SILU = 2          # activation numbers of the feed-forward kernels: 0 exact gelu, 1 tanh gelu, 2 silu
NORM_OFFSET = 1.0   # a norm's weight is stored as its distance from this


class _Layer:
    def __init__(self, mixer, ff, norm1, norm2, conv_w):
        self.mixer, self.ff, self.norm1, self.norm2, self.conv_w = mixer, ff, norm1, norm2, conv_w


class KodezenModel:
    def __init__(self, cfg, w, ops, device):
        self.cfg, self.ops, self.device = cfg, ops, device
        self.vocab, self.width, self.taps = cfg.vocab, cfg.width, cfg.conv_taps
        self.embed = w["embed"].contiguous()
        self.final_w = self._vector(w, "final.norm")
        self.head = FusedLinear([(w["head"], None)], ops, device)
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            pre = f"l{i}."
            if lc.type == "mamba2":
                mixer = StateSpaceDuality(lc.mixer, w, pre + "mix.", ops, device, cfg.norm_eps)
            elif lc.type == "mamba1":
                mixer = SelectiveScan(lc.mixer, w, pre + "mix.", ops, device)
            else:
                mixer = TalkingHeadsAttention(lc.mixer, w, pre + "mix.", ops, device, cfg.norm_eps)
            ff = None
            if isinstance(lc.mlp, ExpertsConfig):
                ff = ExpertsFeedForward(lc.mlp, w, pre + "mlp.", ops, device, activation=SILU, gated=True, sigmoid_scores=True, scale_input=True)
            elif lc.mlp is not None:
                ff = BiasedFeedForward(lc.mlp, w, pre + "mlp.", ops, device)
            conv_w = None
            if pre + "canon1" in w:
                conv_w = w[pre + "canon1"].float().contiguous()
                if tuple(conv_w.shape) != (self.width, self.taps):
                    raise ValueError(f"{pre}canon1 is {tuple(conv_w.shape)}, the configuration says {(self.width, self.taps)}")
            self.layers.append(_Layer(MixerGroup([("mix", mixer, 1.0)], ops, device), ff, self._vector(w, pre + "norm1"),
                                      self._vector(w, pre + "norm2") if ff is not None else None, conv_w))

    def _vector(self, w, name):
        v = w[name].float().contiguous()
        if tuple(v.shape) != (self.width,):
            raise ValueError(f"{name} is {tuple(v.shape)}, the model is {self.width} wide")
        return v

    def state_specs(self):
        """One entry per layer: what its mixer declares, plus the ring of the last taps-1 normed inputs of the mixer."""
        specs = []
        for layer in self.layers:
            spec = layer.mixer.state_spec()
            if self.taps > 1:
                spec["slots"] = spec["slots"] + [("canon", (self.taps - 1, self.width))]
            specs.append(spec)
        return specs

    def forward(self, step, ids, states, rows, n_rows, tap=None):
        """The step's tokens through every layer; returns logits [n_rows][vocab] (fp32) of the batch rows listed in ``rows``."""
        ops, c, T, d = self.ops, self.cfg, step.T, self.width
        xa, xb = step.scratch("stream_a", T * d), step.scratch("stream_b", T * d)      # the residual sum goes from one to the other
        h = step.scratch("normed", T * d)
        y = step.scratch("sub_out", T * d)
        stash = step.scratch("conv_stash", T * d) if self.taps > 1 else None
        scales = step.scratch("seam_scales", T)
        ops.embed(ids, self.embed, self.vocab, d, 1, xa, T, step.st, scale=c.embedding_scale)
        # every seam adds the sublayer result that waits in y (none before the first), norms for the next sublayer and, in front of a
        # mixer, runs the input convolution; the ring a seam read is written by the seam after it
        pending, flush = False, None
        for i, layer in enumerate(self.layers):
            ring = states[i].get("canon")
            if tap is not None and pending:
                ops.seam(step.b, xa, d, step.st, x_out=xb, y=y, post_norm=False)
                xa, xb = xb, xa
                tap(i - 1, xa[:T * d].view(T, d))
                pending = False
            h16 = layer.mixer.proj.operand_rows(step)
            ops.seam(step.b, xa, d, step.st, x_out=xb if pending else None, y=y if pending else None, post_norm=False, pre_g=1.0, eps=c.norm_eps,
                     pre_w=layer.norm1, pre_w_offset=NORM_OFFSET, conv_w=layer.conv_w, taps=self.taps, ring=ring, h=h, h16=h16, stash=stash,
                     flush_ring=flush, flush_taps=self.taps if flush is not None else 0, scales=scales)
            if pending:
                xa, xb = xb, xa
            layer.mixer.forward(step, h, states[i], y, h16_ready=h16 is not None)
            pending, flush = True, ring
            if layer.ff is not None:
                h16 = layer.ff.proj.operand_rows(step)
                ops.seam(step.b, xa, d, step.st, x_out=xb, y=y, post_norm=False, pre_g=1.0, eps=c.norm_eps, pre_w=layer.norm2, pre_w_offset=NORM_OFFSET,
                         h=h, h16=h16, stash=stash, flush_ring=flush, flush_taps=self.taps if flush is not None else 0)
                xa, xb = xb, xa
                layer.ff.forward(step, h, y, h16_ready=h16 is not None)
                flush = None
        # the last residual sum, the model's norm, and the flush of a ring that still waits
        ops.seam(step.b, xa, d, step.st, x_out=xb, y=y, post_norm=False, pre_g=1.0, eps=c.norm_eps, pre_w=self.final_w, pre_w_offset=NORM_OFFSET, h=h,
                 stash=stash, flush_ring=flush, flush_taps=self.taps if flush is not None else 0)
        if tap is not None:
            tap(len(self.layers) - 1, xb[:T * d].view(T, d))
        if n_rows == 0:
            return None
        picked = step.scratch("picked", n_rows * d)
        ops.gather_rows(h, d, rows, n_rows, d, picked, step.st)
        logits = step.scratch("logits", n_rows * self.vocab)
        T_save = step.T
        step.T = n_rows               # the head runs over the picked rows only
        try:
            self.head(step, picked.data_ptr(), d, logits.data_ptr(), self.vocab)
        finally:
            step.T = T_save
        return logits[:n_rows * self.vocab].view(n_rows, self.vocab)
