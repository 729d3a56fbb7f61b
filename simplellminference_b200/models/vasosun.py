"""Vasosun: a decoder-only model whose sublayers each sit between two RMS norms with ONE number as weight, x <- x + norm_b(f(norm_a(x))),
and read their input through a short causal convolution over time (h + conv(h), per channel). The embedding adds a hashed table indexed
by the (previous token, token) pair. Mixers: window attention without rotation (a charge on the logarithm of the distance, a query
temperature), latent attention (queries through a latent, YaRN-scaled rotation, optionally over an earlier layer's cached rows) and the
gated delta rule; feed-forwards: gated (silu) or a mixture of experts with identity experts. The logits are capped by a tanh.

The class only DESCRIBES the model with the mechanisms of ``layers``; cache, state slots, batching and the step loop belong to
``seqengine.SequenceEngine``. Tensor names: ``embed``, ``bigram``, ``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b``,
``l<i>.canon1`` / ``canon2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``."""
from __future__ import annotations

from ..config import ExpertsConfig
from ..layers import ExpertsFeedForward, FusedLinear, GatedDeltaRule, GatedFeedForward, LatentAttention, LogDistanceWindowAttention, MixerGroup


class _Sublayer:
    """f between its two norms: ``pre_g`` / ``post_g`` are the norms' weights, ``conv_w`` [width][taps] the input convolution."""

    def __init__(self, name, body, pre_g, post_g, conv_w):
        self.name, self.body, self.pre_g, self.post_g, self.conv_w = name, body, pre_g, post_g, conv_w


class VasosunModel:
    def __init__(self, cfg, w, ops, device):
        self.cfg, self.ops, self.device = cfg, ops, device
        self.vocab, self.width, self.taps = cfg.vocab, cfg.width, cfg.conv_taps
        self.embed = w["embed"].contiguous()
        self.pairs = w["bigram"].contiguous() if cfg.pair_buckets else None
        if self.pairs is not None and int(self.pairs.shape[0]) != cfg.pair_buckets + 1:
            raise ValueError(f"bigram holds {int(self.pairs.shape[0])} rows, {cfg.pair_buckets} buckets need one more")
        self.final_g = float(w["final.norm"].float().item())
        self.head = FusedLinear([(w["head"], None)], ops, device)
        scalar = lambda n: float(w[n].float().item())   # noqa: E731
        self.layers = []          # per layer: its sublayers in order
        for i, lc in enumerate(cfg.layers):
            pre = f"l{i}."
            if lc.type == "attention":
                mixer = LogDistanceWindowAttention(lc.mixer, w, pre + "mix.", ops, device)
            elif lc.type == "latent_attention":
                mixer = LatentAttention(lc.mixer, w, pre + "mix.", ops, device, cfg.norm_eps)
            else:
                mixer = GatedDeltaRule(lc.mixer, w, pre + "mix.", ops, device, cfg.norm_eps)
            subs = [_Sublayer("mix", MixerGroup([("mix", mixer, 1.0)], ops, device), scalar(pre + "norm1"), scalar(pre + "norm1b"), self._conv(w, pre + "canon1"))]
            if lc.mlp is not None:
                ff = (ExpertsFeedForward if isinstance(lc.mlp, ExpertsConfig) else GatedFeedForward)(lc.mlp, w, pre + "mlp.", ops, device)
                subs.append(_Sublayer("ff", ff, scalar(pre + "norm2"), scalar(pre + "norm2b"), self._conv(w, pre + "canon2")))
            self.layers.append(subs)

    def _conv(self, w, name):
        cw = w[name].float().contiguous()
        if tuple(cw.shape) != (self.width, self.taps):
            raise ValueError(f"{name} is {tuple(cw.shape)}, the configuration says {(self.width, self.taps)}")
        return cw

    def state_specs(self):
        """One entry per layer: what its mixer declares, plus one ring of the last taps-1 normed inputs per sublayer."""
        specs = []
        for subs in self.layers:
            spec = subs[0].body.state_spec()
            if self.taps > 1:
                spec["slots"] = spec["slots"] + [(f"canon.{s.name}", (self.taps - 1, self.width)) for s in subs]
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
        if self.pairs is not None:
            ops.embed_pair(ids, step.prev_ids, self.embed, self.pairs, self.vocab, d, c.pair_buckets, c.pair_mul_prev, c.pair_mul_cur, xa, T, step.st)
        else:
            ops.embed(ids, self.embed, self.vocab, d, 1, xa, T, step.st)
        chain = [(i, sub) for i, subs in enumerate(self.layers) for sub in subs]
        prev, prev_ring = None, None            # the sublayer whose output waits in y, and its ring (the stash holds its last normed rows)
        for k, (i, sub) in enumerate(chain):
            ring = states[i].get(f"canon.{sub.name}")
            h16 = sub.body.proj.operand_rows(step)
            first_of_layer = sub.name == "mix"
            if tap is not None and prev is not None and first_of_layer:
                # inspection of the stream after a layer: the residual sum alone, then the next sublayer's norm and convolution
                ops.seam(step.b, xa, d, step.st, x_out=xb, y=y, post_g=prev.post_g, eps=c.norm_eps)
                xa, xb = xb, xa
                tap(i - 1, xa[:T * d].view(T, d))
                prev = None
            ops.seam(step.b, xa, d, step.st, x_out=xb if prev is not None else None, y=y if prev is not None else None,
                     post_g=prev.post_g if prev is not None else 1.0, pre_g=sub.pre_g, eps=c.norm_eps, conv_w=sub.conv_w, taps=self.taps, ring=ring, h=h,
                     h16=h16, stash=stash, flush_ring=prev_ring, flush_taps=self.taps if prev_ring is not None else 0, scales=scales)
            if prev is not None:
                xa, xb = xb, xa
            if sub.name == "mix":
                sub.body.forward(step, h, states[i], y, h16_ready=h16 is not None)
            else:
                sub.body.forward(step, h, y, h16_ready=h16 is not None)
            prev, prev_ring = sub, ring
        # the last residual sum, the model's norm, and the last ring's flush
        ops.seam(step.b, xa, d, step.st, x_out=xb, y=y, post_g=prev.post_g, pre_g=self.final_g, eps=c.norm_eps, h=h, stash=stash, flush_ring=prev_ring,
                 flush_taps=self.taps if prev_ring is not None else 0)
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
        if c.logit_softcap > 0.0:
            ops.softcap(logits, n_rows * self.vocab, c.logit_softcap, step.st)
        return logits[:n_rows * self.vocab].view(n_rows, self.vocab)
