"""Model-shape presets (reference: include/model/config.h:5-17 hard-codes ONE shape; BASELINE.json names five)."""
from __future__ import annotations

from dataclasses import dataclass, asdict

F32, BF16, INT8 = 0, 1, 2
DTYPE_NAMES = {F32: "f32", BF16: "bf16", INT8: "int8"}


@dataclass(frozen=True)
class ModelShape:
    """Field-for-field the reference's model::LlamaModelConfig."""

    vocab: int
    head_dim: int
    hidden: int
    kv_hidden: int
    inter: int
    max_len: int
    layers: int
    heads: int
    kv_heads: int
    eps: float = 1e-5
    theta: float = 10000.0

    def __post_init__(self):
        if self.heads * self.head_dim != self.hidden:
            raise ValueError("heads*head_dim must equal hidden (the reference's wq/wo are d x d, model.cpp:372-378)")
        if self.kv_heads * self.head_dim != self.kv_hidden or self.heads % self.kv_heads:
            raise ValueError("inconsistent kv dims")

    def n_params(self) -> int:
        d, kv, I, L, V = self.hidden, self.kv_hidden, self.inter, self.layers, self.vocab
        return V * d + (2 * L + 1) * d + L * (2 * d * d + 2 * kv * d + 3 * I * d)

    def step_bytes(self, pos: int, w_dtype: int = BF16, kv_dtype: int = BF16, group: int = 64) -> float:
        """Algorithmic HBM bytes of one decode step at position `pos`."""
        bw = {F32: 4.0, BF16: 2.0, INT8: 1.0 + 4.0 / group}[w_dtype]
        bkv = 4.0 if kv_dtype == F32 else 2.0
        d, kv, I, L, V = self.hidden, self.kv_hidden, self.inter, self.layers, self.vocab
        return (bw * (V * d + L * (2 * d * d + 2 * kv * d + 3 * I * d)) + 4.0 * (2 * L + 1) * d + bw * d
                + bkv * 2 * L * kv * (pos + 1) + bkv * 2 * L * kv)

    def as_dict(self):
        return asdict(self)


# BASELINE.json configs (shapes only; weights are random-init)
PRESETS = {
    "stories15M": ModelShape(32000, 48, 288, 288, 768, 256, 6, 6, 6),
    "stories110M": ModelShape(32000, 64, 768, 768, 2048, 1024, 12, 12, 12),
    "tinyllama-1.1b": ModelShape(32000, 64, 2048, 256, 5632, 2048, 22, 32, 4),
    "llama2-7b": ModelShape(32000, 128, 4096, 4096, 11008, 4096, 32, 32, 32),
    # +8 positions of slack: the reference's GQA RoPE over-run limits the parity domain to pos <= S - H/KVH
    "llama3-8b": ModelShape(128256, 128, 4096, 1024, 14336, 8192 + 8, 32, 32, 8, theta=500000.0),
    # small shapes for tests
    "tiny_gqa": ModelShape(512, 32, 128, 64, 384, 48, 3, 4, 2),
    "tiny_mha_hd48": ModelShape(300, 48, 96, 96, 200, 40, 2, 2, 2),
}


# ---------------------------------------------------------------------------------------------------------------------------
# Models described by a config.json (a folder with config.json + model.safetensors). `architecture` selects the reader here and the
# model class in simplellminference_b200.models; the Llama shapes above stay what the C engine takes.
# ---------------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RotaryConfig:
    """Rotary positions on the first ``dims`` dimensions of a head; ``scaling`` = YaRN-style (factor, original, fast, slow) or None."""
    dims: int
    base: float
    scaling: dict | None = None


@dataclass(frozen=True)
class SoftmaxMixerConfig:
    heads: int
    kv_heads: int
    dim: int          # per-head query / key width
    vdim: int         # per-head value width
    scale: float
    rot: RotaryConfig


@dataclass(frozen=True)
class RecurrentMixerConfig:
    width: int
    blocks: int
    conv: int         # taps of the causal convolution


@dataclass(frozen=True)
class LinearAttentionMixerConfig:
    heads: int
    dim: int
    vdim: int
    tau: float


@dataclass(frozen=True)
class MunazenLayerConfig:
    type: str                                   # "parallel" | "gla"
    left: SoftmaxMixerConfig | None = None      # parallel
    right: RecurrentMixerConfig | None = None   # parallel
    left_scale: float = 1.0
    right_scale: float = 1.0
    gla: LinearAttentionMixerConfig | None = None
    ff: int | None = None                       # width of the dense feed-forward, None = the layer has none


@dataclass(frozen=True)
class MunazenConfig:
    """The Munazen design: every size and every constant that may differ between its models comes from config.json."""
    architecture: str
    vocab: int
    width: int
    streams: int
    norm_eps: float
    norm_groups: int
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    @staticmethod
    def from_dict(c: dict) -> "MunazenConfig":
        layers = []
        for i, l in enumerate(c["layers"]):
            m, mlp = l["mixer"], l.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
            ff = int(mlp["ff"]) if mlp is not None else None
            if l["type"] == "parallel":
                a, r = m["left"], m["right"]
                rot = a["rot"]
                layers.append(MunazenLayerConfig(
                    "parallel",
                    left=SoftmaxMixerConfig(int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"]), float(a["scale"]),
                                            RotaryConfig(int(rot["dims"]), float(rot["base"]), rot.get("scaling") or None)),
                    right=RecurrentMixerConfig(int(r["width"]), int(r["blocks"]), int(r["conv"])),
                    left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]), ff=ff))
            elif l["type"] == "gla":
                layers.append(MunazenLayerConfig("gla", gla=LinearAttentionMixerConfig(int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])),
                                                 ff=ff))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
        loop = c.get("loop") or {}
        start, stop, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
        if not (0 <= start <= stop <= len(layers)) or times < 1:
            raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        norm = c.get("norm") or {}
        return MunazenConfig(c["architecture"], int(c["vocab"]), int(c["width"]), int(c.get("streams", 1)), float(norm.get("eps", 1e-6)),
                             int(norm.get("groups", 1)), tuple(layers), start, stop, times)

    def layer_runs(self) -> list:
        """Layer indices in the order they run: the looped range repeats with the same weights (each pass has its own state)."""
        return (list(range(self.loop_start)) + list(range(self.loop_start, self.loop_stop)) * self.loop_times
                + list(range(self.loop_stop, len(self.layers))))


@dataclass(frozen=True)
class WindowMask:
    """Which earlier positions a query sees: ``size`` None = all of them; else the last ``size`` (itself included) and, whatever the
    distance, the first ``keep_first`` positions of the sequence."""
    size: int | None = None
    keep_first: int = 0

    @staticmethod
    def from_dict(m: dict | None) -> "WindowMask":
        m = m or {}
        size = m.get("size")
        return WindowMask(int(size) if size else None, int(m.get("keep_first") or 0))


@dataclass(frozen=True)
class CappedAttentionConfig:
    """Softmax attention without rotation: unit-rms heads, capped scores, a slope per head on the distance, a window that keeps the first
    positions, values optionally blended with those of the first such layer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float          # 0 = no cap
    mask: WindowMask
    v_mix: bool


@dataclass(frozen=True)
class LatentAttentionConfig:
    """Attention whose keys and values are expanded from one cached latent vector per token (``kv_rank``) plus one rotated key part
    (``rot_dim``) shared by the heads; ``dim`` is the unrotated query / key width of a head."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    mask: WindowMask
    q_rank: int | None = None      # queries go through a normed latent of this width (None: one query projection)
    kv_from: int | None = None     # the layer whose cached rows this one attends over (None: its own)


@dataclass(frozen=True)
class ClampedGluConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class SopetarLayerConfig:
    type: str                                    # "attention" | "latent_attention"
    mixer: object                                # CappedAttentionConfig | LatentAttentionConfig
    mlp: ClampedGluConfig | None = None          # None = the layer has no feed-forward


@dataclass(frozen=True)
class SopetarConfig:
    """The Sopetar design: parallel layers (one layer norm feeds the mixer and the feed-forward), a depth-weighted average of all earlier
    layers' results between layers. Every size and every constant that may differ between its models comes from config.json."""
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple

    @staticmethod
    def from_dict(c: dict) -> "SopetarConfig":
        layers = []
        for i, l in enumerate(c["layers"]):
            m, mlp = l["mixer"], l.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
                ff = ClampedGluConfig(int(mlp["ff"]), float(mlp["limit"]))
            mask = WindowMask.from_dict(m.get("mask"))
            if l["type"] == "attention":
                heads = int(m["heads"])
                kv_heads = int(m.get("kv_heads") or heads)
                if heads % kv_heads:
                    raise ValueError(f"layer {i}: {heads} query heads do not divide over {kv_heads} key/value heads")
                mixer = CappedAttentionConfig(heads, kv_heads, int(m["dim"]), int(m["vdim"]), float(m["scale"]), float(m.get("softcap") or 0.0), mask,
                                              bool(m.get("v_mix")))
            elif l["type"] == "latent_attention":
                rot = m["rot"]
                mixer = LatentAttentionConfig(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]), float(m["scale"]),
                                              RotaryConfig(int(rot["dims"]), float(rot["base"]), None), mask)
                if mixer.rot.dims > mixer.rot_dim or mixer.rot.dims % 2:
                    raise ValueError(f"layer {i}: {mixer.rot.dims} rotary dimensions do not fit a rotated part of {mixer.rot_dim}")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            layers.append(SopetarLayerConfig(l["type"], mixer, ff))
        shared = [l.mixer for l in layers if l.type == "attention" and l.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (shared[0].kv_heads, shared[0].vdim) for m in shared):
            raise ValueError("layers that blend their values with the first such layer's need the same key/value heads and value width")
        return SopetarConfig(c["architecture"], int(c["vocab"]), int(c["width"]), float((c.get("embedding") or {}).get("scale", 1.0)),
                             float((c.get("norm") or {}).get("eps", 1e-6)), tuple(layers))


@dataclass(frozen=True)
class LogDistanceAttentionConfig:
    """Softmax attention without rotation in which positions enter through a charge r1_h * ln(1 + r2_h * distance) on the scores, a
    sliding window, and a query temperature 1 + coef * ln(floor((pos + 1) / every) + 1) (``q_temp_every`` 0 = none)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask: WindowMask
    q_temp_coef: float = 0.0
    q_temp_every: int = 0


@dataclass(frozen=True)
class DeltaRuleConfig:
    """Gated delta rule: ``kv_heads`` query / key heads of width ``dim`` shared by groups of the ``heads`` value heads of width ``vdim``,
    a causal convolution of ``conv`` taps in front of q, k and v."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class GatedFeedForwardConfig:
    ff: int


@dataclass(frozen=True)
class ExpertsConfig:
    """Mixture of experts: ``experts`` feed-forwards of width ``ff`` and ``identity`` experts without weights (their output is their
    input) share one router; a token uses the ``top`` best."""
    experts: int
    identity: int
    top: int
    ff: int


@dataclass(frozen=True)
class VasosunLayerConfig:
    type: str            # "attention" | "latent_attention" | "delta"
    mixer: object        # LogDistanceAttentionConfig | LatentAttentionConfig | DeltaRuleConfig
    mlp: object = None   # GatedFeedForwardConfig | ExpertsConfig | None


@dataclass(frozen=True)
class VasosunConfig:
    """The Vasosun design: every sublayer sits between two RMS norms whose weight is one number and reads its input through a short causal
    convolution; the embedding adds a hashed (previous token, token) table; mixers are window attention with a logarithmic distance
    charge, latent attention (queries through a latent too, YaRN-scaled rotation, optionally over another layer's cache) and the gated
    delta rule; feed-forwards are gated or a mixture of experts. Every size and constant that may differ comes from config.json."""
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    conv_taps: int
    pair_buckets: int
    pair_mul_prev: int
    pair_mul_cur: int
    logit_softcap: float
    layers: tuple

    @staticmethod
    def from_dict(c: dict) -> "VasosunConfig":
        layers = []
        for i, l in enumerate(c["layers"]):
            m, mlp = l["mixer"], l.get("mlp")
            kind = l["type"]
            if kind == "attention":
                heads = int(m["heads"])
                kv_heads = int(m.get("kv_heads") or heads)
                if heads % kv_heads:
                    raise ValueError(f"layer {i}: {heads} query heads do not divide over {kv_heads} key/value heads")
                qt = m.get("q_temp") or {}
                mixer = LogDistanceAttentionConfig(heads, kv_heads, int(m["dim"]), int(m["vdim"]), float(m["scale"]), WindowMask.from_dict(m.get("mask")),
                                                   float(qt.get("coef") or 0.0), int(qt.get("every") or 0))
            elif kind == "latent_attention":
                rot = m["rot"]
                src = m.get("kv_from")
                mixer = LatentAttentionConfig(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]), float(m["scale"]),
                                              RotaryConfig(int(rot["dims"]), float(rot["base"]), rot.get("scaling") or None),
                                              WindowMask.from_dict(m.get("mask")), int(m["q_rank"]) if m.get("q_rank") else None, None if src is None else int(src))
                if mixer.rot.dims > mixer.rot_dim or mixer.rot.dims % 2:
                    raise ValueError(f"layer {i}: {mixer.rot.dims} rotary dimensions do not fit a rotated part of {mixer.rot_dim}")
                if mixer.kv_from is not None:
                    o = layers[mixer.kv_from].mixer if 0 <= mixer.kv_from < i and layers[mixer.kv_from].type == kind else None
                    if o is None or o.kv_from is not None or (o.kv_rank, o.rot_dim, o.rot) != (mixer.kv_rank, mixer.rot_dim, mixer.rot):
                        raise ValueError(f"layer {i}: kv_from {mixer.kv_from} must name an earlier latent-attention layer with a cache of its own "
                                         "and the same latent width and rotation")
            elif kind == "delta":
                heads = int(m["heads"])
                kv_heads = int(m.get("kv_heads") or heads)
                if heads % kv_heads:
                    raise ValueError(f"layer {i}: {heads} value heads do not divide over {kv_heads} key heads")
                mixer = DeltaRuleConfig(heads, kv_heads, int(m["dim"]), int(m["vdim"]), int(m.get("conv") or 1))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            ff = None
            if mlp is not None:
                if mlp.get("kind", "dense") == "dense":
                    ff = GatedFeedForwardConfig(int(mlp["ff"]))
                elif mlp["kind"] == "moe":
                    r = mlp["router"]
                    ff = ExpertsConfig(int(r["experts"]), int(r.get("identity") or 0), int(r["top"]), int(mlp["expert"]["ff"]))
                    if not 1 <= ff.top <= ff.experts + ff.identity:
                        raise ValueError(f"layer {i}: {ff.top} of {ff.experts + ff.identity} experts")
                else:
                    raise ValueError(f"layer {i}: feed-forward kind {mlp['kind']!r} is not part of this design")
            layers.append(VasosunLayerConfig(kind, mixer, ff))
        pair = (c.get("embedding") or {}).get("bigram") or {}
        return VasosunConfig(c["architecture"], int(c["vocab"]), int(c["width"]), float((c.get("norm") or {}).get("eps", 1e-6)),
                             int((c.get("canon") or {}).get("taps") or 1), int(pair.get("buckets") or 0), int(pair.get("mul_prev") or 0),
                             int(pair.get("mul_cur") or 0), float(c.get("logit_softcap") or 0.0), tuple(layers))



@dataclass(frozen=True)
class StateSpaceDualityConfig:
    """Mamba-2: ``heads`` heads of ``vdim`` channels, a state of ``state`` numbers per channel, B and C shared by the heads of each of the
    ``groups`` groups, a causal convolution of ``conv`` taps over x, B and C, the output normed in ``norm_groups`` equal parts."""
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int


@dataclass(frozen=True)
class SelectiveScanConfig:
    """Mamba: ``inner`` channels with a state of ``state`` numbers each, step sizes through a projection of rank ``dt_rank``, a causal
    convolution of ``conv`` taps over x."""
    inner: int
    state: int
    dt_rank: int
    conv: int


@dataclass(frozen=True)
class TalkingHeadsAttentionConfig:
    """Softmax attention with a convolution and a per-head norm on q and k, values that are the keys before the norm, partial rotary
    positions (``rot`` None = none), a sliding window that keeps the first positions, and heads mixed after the softmax."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig | None
    mask: WindowMask
    conv: int


@dataclass(frozen=True)
class BiasedFeedForwardConfig:
    ff: int


@dataclass(frozen=True)
class KodezenLayerConfig:
    type: str            # "mamba2" | "mamba1" | "attention"
    mixer: object        # StateSpaceDualityConfig | SelectiveScanConfig | TalkingHeadsAttentionConfig
    mlp: object = None   # BiasedFeedForwardConfig | ExpertsConfig | None


@dataclass(frozen=True)
class KodezenConfig:
    """The Kodezen design: pre-norm layers (RMS norms whose weights are stored around zero) whose mixer reads its normed input through a
    short causal convolution; mixers are Mamba-2 (state-space duality), Mamba (selective scan) and softmax attention with convolved,
    normed and partly rotated queries and keys, keys as values and heads mixed after the softmax; feed-forwards are dense (biases, exact
    gelu) or a mixture of gated experts whose sigmoid scores multiply the experts' inputs. Every size and constant that may differ
    comes from config.json."""
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    conv_taps: int
    embedding_scale: float
    layers: tuple

    @staticmethod
    def from_dict(c: dict) -> "KodezenConfig":
        layers = []
        for i, l in enumerate(c["layers"]):
            m, mlp = l["mixer"], l.get("mlp")
            kind = l["type"]
            if kind == "mamba2":
                heads, groups = int(m["heads"]), int(m.get("groups") or 1)
                if heads % groups:
                    raise ValueError(f"layer {i}: {heads} heads do not divide over {groups} groups")
                mixer = StateSpaceDualityConfig(heads, int(m["vdim"]), int(m["state"]), groups, int(m.get("norm_groups") or 1), int(m.get("conv") or 1))
            elif kind == "mamba1":
                mixer = SelectiveScanConfig(int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m.get("conv") or 1))
            elif kind == "attention":
                heads = int(m["heads"])
                kv_heads = int(m.get("kv_heads") or heads)
                if heads % kv_heads:
                    raise ValueError(f"layer {i}: {heads} query heads do not divide over {kv_heads} key/value heads")
                rot = m.get("rot")
                rot = RotaryConfig(int(rot["dims"]), float(rot["base"]), None) if rot and int(rot.get("dims") or 0) > 0 else None
                dim = int(m["dim"])
                if rot is not None and (rot.dims > dim or rot.dims % 2):
                    raise ValueError(f"layer {i}: {rot.dims} rotary dimensions do not fit heads of {dim}")
                mixer = TalkingHeadsAttentionConfig(heads, kv_heads, dim, int(m.get("vdim") or dim), float(m["scale"]), rot, WindowMask.from_dict(m.get("mask")),
                                                    int(m.get("conv") or 1))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            ff = None
            if mlp is not None:
                if mlp.get("kind", "dense") == "dense":
                    ff = BiasedFeedForwardConfig(int(mlp["ff"]))
                elif mlp["kind"] == "moe":
                    r = mlp["router"]
                    ff = ExpertsConfig(int(r["experts"]), 0, int(r["top"]), int(mlp["expert"]["ff"]))
                    if not 1 <= ff.top <= ff.experts:
                        raise ValueError(f"layer {i}: {ff.top} of {ff.experts} experts")
                else:
                    raise ValueError(f"layer {i}: feed-forward kind {mlp['kind']!r} is not part of this design")
            layers.append(KodezenLayerConfig(kind, mixer, ff))
        return KodezenConfig(c["architecture"], int(c["vocab"]), int(c["width"]), float((c.get("norm") or {}).get("eps", 1e-6)),
                             int((c.get("canon") or {}).get("taps") or 1), float((c.get("embedding") or {}).get("scale", 1.0)), tuple(layers))


CONFIG_READERS = {"Munazen": MunazenConfig.from_dict, "Sopetar": SopetarConfig.from_dict, "Vasosun": VasosunConfig.from_dict,
                  "Kodezen": KodezenConfig.from_dict}


def read_model_config(model_dir: str):
    """config.json of a model folder -> the config object of its architecture (KeyError names the architectures known here)."""
    import json
    import os
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    arch = c.get("architecture")
    if arch not in CONFIG_READERS:
        raise KeyError(f"architecture {arch!r} is not registered (known: {sorted(CONFIG_READERS)})")
    return CONFIG_READERS[arch](c)
