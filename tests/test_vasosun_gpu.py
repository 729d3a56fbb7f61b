"""Vasosun on the GPU against the plain float64 restatement (tests/vasosun_oracle.py): every mechanism alone, whole prompts with the
stream after every layer, decoding through the cache and the recurrent state, portions down to two tokens, unequal requests in one batch,
pages and slots that are freed and used again, keys that stand out just inside and just outside the window (in prompts and in decoding,
at page borders) and far back, other sizes (also values that happen to be equal or 1), and greedy generation through the scheduler and the
command lines. Small random models, made here; fp32 mode is compared tightly, bf16 mode within the rounding of bf16 operands."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import vasosun_oracle as O  # noqa: E402
import vasosun_testlib as L  # noqa: E402

pytestmark = pytest.mark.gpu

F32_TOL = 2e-5     # relative rms of a vector, fp32 mode: one mechanism
F32_MODEL = 5e-5   # logits of a whole model (a position whose routing or softmax is a near tie multiplies the rounding of the layers before it)
BF16_TOL = 1e-1    # bf16 operands of the products: worst position of a shallow model
BF16_MIXER = 3e-2  # one mixer with bf16 operands and a bf16 cache
BF16_MODEL_TYPICAL = 8e-2

# every mixer and both feed-forwards; a latent layer that attends over an earlier one's cache with other head sizes
CFG_A = L.make_config([L.attention_layer(), L.latent_layer(mlp=L.moe()), L.latent_layer(heads=2, dim=12, vdim=8, kv_from=1, mlp=L.moe(experts=3, identity=1, top=2, ff=20)),
                       L.delta_layer(mlp=L.moe()), L.attention_layer(heads=6, kv_heads=2, size=33, every=0, mlp=None), L.delta_layer(heads=2, kv_heads=2, dim=40, vdim=20, conv=4)])
# values that a model may happen to make equal or 1: one head, a window of one position and none at all, one tap, one expert of one,
# no identity expert, no correction that matters, a temperature that changes at every position, no scaling of the rotation
CFG_ONES = L.make_config([L.delta_layer(heads=1, kv_heads=1, dim=32, vdim=32, conv=1, mlp=L.moe(experts=1, identity=0, top=1, ff=32)),
                          L.attention_layer(heads=1, kv_heads=1, dim=32, vdim=32, size=1, every=1, mlp=None),
                          L.latent_layer(heads=1, dim=16, rot_dim=16, vdim=16, kv_rank=16, q_rank=16, scaling=None, mlp=L.moe(experts=2, identity=3, top=5, ff=8)),
                          L.attention_layer(heads=2, kv_heads=2, dim=16, vdim=16, size=None)], vocab=61, width=32, taps=1, buckets=1, softcap=0)
# head widths the tensor-core attention and products take, enough tokens in the tests for the tensor-core products
CFG_TC = L.make_config([L.latent_layer(heads=4, dim=16, rot_dim=16, vdim=24, kv_rank=48, q_rank=64, mlp=L.moe(experts=6, identity=2, top=3, ff=32)),
                        L.attention_layer(heads=4, kv_heads=2, dim=32, vdim=16, size=40, mlp=L.dense(96)),
                        L.delta_layer(heads=4, kv_heads=2, dim=64, vdim=32, mlp=L.dense(64)),
                        L.latent_layer(heads=2, dim=32, rot_dim=16, vdim=16, kv_rank=48, q_rank=64, kv_from=0, mlp=L.dense(64))], width=64, vocab=128, taps=2)
# sizes that are multiples of nothing
CFG_ODD = L.make_config([L.latent_layer(heads=3, dim=6, rot_dim=10, rot_dims=6, vdim=5, kv_rank=13, q_rank=9, mlp=L.moe(experts=7, identity=3, top=4, ff=11)),
                         L.attention_layer(heads=10, kv_heads=1, dim=6, vdim=10, size=45, scale=0.7, every=3, mlp=L.dense(23)),
                         L.delta_layer(heads=3, kv_heads=1, dim=35, vdim=7, conv=2, mlp=None),
                         L.delta_layer(heads=2, kv_heads=2, dim=70, vdim=9, conv=5, mlp=L.dense(17))], vocab=67, width=50, eps=1e-6, taps=4, buckets=29,
                        mul_prev=1000003, mul_cur=999983)
ALL = [CFG_A, CFG_ONES, CFG_TC, CFG_ODD]
IDS = ["mixed", "ones", "tensorcore", "odd"]


def _engine(tmp_path, cfg, w, dtype="float32", max_tokens=512, max_seqs=4, page_len=32, name="m", **kw):
    from simplellminference_b200.models import build_model
    from simplellminference_b200.seqengine import SequenceEngine
    folder = L.write_model(str(tmp_path / name), cfg, w)
    model = build_model(folder, dtype, "cuda")
    return SequenceEngine(model, max_tokens=max_tokens, max_seqs=max_seqs, page_len=page_len, **kw)


def _logits(eng, slot, toks, want=None):
    want = list(range(len(toks))) if want is None else want
    out = eng.run([(slot, toks, want)])
    return None if out is None else out.cpu().numpy()


def _rel(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.sqrt(((got - want) ** 2).mean()) / max(1e-30, np.sqrt((want ** 2).mean())))


def _w64(w):
    return {k: v.astype(np.float64) for k, v in w.items()}


def _forward(cfg, w, toks):
    return O.forward(toks, _w64(w), cfg)[0]


# ------------------------------------------------------------------------------------------------ mechanisms alone
class _Stub:
    """A model that hands the rows it is given to a function of (step, h, states) and keeps what that returns."""

    def __init__(self, specs, fn, ops, dev):
        self.specs, self.fn, self.ops, self.device = specs, fn, ops, dev
        self.h, self.outs = None, None

    def state_specs(self):
        return self.specs

    def forward(self, step, ids, states, rows, n_rows, tap=None):
        self.outs = [o.clone() for o in self.fn(step, self.h, states)]
        return None


def _feed(stub, rows, portions, max_tokens=1024, page_len=32):
    """rows [T][d] through the stub in portions; returns the concatenated outputs."""
    import torch

    from simplellminference_b200.seqengine import SequenceEngine
    eng = SequenceEngine(stub, max_tokens=max_tokens, page_len=page_len, graphs=False)
    slot, outs, p = eng.admit(), None, 0
    for n in portions:
        stub.h = torch.tensor(rows[p:p + n], dtype=torch.float32, device=stub.device).contiguous().view(-1)
        eng.run([(slot, np.zeros(n, np.int32), [])])
        outs = [[] for _ in stub.outs] if outs is None else outs
        for i, o in enumerate(stub.outs):
            outs[i].append(o.cpu().numpy())
        p += n
    return [np.concatenate(o) for o in outs]


def _mixer_stub(layer_cfgs, w, width, dtype="float32", eps=1e-5):
    import torch

    from simplellminference_b200 import layers
    from simplellminference_b200.config import BF16, F32, VasosunConfig
    from simplellminference_b200.seqops import Ops
    dev = torch.device("cuda")
    ops = Ops(BF16 if dtype == "bfloat16" else F32)
    wt = {k: torch.tensor(v, device=dev, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in w.items()}
    cfg = VasosunConfig.from_dict(L.make_config(layer_cfgs, width=width))
    groups = []
    for i, lc in enumerate(cfg.layers):
        pre = f"l{i}.mix."
        mech = {"attention": lambda: layers.LogDistanceWindowAttention(lc.mixer, wt, pre, ops, dev),
                "latent_attention": lambda: layers.LatentAttention(lc.mixer, wt, pre, ops, dev, eps),
                "delta": lambda: layers.GatedDeltaRule(lc.mixer, wt, pre, ops, dev, eps)}[lc.type]()
        groups.append(layers.MixerGroup([("mix", mech, 1.0)], ops, dev))

    def fn(step, h, states):
        outs = []
        for g, st in zip(groups, states):
            y = step.scratch("sub_out", step.T * width)
            g.forward(step, h, st, y)
            outs.append(y[:step.T * width].view(step.T, width).clone())
        return outs
    return _Stub([g.state_spec() for g in groups], fn, ops, dev)


ALONE = [L.attention_layer(), L.attention_layer(heads=3, kv_heads=3, dim=20, vdim=36, size=9, every=0), L.attention_layer(heads=8, kv_heads=1, dim=8, vdim=8, size=64, scale=1.0, every=2),
         L.attention_layer(size=None), L.latent_layer(), L.latent_layer(heads=1, dim=24, rot_dim=4, vdim=70, kv_rank=72, q_rank=5),
         L.latent_layer(heads=5, dim=4, rot_dim=16, rot_dims=6, vdim=12, kv_rank=20, scaling=None), L.delta_layer(), L.delta_layer(heads=1, kv_heads=1, dim=100, vdim=5, conv=1),
         L.delta_layer(heads=6, kv_heads=2, dim=8, vdim=33, conv=6), L.delta_layer(heads=2, kv_heads=1, dim=300, vdim=5, conv=2),
         L.latent_layer(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=200)]


def _oracle_mixer(layer_cfg, w, h, pre="l0.mix.", kv=None):
    m, h = layer_cfg["mixer"], h.astype(np.float64)
    if layer_cfg["type"] == "attention":
        return O.window_attention(h, _w64(w), pre, m)
    if layer_cfg["type"] == "latent_attention":
        return O.latent_attention(h, _w64(w), pre, m, 1e-5, kv)[0]
    return O.delta_mixer(h, _w64(w), pre, m, 1e-5)


@pytest.mark.parametrize("portions", [[75], [33, 2, 15, 16, 1, 1, 1, 1, 5], [1] * 75])
def test_each_mixer_alone(portions):
    rng = np.random.default_rng(5)
    d, T = 48, 75
    for layer_cfg in ALONE:
        w = L.random_weights(L.make_config([layer_cfg], width=d), seed=11)
        h = rng.standard_normal((T, d)).astype(np.float32)
        got = _feed(_mixer_stub([layer_cfg], w, d), h, portions)[0]
        want = _oracle_mixer(layer_cfg, w, h)
        assert _rel(got, want) < F32_TOL, (layer_cfg["mixer"], _rel(got, want))


@pytest.mark.parametrize("portions", [[80], [40, 2, 37, 1]])
def test_each_mixer_alone_bf16(portions):
    """bf16 matrices, operands and cache; portions of a prompt take the tensor-core attention where the head widths allow it."""
    rng = np.random.default_rng(7)
    d, T = 64, 80
    for layer_cfg in (L.attention_layer(heads=4, kv_heads=2, dim=32, vdim=16, size=30), L.attention_layer(heads=3, kv_heads=1, dim=12, vdim=20, size=None),
                      L.latent_layer(heads=4, dim=16, rot_dim=16, vdim=24, kv_rank=48, q_rank=64), L.latent_layer(), L.delta_layer(), L.delta_layer(dim=64, vdim=32)):
        w = L.random_weights(L.make_config([layer_cfg], width=d), seed=13)
        h = L.bf16_round(rng.standard_normal((T, d))).astype(np.float32)
        got = _feed(_mixer_stub([layer_cfg], w, d, dtype="bfloat16"), h, portions)[0]
        want = _oracle_mixer(layer_cfg, w, h)
        assert _rel(got, want) < BF16_MIXER, (layer_cfg["mixer"], _rel(got, want))


@pytest.mark.parametrize("portions", [[60], [7, 2, 30, 1, 20]])
def test_latent_attention_over_another_layers_cache(portions):
    rng = np.random.default_rng(6)
    d, T = 32, 60
    cfgs = [L.latent_layer(heads=2), L.latent_layer(heads=4, dim=12, vdim=6, q_rank=10, scale=0.5, kv_from=0)]
    w = L.random_weights(L.make_config(cfgs, width=d), seed=12)
    h = rng.standard_normal((T, d)).astype(np.float32)
    got = _feed(_mixer_stub(cfgs, w, d), h, portions)
    kv = O.latent_kv(h.astype(np.float64), _w64(w), "l0.mix.", cfgs[0]["mixer"], 1e-5)
    assert _rel(got[0], _oracle_mixer(cfgs[0], w, h)) < F32_TOL
    assert _rel(got[1], _oracle_mixer(cfgs[1], w, h, "l1.mix.", kv)) < F32_TOL


def _standing_out(kind, d, H, window):
    """A one-mixer layer and weights in which the query of a position reads the first third of its input row and the key the second third,
    through the same map: a query row whose first third repeats the second third of an earlier row gives that position (and no other,
    itself included) a score far above the rest. Returns (layer, weights, third)."""
    t = d // 3
    if kind == "attention":
        layer = L.attention_layer(heads=H, kv_heads=H, dim=16, vdim=16, scale=4.0, size=window, coef=0.1, every=50)
        w = L.random_weights(L.make_config([layer], width=d), seed=3)
        a = L.bf16_round(2.0 * w["l0.mix.q"][:, :t])          # large enough that equal thirds beat every chance alignment
        w["l0.mix.q"][:] = 0.0
        w["l0.mix.k"][:] = 0.0
        w["l0.mix.q"][:, :t] = a
        w["l0.mix.k"][:, t:2 * t] = a
        w["l0.mix.v"][:, :2 * t] = 0.0
        w["l0.mix.r1"][:] = L.bf16_round(np.full(H, 0.5))
    else:
        R, dn = 32, 16
        layer = L.latent_layer(heads=H, dim=dn, rot_dim=4, vdim=16, kv_rank=R, q_rank=R, scale=1.0)
        w = L.random_weights(L.make_config([layer], width=d), seed=3)
        # both latents read through m (the key's from the second third, the query's from the first); head h's unrotated query is
        # 3 W_uk,h c_q: q_h(row i) . k_h(row j) = 3 |W_uk,h c|^2 when row i's first third and row j's second third are equal
        m = w["l0.mix.dkv"][:R, t:2 * t].copy()
        w["l0.mix.dkv"][:R] = 0.0
        w["l0.mix.dkv"][:R, t:2 * t] = m
        w["l0.mix.dq"][:] = 0.0
        w["l0.mix.dq"][:, :t] = m
        uq = np.zeros((H, dn + 4, R), np.float32)
        uq[:, :dn] = L.bf16_round(3.0 * w["l0.mix.uk"].reshape(H, dn, R))
        w["l0.mix.uq"] = uq.reshape(H * (dn + 4), R)
        w["l0.mix.dkv.norm"] = np.ones(R, np.float32)
        w["l0.mix.dq.norm"] = np.ones(R, np.float32)
    return layer, w, t


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
def test_keys_just_inside_and_outside_the_window(decode):
    """The key input of an earlier position is repeated as the query input of a later one: when that position is the oldest one inside the
    window the query's output is essentially its value, one further back it is something else — the restatement says so and the engine
    has to follow it, with the key before, at and after a border of pages of 32."""
    rng = np.random.default_rng(9)
    d, T, H, window = 48, 150, 2, 37
    layer, w, t = _standing_out("attention", d, H, window)
    stub = _mixer_stub([layer], w, d)
    seen = []
    for query in (149, 100, 68, 69, 70):                      # oldest visible key 113 / 64 / 32 / 33 / 34
        for key, visible in ((query - window + 1, True), (query - window, False), (query - 1, True)):
            h = rng.standard_normal((T, d)).astype(np.float32)
            h[key, t:2 * t] *= 2.0                          # a long key: no other key's chance alignment with the query comes close
            h[query, :t] = h[key, t:2 * t]
            want = _oracle_mixer(layer, w, h)
            got = _feed(stub, h, [query] + [1] * (T - query) if decode else [T])[0]
            assert _rel(got, want) < F32_TOL, (query, key, _rel(got, want))
            base = h.copy()
            base[key] = rng.standard_normal(d)
            seen.append((visible, _rel(_oracle_mixer(layer, w, base)[query], want[query])))
    shown = sorted(r for v, r in seen if v)
    assert shown[0] > 0.05 and shown[len(shown) // 2] > 0.5, "a visible repeated position does not stand out: the test would not notice a lost key"
    assert max(r for v, r in seen if not v) < 1e-6, "a hidden position changes the restatement's result"


@pytest.mark.parametrize("kind", ["attention", "latent"])
@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
def test_a_key_far_back_among_hundreds(kind, decode):
    """One position hundreds of tokens back (the first token, one at a page border, one in the middle of a page) towers over all others."""
    rng = np.random.default_rng(10)
    d, T, H = 48, 420, 2
    layer, w, t = _standing_out(kind, d, H, None if kind == "latent" else 400)
    stub = _mixer_stub([layer], w, d)
    shown = []
    for query, key in ((419, 20), (400, 64), (330, 0), (399, 31)):
        h = rng.standard_normal((T, d)).astype(np.float32)
        h[key, t:2 * t] *= 2.0
        h[query, :t] = h[key, t:2 * t]
        want = _oracle_mixer(layer, w, h)
        got = _feed(stub, h, [320] + [1] * (T - 320) if decode else [200, 220])[0]
        assert _rel(got, want) < F32_TOL, (kind, query, key, _rel(got, want))
        base = h.copy()
        base[key] = rng.standard_normal(d)
        shown.append(_rel(_oracle_mixer(layer, w, base)[query], want[query]))
    assert min(shown) > 0.3, "the far position does not stand out"


def test_seam_kernel_alone():
    """Residual sum with a scalar norm, then scalar norm + input convolution, against the restatement; in one piece, in portions that
    are shorter than the convolution's reach, and as the two halves run separately."""
    import torch

    from simplellminference_b200.config import F32
    from simplellminference_b200.seqops import Ops
    rng, dev, ops = np.random.default_rng(2), torch.device("cuda"), Ops(F32)
    for d, taps, T in ((48, 3, 40), (1000, 4, 19), (50, 1, 9), (36, 7, 30), (52, 3, 150)):
        x, y = (3 * rng.standard_normal((T, d))).astype(np.float32), rng.standard_normal((T, d)).astype(np.float32)
        cw = (0.5 * rng.standard_normal((d, taps))).astype(np.float32)
        g_post, g_pre, eps = 0.8, 1.3, 1e-5
        x_new = x.astype(np.float64) + O.scalar_norm(y, g_post, eps)
        want = O.input_conv(O.scalar_norm(x_new, g_pre, eps), cw)
        cwt = torch.tensor(cw, device=dev)
        for split in (False, True):
            def fn(step, h, states):
                n = step.T
                xy = h.view(n, 2 * d)
                xi, yi = xy[:, :d].contiguous(), xy[:, d:].contiguous()
                xo, ho, stash = torch.empty_like(xi), torch.empty_like(xi), step.scratch("stash", n * d)
                ring = states[0].get("ring")
                if split:
                    ops.seam(step.b, xi, d, step.st, x_out=xo, y=yi, post_g=g_post, eps=eps)
                    ops.seam(step.b, xo, d, step.st, pre_g=g_pre, eps=eps, conv_w=cwt, taps=taps, ring=ring, h=ho, stash=stash)
                else:
                    # with scratch for the per-row scales, steps of 64 tokens and more take the two-launch form
                    ops.seam(step.b, xi, d, step.st, x_out=xo, y=yi, post_g=g_post, pre_g=g_pre, eps=eps, conv_w=cwt, taps=taps, ring=ring, h=ho, stash=stash,
                             scales=step.scratch("scales", n))
                tail = torch.empty_like(xi)
                ops.seam(step.b, xo, d, step.st, pre_g=1.0, eps=eps, h=tail, stash=stash, flush_ring=ring, flush_taps=taps if ring is not None else 0)
                return [xo, ho]
            spec = {"pages": [], "slots": [("ring", (taps - 1, d))] if taps > 1 else []}
            stub = _Stub([spec], fn, ops, dev)
            for portions in ([T], [1] * T, [2, 1, 3, T - 6], [T - 3, 3]):
                got = _feed(stub, np.concatenate([x, y], axis=1), portions)
                assert _rel(got[0], x_new) < 1e-6 and _rel(got[1], want) < 2e-6, (d, taps, split, portions[:3], _rel(got[1], want))


def test_feed_forwards_alone():
    """The gated feed-forward and the mixture of experts (routing with a correction, weights without it, identity experts)."""
    import torch

    from simplellminference_b200 import layers
    from simplellminference_b200.config import F32, VasosunConfig
    from simplellminference_b200.seqops import Ops
    rng, d, T = np.random.default_rng(4), 40, 37
    dev, ops = torch.device("cuda"), Ops(F32)
    for mlp in (L.dense(56), L.moe(), L.moe(experts=9, identity=0, top=1, ff=7), L.moe(experts=2, identity=6, top=4, ff=16), L.moe(experts=40, identity=3, top=8, ff=4)):
        cfg = L.make_config([L.attention_layer(mlp=mlp)], width=d)
        w = L.random_weights(cfg, seed=2)
        wt = {k: torch.tensor(v, device=dev) for k, v in w.items()}
        c = VasosunConfig.from_dict(cfg).layers[0].mlp
        ff = (layers.GatedFeedForward if mlp["kind"] == "dense" else layers.ExpertsFeedForward)(c, wt, "l0.mlp.", ops, dev)

        def fn(step, h, states):
            y = step.scratch("sub_out", step.T * d)
            ff.forward(step, h, y)
            return [y[:step.T * d].view(step.T, d)]
        h = (2 * rng.standard_normal((T, d))).astype(np.float32)
        got = _feed(_Stub([{"pages": [], "slots": []}], fn, ops, dev), h, [T])[0]
        h64 = h.astype(np.float64)
        want = O.dense_ff(h64, _w64(w), "l0.mlp.") if mlp["kind"] == "dense" else O.moe_ff(h64, _w64(w), "l0.mlp.", mlp)
        assert _rel(got, want) < F32_TOL, (mlp, _rel(got, want))
        if mlp["kind"] == "moe":        # the correction changes some choices in these weights, else the test would not see it used for the weights
            plain = {**_w64(w), "l0.mlp.correction": np.zeros_like(w["l0.mlp.correction"], dtype=np.float64)}
            if mlp["router"]["top"] < mlp["router"]["experts"] + mlp["router"]["identity"]:
                assert _rel(O.moe_ff(h64, plain, "l0.mlp.", mlp), want) > 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_with_tokens_gathered_per_expert(dtype, monkeypatch):
    """Steps of many tokens multiply a token only with the experts it uses (rows gathered per expert, counts kept on the device): the same
    numbers as the restatement, and as the form that computes every expert, also when an expert gets no token at all."""
    import torch

    from simplellminference_b200 import layers
    from simplellminference_b200.config import BF16, F32, VasosunConfig
    from simplellminference_b200.seqops import Ops
    rng, d, T = np.random.default_rng(14), 64, 300
    dev, ops = torch.device("cuda"), Ops(BF16 if dtype == "bfloat16" else F32)
    for mlp in (L.moe(experts=6, identity=2, top=3, ff=64), L.moe(experts=9, identity=0, top=1, ff=72), L.moe(experts=3, identity=5, top=2, ff=13)):
        cfg = L.make_config([L.attention_layer(mlp=mlp)], width=d)
        w = L.random_weights(cfg, seed=5)
        if mlp["router"]["experts"] == 9:
            w["l0.mlp.router"][4] = 0.0                       # an expert nobody is routed to ...
            w["l0.mlp.correction"][4] = -5.0
        wt = {k: torch.tensor(v, device=dev, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in w.items()}
        ff = layers.ExpertsFeedForward(VasosunConfig.from_dict(cfg).layers[0].mlp, wt, "l0.mlp.", ops, dev)

        def fn(step, h, states):
            y = step.scratch("sub_out", step.T * d)
            ff.forward(step, h, y)
            return [y[:step.T * d].view(step.T, d)]
        h = L.bf16_round(2 * rng.standard_normal((T, d))).astype(np.float32)
        stub = _Stub([{"pages": [], "slots": []}], fn, ops, dev)
        monkeypatch.setattr(layers.ExpertsFeedForward, "gather_min_tokens", 10 ** 9)
        every = _feed(stub, h, [T])[0]
        monkeypatch.setattr(layers.ExpertsFeedForward, "gather_min_tokens", 64)
        monkeypatch.setattr(layers.ExpertsFeedForward, "gather_launch_cost", 0.0)
        assert ff._gathered_pays(T) == (mlp["router"]["top"] < mlp["router"]["experts"])
        gathered = _feed(stub, h, [T])[0]
        want = O.moe_ff(h.astype(np.float64), _w64(w), "l0.mlp.", mlp)
        tol = F32_TOL if dtype == "float32" else BF16_MIXER
        assert _rel(gathered, want) < tol and _rel(every, want) < tol, (mlp, _rel(gathered, want), _rel(every, want))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_chosen_on_the_device_for_single_tokens(dtype, monkeypatch):
    """Steps of one or two tokens stream only the chosen experts' matrices (one launch per projection, the matrix of every (token, choice)
    pair picked on the device): the same numbers as the restatement and as the form that computes every expert."""
    import torch

    from simplellminference_b200 import layers
    from simplellminference_b200.config import BF16, F32, VasosunConfig
    from simplellminference_b200.seqops import Ops
    rng, d = np.random.default_rng(15), 72
    dev, ops = torch.device("cuda"), Ops(BF16 if dtype == "bfloat16" else F32)
    for mlp, T in ((L.moe(experts=7, identity=2, top=3, ff=40), 2), (L.moe(experts=9, identity=0, top=1, ff=64), 8), (L.moe(experts=5, identity=4, top=4, ff=13), 1)):
        cfg = L.make_config([L.attention_layer(mlp=mlp)], width=d)
        w = L.random_weights(cfg, seed=6)
        wt = {k: torch.tensor(v, device=dev, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in w.items()}
        ff = layers.ExpertsFeedForward(VasosunConfig.from_dict(cfg).layers[0].mlp, wt, "l0.mlp.", ops, dev)

        def fn(step, h, states):
            y = step.scratch("sub_out", step.T * d)
            ff.forward(step, h, y)
            return [y[:step.T * d].view(step.T, d)]
        h = L.bf16_round(2 * rng.standard_normal((3 * T, d))).astype(np.float32)
        stub = _Stub([{"pages": [], "slots": []}], fn, ops, dev)
        every = _feed(stub, h, [T, T, T])[0]
        monkeypatch.setattr(layers.ExpertsFeedForward, "index_launch_cost", 0.0)
        assert ff._indexed_pays(T)
        indexed = _feed(stub, h, [T, T, T])[0]
        monkeypatch.undo()
        want = O.moe_ff(h.astype(np.float64), _w64(w), "l0.mlp.", mlp)
        tol = F32_TOL if dtype == "float32" else BF16_MIXER
        assert _rel(indexed, want) < tol and _rel(every, want) < tol, (mlp, _rel(indexed, want), _rel(every, want))


def test_pair_embedding_and_logit_cap(tmp_path):
    """The first token takes the pair table's last row, every other the hashed row of (previous token, token) — also across a cut."""
    cfg = L.make_config([L.attention_layer(mlp=None)], vocab=50, width=32, buckets=7, mul_prev=5, mul_cur=3, softcap=2.0)
    w = L.random_weights(cfg, seed=3)
    w["head"] = (8 * w["head"]).astype(np.float32)           # logits large enough that the cap bends them
    toks = [3, 3, 49, 0, 17, 17, 17, 2]
    want = _forward(cfg, w, toks)
    assert np.abs(want).max() > 1.9
    eng = _engine(tmp_path, cfg, w)
    s = eng.admit()
    got = np.concatenate([_logits(eng, s, toks[:1]), _logits(eng, s, toks[1:5]), _logits(eng, s, toks[5:6]), _logits(eng, s, toks[6:])])
    assert L.logit_error(got, want).max() < F32_TOL
    other = dict(w)
    other["bigram"] = w["bigram"].copy()
    other["bigram"][-1] += 1.0
    assert L.logit_error(_forward(cfg, other, toks)[:1], want[:1]).max() > 1e-2


# ------------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("cfg", ALL, ids=IDS)
def test_whole_prompt_matches_oracle_fp32_and_layers(tmp_path, cfg):
    w = L.random_weights(cfg, seed=1)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=140).tolist()
    want, taps_want = O.forward(toks, _w64(w), cfg)
    eng = _engine(tmp_path, cfg, w)
    taps = []
    got = eng.run([(eng.admit(), toks, list(range(len(toks))))], tap=lambda i, x: taps.append(x.clone().cpu().numpy())).cpu().numpy()
    assert len(taps) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(taps, taps_want)):
        assert _rel(a, b) < F32_MODEL, (i, _rel(a, b))
    assert L.logit_error(got, want).max() < F32_MODEL
    s = eng.admit()                                            # the fused seams give what the separate ones gave
    assert L.logit_error(_logits(eng, s, toks), want).max() < F32_MODEL


@pytest.mark.parametrize("cfg", [CFG_A, CFG_TC, CFG_ODD], ids=["mixed", "tensorcore", "odd"])
def test_bf16_mode_within_operand_rounding(tmp_path, cfg):
    w = L.random_weights(cfg, seed=3)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], size=150).tolist()
    want = _forward(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16")
    s = eng.admit()
    whole = _logits(eng, s, toks)
    eng.release(s)
    s = eng.admit()
    cut = np.concatenate([_logits(eng, s, toks[:100]), _logits(eng, s, toks[100:102])] + [_logits(eng, s, toks[p:p + 1]) for p in range(102, 150)])
    # Six layers deep, rounding of the operands is multiplied by what follows it, and a choice of experts that is a near tie may fall the
    # other way (the position, and through attention and state some later ones, then differ visibly): the typical position is held to
    # the rounding, outliers are few. The mechanisms alone are held to the rounding itself in test_each_mixer_alone_bf16.
    for got in (whole, cut):
        e = L.logit_error(got, want)
        assert np.median(e) < BF16_MODEL_TYPICAL and (e > 0.3).mean() < 0.1, (np.median(e), (e > 0.3).mean())
    e = L.logit_error(cut, whole)
    assert np.median(e) < BF16_MODEL_TYPICAL, np.median(e)


@pytest.mark.parametrize("cfg", ALL, ids=IDS)
def test_prefill_against_token_by_token_and_portions(tmp_path, cfg):
    w = L.random_weights(cfg, seed=5)
    toks = np.random.default_rng(6).integers(0, cfg["vocab"], size=120).tolist()
    want = _forward(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w)
    for portions in ([1] * 120, [2] * 60, [31, 2, 33, 1, 1, 40, 12], [64, 56], [119, 1], [3, 1, 2, 114]):
        s, outs, p = eng.admit(), [], 0
        for n in portions:
            outs.append(_logits(eng, s, toks[p:p + n]))
            p += n
        eng.release(s)
        assert L.logit_error(np.concatenate(outs), want).max() < F32_MODEL, portions[:3]


@pytest.mark.parametrize("cfg", [CFG_A, CFG_ODD], ids=["mixed", "odd"])
def test_unequal_requests_in_one_batch_and_reuse_of_pages_and_slots(tmp_path, cfg):
    """Seven requests of unequal length through three slots and ten pages of 32: portions of prompts beside single tokens of others, every
    request's logits equal the restatement's of that request alone; pages and slots go from finished requests to new ones."""
    w = L.random_weights(cfg, seed=7)
    rng = np.random.default_rng(8)
    lens = [70, 33, 5, 96, 64, 1, 47]
    reqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lens]
    want = [_forward(cfg, w, r) for r in reqs]
    eng = _engine(tmp_path, cfg, w, max_tokens=320, max_seqs=3, page_len=32)
    waiting, slots, fed, got = list(range(len(reqs))), {}, [0] * len(reqs), [[] for _ in reqs]
    used_slots, page_users, step = [], {}, 0
    sizes = [17, 2, 32, 5, 40, 3]
    while waiting or slots:
        while waiting and len(slots) < 3 and eng.free_pages >= -(-lens[waiting[0]] // 32) + sum(-(-lens[i] // 32) - eng.pages.held(s) for i, s in slots.items()):
            i = waiting.pop(0)
            slots[i] = eng.admit()
            used_slots.append(slots[i])
        entries, order = [], []
        for i, s in slots.items():
            left = lens[i] - fed[i]
            n = 1 if (fed[i] > lens[i] // 2) else min(left, sizes[(step + i) % len(sizes)])   # portions first, single tokens later
            entries.append((s, reqs[i][fed[i]:fed[i] + n], list(range(n))))
            order.append((i, n))
        out = eng.run(entries).cpu().numpy()
        table = eng.pages.table()
        for i, sl in slots.items():
            for pg in table[sl]:
                if pg >= 0:
                    page_users.setdefault(int(pg), set()).add(i)
        r = 0
        for i, n in order:
            got[i].append(out[r:r + n])
            r += n
            fed[i] += n
        for i in [i for i in slots if fed[i] == lens[i]]:
            eng.release(slots.pop(i))
        step += 1
    assert len(used_slots) > len(set(used_slots)), "no slot was used twice: the test does not test reuse"
    assert eng.free_pages == 10 and any(len(u) > 1 for u in page_users.values()), "no page went from one request to another"
    for i in range(len(reqs)):
        assert L.logit_error(np.concatenate(got[i]), want[i]).max() < F32_MODEL, i


def test_long_decoding_over_page_borders_and_past_the_window(tmp_path):
    cfg = L.make_config([L.attention_layer(size=50), L.delta_layer(mlp=L.moe()), L.latent_layer(), L.attention_layer(size=130, every=64, mlp=L.moe()),
                         L.latent_layer(heads=2, kv_from=2)])
    w = L.random_weights(cfg, seed=8)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], size=330).tolist()
    want = _forward(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, max_tokens=384, page_len=64)
    s = eng.admit()
    outs = [_logits(eng, s, toks[:60])] + [_logits(eng, s, toks[p:p + 1]) for p in range(60, 330)]
    assert eng.graph_replays > 200
    assert L.logit_error(np.concatenate(outs), want).max() < F32_MODEL


def test_first_tokens_of_a_sequence_after_a_used_slot(tmp_path):
    """A slot (recurrent state, convolution rings, previous token) and pages that held a long request serve the next one: its first
    tokens equal the restatement's."""
    w = L.random_weights(CFG_A, seed=9)
    rng = np.random.default_rng(10)
    eng = _engine(tmp_path, CFG_A, w, max_seqs=1, max_tokens=96)
    for n in (90, 4, 1, 2, 35):
        toks = rng.integers(0, CFG_A["vocab"], size=n).tolist()
        s = eng.admit()
        got = np.concatenate([_logits(eng, s, toks[:1]), _logits(eng, s, toks[1:])]) if n > 1 else _logits(eng, s, toks)
        eng.release(s)
        assert L.logit_error(got, _forward(CFG_A, w, toks)).max() < F32_MODEL, n


def _follows_greedy(cfg, w, prompt, produced):
    seq = list(prompt)
    for k, tok in enumerate(produced):
        lg = _forward(cfg, w, seq)[-1]
        order = np.argsort(lg)
        close = lg[order[-1]] - lg[order[-2]] <= 1e-3 * np.abs(lg).max()      # a near tie may fall either way: follow the engine
        assert tok == int(order[-1]) or (close and tok == int(order[-2])), (prompt[:4], k)
        seq.append(tok)


def test_greedy_generation_through_the_scheduler(tmp_path):
    """Requests of unequal length through ContinuousBatcher over SequenceDecoder (prompts in portions beside decoding requests, more
    requests than slots): every request's tokens are the restatement's greedy continuation of that prompt alone."""
    from simplellminference_b200.scheduler import ContinuousBatcher
    from simplellminference_b200.seqengine import SequenceDecoder
    cfg = CFG_A
    w = L.random_weights(cfg, seed=12)
    rng = np.random.default_rng(13)
    prompts = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (5, 40, 1, 23, 64, 7)]
    new = 10
    eng = _engine(tmp_path, cfg, w, max_tokens=6 * 32, max_seqs=3, page_len=32)
    cb = ContinuousBatcher(SequenceDecoder(eng, prefill_chunk=16), chunk=4)
    ids = [cb.submit(p, new) for p in prompts]
    out = cb.run()
    assert cb.stats.max_live == 3 and eng.free_pages == 6
    for rid, p in zip(ids, prompts):
        got = [int(t) for t in out[rid]]
        assert got[:len(p) - 1] == p[1:]
        _follows_greedy(cfg, w, p, got[len(p) - 1:])


def test_trace_replayer_command(tmp_path):
    """bin/trace_run end to end on a Vasosun folder: the model class comes from config.json."""
    import json
    import subprocess
    cfg = CFG_ODD
    w = L.random_weights(cfg, seed=15)
    folder = L.write_model(str(tmp_path / "model"), cfg, w)
    rng = np.random.default_rng(16)
    a, b = rng.integers(0, cfg["vocab"], size=70).tolist(), rng.integers(0, cfg["vocab"], size=9).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b, "want": [8]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:], "want": [38]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [0, 8]}], "end": ["c"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out_dir = tmp_path / "out"
    for dtype, tol in (("float32", F32_MODEL), ("bfloat16", BF16_TOL)):
        r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out_dir), "--max-tokens", "128"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        wa, wb = _forward(cfg, w, a), _forward(cfg, w, b)
        V = cfg["vocab"]
        got = [np.fromfile(out_dir / f"{n}.f32", dtype="<f4").reshape(-1, V) for n in range(4)]
        assert L.logit_error(got[0], wa[[0, 29]]).max() < tol and L.logit_error(got[1], np.stack([wa[30], wb[8]])).max() < tol
        assert L.logit_error(got[2], wa[[69]]).max() < tol and L.logit_error(got[3], wb[[0, 8]]).max() < tol


def test_generation_command_line(tmp_path):
    """python -m simplellminference_b200.generate on a Vasosun folder: registry, engine, scheduler, device arg-max."""
    import json
    import subprocess
    cfg = CFG_TC
    w = L.random_weights(cfg, seed=21)
    folder = L.write_model(str(tmp_path / "model"), cfg, w)
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [7]]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "simplellminference_b200.generate", "--model", folder, "--dtype", "float32", "--max-new-tokens", "6", "--prefill-chunk", "3"]
    for p in prompts:
        cmd += ["--prompt", ",".join(str(t) for t in p)]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert [ln["prompt"] for ln in lines] == prompts
    for ln in lines:
        assert len(ln["tokens"]) == 6
        _follows_greedy(cfg, w, ln["prompt"], ln["tokens"])
