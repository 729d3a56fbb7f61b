"""Kodezen on the GPU against the plain float64 restatement (tests/kodezen_oracle.py): every mechanism alone, whole prompts with the
stream after every layer, decoding through the cache and the recurrent state, portions down to two tokens, unequal requests in one batch,
pages and slots that are freed and used again, keys that stand out just inside and just outside the window and among the kept first
positions (in prompts and in decoding, at page borders) and far back, other sizes (also values that happen to be equal or 1), and greedy
generation through the scheduler and the command lines. Small random models, made here; fp32 mode is compared tightly, bf16 mode within
the rounding of bf16 operands."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import kodezen_oracle as O  # noqa: E402
import kodezen_testlib as L  # noqa: E402

pytestmark = pytest.mark.gpu

F32_TOL = 2e-5     # relative rms of a vector, fp32 mode: one mechanism
F32_MODEL = 5e-5   # logits of a whole model
BF16_TOL = 1e-1    # bf16 operands of the products: worst position of a shallow model
BF16_MIXER = 3e-2  # one mixer with bf16 operands and a bf16 cache
BF16_MODEL_TYPICAL = 8e-2
EPS = 1e-5

# every mixer and both feed-forwards
CFG_A = L.make_config([L.mamba2_layer(), L.mamba1_layer(mlp=L.moe()), L.attention_layer(mlp=L.moe(experts=6, top=3, ff=10)),
                       L.mamba2_layer(heads=6, vdim=4, state=5, groups=3, norm_groups=1, conv=2, mlp=None), L.attention_layer(heads=6, kv_heads=3, size=33, keep_first=0, conv=2),
                       L.mamba1_layer(inner=24, state=9, dt_rank=2, conv=4, mlp=L.moe(experts=3, top=1, ff=20))])
# values that a model may happen to make equal or 1: one head, one group, one state, one tap everywhere, a window of one position and none
# at all, one expert of one, no rotation, every dimension rotated, an embedding scale of one
CFG_ONES = L.make_config([L.mamba2_layer(heads=1, vdim=32, state=1, groups=1, norm_groups=1, conv=1, mlp=L.moe(experts=1, top=1, ff=32)),
                          L.attention_layer(heads=1, kv_heads=1, dim=32, size=1, keep_first=0, rot_dims=32, conv=1, mlp=None),
                          L.mamba1_layer(inner=32, state=1, dt_rank=1, conv=1, mlp=L.moe(experts=4, top=4, ff=8)),
                          L.attention_layer(heads=2, kv_heads=2, dim=16, size=None, rot_dims=0, conv=1),
                          L.attention_layer(heads=2, kv_heads=1, dim=16, size=4, keep_first=4, rot_dims=2)], vocab=61, width=32, taps=1, scale=1.0)
# head widths the tensor-core attention and products take, enough tokens in the tests for the tensor-core products
CFG_TC = L.make_config([L.mamba2_layer(heads=4, vdim=16, state=16, groups=1, norm_groups=4, mlp=L.moe(experts=6, top=2, ff=32)),
                        L.attention_layer(heads=4, kv_heads=2, dim=32, size=40, keep_first=5, rot_dims=16, mlp=L.dense(96)),
                        L.mamba1_layer(inner=128, state=16, dt_rank=8, mlp=L.dense(64)),
                        L.attention_layer(heads=2, kv_heads=1, dim=64, size=None, rot_dims=64, mlp=L.moe(experts=4, top=1, ff=64))], width=64, vocab=128, taps=2)
# sizes that are multiples of nothing
CFG_ODD = L.make_config([L.mamba1_layer(inner=35, state=11, dt_rank=3, conv=2, mlp=L.moe(experts=7, top=4, ff=11)),
                         L.attention_layer(heads=10, kv_heads=1, dim=6, size=45, keep_first=7, rot_dims=2, scale=0.7, conv=5, mlp=L.dense(23)),
                         L.mamba2_layer(heads=3, vdim=7, state=35, groups=1, norm_groups=3, conv=5, mlp=None),
                         L.mamba2_layer(heads=9, vdim=5, state=70, groups=3, norm_groups=5, conv=2, mlp=L.dense(17)),
                         L.attention_layer(heads=9, kv_heads=3, dim=10, size=17, keep_first=1, rot_dims=6, base=77.0, conv=4, mlp=None)], vocab=67, width=50, eps=1e-6,
                        taps=4, scale=2.5)
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


def _forward(cfg, w, toks, layer_outputs=None):
    return O.forward(cfg, _w64(w), toks, layer_outputs)


# ------------------------------------------------------------------------------------------------ mechanisms alone
def _mixer_stub(layer_cfgs, w, width, dtype="float32", eps=EPS):
    import torch

    from simplellminference_b200 import layers
    from simplellminference_b200.config import BF16, F32, KodezenConfig
    from simplellminference_b200.seqops import Ops
    dev = torch.device("cuda")
    ops = Ops(BF16 if dtype == "bfloat16" else F32)
    wt = {k: torch.tensor(v, device=dev, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in w.items()}
    cfg = KodezenConfig.from_dict(L.make_config(layer_cfgs, width=width))
    groups = []
    for i, lc in enumerate(cfg.layers):
        pre = f"l{i}.mix."
        mech = {"mamba2": lambda: layers.StateSpaceDuality(lc.mixer, wt, pre, ops, dev, eps),
                "mamba1": lambda: layers.SelectiveScan(lc.mixer, wt, pre, ops, dev),
                "attention": lambda: layers.TalkingHeadsAttention(lc.mixer, wt, pre, ops, dev, eps)}[lc.type]()
        groups.append(layers.MixerGroup([("mix", mech, 1.0)], ops, dev))

    def fn(step, h, states):
        outs = []
        for g, st in zip(groups, states):
            y = step.scratch("sub_out", step.T * width)
            g.forward(step, h, st, y)
            outs.append(y[:step.T * width].view(step.T, width).clone())
        return outs
    return L.Stub([g.state_spec() for g in groups], fn, ops, dev)


ALONE = [L.mamba2_layer(), L.mamba2_layer(heads=1, vdim=40, state=3, groups=1, norm_groups=5, conv=1), L.mamba2_layer(heads=6, vdim=5, state=33, groups=2, norm_groups=3, conv=6),
         L.mamba2_layer(heads=2, vdim=33, state=130, groups=2, norm_groups=1, conv=2), L.mamba2_layer(heads=8, vdim=80, state=4, groups=1, norm_groups=1, conv=2),
         L.mamba2_layer(heads=16, vdim=64, state=3, groups=2, norm_groups=2, conv=3), L.mamba1_layer(), L.mamba1_layer(inner=70, state=1, dt_rank=1, conv=1),
         L.mamba1_layer(inner=33, state=20, dt_rank=7, conv=6), L.mamba1_layer(inner=8, state=100, dt_rank=3, conv=2), L.mamba1_layer(inner=12, state=203, dt_rank=2, conv=3), L.attention_layer(),
         L.attention_layer(heads=3, kv_heads=3, dim=20, size=9, keep_first=0, rot_dims=20, conv=1), L.attention_layer(heads=8, kv_heads=1, dim=8, size=64, keep_first=10, scale=1.0, rot_dims=2),
         L.attention_layer(heads=6, kv_heads=3, dim=12, size=None, rot_dims=0, conv=5), L.attention_layer(heads=2, kv_heads=2, dim=36, size=5, keep_first=9, conv=2)]


def _oracle_mixer(layer_cfg, w, h, pre="l0.mix.", eps=EPS):
    m, h = layer_cfg["mixer"], h.astype(np.float64)
    if layer_cfg["type"] == "mamba2":
        return O.state_space_duality(h, _w64(w), pre, m, eps)
    if layer_cfg["type"] == "mamba1":
        return O.selective_scan(h, _w64(w), pre, m)
    return O.talking_attention(h, _w64(w), pre, m, eps)


@pytest.mark.parametrize("portions", [[75], [33, 2, 15, 16, 1, 1, 1, 1, 5], [1] * 75])
def test_each_mixer_alone(portions):
    rng = np.random.default_rng(5)
    d, T = 48, 75
    for layer_cfg in ALONE:
        w = L.random_weights(L.make_config([layer_cfg], width=d), seed=11)
        h = rng.standard_normal((T, d)).astype(np.float32)
        got = L.feed(_mixer_stub([layer_cfg], w, d), h, portions)[0]
        want = _oracle_mixer(layer_cfg, w, h)
        assert _rel(got, want) < F32_TOL, (layer_cfg["mixer"], _rel(got, want))


@pytest.mark.parametrize("portions", [[80], [40, 2, 37, 1]])
def test_each_mixer_alone_bf16(portions):
    """bf16 matrices, operands and cache; portions of a prompt take the tensor-core attention where the head widths allow it."""
    rng = np.random.default_rng(7)
    d, T = 64, 80
    for layer_cfg in (L.attention_layer(heads=4, kv_heads=2, dim=32, size=30), L.attention_layer(heads=3, kv_heads=1, dim=12, size=None), L.mamba2_layer(),
                      L.mamba2_layer(heads=4, vdim=16, state=16, groups=1), L.mamba1_layer(), L.mamba1_layer(inner=128, state=16, dt_rank=8)):
        w = L.random_weights(L.make_config([layer_cfg], width=d), seed=13)
        h = L.bf16_round(rng.standard_normal((T, d))).astype(np.float32)
        got = L.feed(_mixer_stub([layer_cfg], w, d, dtype="bfloat16"), h, portions)[0]
        want = _oracle_mixer(layer_cfg, w, h)
        assert _rel(got, want) < BF16_MIXER, (layer_cfg["mixer"], _rel(got, want))


def test_recurrences_over_long_portions_beside_short_ones():
    """Portions longer than a range of the scans (the recurrences then run as passes over ranges: every range from zero, a carry, every
    range again) beside single tokens and short portions of another sequence, cut at, just before and just after the ranges' borders; the
    state a long portion leaves is the one the next step starts from."""
    import torch

    from simplellminference_b200.seqengine import SequenceEngine
    rng = np.random.default_rng(21)
    d, TA, TB = 48, 700, 300
    for layer_cfg in (L.mamba1_layer(), L.mamba1_layer(inner=70, state=1, dt_rank=1, conv=1), L.mamba1_layer(inner=33, state=20, dt_rank=7, conv=6),
                      L.mamba1_layer(inner=8, state=100, dt_rank=3, conv=2), L.mamba2_layer(), L.mamba2_layer(heads=6, vdim=5, state=33, groups=2, norm_groups=3, conv=6)):
        w = L.random_weights(L.make_config([layer_cfg], width=d), seed=17)
        stub = _mixer_stub([layer_cfg], w, d)
        ha, hb = rng.standard_normal((TA, d)).astype(np.float32), rng.standard_normal((TB, d)).astype(np.float32)
        eng = SequenceEngine(stub, max_tokens=1280, max_seqs=2, page_len=32, graphs=False)
        sa, sb = eng.admit(), eng.admit()
        # (tokens of a, tokens of b) per step
        steps = [(129, 1), (1, 128), (256, 1), (127, 130), (2, 1), (185, 39)]
        assert sum(a for a, _ in steps) == TA and sum(b for _, b in steps) == TB
        got_a, got_b, pa, pb = [], [], 0, 0
        for na, nb in steps:
            stub.h = torch.tensor(np.concatenate([ha[pa:pa + na], hb[pb:pb + nb]]), dtype=torch.float32, device=stub.device).contiguous().view(-1)
            eng.run([(sa, np.zeros(na, np.int32), []), (sb, np.zeros(nb, np.int32), [])])
            out = stub.outs[0].cpu().numpy()
            got_a.append(out[:na]); got_b.append(out[na:na + nb])
            pa, pb = pa + na, pb + nb
        assert _rel(np.concatenate(got_a), _oracle_mixer(layer_cfg, w, ha)) < F32_TOL, layer_cfg["mixer"]
        assert _rel(np.concatenate(got_b), _oracle_mixer(layer_cfg, w, hb)) < F32_TOL, layer_cfg["mixer"]


def test_recurrent_state_and_rings_of_a_slot_used_again():
    """A slot that carried one sequence's state and convolution inputs serves another: its first tokens see zeros, not the old state."""
    rng = np.random.default_rng(3)
    d = 48
    from simplellminference_b200.seqengine import SequenceEngine
    for layer_cfg in (L.mamba2_layer(), L.mamba1_layer(), L.attention_layer()):
        w = L.random_weights(L.make_config([layer_cfg], width=d), seed=4)
        stub = _mixer_stub([layer_cfg], w, d)
        eng = SequenceEngine(stub, max_tokens=128, max_seqs=1, page_len=32, graphs=False)
        for T, portions in ((50, [50]), (3, [1, 2]), (40, [2, 38]), (1, [1])):
            h = rng.standard_normal((T, d)).astype(np.float32)
            got = L.feed(stub, h, portions, engine=eng)[0]
            assert _rel(got, _oracle_mixer(layer_cfg, w, h)) < F32_TOL, (layer_cfg["type"], T)


def _standing_out(d, H, window, keep_first):
    """An attention layer and weights in which the query of a position reads the first third of its input row and the key the second
    third, through the same map, with no convolution reaching back, no rotation and a norm without weights: a query row whose first third
    repeats the second third of an earlier row gives that position (and no other, itself included) a score far above the rest.
    The heads are mixed by a full matrix. Returns (layer, weights, third)."""
    t = d // 3
    layer = L.attention_layer(heads=H, kv_heads=H // 2, dim=16, scale=3.0, size=window, keep_first=keep_first, rot_dims=0, conv=2)
    w = L.random_weights(L.make_config([layer], width=d), seed=3)
    a = w["l0.mix.k"][:, :t].copy()
    w["l0.mix.q"][:] = 0.0
    w["l0.mix.k"][:] = 0.0
    # the query heads of a group read through their key head's map
    w["l0.mix.q"][:, :t] = np.repeat(a.reshape(H // 2, 1, 16, t), 2, axis=1).reshape(H * 16, t)
    w["l0.mix.k"][:, t:2 * t] = a
    for n in ("q", "k"):                                    # the convolution passes the current token only
        w[f"l0.mix.{n}.conv"][:] = 0.0
        w[f"l0.mix.{n}.conv"][:, -1] = 1.0
        w[f"l0.mix.{n}.norm"][:] = 1.0
    return layer, w, t


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
def test_keys_just_inside_and_outside_the_window_and_the_kept_first(decode):
    """The key input of an earlier position is repeated as the query input of a later one: when that position is the oldest one inside the
    window, or the last of the kept first positions, the query's output is essentially its value; one further back (or the first position
    that is not kept) it is something else — the restatement says so and the engine has to follow it, with the key before, at and after a
    border of pages of 32."""
    rng = np.random.default_rng(9)
    d, T, H, window, keep = 48, 150, 4, 37, 5
    layer, w, t = _standing_out(d, H, window, keep)
    stub = _mixer_stub([layer], w, d)
    seen = []
    for query in (149, 100, 68, 69, 70):                      # oldest visible key 113 / 64 / 32 / 33 / 34
        for key, visible in ((query - window + 1, True), (query - window, False), (query - 1, True), (keep - 1, True), (keep, False), (0, True)):
            h = rng.standard_normal((T, d)).astype(np.float32)
            h[key, t:2 * t] *= 2.0                          # a long key: no other key's chance alignment with the query comes close
            h[query, :t] = h[key, t:2 * t]
            want = _oracle_mixer(layer, w, h)
            got = L.feed(stub, h, [query] + [1] * (T - query) if decode else [T])[0]
            assert _rel(got, want) < F32_TOL, (query, key, _rel(got, want))
            base = h.copy()
            base[key] = rng.standard_normal(d)
            seen.append((visible, _rel(_oracle_mixer(layer, w, base)[query], want[query])))
    shown = sorted(r for v, r in seen if v)
    assert shown[0] > 0.05 and shown[len(shown) // 2] > 0.3, "a visible repeated position does not stand out: the test would not notice a lost key"
    assert max(r for v, r in seen if not v) < 1e-6, "a hidden position changes the restatement's result"


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
def test_a_key_far_back_among_hundreds(decode):
    """One position hundreds of tokens back (the first token, one at a page border, one in the middle of a page) towers over all others."""
    rng = np.random.default_rng(10)
    d, T, H = 48, 420, 4
    layer, w, t = _standing_out(d, H, 400, 0)
    stub = _mixer_stub([layer], w, d)
    shown = []
    for query, key in ((419, 20), (400, 64), (330, 0), (399, 31)):
        h = rng.standard_normal((T, d)).astype(np.float32)
        h[key, t:2 * t] *= 2.0
        h[query, :t] = h[key, t:2 * t]
        want = _oracle_mixer(layer, w, h)
        got = L.feed(stub, h, [320] + [1] * (T - 320) if decode else [200, 220])[0]
        assert _rel(got, want) < F32_TOL, (query, key, _rel(got, want))
        base = h.copy()
        base[key] = rng.standard_normal(d)
        shown.append(_rel(_oracle_mixer(layer, w, base)[query], want[query]))
    assert min(shown) > 0.3, "the far position does not stand out"


def test_mixed_heads_read_other_heads_weights():
    """With a mixing matrix that gives head 0 the weights of the last head only (another key/value head's query), head 0's output is that
    head's weights on head 0's OWN values: the restatement and the engine agree, and differ from the unmixed result."""
    rng = np.random.default_rng(12)
    d, T = 48, 60
    layer = L.attention_layer(heads=4, kv_heads=2, dim=16, size=None)
    w = L.random_weights(L.make_config([layer], width=d), seed=5)
    talk = np.eye(4, dtype=np.float32)
    talk[0] = [0, 0, 0, 1]
    w["l0.mix.talk"] = talk
    h = rng.standard_normal((T, d)).astype(np.float32)
    want = _oracle_mixer(layer, w, h)
    for portions in ([T], [20] + [1] * 40):
        assert _rel(L.feed(_mixer_stub([layer], w, d), h, portions)[0], want) < F32_TOL
    plain = dict(w)
    plain["l0.mix.talk"] = np.eye(4, dtype=np.float32)
    assert _rel(_oracle_mixer(layer, plain, h), want) > 0.05


def test_long_memory_of_the_recurrent_state():
    """A decay close to one: what a token wrote hundreds of positions back still shows in the output, in a prompt cut into portions and
    in decoding, as the restatement says."""
    rng = np.random.default_rng(14)
    d, T = 48, 400
    for layer_cfg in (L.mamba2_layer(), L.mamba1_layer()):
        w = L.random_weights(L.make_config([layer_cfg], width=d), seed=6)
        if layer_cfg["type"] == "mamba2":
            w["l0.mix.A_log"][:] = -6.0
        else:
            w["l0.mix.A_log"][:] = -6.0
        h = rng.standard_normal((T, d)).astype(np.float32)
        want = _oracle_mixer(layer_cfg, w, h)
        for portions in ([T], [130, 2, 200, 68], [300] + [1] * 100):
            got = L.feed(_mixer_stub([layer_cfg], w, d), h, portions)[0]
            assert _rel(got, want) < F32_TOL, (layer_cfg["type"], portions[:2], _rel(got, want))
        other = h.copy()
        other[3] = rng.standard_normal(d)
        assert _rel(_oracle_mixer(layer_cfg, w, other)[-1], want[-1]) > 1e-3, "the early token has faded: the test would not notice a lost state"


def test_seam_with_channel_weights_alone():
    """Plain residual sum, then the norm with a weight per channel stored around zero and the input convolution, against the restatement;
    in one piece, in portions shorter than the convolution's reach, and as the two halves run separately."""
    import torch

    from simplellminference_b200.config import F32
    from simplellminference_b200.seqops import Ops
    rng, dev, ops = np.random.default_rng(2), torch.device("cuda"), Ops(F32)
    for d, taps, T in ((48, 3, 40), (1000, 4, 19), (50, 1, 9), (36, 7, 30), (52, 3, 150)):
        x, y = (3 * rng.standard_normal((T, d))).astype(np.float32), rng.standard_normal((T, d)).astype(np.float32)
        cw = (0.5 * rng.standard_normal((d, taps))).astype(np.float32)
        nw = (0.3 * rng.standard_normal(d)).astype(np.float32)
        eps = 1e-5
        x_new = x.astype(np.float64) + y
        want = O.input_conv(O.offset_norm(x_new, nw, eps), cw)
        cwt, nwt = torch.tensor(cw, device=dev), torch.tensor(nw, device=dev)
        for split in (False, True):
            def fn(step, h, states):
                n = step.T
                xy = h.view(n, 2 * d)
                xi, yi = xy[:, :d].contiguous(), xy[:, d:].contiguous()
                xo, ho, stash = torch.empty_like(xi), torch.empty_like(xi), step.scratch("stash", n * d)
                ring = states[0].get("ring")
                if split:
                    ops.seam(step.b, xi, d, step.st, x_out=xo, y=yi, post_norm=False)
                    ops.seam(step.b, xo, d, step.st, pre_g=1.0, pre_w=nwt, pre_w_offset=1.0, eps=eps, conv_w=cwt, taps=taps, ring=ring, h=ho, stash=stash)
                else:
                    # with scratch for the per-row scales, steps of 64 tokens and more take the two-launch form
                    ops.seam(step.b, xi, d, step.st, x_out=xo, y=yi, post_norm=False, pre_g=1.0, pre_w=nwt, pre_w_offset=1.0, eps=eps, conv_w=cwt, taps=taps,
                             ring=ring, h=ho, stash=stash, scales=step.scratch("scales", n))
                tail = torch.empty_like(xi)
                ops.seam(step.b, xo, d, step.st, pre_g=1.0, eps=eps, h=tail, stash=stash, flush_ring=ring, flush_taps=taps if ring is not None else 0)
                return [xo, ho]
            spec = {"pages": [], "slots": [("ring", (taps - 1, d))] if taps > 1 else []}
            stub = L.Stub([spec], fn, ops, dev)
            for portions in ([T], [1] * T, [2, 1, 3, T - 6], [T - 3, 3]):
                got = L.feed(stub, np.concatenate([x, y], axis=1), portions)
                assert _rel(got[0], x_new) < 1e-6 and _rel(got[1], want) < 2e-6, (d, taps, split, portions[:3], _rel(got[1], want))


def _ff_stub(mlp, w, d, dtype="float32"):
    import torch

    from simplellminference_b200 import layers
    from simplellminference_b200.config import BF16, F32, KodezenConfig
    from simplellminference_b200.seqops import Ops
    dev, ops = torch.device("cuda"), Ops(BF16 if dtype == "bfloat16" else F32)
    wt = {k: torch.tensor(v, device=dev, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in w.items()}
    c = KodezenConfig.from_dict(L.make_config([L.mamba2_layer(mlp=mlp)], width=d)).layers[0].mlp
    if mlp["kind"] == "dense":
        ff = layers.BiasedFeedForward(c, wt, "l0.mlp.", ops, dev)
    else:
        ff = layers.ExpertsFeedForward(c, wt, "l0.mlp.", ops, dev, activation=2, gated=True, sigmoid_scores=True, scale_input=True)

    def fn(step, h, states):
        y = step.scratch("sub_out", step.T * d)
        ff.forward(step, h, y)
        return [y[:step.T * d].view(step.T, d)]
    return L.Stub([{"pages": [], "slots": []}], fn, ops, dev), ff


def _oracle_ff(mlp, w, h):
    h = h.astype(np.float64)
    return O.dense_ff(h, _w64(w), "l0.mlp.") if mlp["kind"] == "dense" else O.experts_ff(h, _w64(w), "l0.mlp.", mlp)


def test_feed_forwards_alone():
    """The feed-forward with biases and the mixture of gated experts (sigmoid scores, not renormalised, on the experts' inputs)."""
    rng, d, T = np.random.default_rng(4), 40, 37
    for mlp in (L.dense(56), L.moe(), L.moe(experts=9, top=1, ff=7), L.moe(experts=2, top=2, ff=16), L.moe(experts=40, top=8, ff=4), L.moe(experts=1, top=1, ff=5)):
        w = L.random_weights(L.make_config([L.mamba2_layer(mlp=mlp)], width=d), seed=2)
        stub, _ = _ff_stub(mlp, w, d)
        h = (2 * rng.standard_normal((T, d))).astype(np.float32)
        for portions in ([T], [1] * 5 + [T - 5]):
            assert _rel(L.feed(stub, h, portions)[0], _oracle_ff(mlp, w, h)) < F32_TOL, mlp


def test_score_multiplies_the_experts_input_not_its_output():
    """The restatement with the score moved to the output differs visibly: the engine follows the one that scales the input."""
    rng, d, T = np.random.default_rng(8), 40, 20
    mlp = L.moe(experts=4, top=2, ff=16)
    w = L.random_weights(L.make_config([L.mamba2_layer(mlp=mlp)], width=d), seed=3)
    h = (2 * rng.standard_normal((T, d))).astype(np.float64)
    want = O.experts_ff(h, _w64(w), "l0.mlp.", mlp)
    chosen, score = O.route(h, _w64(w), "l0.mlp.", 2)
    other = np.zeros_like(h)
    for t in range(T):
        for e, s in zip(chosen[t], score[t]):
            p = f"l0.mlp.e{int(e)}."
            other[t] += s * ((O.silu(w[p + "gate"].astype(np.float64) @ h[t]) * (w[p + "up"].astype(np.float64) @ h[t])) @ w[p + "down"].astype(np.float64).T)
    assert _rel(other, want) > 0.05
    stub, _ = _ff_stub(mlp, w, d)
    assert _rel(L.feed(stub, h.astype(np.float32), [T])[0], want) < F32_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_with_the_tokens_gathered_per_expert(dtype, monkeypatch):
    """Steps of many tokens multiply a token only with the experts it uses: the same numbers as the form that computes every expert."""
    from simplellminference_b200 import layers
    rng, d, T = np.random.default_rng(14), 64, 150
    for mlp in (L.moe(experts=6, top=2, ff=32), L.moe(experts=5, top=1, ff=24), L.moe(experts=3, top=3, ff=16)):
        w = L.random_weights(L.make_config([L.mamba2_layer(mlp=mlp)], width=d), seed=5)
        stub, ff = _ff_stub(mlp, w, d, dtype)
        h = L.bf16_round(2 * rng.standard_normal((T, d))).astype(np.float32)
        monkeypatch.setattr(layers.ExpertsFeedForward, "gather_min_tokens", 10 ** 9)
        every = L.feed(stub, h, [T])[0]
        monkeypatch.setattr(layers.ExpertsFeedForward, "gather_min_tokens", 64)
        monkeypatch.setattr(layers.ExpertsFeedForward, "gather_launch_cost", 0.0)
        assert ff._gathered_pays(T) == (mlp["router"]["top"] < mlp["router"]["experts"])
        gathered = L.feed(stub, h, [T])[0]
        want = _oracle_ff(mlp, w, h)
        tol = F32_TOL if dtype == "float32" else BF16_MIXER
        assert _rel(gathered, want) < tol and _rel(every, want) < tol, (mlp, _rel(gathered, want), _rel(every, want))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_chosen_on_the_device_in_steps_of_few_tokens(dtype, monkeypatch):
    """Decoding steps stream only the chosen experts' matrices (one launch for all first products, one for all second ones); the score on
    the expert's input is applied to the results of the first products. The same numbers as the form that computes every expert."""
    from simplellminference_b200 import layers
    rng, d = np.random.default_rng(15), 64
    for mlp, T in ((L.moe(experts=12, top=2, ff=32), 3), (L.moe(experts=9, top=1, ff=24), 8), (L.moe(experts=7, top=3, ff=20), 2), (L.moe(experts=5, top=4, ff=8), 1)):
        w = L.random_weights(L.make_config([L.mamba2_layer(mlp=mlp)], width=d), seed=6)
        stub, ff = _ff_stub(mlp, w, d, dtype)
        h = L.bf16_round(2 * rng.standard_normal((T, d))).astype(np.float32)
        monkeypatch.setattr(layers.ExpertsFeedForward, "index_launch_cost", 1e9)
        assert not ff._indexed_pays(T)
        every = L.feed(stub, h, [T])[0]
        monkeypatch.setattr(layers.ExpertsFeedForward, "index_launch_cost", 0.0)
        assert ff._indexed_pays(T)
        indexed = L.feed(stub, h, [T])[0]
        want = _oracle_ff(mlp, w, h)
        tol = F32_TOL if dtype == "float32" else BF16_MIXER
        assert _rel(indexed, want) < tol and _rel(every, want) < tol, (mlp, _rel(indexed, want), _rel(every, want))


# ------------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("cfg", ALL, ids=IDS)
def test_whole_prompt_matches_oracle_fp32_and_layers(tmp_path, cfg):
    w = L.random_weights(cfg, seed=1)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=140).tolist()
    taps_want = []
    want = _forward(cfg, w, toks, taps_want)
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
    # Several layers deep, rounding of the operands is multiplied by what follows it, and a choice of experts that is a near tie may fall
    # the other way: the typical position is held to the rounding, outliers are few. The mechanisms alone are held to the rounding
    # itself in test_each_mixer_alone_bf16.
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
    cfg = L.make_config([L.attention_layer(size=50, keep_first=2), L.mamba2_layer(mlp=L.moe()), L.mamba1_layer(), L.attention_layer(size=130, keep_first=40, mlp=L.moe())])
    w = L.random_weights(cfg, seed=8)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], size=330).tolist()
    want = _forward(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, max_tokens=384, page_len=64)
    s = eng.admit()
    outs = [_logits(eng, s, toks[:60])] + [_logits(eng, s, toks[p:p + 1]) for p in range(60, 330)]
    assert eng.graph_replays > 200
    assert L.logit_error(np.concatenate(outs), want).max() < F32_MODEL


def test_first_tokens_of_a_sequence_after_a_used_slot(tmp_path):
    """A slot (recurrent states, convolution rings) and pages that held a long request serve the next one: its first tokens equal the
    restatement's."""
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
    """bin/trace_run end to end on a Kodezen folder: the model class comes from config.json."""
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
    """python -m simplellminference_b200.generate on a Kodezen folder: registry, engine, scheduler, device arg-max."""
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
