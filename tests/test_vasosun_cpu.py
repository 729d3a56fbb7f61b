"""CPU-side checks of the Vasosun integration: config reader and registry, the scaled rotary frequencies against the plain restatement,
and the restatement's own properties (visibility through the window, causality, the delta rule's memory, routing)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import vasosun_oracle as O  # noqa: E402
import vasosun_testlib as L  # noqa: E402


def test_config_reader(tmp_path):
    from simplellminference_b200.config import DeltaRuleConfig, ExpertsConfig, GatedFeedForwardConfig, VasosunConfig, read_model_config
    cfg = L.make_config([L.attention_layer(), L.latent_layer(mlp=L.moe()), L.latent_layer(heads=5, kv_from=1, mlp=None), L.delta_layer(conv=4),
                         L.attention_layer(size=None, every=0)])
    folder = L.write_model(str(tmp_path / "m"), cfg, {"embed": np.zeros((2, 2), np.float32)})
    c = read_model_config(folder)
    assert isinstance(c, VasosunConfig) and (c.vocab, c.width, c.norm_eps, c.conv_taps, c.logit_softcap) == (83, 48, 1e-5, 3, 12.0)
    assert (c.pair_buckets, c.pair_mul_prev, c.pair_mul_cur) == (53, 31, 7)
    a, b, e, f, g = (l.mixer for l in c.layers)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.mask.size, a.q_temp_coef, a.q_temp_every) == (4, 2, 16, 24, 0.3, 20, 0.4, 7)
    assert (b.heads, b.dim, b.rot_dim, b.vdim, b.kv_rank, b.q_rank, b.kv_from, b.mask.size) == (3, 8, 12, 20, 40, 24, None, None)
    assert b.rot.scaling == {"factor": 4.0, "original": 24, "fast": 4.0, "slow": 1.0} and (e.heads, e.kv_from) == (5, 1)
    assert f == DeltaRuleConfig(4, 2, 16, 12, 4) and g.mask.size is None and g.q_temp_every == 0
    assert c.layers[0].mlp == GatedFeedForwardConfig(40) and c.layers[1].mlp == ExpertsConfig(5, 2, 3, 12) and c.layers[2].mlp is None
    with pytest.raises(ValueError, match="unknown mixer type"):
        VasosunConfig.from_dict(L.make_config([dict(L.delta_layer(), type="conv")]))
    with pytest.raises(ValueError, match="not part of this design"):
        VasosunConfig.from_dict(L.make_config([L.delta_layer(mlp={"kind": "sparse"})]))
    with pytest.raises(ValueError, match="kv_from"):
        VasosunConfig.from_dict(L.make_config([L.latent_layer(kv_from=1), L.latent_layer()]))
    with pytest.raises(ValueError, match="kv_from"):
        VasosunConfig.from_dict(L.make_config([L.latent_layer(), L.latent_layer(kv_rank=8, kv_from=0)]))
    with pytest.raises(ValueError, match="kv_from"):
        VasosunConfig.from_dict(L.make_config([L.latent_layer(), L.latent_layer(kv_from=0), L.latent_layer(kv_from=1)]))
    with pytest.raises(ValueError, match="do not divide"):
        VasosunConfig.from_dict(L.make_config([L.delta_layer(heads=5, kv_heads=2)]))
    with pytest.raises(ValueError, match="experts"):
        VasosunConfig.from_dict(L.make_config([L.delta_layer(mlp=L.moe(experts=2, identity=1, top=4))]))


def test_registry_knows_the_design():
    from simplellminference_b200.config import CONFIG_READERS
    from simplellminference_b200.models import MODEL_CLASSES
    assert all(n in MODEL_CLASSES and n in CONFIG_READERS for n in ("Vasosun", "Sopetar", "Munazen"))


@pytest.mark.parametrize("scaling", [None, {"factor": 4.0, "original": 24, "fast": 4.0, "slow": 1.0}, {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0}])
def test_scaled_frequencies(scaling):
    from simplellminference_b200.layers import yarn_frequencies
    for dims, base in ((4, 100.0), (16, 1e6), (64, 1e4)):
        f, mag = yarn_frequencies(dims, base, scaling)
        fo, mo = O.yarn_table(dims, base, scaling)
        np.testing.assert_allclose(f, fo, rtol=1e-14)
        assert abs(mag - mo) < 1e-15
        if scaling:
            assert f[0] <= base ** 0 and f[-1] >= base ** (-2.0 * (dims // 2 - 1) / dims) / scaling["factor"] * (1 - 1e-12)


def test_window_and_causality_of_the_restatement():
    rng = np.random.default_rng(0)
    d, n = 24, 30
    layer = L.attention_layer(heads=2, kv_heads=1, dim=8, vdim=8, size=5)
    w = {k: v.astype(np.float64) for k, v in L.random_weights(L.make_config([layer], width=d), seed=1).items()}
    h = rng.standard_normal((n, d))
    base = O.window_attention(h, w, "l0.mix.", layer["mixer"])
    for changed, first_moved in ((10, 10), (29, 29)):
        h2 = h.copy()
        h2[changed] += 1.0
        moved = np.abs(O.window_attention(h2, w, "l0.mix.", layer["mixer"]) - base).max(axis=1) > 1e-12
        assert moved[:first_moved].sum() == 0 and moved[changed] and moved[changed + 5:].sum() == 0       # nothing earlier, nothing beyond the window
        assert moved[changed:changed + 5].all()


def test_delta_rule_of_the_restatement():
    """With beta = 1, no decay and unit keys the rule stores v under k exactly: reading with the same key returns v, an orthogonal key 0."""
    k = np.eye(4)[[0, 1, 0]]
    v = np.array([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    o = O.delta_rule(k, k, v, np.ones(3), np.ones(3))
    np.testing.assert_allclose(o, v)                        # position 2 overwrote what position 0 stored under the same key
    o = O.delta_rule(np.eye(4)[[2, 2, 1]], k, v, np.ones(3), np.ones(3))
    np.testing.assert_allclose(o, [[0, 0], [0, 0], [3, 4]])
    o = O.delta_rule(k, k, v, np.ones(3), np.array([1.0, 0.5, 0.5]))
    np.testing.assert_allclose(o[2], v[2])                  # the decay shrinks what is stored, the write corrects to v again


def test_routing_of_the_restatement():
    w = {"r.router": np.array([[1.0], [2.0], [0.0], [1.5]]), "r.correction": np.array([0.0, -1.0, 1.0, 0.0])}
    chosen, weight = O.route(np.array([[1.0]]), w, "r.", 2)
    s = O.softmax(np.array([[1.0, 2.0, 0.0, 1.5]]))
    assert sorted(chosen[0].tolist()) == [2, 3]              # the correction moves the choice from expert 1 to expert 2 ...
    np.testing.assert_allclose(sorted(weight[0]), sorted(s[0, [2, 3]]))   # ... and stays out of the weights, which do not sum to one
    h = np.array([[2.0, -1.0]])
    mlp = {"router": {"experts": 0, "identity": 2, "top": 1}, "expert": {"ff": 1}}
    out = O.moe_ff(h, {"m.router": np.array([[1.0, 0.0], [0.0, 1.0]]), "m.correction": np.zeros(2)}, "m.", mlp)
    np.testing.assert_allclose(out, O.softmax(np.array([[2.0, -1.0]]))[0, 0] * h)     # an identity expert returns its input times the weight


def test_pair_rows_of_the_restatement():
    table, pairs = np.zeros((5, 2)), np.arange(8, dtype=np.float64).reshape(4, 2)      # 3 buckets + the first token's row
    x = O.embed([4, 1, 1], table, pairs, 3, 2, 5)
    np.testing.assert_allclose(x, pairs[[3, (4 * 2 + 1 * 5) % 3, (1 * 2 + 1 * 5) % 3]])
