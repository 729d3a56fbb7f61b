"""CPU-side checks of the Kodezen integration: config reader and registry, and the restatement's own properties (visibility through the
window and the kept first positions, causality, the two recurrences against their closed forms, routing, the convolution's reach)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import kodezen_oracle as O  # noqa: E402
import kodezen_testlib as L  # noqa: E402


def test_config_reader(tmp_path):
    from simplellminference_b200.config import (BiasedFeedForwardConfig, ExpertsConfig, KodezenConfig, SelectiveScanConfig, StateSpaceDualityConfig,
                                                read_model_config)
    cfg = L.make_config([L.mamba2_layer(), L.mamba1_layer(mlp=L.moe()), L.attention_layer(mlp=None), L.attention_layer(size=None, rot_dims=0, conv=1)])
    folder = L.write_model(str(tmp_path / "m"), cfg, {"embed": np.zeros((2, 2), np.float32)})
    c = read_model_config(folder)
    assert isinstance(c, KodezenConfig) and (c.vocab, c.width, c.norm_eps, c.conv_taps, c.embedding_scale) == (83, 48, 1e-5, 3, 3.0)
    a, b, e, f = (l.mixer for l in c.layers)
    assert a == StateSpaceDualityConfig(4, 8, 12, 2, 2, 4) and b == SelectiveScanConfig(40, 6, 5, 3)
    assert (e.heads, e.kv_heads, e.dim, e.vdim, e.scale, e.mask.size, e.mask.keep_first, e.rot.dims, e.rot.base, e.conv) == (4, 2, 16, 16, 0.3, 20, 3, 8, 1000.0, 3)
    assert f.rot is None and f.mask.size is None and f.conv == 1
    assert c.layers[0].mlp == BiasedFeedForwardConfig(40) and c.layers[1].mlp == ExpertsConfig(5, 0, 2, 12) and c.layers[2].mlp is None
    bare = KodezenConfig.from_dict({"architecture": "Kodezen", "vocab": 5, "width": 4, "layers": []})      # what is not named does not exist
    assert (bare.conv_taps, bare.embedding_scale, bare.norm_eps) == (1, 1.0, 1e-6)
    with pytest.raises(ValueError, match="unknown mixer type"):
        KodezenConfig.from_dict(L.make_config([dict(L.mamba1_layer(), type="conv")]))
    with pytest.raises(ValueError, match="not part of this design"):
        KodezenConfig.from_dict(L.make_config([L.mamba1_layer(mlp={"kind": "sparse"})]))
    with pytest.raises(ValueError, match="do not divide"):
        KodezenConfig.from_dict(L.make_config([L.mamba2_layer(heads=5, groups=2)]))
    with pytest.raises(ValueError, match="do not divide"):
        KodezenConfig.from_dict(L.make_config([L.attention_layer(heads=5, kv_heads=2)]))
    with pytest.raises(ValueError, match="rotary"):
        KodezenConfig.from_dict(L.make_config([L.attention_layer(dim=8, rot_dims=10)]))
    with pytest.raises(ValueError, match="experts"):
        KodezenConfig.from_dict(L.make_config([L.mamba1_layer(mlp=L.moe(experts=2, top=4))]))


def test_registry_knows_the_design():
    from simplellminference_b200.config import CONFIG_READERS
    from simplellminference_b200.models import MODEL_CLASSES
    assert all(n in MODEL_CLASSES and n in CONFIG_READERS for n in ("Kodezen", "Vasosun", "Sopetar", "Munazen"))


def test_window_kept_positions_and_causality_of_the_restatement():
    rng = np.random.default_rng(0)
    d, n = 24, 30
    layer = L.attention_layer(heads=2, kv_heads=1, dim=8, size=5, keep_first=2, conv=2)
    w = {k: v.astype(np.float64) for k, v in L.random_weights(L.make_config([layer], width=d), seed=1).items()}
    h = rng.standard_normal((n, d))
    base = O.talking_attention(h, w, "l0.mix.", layer["mixer"], 1e-5)
    # a change at position c reaches c's key and, through the convolution of two taps, the key of c + 1: the window of 5 carries it to c + 5
    h2 = h.copy()
    h2[10] += 1.0
    moved = np.abs(O.talking_attention(h2, w, "l0.mix.", layer["mixer"], 1e-5) - base).max(axis=1) > 1e-12
    assert moved[:10].sum() == 0 and moved[10:16].all() and moved[16:].sum() == 0
    # position 0 is kept: every later position sees it; position 2 is not, and its key leaves with the window
    h2 = h.copy()
    h2[0] += 1.0
    assert (np.abs(O.talking_attention(h2, w, "l0.mix.", layer["mixer"], 1e-5) - base).max(axis=1) > 1e-12).all()
    see = O.visible(12, 5, 2)
    assert see[11, 0] and see[11, 1] and not see[11, 2] and not see[11, 6] and see[11, 7] and not see[3, 4]


def test_rotation_of_the_restatement():
    x = np.zeros((3, 1, 6))
    x[:, 0, 0] = x[:, 0, 4] = 1.0
    y = O.rotate_pairs(x, np.arange(3), 4, 100.0)
    np.testing.assert_allclose(y[2, 0, :2], [np.cos(2.0), np.sin(2.0)])        # pair (0, 1) turns by pos * 1
    np.testing.assert_allclose(y[:, 0, 4], 1.0)                                # beyond the rotary dimensions nothing turns
    a, b = np.random.default_rng(1).standard_normal((2, 1, 1, 6))
    dots = [float(O.rotate_pairs(a, [p], 6, 50.0)[0, 0] @ O.rotate_pairs(b, [p - 3], 6, 50.0)[0, 0]) for p in (3, 10, 40)]
    np.testing.assert_allclose(dots, dots[0])                                  # a score depends on the distance only


def test_recurrences_of_the_restatement():
    """One head, one channel: the state-space form and the selective scan against their sums written out."""
    n = 6
    rng = np.random.default_rng(2)
    m = {"heads": 1, "vdim": 1, "state": 2, "groups": 1, "norm_groups": 1, "conv": 1}
    d = 3
    W = {k: v.astype(np.float64) for k, v in L.random_weights(L.make_config([dict(L.mamba2_layer(), mixer=m)], width=d), seed=3).items()}
    h = rng.standard_normal((n, d))
    u = h @ W["l0.mix.in"].T
    z, xbc, dt = u[:, :1], O.silu(u[:, 1:6] * W["l0.mix.conv"][:, 0] + W["l0.mix.conv.b"]), O.softplus(u[:, 6] + W["l0.mix.dt_bias"][0])
    x, B, C = xbc[:, 0], xbc[:, 1:3], xbc[:, 3:5]
    a = np.exp(-np.exp(W["l0.mix.A_log"][0]) * dt)
    y = np.array([sum(np.prod(a[s + 1:t + 1]) * dt[s] * x[s] * (B[s] @ C[t]) for s in range(t + 1)) + W["l0.mix.D"][0] * x[t] for t in range(n)])
    y = (y * O.silu(z[:, 0]))[:, None]
    want = (y / np.sqrt(y * y + 1e-5) * W["l0.mix.norm"]) @ W["l0.mix.o"].T
    np.testing.assert_allclose(O.state_space_duality(h, W, "l0.mix.", m, 1e-5), want, rtol=1e-10, atol=1e-12)
    m = {"inner": 1, "state": 2, "dt_rank": 1, "conv": 1}
    W = {k: v.astype(np.float64) for k, v in L.random_weights(L.make_config([dict(L.mamba1_layer(), mixer=m)], width=d), seed=4).items()}
    u = h @ W["l0.mix.in"].T
    x, z = O.silu(u[:, 0] * W["l0.mix.conv"][0, 0] + W["l0.mix.conv.b"][0]), u[:, 1]
    low = x[:, None] * W["l0.mix.x"][:, 0]
    dt = O.softplus(low[:, 0] * W["l0.mix.dt"][0, 0] + W["l0.mix.dt.b"][0])
    A = -np.exp(W["l0.mix.A_log"][0])
    y = np.array([sum(np.exp(dt[s + 1:t + 1].sum() * A[k]) * dt[s] * x[s] * low[s, 1 + k] * low[t, 3 + k] for s in range(t + 1) for k in range(2))
                  + W["l0.mix.D"][0] * x[t] for t in range(n)])
    np.testing.assert_allclose(O.selective_scan(h, W, "l0.mix.", m), (y * O.silu(z))[:, None] @ W["l0.mix.o"].T, rtol=1e-10, atol=1e-12)


def test_routing_of_the_restatement():
    w = {"r.router": np.array([[1.0], [2.0], [-3.0], [1.5]])}
    chosen, weight = O.route(np.array([[1.0]]), w, "r.", 2)
    assert chosen[0].tolist() == [1, 3]
    np.testing.assert_allclose(weight[0], O.sigmoid(np.array([2.0, 1.5])))     # each score by itself: they do not sum to one
    # one expert whose matrices are ones: silu(s * sum h) * (s * sum h), for each output channel
    mlp = {"router": {"experts": 1, "top": 1}, "expert": {"ff": 1}}
    W = {"m.router": np.array([[0.5, 0.5]]), "m.e0.gate": np.ones((1, 2)), "m.e0.up": np.ones((1, 2)), "m.e0.down": np.ones((2, 1))}
    h = np.array([[2.0, -1.0]])
    s = O.sigmoid(0.5)
    np.testing.assert_allclose(O.experts_ff(h, W, "m.", mlp), np.full((1, 2), O.silu(s) * s))


def test_convolutions_of_the_restatement():
    h = np.arange(1.0, 5.0)[:, None]
    w = np.array([[100.0, 10.0, 1.0]])                       # the last column is the current token's
    np.testing.assert_allclose(O.causal_conv(h, w)[:, 0], [1, 12, 123, 234])
    np.testing.assert_allclose(O.input_conv(h, w)[:, 0], [2, 14, 126, 238])
    np.testing.assert_allclose(O.causal_conv(h, w, [0.5])[:, 0], [1.5, 12.5, 123.5, 234.5])
    np.testing.assert_allclose(O.offset_norm(np.array([[3.0, 4.0]]), np.array([0.0, 1.0]), 0.0), [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])


def test_bench_geometries_are_valid_configurations():
    """The sizes of ``bench.py --kodezen`` parse, keep the layer pattern and differ from one another only in width and depth."""
    from simplellminference_b200.bench_kodezen import SIZES, kodezen_config
    from simplellminference_b200.config import KodezenConfig
    for name, size in SIZES.items():
        cfg = KodezenConfig.from_dict(kodezen_config(size["width"], size["repeats"]))
        assert cfg.width == size["width"] and len(cfg.layers) == 4 * size["repeats"], name
        assert [l.type for l in cfg.layers[:4]] == ["mamba2", "mamba1", "mamba2", "attention"]
        assert all(l.mixer.heads * l.mixer.vdim == 2 * cfg.width for l in cfg.layers if l.type == "mamba2")
