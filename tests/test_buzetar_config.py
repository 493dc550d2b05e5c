"""Buzetar without a GPU: its configuration reader, what the builder asks of weights and cache, and the plain
implementation's mechanisms against closed forms."""
import copy

import numpy as np
import pytest

import plain_buzetar as plain

CFG = {
    "architecture": "Buzetar", "vocab": 120, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0}, "logit_scale": 0.5,
    "layers": [
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "conv": 3}, "mlp": {"kind": "dense", "ff": 40, "limit": 1.5}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "rot_dim": 6, "vdim": 10, "q_rank": 20, "kv_rank": 14, "scale": 0.3,
                                               "rot": {"base": 10000.0, "dims": 4}, "mask": {"size": 9}}, "mlp": None},
        {"type": "lightning", "mixer": {"heads": 2, "dim": 6, "vdim": 5, "decay": [1.0, 0.5]}, "mlp": {"kind": "dense", "ff": 16, "limit": 2.0}},
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 8, "rot_dim": 4, "vdim": 8, "q_rank": 8, "kv_rank": 8, "scale": 1.0,
                                               "rot": {"base": 100.0, "dims": 4}}, "mlp": None},
    ]}


def test_configuration_is_read_written_back_and_refused_by_name():
    from llmx_b200.config import BuzetarConfig, ConfigError
    c = BuzetarConfig.from_dict(CFG)
    assert BuzetarConfig.from_dict(c.to_dict()) == c
    assert c.layers[1].mixer.window == 9 and c.layers[3].mixer.window is None and c.layers[1].mixer.rot_dims == 4
    assert c.layers[1].mlp is None and c.layers[2].mlp.ff == 16 and c.layers[2].mixer.decay == (1.0, 0.5)
    assert BuzetarConfig.from_dict(dict(CFG, note="x")).ignored == ("note",)

    def broken(path, value):
        raw = copy.deepcopy(CFG)
        node = raw
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        return raw

    for path, value, word in ((("layers", 0, "type"), "conv", "mixer type"), (("layers", 2, "mixer", "decay"), [0.5], "decay"),
                              (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 1, "mixer", "rot", "dims"), 3, "rot.dims"),
                              (("layers", 1, "mixer", "rot", "dims"), 8, "rot.dims"), (("layers", 0, "mlp", "kind"), "routed", "mlp.kind"),
                              (("layers", 1, "mixer", "mask"), {"size": 0}, "mask.size"), (("width",), 0, "width"),
                              (("layers",), [], "layers"), (("norm",), None, "norm"), (("layers", 0, "mixer", "conv"), 0, "conv")):
        with pytest.raises(ConfigError) as e:
            BuzetarConfig.from_dict(broken(path, value))
        assert word in str(e.value), (path, str(e.value))


def test_registry_builds_the_model_and_names_its_tensors_and_cache_needs():
    from llmx_b200.cache import CacheManager, KVSpec, StateSpec
    from llmx_b200.registry import architecture_of
    entry = architecture_of(CFG)
    model = entry.build(entry.config_cls.from_dict(CFG))
    specs = model.tensor_specs()
    assert specs["embed"].shape == (120, 48) and specs["head"].shape == (120, 48) and specs["final.norm"].shape == (48,)
    assert specs["l0.norm1"].shape == (48,) and specs["l0.mix.q.conv"].shape == (24, 3) and specs["l0.mix.v.conv"].shape == (40, 3)
    assert specs["l0.mix.b"].shape == (4, 48) and specs["l0.mix.A_log"].shape == (4,) and specs["l0.mix.norm"].shape == (10,)
    assert specs["l1.mix.dkv"].shape == (20, 48) and specs["l1.mix.dkv.norm"].shape == (14,) and specs["l1.mix.uq"].shape == (42, 20)
    assert specs["l1.mix.uk"].shape == (24, 14) and specs["l1.mix.uv"].shape == (30, 14) and specs["l1.mix.o"].shape == (48, 30)
    assert specs["l2.mix.q"].shape == (12, 48) and specs["l2.mix.v"].shape == (10, 48) and specs["l2.mix.norm"].shape == (10,)
    assert "l1.mlp.gate" not in specs and specs["l2.mlp.down"].shape == (48, 16)
    needs = model.cache_entry_specs()
    assert needs[0] == StateSpec((4 * 10 * 12 + 2 * (24 + 24 + 40),), "float32")
    assert needs[1] == KVSpec(1, 20, 9, planes=1) and needs[3] == KVSpec(1, 12, None, planes=1)
    assert needs[2] == StateSpec((2 * 5 * 6,), "float32")
    import torch
    cache = CacheManager(needs, 4, 64, 2, kv_dtype=torch.float32, device="cpu")
    assert sorted(tuple(g.storage.shape) for g in cache.groups) == [(1, 16, 1, 1, 4, 12), (1, 16, 1, 1, 4, 20)]
    assert cache.state_slots.num_slots == 4


def test_plain_decayed_recurrence_is_the_weighted_sum_over_the_past():
    rng = np.random.default_rng(0)
    T, H, D, V = 9, 2, 3, 4
    q, k, v = rng.normal(size=(T, H, D)), rng.normal(size=(T, H, D)), rng.normal(size=(T, H, V))
    decay = np.array([0.7, 1.0])
    got = plain.decayed_linear_attention(q, k, v, decay)
    for h in range(H):
        for t in range(T):
            want = sum(decay[h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert np.allclose(got[t, h], want)


def test_plain_delta_rule_stores_and_overwrites():
    """With unit keys, beta 1 and no decay, writing v under key k and reading with q = k returns v; writing again under
    the same key replaces it; an orthogonal key leaves it."""
    e0, e1 = np.array([1.0, 0, 0]), np.array([0, 1.0, 0])
    k = np.stack([e0, e1, e0, e0])[:, None, :]
    v = np.array([[1.0, 2], [3, 4], [5, 6], [7, 8]])[:, None, :]
    q = np.stack([e0, e0, e0, e1])[:, None, :]
    one = np.ones((4, 1))
    out = plain.gated_delta_rule(q, k, v, one, one)[:, 0]
    assert np.allclose(out, [[1, 2], [1, 2], [5, 6], [3, 4]])
    half = plain.gated_delta_rule(q, k, v, 0.5 * one, one)[:, 0]
    assert np.allclose(half[0], [0.5, 1.0]) and np.allclose(half[2], [0.5 * 0.5 + 0.5 * 5, 0.5 * 1.0 + 0.5 * 6])
    decayed = plain.gated_delta_rule(q, k, v, one, 0.5 * one)[:, 0]
    assert np.allclose(decayed[1], [0.5, 1.0])          # read after one decay of the first write


def test_plain_window_rotation_and_filter():
    rng = np.random.default_rng(1)
    T = 12
    q, k, v = rng.normal(size=(T, 1, 4)), rng.normal(size=(T, 1, 4)), rng.normal(size=(T, 1, 3))
    full = plain.windowed_softmax_attention(q, k, v, 0.5, None)
    win = plain.windowed_softmax_attention(q, k, v, 0.5, 5)
    assert np.allclose(full[:5], win[:5]) and not np.allclose(full[5], win[5])
    v2 = v.copy()
    v2[2] += 1.0
    win2 = plain.windowed_softmax_attention(q, k, v2, 0.5, 5)
    assert not np.allclose(win[6], win2[6]) and np.array_equal(win[7:], win2[7:])       # position 6 still sees 2; 7 does not
    # Rotation: lengths are kept, the unrotated rest passes, and a product depends on the distance alone.
    x, y = rng.normal(size=(1, 8)), rng.normal(size=(1, 8))
    dots = []
    for p in (0, 5, 40):
        a, b = plain.rotate_interleaved(x, [p + 3], 100.0, 6), plain.rotate_interleaved(y, [p], 100.0, 6)
        assert np.allclose(np.linalg.norm(a), np.linalg.norm(x)) and np.array_equal(a[:, 6:], x[:, 6:])
        dots.append(float(a[0] @ b[0]))
    assert np.allclose(dots, dots[0])
    u = plain.rotate_interleaved(np.array([[1.0, 0.0]]), [1], 10.0, 2)
    assert np.allclose(u, [[np.cos(1.0), np.sin(1.0)]])
    # The filter: the last tap weighs the current token; nothing before the start.
    xs = rng.normal(size=(6, 2))
    taps = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = plain.causal_conv(xs, taps)
    assert np.allclose(y[:, 1], xs[:, 1]) and np.isclose(y[0, 0], 100 * xs[0, 0]) and np.isclose(y[2, 0], xs[0, 0] + 10 * xs[1, 0] + 100 * xs[2, 0])
