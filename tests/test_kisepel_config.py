"""Kisepel without a GPU: its configuration reader, what the builder asks of weights and cache, the order its layers
run in, pages given back at the edge of a chunk, and the plain implementation's mechanisms against closed forms."""
import copy

import numpy as np
import pytest

import plain_kisepel as plain

MOE = {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24}, "shared": {"ff": 40}}
CFG = {
    "architecture": "Kisepel", "vocab": 130, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0}, "logit_scale": 0.5,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "lightning", "mixer": {"heads": 2, "dim": 6, "vdim": 5, "decay": [1.0, 0.5]}, "mlp": MOE},
        {"type": "mamba2", "mixer": {"heads": 6, "vdim": 4, "state": 10, "groups": 3, "conv": 4, "norm_groups": 2}, "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.3, "mask": {"size": 9},
                     "rot": {"base": 10000.0, "dims": 8, "scaling": {"factor": 2.0}}},
            "right": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "conv": 3, "decay_rank": 7, "gate_rank": 5}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 16}, "shared": None}},
        {"type": "mamba2", "mixer": {"heads": 2, "vdim": 8, "state": 4, "groups": 1, "conv": 2, "norm_groups": 1}, "mlp": MOE},
    ]}


def test_configuration_is_read_written_back_and_refused_by_name():
    from llmx_b200.config import ConfigError, KisepelConfig
    c = KisepelConfig.from_dict(CFG)
    assert KisepelConfig.from_dict(c.to_dict()) == c
    left, right = c.layers[2].mixer.left, c.layers[2].mixer.right
    assert left.chunk == 9 and left.rot_dims == 8 and left.rot_factor == 2.0 and left.vdim == 10 and right.decay_rank == 7
    assert c.layers[1].mlp is None and c.layers[2].mlp.shared_ff is None and c.layers[0].mlp.shared_ff == 40 and c.layers[0].mlp.top == 2
    assert c.loop.start == 1 and c.loop.times == 3 and c.layers[1].mixer.norm_groups == 2
    assert KisepelConfig.from_dict(dict(CFG, note="x")).ignored == ("note",)
    bare = copy.deepcopy(CFG)
    del bare["loop"], bare["layers"][2]["mixer"]["left"]["rot"]["scaling"], bare["layers"][2]["mixer"]["left"]["mask"]
    del bare["layers"][2]["mixer"]["right"]["decay_rank"], bare["layers"][2]["mixer"]["right"]["gate_rank"]
    b = KisepelConfig.from_dict(bare)
    assert b.loop.times == 1 and b.layers[2].mixer.left.chunk is None and b.layers[2].mixer.left.rot_factor == 1.0
    assert b.layers[2].mixer.right.decay_rank is None and [i for i, _ in b.layer_runs()] == [0, 1, 2, 3]

    def broken(path, value):
        raw = copy.deepcopy(CFG)
        node = raw
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        return raw

    for path, value, word in ((("layers", 0, "type"), "conv", "mixer type"), (("layers", 0, "mixer", "decay"), [0.5], "decay"),
                              (("layers", 1, "mixer", "groups"), 4, "groups"), (("layers", 1, "mixer", "norm_groups"), 5, "norm_groups"),
                              (("layers", 2, "mixer", "left", "rot", "dims"), 3, "rot.dims"), (("layers", 2, "mixer", "left", "rot", "dims"), 14, "rot.dims"),
                              (("layers", 2, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("layers", 2, "mixer", "right", "kv_heads"), 3, "kv_heads"),
                              (("layers", 2, "mixer", "left", "mask"), {"size": 0}, "mask.size"), (("layers", 0, "mlp", "kind"), "dense", "mlp.kind"),
                              (("layers", 0, "mlp", "router", "top"), 6, "top"), (("loop",), {"start": 2, "stop": 1, "times": 2}, "loop"),
                              (("loop",), {"start": 0, "stop": 5, "times": 2}, "loop"), (("loop", "times"), 0, "times"),
                              (("width",), 0, "width"), (("layers",), [], "layers"), (("norm",), None, "norm"),
                              (("layers", 1, "mixer", "conv"), 0, "conv"), (("layers", 2, "mixer", "left", "rot", "scaling"), {"factor": 0}, "factor")):
        with pytest.raises(ConfigError) as e:
            KisepelConfig.from_dict(broken(path, value))
        assert word in str(e.value), (path, str(e.value))


def test_registry_builds_the_model_and_names_its_tensors_cache_needs_and_order():
    from llmx_b200.cache import KVSpec, StateSpec
    from llmx_b200.registry import architecture_of
    entry = architecture_of(CFG)
    model = entry.build(entry.config_cls.from_dict(CFG))
    specs = model.tensor_specs()
    assert specs["embed"].shape == (130, 48) and "head" not in specs and specs["final.norm"].shape == (48,)
    assert specs["l0.mix.q"].shape == (12, 48) and specs["l0.mix.v"].shape == (10, 48) and specs["l0.mix.norm"].shape == (10,)
    assert specs["l0.mlp.table"].shape == (130, 2) and specs["l0.mlp.table"].kind == "int_table"
    assert specs["l0.mlp.e4.gate"].shape == (24, 48) and specs["l0.mlp.e0.down"].shape == (48, 24) and specs["l0.mlp.shared.up"].shape == (40, 48)
    assert "l0.mlp.e5.gate" not in specs and "l1.mlp.table" not in specs and "l2.mlp.shared.gate" not in specs
    assert specs["l1.mix.in"].shape == (2 * 24 + 2 * 30 + 6, 48) and specs["l1.mix.conv"].shape == (24 + 60, 4)
    assert specs["l1.mix.conv.b"].shape == (84,) and specs["l1.mix.D"].shape == (6,) and specs["l1.mix.norm"].shape == (24,)
    assert specs["l2.mix.left.q"].shape == (48, 48) and specs["l2.mix.left.k"].shape == (24, 48) and specs["l2.mix.left.v"].shape == (20, 48)
    assert specs["l2.mix.left.o"].shape == (48, 40) and specs["l2.mix.left.q.norm"].shape == (12,) and specs["l2.mix.left.out"].shape == (48,)
    assert specs["l2.mix.right.q"].shape == (12, 48) and specs["l2.mix.right.v"].shape == (40, 48) and specs["l2.mix.right.v.conv"].shape == (40, 3)
    assert specs["l2.mix.right.a1"].shape == (7, 48) and specs["l2.mix.right.a2"].shape == (24, 7) and specs["l2.mix.right.dt_bias"].shape == (24,)
    assert specs["l2.mix.right.g1"].shape == (5, 48) and specs["l2.mix.right.g2"].shape == (40, 5) and specs["l2.mix.right.norm"].shape == (10,)
    assert specs["l2.mix.right.b"].shape == (4, 48) and specs["l2.mix.right.A_log"].shape == (4,) and specs["l2.mix.right.out"].shape == (48,)
    # Layers 1 and 2 run three times, each run with cache entries of its own; the embedding output joins before the
    # second and third pass.
    assert [(s.block, s.add_embedding) for s in model.order] == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert [s.cache_entry for s in model.order] == [0, 1, (2, 3), 4, (5, 6), 7, (8, 9), 10]
    needs = model.cache_entry_specs()
    assert needs[0] == StateSpec((2 * 6 * 5,), "float32")
    assert needs[1] == needs[4] == needs[7] == StateSpec((6 * 4 * 10 + 3 * 84,), "float32")
    assert needs[2] == needs[5] == KVSpec(2, 12 + 10, None, planes=1, chunk=9)
    assert needs[3] == StateSpec((4 * 10 * 6 + 2 * (12 + 12 + 40),), "float32")
    # Ranks the configuration does not name are left open for the stored tensors to give.
    bare = copy.deepcopy(CFG)
    del bare["layers"][2]["mixer"]["right"]["decay_rank"], bare["layers"][2]["mixer"]["right"]["gate_rank"]
    open_specs = entry.build(entry.config_cls.from_dict(bare)).tensor_specs()
    assert open_specs["l2.mix.right.a1"].shape == (-1, 48) and open_specs["l2.mix.right.g2"].shape == (40, -1)


def test_random_tables_name_different_experts_in_every_row():
    from llmx_b200.weights import RandomSource
    from llmx_b200.weights.spec import TensorSpec
    src = RandomSource({"t": TensorSpec((500, 3), "int_table", init="distinct_rows", bound=5)}, seed=4)
    t = src.tensor("t").numpy()
    assert t.min() == 0 and t.max() == 4 and all(len(set(row)) == 3 for row in t)
    assert len({tuple(r) for r in t}) > 20


def test_pages_below_the_chunk_of_the_next_position_are_given_back():
    from llmx_b200.cache.pages import RELEASED, BlockTable, PagePool
    pool = PagePool(16)
    t = BlockTable(pool, 4, chunk=10)
    t.prepare(9)
    t.commit()
    assert t.held_pages == 3                      # position 9 still sees 0..8
    t.prepare(1)
    t.commit()                                    # ten tokens: position 10 starts a chunk, nothing below it is seen again
    assert t.pages[:2] == [RELEASED, RELEASED] and t.held_pages == 1      # page 2 holds positions 8..11
    t.prepare(25)                                 # a portion that crosses two chunk edges keeps its pages until it is committed
    assert t.held_pages == 7
    t.commit()                                    # 35 tokens: the next position's chunk starts at 30
    assert t._first_live == 7 and t.slot_of(30) == t.pages[7] * 4 + 2
    with pytest.raises(RuntimeError):
        t.slot_of(27)
    t.free()
    assert pool.free_pages == 16
    both = BlockTable(pool, 4, window=6, chunk=20)
    both.prepare(19)
    both.commit()
    assert both._first_live == 3                  # the window (keys 14..) is the tighter of the two here
    both.prepare(2)
    both.commit()
    assert both._first_live == 5                  # 21 tokens: the chunk (keys 20..) is
    both.free()


# ---- the plain implementation's mechanisms against closed forms ----------------------------------------------------
def test_plain_state_space_against_a_closed_form():
    """One head, constant inputs: S_t = a S_{t-1} + dt B x^T is a geometric sum."""
    T, N, V = 6, 3, 2
    B, C, x = np.array([1.0, 2.0, 0.5]), np.array([0.5, -1.0, 2.0]), np.array([3.0, -2.0])
    dt, a_log, skip = 0.7, np.log(0.4), 1.5
    a = np.exp(-0.4 * dt)
    y = plain.selective_scan(np.tile(x, (T, 1, 1)), np.tile(B, (T, 1, 1)), np.tile(C, (T, 1, 1)), np.full((T, 1), dt), np.array([a_log]), np.array([skip]))
    for t in range(T):
        geo = sum(a ** i for i in range(t + 1))
        assert np.allclose(y[t, 0], geo * dt * (B @ C) * x + skip * x)


def test_plain_channel_gated_delta_rule_against_a_hand_computation():
    q = np.array([[[1.0, 0.0]], [[0.0, 1.0]]])
    k = np.array([[[1.0, 0.0]], [[1.0, 1.0]]])
    v = np.array([[[2.0]], [[3.0]]])
    beta = np.array([[0.5], [1.0]])
    g = np.array([[[0.9, 0.8]], [[0.5, 0.25]]])
    o = plain.channel_gated_delta_rule(q, k, v, beta, g)
    # t = 0: S = 0; u = 0.5 * 2 = 1; S = [[1], [0]]; o = 1.   t = 1: S = [[0.5], [0]]; u = 3 - 0.5 = 2.5; S = [[3], [2.5]]; o = 2.5.
    assert np.allclose(o[:, 0, 0], [1.0, 2.5])


def test_plain_rotation_pairs_the_halves_and_leaves_the_rest():
    x = np.arange(1.0, 7.0).reshape(1, 1, 6)
    y = plain.rotate_half(np.tile(x, (3, 1, 1)), [0, 1, 2], base=100.0, dims=4, factor=2.0)
    assert np.allclose(y[0], x[0]) and np.allclose(y[:, :, 4:], x[:, :, 4:])
    for p in (1, 2):
        for i, f in enumerate((1.0 / 2.0, 100.0 ** -0.5 / 2.0)):
            u, v = x[0, 0, i], x[0, 0, i + 2]
            assert np.isclose(y[p, 0, i], u * np.cos(p * f) - v * np.sin(p * f)) and np.isclose(y[p, 0, i + 2], v * np.cos(p * f) + u * np.sin(p * f))


def test_plain_chunks_are_counted_from_the_first_position():
    rng = np.random.default_rng(0)
    T, chunk = 11, 4
    q, k, v = rng.normal(size=(T, 2, 3)), rng.normal(size=(T, 1, 3)), rng.normal(size=(T, 1, 5))
    o = plain.chunked_softmax_attention(q, k, v, 0.5, chunk)
    for i in (4, 8):                                # a chunk's first position sees itself alone
        assert np.allclose(o[i, 0], v[i, 0]) and np.allclose(o[i, 1], v[i, 0])
    k2, v2 = k.copy(), v.copy()
    k2[3], v2[3] = 9.0, 9.0                         # the last position of the first chunk
    o2 = plain.chunked_softmax_attention(q, k2, v2, 0.5, chunk)
    assert np.array_equal(o[:3], o2[:3]) and not np.allclose(o[3], o2[3]) and np.array_equal(o[4:], o2[4:])


def test_plain_experts_follow_the_table_and_loop_order():
    rng = np.random.default_rng(1)
    E, ff, n = 6, 4, 3
    w = {f"m.e{e}.{r}": rng.normal(size=(ff, E) if r != "down" else (E, ff)) for e in range(n) for r in ("gate", "up", "down")}
    w["m.table"] = np.array([[0, 1], [2, 0], [1, 2]], dtype=np.int32)
    h = rng.normal(size=(2, E))
    mlp = {"router": {"experts": n, "top": 2}, "shared": None}
    out = plain.table_routed_experts(h, [1, 2], w, "m.", mlp)
    assert np.allclose(out[0], 0.5 * (plain.gated_unit(h[:1], w, "m.e2.") + plain.gated_unit(h[:1], w, "m.e0."))[0])
    assert np.allclose(out[1], 0.5 * (plain.gated_unit(h[1:], w, "m.e1.") + plain.gated_unit(h[1:], w, "m.e2."))[0])
    assert plain.layer_runs(CFG) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert plain.layer_runs({"layers": [0, 0, 0]}) == [(0, False), (1, False), (2, False)]


def test_layer_order_with_several_entries_a_step_is_checked():
    from llmx_b200.models import LayerStep, Model
    from llmx_b200.registry import architecture_of
    entry = architecture_of(CFG)
    m = entry.build(entry.config_cls.from_dict(CFG))
    kw = dict(embedding=m.embedding, blocks=m.blocks, head=m.head, vocab_size=130, max_positions=64)
    with pytest.raises(ValueError, match="needs 2 cache entries, 1 named"):
        Model(order=[LayerStep(2, 0)], **kw)
    with pytest.raises(ValueError, match="needs a cache entry, 2 named"):
        Model(order=[LayerStep(0, (0, 1))], **kw)
    with pytest.raises(ValueError, match="both write"):
        Model(order=[LayerStep(2, (0, 1)), LayerStep(0, 1)], **kw)
    ok = Model(order=[LayerStep(2, (1, 0)), LayerStep(2, (3, 2), add_embedding=True)], **kw)
    assert [type(s).__name__ for s in ok.cache_entry_specs()] == ["StateSpec", "KVSpec", "StateSpec", "KVSpec"]
    assert ok.native is None
