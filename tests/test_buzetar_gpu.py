"""Buzetar on the GPU against the plain implementation (tests/plain_buzetar.py): every mechanism alone, whole models
under every cutting, windows' and pages' edges, slots used again, long decoding, generation through the scheduler.

The configurations are this file's own: sizes that differ from one another everywhere (head counts, key / value /
rotated widths, ranks, windows, filter lengths, feed-forward widths that are not the model's width, layers without a
feed-forward or without a window, a rotation over part of the rotated part), and weights scaled up so that
activations are of order one and attention is far from uniform.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_buzetar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

MLP = {"kind": "dense", "ff": 72, "limit": 1.5}


def lightning(heads=3, dim=20, vdim=12, decay=(1.0, 0.97, 0.6), mlp=MLP):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def latent(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=48, window=20, rot_dims=None, base=10000.0, scale=0.3, mlp=MLP):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def delta(heads=4, kv_heads=2, dim=24, vdim=20, conv=3, mlp=MLP):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def config(layers, width=96, vocab=200, eps=1e-5, emb=3.0, logit=0.5):
    return {"architecture": "Buzetar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb},
            "logit_scale": logit, "layers": layers}


# Two whole models.  P: every mixer kind twice with different sizes, one layer without a feed-forward, one attention
# layer without a window and with only part of its rotated part rotated, a filter of two taps and one of five.
MODEL_P = config([delta(), latent(), lightning(), latent(heads=2, dim=24, rot_dim=12, vdim=10, q_rank=24, kv_rank=36, window=None, rot_dims=8, scale=0.25),
                  delta(heads=2, kv_heads=2, dim=16, vdim=36, conv=2, mlp=None), lightning(heads=2, dim=36, vdim=40, decay=(0.999, 0.9), mlp={"kind": "dense", "ff": 50, "limit": 0.8})])
# Q: a width and a vocabulary that are no multiples of 8 (products off the tensor cores), one head, a window of one page.
MODEL_Q = config([latent(heads=1, dim=10, rot_dim=6, vdim=14, q_rank=12, kv_rank=20, window=8, scale=0.5, mlp={"kind": "dense", "ff": 30, "limit": 3.0}),
                  lightning(heads=1, dim=9, vdim=7, decay=(0.8,), mlp=None), delta(heads=3, kv_heads=1, dim=10, vdim=6, conv=5)],
                 width=50, vocab=101, eps=1e-6, emb=1.0, logit=2.0)


def make_folder(tmp, cfg, seed, dtype=torch.float32, gain=5.0, sharpen=1.0):
    """A model folder with random weights of order one: matrices N(0, 0.02) x gain (query maps x sharpen on top)."""
    from llmx_b200.config import BuzetarConfig
    from llmx_b200.registry import architecture_of
    from llmx_b200.weights import RandomSource, write_safetensors
    c = BuzetarConfig.from_dict(cfg)
    model = architecture_of(cfg).build(c)
    specs = model.tensor_specs()
    src = RandomSource(specs, seed, dtype=torch.float32)
    tensors = {}
    for n in src.names():
        t = src.tensor(n)
        if specs[n].kind in ("matrix", "table") and not n.endswith(".conv"):
            t = t * gain
        if n.endswith(".uq"):
            t = t * sharpen
        tensors[n] = t.to(dtype)
    os.makedirs(tmp, exist_ok=True)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(tmp, "model.safetensors"), tensors)
    return {n: t.to(torch.float32).numpy() for n, t in tensors.items()}


def engine_of(folder, dtype, kv_tokens, page=4, requests=4):
    from llmx_b200.engine import Engine, EngineOptions
    return Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_tokens=kv_tokens, page_size=page, max_requests=requests))


def worst_error(got, refs):
    worst, where = 0.0, None
    for key, row in got.items():
        d = float(np.abs(row - refs[key[0]][key[1]]).max())
        if not np.isfinite(d):
            return float("inf"), key
        if d > worst:
            worst, where = d, key
    return worst, where


CUTTINGS = (helpers.trace_whole, helpers.trace_tail_decoded, helpers.trace_portions, helpers.trace_mixed)


def run_cuttings(folder, cfg, w, dtype, lengths, tol, page=4, seed=0):
    requests = {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed=seed + i) for i, n in enumerate(lengths)}
    refs = {rid: plain.forward(cfg, w, ids) for rid, ids in requests.items()}
    scale = max(float(np.abs(r).max()) for r in refs.values())
    measured = {}
    for make in CUTTINGS:
        steps = make(requests)
        engine = engine_of(folder, dtype, helpers.tokens_needed(steps), page)
        got = helpers.run_trace(engine, steps)
        engine.cache.check()
        assert all(u == 0 for u in engine.cache.used_pages())
        assert engine.cache.state_slots.free_slots == engine.cache.state_slots.num_slots
        worst, where = worst_error(got, refs)
        measured[make.__name__] = worst / scale
        assert len(got) == sum(lengths)
        assert worst <= tol * scale, f"{make.__name__}: {worst:.3e} at {where} (scale {scale:.3f})"
    return measured


# ---- every mechanism alone: one-layer models -----------------------------------------------------------------------
ONE_LAYER = {
    "lightning": lightning(),
    "lightning_no_mlp": lightning(heads=2, dim=40, vdim=9, decay=(0.999, 0.5), mlp=None),
    "latent_window": latent(),
    "latent_full_partial_rotation": latent(heads=2, dim=12, rot_dim=16, vdim=20, q_rank=30, kv_rank=28, window=None, rot_dims=6),
    "delta": delta(),
    "delta_one_tap_group_of_three": delta(heads=6, kv_heads=2, dim=12, vdim=16, conv=1, mlp=None),
    "delta_long_filter": delta(heads=1, kv_heads=1, dim=32, vdim=8, conv=6),
    "delta_rows_off_16_bytes": delta(heads=3, kv_heads=3, dim=8, vdim=5, conv=2),          # q/k widths of 4s in rows that are not
    "latent_18_heads": latent(heads=18, dim=8, rot_dim=4, vdim=6, q_rank=20, kv_rank=24, window=30),      # two groups of heads a tile
    "lightning_wide_heads": lightning(heads=2, dim=160, vdim=24, decay=(0.99, 0.9)),       # more than four values a lane
    "delta_very_wide_heads": delta(heads=2, kv_heads=1, dim=320, vdim=6, conv=3, mlp=None),
    "latent_window_of_one": latent(heads=2, dim=8, rot_dim=8, vdim=8, q_rank=16, kv_rank=16, window=1),
    "latent_nothing_rotated": latent(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=16, kv_rank=16, window=25, rot_dims=0),
}


@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_mixer_under_every_cutting_float32(tmp_path, name):
    cfg = config([ONE_LAYER[name]])
    w = make_folder(str(tmp_path), cfg, seed=7)
    run_cuttings(str(tmp_path), cfg, w, "float32", [50, 3, 77, 20, 1, 64], 1e-4)


def test_row_kernels_against_the_plain_functions():
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(3)
    for width in (50, 96, 4100):
        x = torch.randn(5, width, generator=g) * 3 + 1.5
        wt = torch.rand(width, generator=g) + 0.5
        for out_dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 2 ** -8)):
            out = torch.empty(5, width, dtype=out_dtype, device=DEV)
            ops.layernorm(x.to(DEV), wt.to(DEV), 1e-5, out)
            ref = plain.layer_norm(x.numpy(), wt.numpy(), 1e-5)
            assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
        idx = torch.tensor([4, 0, 4], dtype=torch.int32)
        out = torch.empty(3, width, dtype=torch.float32, device=DEV)
        ops.layernorm(x.to(DEV), wt.to(DEV), 1e-5, out, row_index=idx.to(DEV))
        assert np.abs(out.cpu().numpy() - plain.layer_norm(x.numpy()[[4, 0, 4]], wt.numpy(), 1e-5)).max() <= 1e-5
    # A buffer handed to the norm's launch is cleared by it, whatever its size against the rows'.
    for count in (4, 1000, 1 << 20):
        junk = torch.full((count,), 7.0, dtype=torch.float32, device=DEV)
        x = torch.randn(3, 96, generator=g)
        out = torch.empty(3, 96, dtype=torch.float32, device=DEV)
        ops.layernorm(x.to(DEV), torch.ones(96, device=DEV), 1e-5, out, zero=junk)
        assert float(junk.abs().max()) == 0.0
        assert np.abs(out.cpu().numpy() - plain.layer_norm(x.numpy(), np.ones(96), 1e-5)).max() <= 1e-5
    # The clamped gated unit: values on both sides of the limit on both branches.
    gu = torch.randn(6, 2 * 37, generator=g) * 3
    out = torch.empty(6, 37, dtype=torch.float32, device=DEV)
    ops.clamped_glu(gu.to(DEV), out, 1.5, 1.702)
    gg, uu = np.minimum(gu[:, :37].numpy().astype(np.float64), 1.5), np.clip(gu[:, 37:].numpy().astype(np.float64), -1.5, 1.5)
    ref = gg * plain.sigmoid(1.702 * gg) * (uu + 1.0)
    assert (gu[:, :37] > 1.5).any() and (gu[:, 37:] < -1.5).any() and np.abs(out.cpu().numpy() - ref).max() <= 1e-5
    # The gated norm: one group (the row) with a sigmoid gate; groups of a head with a shared weight and a silu gate.
    o = torch.randn(4, 60, generator=g)
    wide = torch.randn(4, 100, generator=g)
    gate = wide[:, 30:90]
    for group, wlen, kind in ((60, 60, "sigmoid"), (12, 12, "silu")):
        wt = torch.rand(wlen, generator=g) + 0.5
        out = torch.empty(4, 60, dtype=torch.float32, device=DEV)
        ops.gated_rmsnorm(o.to(DEV), wide.to(DEV)[:, 30:90], wt.to(DEV), 1e-5, group, kind, out)
        normed = plain.rms_norm(o.numpy().reshape(4, 60 // group, group), wt.numpy(), 1e-5).reshape(4, 60)
        gv = gate.numpy().astype(np.float64)
        ref = normed * (plain.sigmoid(gv) if kind == "sigmoid" else plain.silu(gv))
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5
    table = torch.randn(9, 20, generator=g)
    ids = torch.tensor([3, 8, 0], dtype=torch.int32, device=DEV)
    x = ops.embed_scaled(table.to(DEV), ids, torch.empty(3, 20, dtype=torch.float32, device=DEV), 2.5)
    assert torch.equal(x.cpu(), table[[3, 8, 0]] * 2.5)


# ---- whole models ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("which", ["P", "Q"])
def test_whole_models_under_every_cutting_float32(tmp_path, which):
    cfg = MODEL_P if which == "P" else MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=11)
    run_cuttings(str(tmp_path), cfg, w, "float32", [50, 3, 77, 20, 1, 64, 133], 1e-4, page=4 if which == "P" else 8)


# Twice the error measured when the budget was frozen, as a fraction of the logit scale (the plain implementation is
# exact; the path rounds the inputs of products and the cached latents to bfloat16).
BF16_BUDGET = {"P": 3.6e-2, "Q": 2.5e-2}     # measured: P 1.8e-2, Q 1.2e-2, the same under every cutting


@pytest.mark.parametrize("which", ["P", "Q"])
def test_whole_models_under_every_cutting_bfloat16(tmp_path, which):
    cfg = MODEL_P if which == "P" else MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=11, dtype=torch.bfloat16)
    measured = run_cuttings(str(tmp_path), cfg, w, "bfloat16", [50, 3, 77, 20, 1, 64, 133], BF16_BUDGET[which], page=16)
    print("bfloat16 error / scale:", which, measured)


def test_a_request_in_a_batch_equals_the_request_alone(tmp_path):
    """Unequal requests in one step (a long portion, a short one, single tokens after history) against each alone."""
    from llmx_b200.engine import StepEntry
    cfg = MODEL_P
    make_folder(str(tmp_path), cfg, seed=5)
    ids = {r: helpers.random_ids(cfg["vocab"], n, seed=40 + i) for i, (r, n) in enumerate({"a": 90, "b": 31, "c": 12, "d": 2}.items())}
    alone = {}
    for r, t in ids.items():
        e = engine_of(str(tmp_path), "float32", 256)
        cut = len(t) // 2
        e.step([StepEntry(r, t[:cut], [])])
        alone[r] = e.step([StepEntry(r, t[cut:], list(range(len(t) - cut)))]).cpu().numpy()
    e = engine_of(str(tmp_path), "float32", 512)
    e.step([StepEntry(r, t[:len(t) // 2], []) for r, t in ids.items()])
    got = e.step([StepEntry(r, t[len(t) // 2:], list(range(len(t) - len(t) // 2))) for r, t in ids.items()]).cpu().numpy()
    at = 0
    for r, t in ids.items():
        n = len(t) - len(t) // 2
        assert np.abs(got[at:at + n] - alone[r]).max() <= 1e-5 * np.abs(alone[r]).max(), r
        at += n


# ---- edges of windows and pages ------------------------------------------------------------------------------------
@pytest.mark.parametrize("window,page", [(20, 4), (16, 16), (33, 8), (300, 16)])
def test_a_token_is_seen_exactly_while_the_window_holds_it(tmp_path, window, page):
    """One attention layer: changing token j changes the logits at j .. j + window - 1 and leaves those from
    j + window on bit for bit as they were, in a prompt taken whole, in portions that cut the window, and decoded;
    j and the window's edges lie at page borders and off them."""
    from llmx_b200.engine import StepEntry
    cfg = config([latent(window=window, mlp=None)])
    make_folder(str(tmp_path), cfg, seed=3, sharpen=0.5)        # flat attention: every key of the window carries weight
    n = window + 45
    base = helpers.random_ids(cfg["vocab"], n, seed=1)
    for j in (0, 5, page, 2 * page - 1):
        other = list(base)
        other[j] = (base[j] + 1) % cfg["vocab"]
        for how in ("whole", "portions", "decoded"):
            rows = []
            for ids in (base, other):
                e = engine_of(str(tmp_path), "float32", 1024, page)
                if how == "whole":
                    out = e.step([StepEntry("r", ids, list(range(n)))]).cpu().numpy()
                elif how == "portions":
                    cuts, out, at = [j + window - 1, 2, 1, 7], [], 0
                    k = 0
                    while at < n:
                        p = max(1, min(cuts[k % 4], n - at))
                        out.append(e.step([StepEntry("r", ids[at:at + p], list(range(p)))]).cpu().numpy())
                        at, k = at + p, k + 1
                    out = np.concatenate(out)
                else:
                    head = min(j + 3, n)
                    out = [e.step([StepEntry("r", ids[:head], list(range(head)))]).cpu().numpy()]
                    out += [e.step([StepEntry("r", [t], [0])]).cpu().numpy() for t in ids[head:]]
                    out = np.concatenate(out)
                e.cache.check()
                rows.append(out)
            a, b = rows
            last_inside, first_outside = j + window - 1, j + window
            assert not np.array_equal(a[last_inside], b[last_inside]), (how, j, "the window's last position must see the token")
            assert np.abs(a[last_inside] - b[last_inside]).max() > 1e-5 * np.abs(a).max(), (how, j)
            assert np.array_equal(a[first_outside:], b[first_outside:]), (how, j, "a token past the window was seen")
            assert np.array_equal(a[:j], b[:j])


@pytest.mark.parametrize("kv_rank,rot_dim,heads,window", [(128, 32, 3, 40), (256, 64, 20, None), (512, 64, 5, 150)])
@pytest.mark.parametrize("sharpen,tol", [(0.25, 5e-5), (2.0, 5e-4)])
def test_tensor_core_scores_equal_the_cuda_core_scores(tmp_path, kv_rank, rot_dim, heads, window, sharpen, tol):
    """Latents of 128, 256 and 512 values in a bfloat16 cache: the scores step on the tensor cores (32-bit factors as
    sums of three bfloat16 values) against the same step on the CUDA cores, over the same cache, under every cutting:
    whole prompts, portions that cut windows and tiles, single tokens after long histories (key ranges).  With flat
    scores the two agree as two orders of 32-bit sums do; with scores of tens, the tensor core's cut-off additions show
    in the exponentials (an absolute error of a score is a relative error of its weight), far below what a key at the
    wrong place or a lost row would do."""
    from llmx_b200.engine import Engine, EngineOptions
    cfg = config([latent(heads=heads, dim=24, rot_dim=rot_dim, vdim=16, q_rank=40, kv_rank=kv_rank, window=window, scale=0.2),
                  lightning(), latent(heads=2, dim=16, rot_dim=rot_dim, vdim=24, q_rank=32, kv_rank=kv_rank, window=window, rot_dims=rot_dim // 2, mlp=None)])
    make_folder(str(tmp_path), cfg, seed=21, sharpen=sharpen)
    requests = {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed=70 + i) for i, n in enumerate([330, 3, 77, 200, 1, 64])}
    for make in CUTTINGS:
        steps = make(requests)
        got = []
        for plain_cores in (False, True):
            engine = Engine.from_dir(str(tmp_path), EngineOptions(dtype="float32", kv_dtype="bfloat16", kv_tokens=helpers.tokens_needed(steps),
                                                                  page_size=16, max_requests=4))
            for block in engine.model.blocks:
                if hasattr(block.mixer, "plain_cores"):
                    block.mixer.plain_cores = plain_cores
            got.append(helpers.run_trace(engine, steps))
            engine.cache.check()
        scale = max(float(np.abs(r).max()) for r in got[1].values())
        worst = max(float(np.abs(got[0][k] - got[1][k]).max()) for k in got[1])
        assert len(got[0]) == len(got[1]) == sum(len(v) for v in requests.values())
        assert np.isfinite(worst) and worst <= tol * scale, (make.__name__, worst, scale)


def test_far_keys_without_a_window(tmp_path):
    """Attention without a window over hundreds of keys across many pages: sharpened so that single far keys decide."""
    cfg = config([latent(window=None, rot_dims=4), lightning(decay=(1.0, 0.999, 0.99))])
    w = make_folder(str(tmp_path), cfg, seed=9, sharpen=6.0)
    run_cuttings(str(tmp_path), cfg, w, "float32", [700, 333], 1e-4, page=16)


def test_slots_and_pages_used_again_start_from_nothing(tmp_path):
    """Requests follow one another through the same two state slots and the same few pages; each equals the plain
    implementation from its first token (which sees zeros before the start, whatever the slot held)."""
    from llmx_b200.engine import StepEntry
    cfg = MODEL_P
    w = make_folder(str(tmp_path), cfg, seed=2)
    e = engine_of(str(tmp_path), "float32", 64, page=4, requests=1)
    for i in range(5):
        ids = helpers.random_ids(cfg["vocab"], 40 + 5 * i, seed=90 + i)
        ref = plain.forward(cfg, w, ids)
        got = np.concatenate([e.step([StepEntry(i, ids[:3], [0, 1, 2])]).cpu().numpy(),
                              e.step([StepEntry(i, ids[3:], list(range(len(ids) - 3)))]).cpu().numpy()])
        e.end(i)
        e.cache.check()
        assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max(), i


def test_long_decoding(tmp_path):
    cfg = MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=4)
    ids = helpers.random_ids(cfg["vocab"], 400, seed=8)
    ref = plain.forward(cfg, w, ids)
    steps = helpers.trace_tail_decoded({"r": ids}, tail=390)
    e = engine_of(str(tmp_path), "float32", 512, page=16)
    got = helpers.run_trace(e, steps)
    worst, where = worst_error(got, {"r": ref})
    assert worst <= 1e-4 * np.abs(ref).max(), where


# ---- the framework's entry points ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(tmp_path, dtype):
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    cfg = MODEL_P
    w = make_folder(str(tmp_path), cfg, seed=6, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    prompts = [helpers.random_ids(cfg["vocab"], n, seed=n) for n in (5, 17, 33, 60)]
    llm = LLM(str(tmp_path), dtype=dtype, kv_tokens=512, page_size=16, ubatch=24, max_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=24, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True))
    assert [len(o.tokens) for o in outs] == [24] * 4
    for p, o in zip(prompts, outs):
        ids = list(p)
        for t in o.tokens:
            logits = plain.forward(cfg, w, ids)[-1]
            best = int(np.argmax(logits))
            gap = 2 * BF16_BUDGET["P"] if dtype == "bfloat16" else 1e-4
            assert t == best or logits[best] - logits[t] <= gap * np.abs(logits).max(), (len(ids), t, best)
            ids.append(t)
    assert all(u == 0 for u in llm.engine.cache.used_pages())
    assert llm.engine.cache.state_slots.free_slots == llm.engine.cache.state_slots.num_slots


def test_recorded_steps_equal_plain_steps(tmp_path):
    """Steps whose shape keeps coming are recorded as CUDA graphs and replayed: the same logits as the plain
    implementation, portions and decoded tokens, with the tiled attention's plan made for the recording's room."""
    from llmx_b200.engine import Engine, EngineOptions
    cfg = MODEL_P
    w = make_folder(str(tmp_path), cfg, seed=14)
    requests = {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed=30 + i) for i, n in enumerate([70, 70, 70, 41])}
    refs = {rid: plain.forward(cfg, w, ids) for rid, ids in requests.items()}
    steps = helpers.trace_portions(requests, portions=[7, 7, 7, 7, 7, 7, 7, 7, 7, 1, 1, 1, 1, 1, 1, 1])
    engine = Engine.from_dir(str(tmp_path), EngineOptions(dtype="float32", kv_tokens=256, page_size=16, max_requests=2, record_after=1))
    assert engine.model.recordable
    got = helpers.run_trace(engine, steps, record=True)
    assert len(engine.step_recordings) >= 2          # the portion of seven rows and the single row, at least
    worst, where = worst_error(got, refs)
    assert worst <= 1e-4 * max(float(np.abs(r).max()) for r in refs.values()), where
    engine.cache.check()


def test_command_line_generates_from_a_folder(tmp_path):
    cfg = MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=15, dtype=torch.bfloat16)
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmx"), "generate", str(tmp_path), "5,17,3,99", "-n", "6", "--temp", "0",
                          "--ignore-eos", "--dtype", "f32"], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    ids = next(l for l in run.stdout.splitlines() if l.startswith("ids: "))
    tokens = [int(t) for t in ids[5:].split(",")]
    assert len(tokens) == 6
    seq = [5, 17, 3, 99]
    for t in tokens:
        logits = plain.forward(cfg, w, seq)[-1]
        best = int(np.argmax(logits))
        assert t == best or logits[best] - logits[t] <= 1e-4 * np.abs(logits).max()
        seq.append(t)


def test_command_line_logits_and_bench_take_the_folder(tmp_path):
    make_folder(str(tmp_path), MODEL_Q, seed=16, dtype=torch.bfloat16)
    exe = [sys.executable, os.path.join(ROOT, "bin", "llmx")]
    logits = subprocess.run(exe + ["logits", str(tmp_path), "5,17,3,99", "--top", "3", "--dtype", "f32"], capture_output=True, text=True, timeout=600)
    assert logits.returncode == 0 and logits.stdout.strip(), logits.stderr[-2000:]
    bench = subprocess.run(exe + ["bench", "--model", str(tmp_path), "--p", "64", "--n", "8", "--r", "1"], capture_output=True, text=True, timeout=600)
    assert bench.returncode == 0 and "tok" in bench.stdout, bench.stderr[-2000:]


def test_temperature_sampling_is_reproducible_and_independent_of_the_batch(tmp_path):
    """Four requests as mixed portions and decoded tokens, temperature 0.8 with fixed seeds: the same seeds give the same
    replies, and a request's reply is the one it gets alone (its state and latents are its own, whatever shares the step)."""
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    cfg = MODEL_P
    make_folder(str(tmp_path), cfg, seed=17)
    prompts = [helpers.random_ids(cfg["vocab"], n, seed=n) for n in (1, 9, 40, 70)]
    params = [SamplingParams(max_tokens=12, temp=0.8, top_k=40, top_p=0.95, seed=100 + i, ignore_eos=True) for i in range(4)]
    llm = LLM(str(tmp_path), dtype="float32", kv_tokens=512, page_size=16, ubatch=32, max_seqs=4)
    first = [o.tokens for o in llm.generate(prompts, params)]
    again = [o.tokens for o in llm.generate(prompts, params)]
    assert first == again
    for i in range(4):
        alone = LLM(str(tmp_path), dtype="float32", kv_tokens=256, page_size=16, ubatch=32, max_seqs=1).generate([prompts[i]], [params[i]])
        assert alone[0].tokens == first[i], i


def test_trace_run_program(tmp_path):
    cfg = MODEL_Q
    w = make_folder(str(tmp_path / "m"), cfg, seed=12, dtype=torch.bfloat16)
    requests = {f"q{i}": helpers.random_ids(cfg["vocab"], n, seed=50 + i) for i, n in enumerate([45, 3, 80, 20, 64])}
    steps = helpers.trace_mixed(requests, tail=5)
    for dtype, tol in (("float32", 1e-4), ("bfloat16", BF16_BUDGET["Q"])):
        out = tmp_path / ("out_" + dtype)
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype,
                               "--out", str(out), "--max-tokens", str(helpers.tokens_needed(steps))],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
        got = helpers.read_trace_output(steps, str(out), cfg["vocab"])
        refs = {rid: plain.forward(cfg, w, ids) for rid, ids in requests.items()}
        worst, where = worst_error(got, refs)
        assert worst <= tol * max(float(np.abs(r).max()) for r in refs.values()), (dtype, worst, where)
