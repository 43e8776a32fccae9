"""The plain Gatuzen restatement (oracle/gatuzen.py) checked against closed forms, and the host-side pieces that need no GPU:
synthetic checkpoints, integer tables through the safetensors reader, the choice of the executor by config.json."""
import json
import math
import os

import numpy as np

from aha_b200 import synth
from oracle import gatuzen as Z


def test_group_norm_normalises_every_part_on_its_own():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 12)) * np.array([1.0] * 4 + [50.0] * 4 + [0.01] * 4)
    w = rng.standard_normal(12)
    y = Z.group_norm(x, w, 3, 0.0)
    for g in range(3):
        part = y[:, 4 * g:4 * g + 4] / w[4 * g:4 * g + 4]
        assert np.allclose((part * part).mean(axis=1), 1.0)
    # one group is the ordinary RMS norm; eps sits inside the root
    assert np.allclose(Z.group_norm(x, w, 1, 0.5), x / np.sqrt((x * x).mean(axis=1, keepdims=True) + 0.5) * w)


def test_causal_conv_is_a_correlation_with_state():
    rng = np.random.default_rng(1)
    u, w, b = rng.standard_normal((11, 3)), rng.standard_normal((3, 4)), rng.standard_normal(3)
    y, tail = Z.causal_conv(u, w, np.zeros((3, 3)), b)
    for c in range(3):
        ext = np.concatenate([np.zeros(3), u[:, c]])
        assert np.allclose(y[:, c], [b[c] + sum(w[c, j] * ext[t + j] for j in range(4)) for t in range(11)])     # the last column is the current token's
    assert np.allclose(tail, u[-3:])
    t2, parts = np.zeros((3, 3)), []
    for a, e in [(0, 1), (1, 3), (3, 4), (4, 11)]:          # portions shorter than the tail
        yy, t2 = Z.causal_conv(u[a:e], w, t2, b)
        parts.append(yy)
    assert np.allclose(np.concatenate(parts), y) and np.allclose(t2, tail)
    st = {}
    assert np.allclose(Z.input_conv(u, w, st, "k"), u + y - b)      # the sublayer reads h + conv(h)
    one = np.ones((2, 1))
    assert Z.causal_conv(u[:4, :2], one, np.zeros((0, 2)))[0].shape == (4, 2)     # a single tap keeps no state


def test_diag_recurrence_closed_forms():
    # constant decay a, key k, value v: S_t = k v (1 - a^t) / (1 - a) per row
    T = 9
    a, k, q = np.array([0.5, 0.9, 0.0]), np.array([1.0, -2.0, 3.0]), np.array([1.0, 0.5, -2.0])
    v = np.array([2.0, -1.0])
    S = np.zeros((3, 2))
    o = Z.diag_recurrence(np.tile(q, (T, 1)), np.tile(k, (T, 1)), np.tile(v, (T, 1)), np.tile(a, (T, 1)), S)
    for t in range(T):
        geo = np.where(a == 1.0, t + 1, (1 - a ** (t + 1)) / (1 - a))
        assert np.allclose(o[t], (q * k * geo).sum() * v)
    # decay one and key one: a running sum; decay zero: only the current token
    x = np.random.default_rng(2).standard_normal((6, 1, 4))
    ones = np.ones((6, 1))
    assert np.allclose(Z.diag_recurrence(ones, ones, x[:, 0], ones, np.zeros((1, 4))), np.cumsum(x[:, 0], axis=0))
    assert np.allclose(Z.diag_recurrence(ones, ones, x[:, 0], 0 * ones, np.zeros((1, 4))), x[:, 0])


def test_rotary_table_and_rotation():
    f, m = Z.rotary_table({"dims": 8, "base": 100.0})
    assert np.allclose(f, 100.0 ** (-np.arange(4) / 4.0)) and m == 1.0
    sc = {"factor": 8.0, "original": 16, "fast": 1.5, "slow": 0.25}
    f2, m2 = Z.rotary_table({"dims": 16, "base": 50.0, "scaling": sc})
    plain = 50.0 ** (-np.arange(8) / 8.0)
    d = lambda t: 16 * math.log(16 / (2 * math.pi * t)) / (2 * math.log(50.0))
    lo, hi = math.floor(d(1.5)), math.ceil(d(0.25))
    assert (lo, hi) == (1, 5)
    assert np.allclose(f2[:2], plain[:2]) and np.allclose(f2[5:], plain[5:] / 8.0)        # fast pairs kept, slow pairs divided by the factor
    assert np.allclose(f2[3], plain[3] * (0.5 / 8.0 + 0.5)) and np.isclose(m2, 0.1 * math.log(8.0) + 1.0)
    # a rotation keeps lengths (times the factor), passes the coordinates after the rotated ones, and depends on position differences only
    rng = np.random.default_rng(3)
    x, y = rng.standard_normal((1, 10)), rng.standard_normal((1, 10))
    fr = np.array([1.0, 0.3, 0.01])
    r = Z.rotate_pairs(x, np.array([7]), fr, 1.25)
    assert np.allclose(np.linalg.norm(r[0, :6]), 1.25 * np.linalg.norm(x[0, :6])) and np.array_equal(r[0, 6:], x[0, 6:])
    dot = lambda p, q: (Z.rotate_pairs(x, np.array([p]), fr, 1.0)[0, :6] * Z.rotate_pairs(y, np.array([q]), fr, 1.0)[0, :6]).sum()
    assert np.isclose(dot(12, 5), dot(107, 100))
    assert np.allclose(Z.rotate_pairs(x, np.array([0]), fr, 1.0), x)
    u = np.zeros((1, 2)); u[0, 0] = 1.0
    assert np.allclose(Z.rotate_pairs(u, np.array([1]), np.array([0.5]), 1.0), [[math.cos(0.5), math.sin(0.5)]])    # (u, v) -> (u cos - v sin, v cos + u sin)


def test_table_experts_average_the_rows_chosen_by_the_token_id():
    rng = np.random.default_rng(4)
    W, ff, E = 6, 5, 4
    wts = {"table": np.array([[1, 3], [0, 2], [3, 1]])}
    for e in range(E):
        for nm, shp in (("gate", (ff, W)), ("up", (ff, W)), ("down", (W, ff))):
            wts["e%d.%s" % (e, nm)] = rng.standard_normal(shp)
    h = rng.standard_normal((3, W))
    ml = {"router": {"experts": E, "top": 2}, "expert": {"ff": ff}}
    out = Z.table_moe(h, [2, 0, 2], wts, ml)
    ex = lambda e, x: (Z.silu(wts["e%d.gate" % e] @ x) * (wts["e%d.up" % e] @ x)) @ wts["e%d.down" % e].T
    assert np.allclose(out[0], 0.5 * (ex(3, h[0]) + ex(1, h[0]))) and np.allclose(out[1], 0.5 * (ex(1, h[1]) + ex(3, h[1])))
    assert np.allclose(Z.table_moe(h[:1], [1], wts, ml)[0], 0.5 * (ex(0, h[0]) + ex(2, h[0])))


def test_latent_attention_equals_attention_over_expanded_keys_and_is_causal():
    cfg = synth.gatuzen_config([{"type": "latent_attention", "heads": 2, "dim": 4, "rot_dim": 4, "vdim": 6, "kv_rank": 5, "base": 10.0, "scaling": None}], width=8, vocab=11, taps=0)
    w = {k: synth.bf16_to_f32(v) for k, v in synth.make_gatuzen(cfg, 1).items()}
    W = {k[len("l0.mix."):]: np.asarray(v, np.float64) for k, v in w.items() if k.startswith("l0.mix.")}
    mx = cfg["layers"][0]["mixer"]
    h = np.random.default_rng(5).standard_normal((7, 8))
    whole = Z.latent_attention_mixer(h, W, mx, 1e-5, {}, 0)
    st, parts = {}, []
    for a, b in [(0, 3), (3, 4), (4, 7)]:
        parts.append(Z.latent_attention_mixer(h[a:b], W, mx, 1e-5, st, a))
    assert np.allclose(np.concatenate(parts), whole)
    h2 = h.copy(); h2[5] += 1.0
    other = Z.latent_attention_mixer(h2, W, mx, 1e-5, {}, 0)
    assert np.allclose(other[:5], whole[:5]) and not np.allclose(other[6], whole[6])
    assert st["c"].shape == (7, 5) and st["kr"].shape == (7, 4)        # what a cache has to hold per token


def test_loop_runs_and_portions_equal_the_whole_prompt():
    layers = [{"type": "gla", "heads": 2, "dim": 4, "vdim": 6, "tau": 4.0, "rank": 2, "moe": {"experts": 3, "top": 2, "ff": 8}},
              {"type": "mamba2", "heads": 2, "vdim": 4, "state": 4, "groups": 1, "norm_groups": 2, "conv": 3, "moe": None},
              {"type": "latent_attention", "heads": 2, "dim": 4, "rot_dim": 2, "vdim": 4, "kv_rank": 6, "scaling": {"factor": 2.0, "original": 8, "fast": 2.0, "slow": 1.0}, "moe": None}]
    cfg = synth.gatuzen_config(layers, width=16, vocab=23, groups=2, taps=3, loop=(1, 3, 3))
    w = synth.make_gatuzen(cfg, 3)
    assert w["loop.step"].shape == (3, 16) and w["l0.mlp.table"].shape == (23, 2) and "l1.mlp.table" not in w and w["l0.mix.a1"].shape == (2, 16)
    assert w["l1.mix.in"].shape == (2 * 8 + 2 * 4 + 2, 16) and w["l1.mix.conv"].shape == (8 + 8, 3) and w["l2.mix.dkv"].shape == (8, 16)
    assert all(len(set(r)) == 2 for r in np.asarray(w["l0.mlp.table"]))      # the entries of a row differ
    f = {k: (np.asarray(v) if k.endswith("table") else synth.bf16_to_f32(v)) for k, v in w.items()}
    o = Z.Gatuzen(cfg, f)
    assert [l for l, _ in o.runs] == [0, 1, 2, 1, 2, 1, 2] and [t for _, t in o.runs] == [None, 0, None, 1, None, 2, None]
    ids = np.random.default_rng(0).integers(0, 23, 40)
    trace = []
    whole = o.forward(ids, None, trace)
    assert len(trace) == 7
    st, parts = o.new_state(), []
    for a, b in [(0, 7), (7, 9), (9, 10), (10, 33), (33, 40)]:
        parts.append(o.forward(ids[a:b], st))
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-10
    assert len(o.greedy(ids[:5], 4)) == 4
    # the vector before a pass matters, and each pass has a state of its own (the second pass does not continue the first one's)
    f2 = dict(f); f2["loop.step"] = f["loop.step"] * 0.0
    assert np.abs(Z.Gatuzen(cfg, f2).forward(ids) - whole).max() > 1e-3
    big = synth.gatuzen_shape(256, 6, 4, 32, 64, 8, 2, vocab=500, loop=(0, 3, 2))
    assert [l["type"] for l in big["layers"]] == ["gla", "mamba2", "latent_attention"] * 2 and big["loop"]["times"] == 2


def test_safetensors_roundtrip_with_integer_table_and_kind(tmp_path):
    from aha_b200 import checkpoint
    cfg = synth.gatuzen_config([{"type": "gla", "heads": 1, "dim": 4, "vdim": 4, "moe": {"experts": 3, "top": 2, "ff": 4}}], width=8, vocab=9)
    w = synth.make_gatuzen(cfg, 0)
    stored = dict(w)
    stored["l0.mlp.table"] = np.asarray(w["l0.mlp.table"]).astype(np.int32)     # checkpoints hold the table as 32-bit integers
    p = os.path.join(tmp_path, "model.safetensors")
    checkpoint.write_safetensors(p, stored)
    r = checkpoint.read_safetensors(p)
    assert sorted(r) == sorted(w)
    for k in w:
        assert r[k].shape == w[k].shape and np.array_equal(np.asarray(r[k]).view(np.ndarray), np.asarray(w[k]).view(np.ndarray))
    assert checkpoint.model_kind(cfg) == "gatuzen"
    json.dumps(cfg)
