"""The plain Malasun restatement (oracle/malasun.py) checked against closed forms, and the host-side pieces of the layered
engine that need no GPU: synthetic checkpoints, the safetensors reader, the choice of the executor by config.json."""
import json
import os

import numpy as np
import pytest

from aha_b200 import synth
from oracle import malasun as M


def test_xielu_branches_and_continuity():
    p, q = 0.3, -0.4
    ap, aq = np.log1p(np.exp(p)), 0.5 + np.log1p(np.exp(q))
    z = np.array([-3.0, -1e-9, 0.0, 1e-9, 2.0])
    y = M.xielu(z, p, q)
    assert np.allclose(y[4], ap * 4.0 + 1.0)
    assert np.allclose(y[0], aq * (np.exp(-3.0) - 1.0 + 3.0) - 1.5)
    assert abs(y[1]) < 1e-8 and y[2] == 0.0 and abs(y[3]) < 1e-8          # both branches meet at 0 with slope 1/2


def test_short_conv_is_a_causal_correlation_with_state():
    rng = np.random.default_rng(0)
    u, w = rng.standard_normal((11, 3)), rng.standard_normal((3, 4))
    y, tail = M.short_conv(u, w, np.zeros((3, 3)))
    for c in range(3):
        ext = np.concatenate([np.zeros(3), u[:, c]])
        want = [sum(w[c, j] * ext[t + j] for j in range(4)) for t in range(11)]
        assert np.allclose(y[:, c], want)
    assert np.allclose(tail, u[-3:])
    # fed in portions (down to one token, shorter than the tail) the result is the same
    t2 = np.zeros((3, 3))
    parts = []
    for a, b in [(0, 1), (1, 3), (3, 4), (4, 11)]:
        yy, t2 = M.short_conv(u[a:b], w, t2)
        parts.append(yy)
    assert np.allclose(np.concatenate(parts), y) and np.allclose(t2, tail)


def test_hgrn2_recurrence_closed_form_for_constant_gates():
    # constant f and v: S_t = (1 - f^t) v per row, o_t = sum_i (1 - f_i^t) q_i v
    T, D, Dv = 9, 3, 2
    f = np.tile(np.array([0.5, 0.9, 0.0]), (T, 1))
    v = np.tile(np.array([2.0, -1.0]), (T, 1))
    q = np.tile(np.array([1.0, 0.5, -2.0]), (T, 1))
    S = np.zeros((D, Dv))
    o = M.hgrn2_recurrence(q, f, v, S)
    for t in range(T):
        want = sum((1 - f[0, i] ** (t + 1)) * q[0, i] for i in range(D)) * v[0]
        assert np.allclose(o[t], want)


def test_window_attention_sees_exactly_the_window():
    rng = np.random.default_rng(1)
    N, H, G, D, Dv, win = 12, 2, 1, 4, 3, 5
    q, k, v = rng.standard_normal((N, H, D)), rng.standard_normal((N, G, D)), rng.standard_normal((N, G, Dv))
    out = M.window_attention(q, k, v, 0, 0.5, win)
    for h in range(H):
        slope = 2.0 ** (-8.0 * (h + 1) / H)
        for i in range(N):
            s = np.full(N, -np.inf)
            for j in range(N):
                if 0 <= i - j < win:
                    s[j] = q[i, h] @ k[j, 0] * 0.5 - slope * (i - j)
            w = np.exp(s - s.max()); w /= w.sum()
            assert np.allclose(out[i, h], w @ v[:, 0])
    # a value just outside the window has no influence, one just inside has
    v2 = v.copy(); v2[3] += 100.0
    out2 = M.window_attention(q, k, v2, 0, 0.5, win)
    assert np.allclose(out2[8], out[8]) and not np.allclose(out2[7], out[7])


def test_portions_equal_the_whole_prompt_and_greedy_runs():
    cfg = synth.get_config("malasun", "tiny")
    w = {k: synth.bf16_to_f32(v) for k, v in synth.make_malasun(cfg, 3).items()}
    o = M.Malasun(cfg, w)
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], 50)
    whole = o.forward(ids)
    st, parts = o.new_state(), []
    for a, b in [(0, 7), (7, 9), (9, 10), (10, 43), (43, 50)]:
        parts.append(o.forward(ids[a:b], st))
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-10
    assert len(o.greedy(ids[:5], 4)) == 4


def test_synthetic_checkpoint_names_and_shapes():
    cfg = synth.get_config("malasun", "tiny")
    w = synth.make_malasun(cfg, 0)
    assert w["embed"].shape == (cfg["vocab"], cfg["width"]) and w["l0.norm1"].shape == ()
    assert "l2.mix.k" not in w and "l2.mix.q.conv" in w and "l4.mix.q.conv" not in w      # shared cache: no k / v tensors; layer 4 has no convolution
    assert w["l1.mix.lower"].shape == (3 * 16,) and w["l0.mlp.act"].shape == (2,)
    big = synth.malasun_shape(512, 6, 8, 2, 64, 256, 1024, 4, 64, vocab=1000)
    kinds = [(l["type"], l["mixer"].get("kv_from")) for l in big["layers"]]
    assert kinds == [("hgrn2", None), ("attention", None), ("hgrn2", None), ("attention", 1), ("hgrn2", None), ("attention", None)]


def test_safetensors_roundtrip_and_kind(tmp_path):
    from aha_b200 import checkpoint
    cfg = synth.get_config("malasun", "tiny")
    w = synth.make_malasun(cfg, 0)
    p = os.path.join(tmp_path, "model.safetensors")
    checkpoint.write_safetensors(p, w)
    r = checkpoint.read_safetensors(p)
    assert sorted(r) == sorted(w)
    for k in w:
        assert r[k].shape == w[k].shape and np.array_equal(np.asarray(r[k]).view(np.ndarray), np.asarray(w[k]).view(np.ndarray))
    assert checkpoint.model_kind(cfg) == "malasun"
    assert checkpoint.model_kind({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3"}) == "qwen3"
    with pytest.raises(ValueError):
        checkpoint.model_kind({"model_type": "other"})
    json.dumps(cfg)
