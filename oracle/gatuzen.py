"""Plain numpy restatement of the Gatuzen decoder (float64 arithmetic on the checkpoint's values): test infrastructure only.

A Gatuzen model is a list of layers read from config["layers"], a span of which ("loop": start, stop, times) may run several
times in a row with the same weights and a state of its own per pass; before every pass a learned vector is added to the stream.
A layer is a sandwich around each sublayer,

    x += m * post_norm(sublayer(h + conv(h))),     h = pre_norm(x),

with grouped RMS norms (the vector is cut into equal consecutive parts, each divided by its own root mean square, then a
per-coordinate gain) and a short causal per-channel convolution on what the sublayer reads.  Three mixers:

  gla               gated linear attention: S <- diag(alpha) S + k v^T per head, o = S^T q, alpha = sigmoid(z)^(1/tau)
  mamba2            selective state space: S <- exp(-exp(A_log) dt) S + dt B x^T per head, y = S^T C + D x
  latent_attention  softmax attention whose keys / values are expanded from one cached low-rank latent per token plus one
                    rotated key part shared by the heads (rotary with YaRN frequency interpolation)

and one feed-forward: gated experts chosen by a lookup table on the token id (no router), equal weights.
One function per mechanism; `Gatuzen.forward` carries a per-sequence state so that a prompt may be fed in portions.
"""
import math

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def group_norm(x, w, groups, eps):
    """RMS norm in `groups` equal consecutive parts of the last axis, then the gain w (one number per coordinate)."""
    T, C = x.shape
    return rms_unit(x.reshape(T, groups, C // groups), eps).reshape(T, C) * w


def causal_conv(u, w, tail, bias=None):
    """y_t = sum_j w[:, j] u_{t - taps + 1 + j} (+ bias).  u [T, C]; w [C, taps]; tail [taps - 1, C]: the inputs before this call
    (zeros at a sequence's start).  Returns y and the new tail."""
    taps = w.shape[1]
    full = np.concatenate([tail, u], axis=0)
    T = u.shape[0]
    y = np.zeros_like(u)
    for j in range(taps):
        y += full[j:j + T] * w[:, j]
    if bias is not None:
        y = y + bias
    return y, full[full.shape[0] - (taps - 1):].copy()


def input_conv(h, w, st, key):
    """h + conv(h) with the convolution's last inputs kept in st[key]."""
    if key not in st:
        st[key] = np.zeros((w.shape[1] - 1, h.shape[1]), F)
    y, st[key] = causal_conv(h, w, st[key])
    return h + y


def diag_recurrence(q, k, v, decay, S):
    """One head of  S <- diag(decay_t) S + k_t v_t^T,  o_t = S^T q_t.  q, k, decay [T, dk]; v [T, dv]; S [dk, dv] in place."""
    T = q.shape[0]
    o = np.zeros((T, v.shape[1]), F)
    for t in range(T):
        S *= decay[t][:, None]
        S += k[t][:, None] * v[t][None, :]
        o[t] = S.T @ q[t]
    return o


def gla_mixer(h, W, mx, eps, st):
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W["k"].T).reshape(T, H, D)
    v = (h @ W["v"].T).reshape(T, H, Dv)
    z = ((h @ W["a1"].T) @ W["a2"].T + W["a2.b"]).reshape(T, H, D)
    alpha = np.exp(-softplus(-z) / mx["tau"])          # sigmoid(z) ** (1 / tau)
    if "S" not in st:
        st["S"] = np.zeros((H, D, Dv), F)
    o = np.zeros((T, H, Dv), F)
    for hd in range(H):
        o[:, hd] = rms_unit(diag_recurrence(q[:, hd], k[:, hd], v[:, hd], alpha[:, hd], st["S"][hd]), eps) * W["norm"]
    return (o.reshape(T, H * Dv) * silu(h @ W["g"].T)) @ W["o"].T


def mamba2_mixer(h, W, mx, eps, st):
    H, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = H * P
    T = h.shape[0]
    u = h @ W["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    if "conv" not in st:
        st["conv"] = np.zeros((W["conv"].shape[1] - 1, xbc.shape[1]), F)
        st["S"] = np.zeros((H, N, P), F)
    xbc, st["conv"] = causal_conv(xbc, W["conv"], st["conv"], W["conv.b"])
    xbc = silu(xbc)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W["dt_bias"])                   # [T, H]
    a = np.exp(-np.exp(W["A_log"]) * dt)
    y = np.zeros((T, H, P), F)
    for hd in range(H):
        g = hd // (H // G)
        dec = np.repeat(a[:, hd:hd + 1], N, axis=1)
        y[:, hd] = diag_recurrence(C[:, g], dt[:, hd:hd + 1] * B[:, g], x[:, hd], dec, st["S"][hd]) + W["D"][hd] * x[:, hd]
    y = y.reshape(T, inner) * silu(z)
    return group_norm(y, W["norm"], mx["norm_groups"], eps) @ W["o"].T


def rotary_table(rot):
    """Frequencies [dims / 2] and the factor on cos / sin.  With 'scaling': YaRN -- low frequencies are divided by `factor`, high
    ones kept, a linear ramp between the dimensions whose wavelengths fit `fast` and `slow` times into the original length."""
    dims, base = rot["dims"], float(rot["base"])
    i = np.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(sc["fast"])), 0)
    hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, pos, freqs, mult):
    """x [T, ..., n]: coordinates (2i, 2i + 1), i < len(freqs), turn by pos * freqs[i]; cos and sin carry `mult`; the rest passes."""
    out = x.copy()
    n = 2 * len(freqs)
    ang = pos.astype(F)[:, None] * freqs[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (len(freqs),)
    c, s = (np.cos(ang) * mult).reshape(shape), (np.sin(ang) * mult).reshape(shape)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def latent_attention_mixer(h, W, mx, eps, st, pos0):
    H, D, R, Dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    pos = pos0 + np.arange(T)
    freqs, mult = rotary_table(mx["rot"])
    q = (h @ W["q"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, freqs, mult)
    d = h @ W["dkv"].T
    c = rms_unit(d[:, :rank], eps) * W["dkv.norm"]
    k_rot = rotate_pairs(d[:, rank:], pos, freqs, mult)
    if "c" not in st:
        st["c"], st["kr"] = np.zeros((0, rank), F), np.zeros((0, R), F)
    st["c"] = np.concatenate([st["c"], c])
    st["kr"] = np.concatenate([st["kr"], k_rot])
    S = st["c"].shape[0]
    k_plain = (st["c"] @ W["uk"].T).reshape(S, H, D)
    val = (st["c"] @ W["uv"].T).reshape(S, H, Dv)
    o = np.zeros((T, H, Dv), F)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ st["kr"].T) * mx["scale"]
        s = np.where(np.arange(S)[None, :] <= pos[:, None], s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        o[:, hd] = (p / p.sum(axis=1, keepdims=True)) @ val[:, hd]
    return (o.reshape(T, H * Dv) * sigmoid(h @ W["g"].T)) @ W["o"].T


def table_moe(h, tokens, W, ml):
    """Every token's experts come from a table row of its id; the chosen experts' outputs are averaged."""
    top = ml["router"]["top"]
    table = np.asarray(W["table"]).astype(np.int64)
    out = np.zeros_like(h)
    for t, tok in enumerate(tokens):
        for e in table[int(tok)][:top]:
            p = "e%d." % e
            out[t] += (silu(h[t] @ W[p + "gate"].T) * (h[t] @ W[p + "up"].T)) @ W[p + "down"].T / top
    return out


class Gatuzen:
    def __init__(self, config, weights):
        self.cfg = config
        self.w = {k: np.asarray(v, F) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])
        self.groups = int(config["norm"].get("groups", 1))
        self.mult = float(config.get("residual_mult", 1.0))
        L = len(config["layers"])
        lp = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
        # (layer, pass number when the run opens a pass else None)
        self.runs = [(l, None) for l in range(lp["start"])]
        for t in range(lp["times"] if lp["stop"] > lp["start"] else 0):
            self.runs += [(l, t if l == lp["start"] else None) for l in range(lp["start"], lp["stop"])]
        self.runs += [(l, None) for l in range(max(lp["stop"], lp["start"]), L)]

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        return {"pos": 0, "runs": [dict() for _ in self.runs]}

    def forward(self, tokens, state=None, trace=None):
        """tokens [T] of ONE sequence, appended to what `state` holds (None: a new sequence).  Returns logits [T, vocab] (float64).
        trace: a list that receives the stream after every layer run."""
        cfg, w = self.cfg, self.w
        if state is None:
            state = self.new_state()
        tokens = np.asarray(tokens, np.int64)
        x = w["embed"][tokens] * float(cfg.get("embedding", {}).get("scale", 1.0))
        pos0 = state["pos"]
        for r, (l, opens) in enumerate(self.runs):
            ly, st, p = cfg["layers"][l], state["runs"][r], "l%d." % l
            if opens is not None:
                x = x + w["loop.step"][opens]
            h = group_norm(x, w[p + "norm1"], self.groups, self.eps)
            if p + "canon1" in w:
                h = input_conv(h, w[p + "canon1"], st, "canon1")
            W = self.sub(p + "mix.")
            if ly["type"] == "gla":
                y = gla_mixer(h, W, ly["mixer"], self.eps, st)
            elif ly["type"] == "mamba2":
                y = mamba2_mixer(h, W, ly["mixer"], self.eps, st)
            elif ly["type"] == "latent_attention":
                y = latent_attention_mixer(h, W, ly["mixer"], self.eps, st, pos0)
            else:
                raise ValueError(ly["type"])
            x = x + self.mult * group_norm(y, w[p + "norm1b"], self.groups, self.eps)
            if ly.get("mlp"):
                h = group_norm(x, w[p + "norm2"], self.groups, self.eps)
                if p + "canon2" in w:
                    h = input_conv(h, w[p + "canon2"], st, "canon2")
                y = table_moe(h, tokens, self.sub(p + "mlp."), ly["mlp"])
                x = x + self.mult * group_norm(y, w[p + "norm2b"], self.groups, self.eps)
            if trace is not None:
                trace.append(x.copy())
        state["pos"] = pos0 + len(tokens)
        x = group_norm(x, w["final.norm"], self.groups, self.eps)
        return (x @ w["head"].T) * float(cfg.get("logit_scale", 1.0))

    def greedy(self, prompt, n):
        """n tokens of greedy decoding after `prompt` (the first of equal maxima wins)."""
        st = self.new_state()
        lg = self.forward(prompt, st)[-1]
        out = []
        for _ in range(n):
            out.append(int(np.argmax(lg.astype(np.float32))))
            lg = self.forward([out[-1]], st)[-1]
        return out
