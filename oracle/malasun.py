"""Plain numpy restatement of the Malasun decoder (float64 arithmetic on the checkpoint's values): test infrastructure only.

A Malasun model is a list of layers read from config["layers"]; every layer is  x += norm1(mixer(x))  and, when it has a
feed-forward,  x += norm2(ff(x))  -- the scalar-gain RMS norms sit on the sublayer OUTPUTS, the sublayers read x itself.
Two mixers exist:

  hgrn2      gated linear recurrence per head with a [dim, vdim] state:  S[i, j] <- f[i] S[i, j] + (1 - f[i]) v[j],
             o[j] = sum_i S[i, j] q[i],  with the gate f = lo + (1 - lo) sigmoid(f_raw) and q = silu(q_raw)
  attention  grouped-query softmax attention over a sliding window with a linear distance penalty slope_h (i - j),
             biased q/k/v projections, a short causal convolution on q, k and v, RMS norm of q and k over the whole
             projection, a sigmoid output gate, and optionally the keys / values of an earlier layer ("kv_from")

One function per mechanism; `Malasun.forward` carries a per-sequence state so that a prompt may be fed in portions.
"""
import numpy as np

F = np.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is ONE number for all coordinates."""
    return rms_unit(x, eps) * F(np.asarray(g).reshape(-1)[0])


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def silu(z):
    return z * sigmoid(z)


def xielu(z, p, q):
    """a_p z^2 + z/2 for positive z, a_n (e^z - 1 - z) + z/2 otherwise; a_p = softplus(p), a_n = 1/2 + softplus(q)."""
    ap, aq = softplus(F(p)), 0.5 + softplus(F(q))
    pos = ap * z * z + 0.5 * z
    neg = aq * (np.expm1(np.minimum(z, 0.0)) - z) + 0.5 * z
    return np.where(z > 0, pos, neg)


def hgrn2_recurrence(q, f, v, S):
    """One head.  q, f: [T, dim]; v: [T, vdim]; S: [dim, vdim] (updated in place).  Returns o [T, vdim]."""
    T = q.shape[0]
    o = np.zeros((T, v.shape[1]), F)
    for t in range(T):
        S *= f[t][:, None]
        S += (1.0 - f[t])[:, None] * v[t][None, :]
        o[t] = S.T @ q[t]
    return o


def hgrn2_mixer(h, W, mx, eps, st):
    """h [T, width]; W: the layer's '.mix.*' tensors; st: {'S': [heads, dim, vdim]} carried between calls."""
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = silu(h @ W["q"].T).reshape(T, H, D)
    lo = W["lower"].reshape(H, D)
    f = lo + (1.0 - lo) * sigmoid((h @ W["f"].T + W["f.b"]).reshape(T, H, D))
    v = (h @ W["v"].T).reshape(T, H, Dv)
    if "S" not in st:
        st["S"] = np.zeros((H, D, Dv), F)
    out = np.zeros((T, H, Dv), F)
    for hd in range(H):
        o = hgrn2_recurrence(q[:, hd], f[:, hd], v[:, hd], st["S"][hd])
        out[:, hd] = rms_unit(o, eps) * W["norm"]
    return out.reshape(T, H * Dv) @ W["o"].T


def short_conv(u, w, tail):
    """Causal depthwise convolution.  u [T, C] (this call's projected values), w [C, taps], tail [taps-1, C] = the values
    projected before this call (zeros at a sequence's start).  y_t = sum_j w[:, j] u_{t - taps + 1 + j}.  Returns y, new tail."""
    taps = w.shape[1]
    ext = np.concatenate([tail, u], axis=0)
    T = u.shape[0]
    y = np.zeros_like(u)
    for j in range(taps):
        y += ext[j:j + T] * w[:, j][None, :]
    return y, ext[ext.shape[0] - (taps - 1):].copy()


def window_attention(q, k, v, pos0, scale, window):
    """q [T, H, D] at positions pos0 .. pos0+T-1; k [N, G, D], v [N, G, Dv] hold positions 0 .. N-1 (N = pos0 + T).
    score = q.k * scale - slope_h (i - j), slope_h = 2^(-8 (h+1) / H); visible: 0 <= i - j < window (None = all earlier)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), F)
    for hd in range(H):
        g = hd // (H // G)
        slope = 2.0 ** (-8.0 * (hd + 1) / H)
        for t in range(T):
            i = pos0 + t
            j0 = 0 if window is None else max(0, i - window + 1)
            js = np.arange(j0, i + 1)
            s = (k[js, g] @ q[t, hd]) * scale - slope * (i - js)
            s = s - s.max()
            w = np.exp(s)
            w /= w.sum()
            out[t, hd] = w @ v[js, g]
    return out


def attention_mixer(h, W, mx, eps, st, kv_of):
    """st: this layer's {'tail_q', 'tail_k', 'tail_v', 'k', 'v', 'n'}; kv_of: the state dict that owns the keys / values
    this layer reads (its own, or the one of layer mx['kv_from'], which has already run in this call)."""
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    pos0 = st.get("n", 0)
    taps = mx.get("conv")

    def proj(name, n):
        u = h @ W[name].T
        if name + ".b" in W:
            u = u + W[name + ".b"]
        if taps:
            tail = st.get("tail_" + name, np.zeros((taps - 1, n), F))
            u, st["tail_" + name] = short_conv(u, W[name + ".conv"], tail)
        return u

    q = proj("q", H * D)
    if "q.norm" in W:
        q = rms_unit(q, eps) * W["q.norm"]
    if "kv_from" not in mx:
        k = proj("k", G * D)
        if "k.norm" in W:
            k = rms_unit(k, eps) * W["k.norm"]
        v = proj("v", G * Dv)
        st["k"] = np.concatenate([st.get("k", np.zeros((0, G, D), F)), k.reshape(T, G, D)])
        st["v"] = np.concatenate([st.get("v", np.zeros((0, G, Dv), F)), v.reshape(T, G, Dv)])
    window = mx["mask"]["size"] if mx.get("mask") else None
    o = window_attention(q.reshape(T, H, D), kv_of["k"], kv_of["v"], pos0, F(mx["scale"]), window)
    o = o.reshape(T, H * Dv) * sigmoid(h @ W["g"].T)
    st["n"] = pos0 + T
    return o @ W["o"].T


def dense_ff(h, W):
    return xielu(h @ W["up"].T, W["act"][0], W["act"][1]) @ W["down"].T


class Malasun:
    def __init__(self, config, weights):
        """weights: name -> numpy array (any float dtype; values are used as they are, in float64)."""
        self.cfg = config
        self.eps = F(config["norm"]["eps"])
        self.w = {k: np.asarray(v, F) for k, v in weights.items()}
        self.layers = config["layers"]

    def sub(self, prefix):
        n = len(prefix)
        return {k[n:]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        return [dict() for _ in self.layers]

    def forward(self, tokens, state=None, trace=None):
        """Feeds `tokens` after whatever `state` already holds.  Returns logits [T, vocab]; `trace` (a list) receives the
        residual stream after every layer."""
        if state is None:
            state = self.new_state()
        x = self.w["embed"][np.asarray(tokens, np.int64)]
        for i, ly in enumerate(self.layers):
            p = "l%d." % i
            mx = ly["mixer"]
            W = self.sub(p + "mix.")
            if ly["type"] == "hgrn2":
                y = hgrn2_mixer(x, W, mx, self.eps, state[i])
            elif ly["type"] == "attention":
                y = attention_mixer(x, W, mx, self.eps, state[i], state[mx["kv_from"]] if "kv_from" in mx else state[i])
            else:
                raise ValueError("unknown mixer " + ly["type"])
            x = x + scalar_norm(y, self.w[p + "norm1"], self.eps)
            if ly.get("mlp"):
                if ly["mlp"]["kind"] != "dense":
                    raise ValueError("unknown feed-forward " + ly["mlp"]["kind"])
                x = x + scalar_norm(dense_ff(x, self.sub(p + "mlp.")), self.w[p + "norm2"], self.eps)
            if trace is not None:
                trace.append(x.copy())
        return scalar_norm(x, self.w["final.norm"], self.eps) @ self.w["head"].T

    def greedy(self, prompt, n):
        st = self.new_state()
        lg = self.forward(prompt, st)
        out = [int(np.argmax(lg[-1]))]
        for _ in range(n - 1):
            lg = self.forward([out[-1]], st)
            out.append(int(np.argmax(lg[-1])))
        return out
