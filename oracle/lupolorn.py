"""Plain numpy restatement of the Lupolorn decoder (float64 arithmetic on the checkpoint's values): test infrastructure only.

A Lupolorn model is a list of layers read from config["layers"].  A layer wraps each sublayer in two RMS norms with a gain per
channel,

    x += norm_after(sublayer(norm_before(x))),

first the mixer, then the feed-forward (if the layer has one).  Three mixers:

  mingru            elementwise gated recurrence  S_t = (1 - z_t) S_{t-1} + z_t c_t  whose gate and candidate read the current token only
  latent_attention  sliding-window softmax attention without positions; queries, keys and values are expanded from normed low-rank latents,
                    one latent per token is all a cache has to hold
  attention         causal attention with grouped key / value heads, rotary positions on interleaved pairs (frequencies rescaled band by band),
                    unit-RMS queries and keys, a softmax whose denominator holds an extra 1, and a sigmoid gate per head on the output

and two feed-forwards with the squared relu: dense, and routed experts (softmax router, the `top` best scores used as they are) plus a
shared expert behind a sigmoid gate.  The embedding table, unscaled, is also the output projection.
One function per mechanism; `Lupolorn.forward` carries a per-sequence state so that a prompt may be fed in portions.
"""
import math

import numpy as np

F = np.float64


def sigmoid(z):
    return 0.5 * (1.0 + np.tanh(0.5 * np.asarray(z, F)))


def silu(z):
    return z * sigmoid(z)


def relu2(z):
    return np.square(np.maximum(z, 0.0))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def mingru_candidate(u):
    """u + 1/2 on the non-negative side, the logistic function on the negative side (the two meet at 1/2)."""
    return np.where(u >= 0.0, u + 0.5, sigmoid(np.minimum(u, 0.0)))


def mingru_mixer(h, W, st):
    """h [T, width]; st["S"] is the running state [n] of the sequence."""
    z = sigmoid(h @ W["z"].T + W["z.b"])
    cand = mingru_candidate(h @ W["x"].T + W["x.b"])
    S = st.get("S")
    if S is None:
        S = np.zeros(z.shape[1], F)
    out = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S
    st["S"] = S
    return (out * silu(h @ W["g"].T)) @ W["o"].T


def softmax_rows(s, visible, sink=False):
    """Rows of s over the visible entries; sink: an extra entry of score 0 (and no value) takes part in the denominator."""
    s = np.where(visible, s, -np.inf)
    m = s.max(axis=1, keepdims=True)
    if sink:
        m = np.maximum(m, 0.0)
    p = np.exp(s - m)
    den = p.sum(axis=1, keepdims=True)
    if sink:
        den = den + np.exp(-m)
    return p / den


def latent_attention_mixer(h, W, mx, eps, st, pos0):
    H, D, Dv, window = mx["heads"], mx["dim"], mx["vdim"], mx["mask"]["size"]
    T = h.shape[0]
    pos = pos0 + np.arange(T)
    cq = rms_norm(h @ W["dq"].T, W["dq.norm"], eps)
    q = (cq @ W["uq"].T).reshape(T, H, D)
    c = rms_norm(h @ W["dkv"].T, W["dkv.norm"], eps)
    st["c"] = c if "c" not in st else np.concatenate([st["c"], c])
    S = st["c"].shape[0]
    k = (st["c"] @ W["uk"].T).reshape(S, H, D)
    val = (st["c"] @ W["uv"].T).reshape(S, H, Dv)
    j = np.arange(S)[None, :]
    visible = (j <= pos[:, None]) & (pos[:, None] - j < window)
    o = np.zeros((T, H, Dv), F)
    for hd in range(H):
        o[:, hd] = softmax_rows(q[:, hd] @ k[:, hd].T * mx["scale"], visible) @ val[:, hd]
    return o.reshape(T, H * Dv) @ W["o"].T


def banded_frequencies(rot):
    """f_i = base^(-2i/dims); with "scaling": short waves (below original / high) are kept, long ones (above original / low) divided by
    `factor`, those between move linearly, in original / wavelength, from the one to the other."""
    dims = rot["dims"]
    f = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)], F)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wl = 2.0 * math.pi / fi
        if wl < orig / high:
            out[i] = fi
        elif wl > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / wl - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_pairs(x, pos, freqs):
    """x [T, heads, dim]: coordinates (2i, 2i + 1) of the first 2 len(freqs) are turned by pos * f_i; the rest pass."""
    out = x.copy()
    n = 2 * len(freqs)
    ang = pos[:, None].astype(F) * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def attention_mixer(h, W, mx, eps, st, pos0):
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    pos = pos0 + np.arange(T)
    freqs = banded_frequencies(mx["rot"]) if mx.get("rot") and mx["rot"]["dims"] > 0 else np.zeros(0, F)
    q = rms_unit(rotate_pairs((h @ W["q"].T).reshape(T, H, D), pos, freqs), eps)
    k = rms_unit(rotate_pairs((h @ W["k"].T).reshape(T, G, D), pos, freqs), eps)
    v = (h @ W["v"].T).reshape(T, G, Dv)
    if "k" in st:
        k, v = np.concatenate([st["k"], k]), np.concatenate([st["v"], v])
    st["k"], st["v"] = k, v
    S = k.shape[0]
    visible = np.arange(S)[None, :] <= pos[:, None]
    gate = sigmoid(h @ W["g"].T)                # [T, H]
    o = np.zeros((T, H, Dv), F)
    for hd in range(H):
        g = hd // (H // G)
        o[:, hd] = (softmax_rows(q[:, hd] @ k[:, g].T * mx["scale"], visible, sink=True) @ v[:, g]) * gate[:, hd:hd + 1]
    return o.reshape(T, H * Dv) @ W["o"].T


def ff_unit(h, W, p=""):
    return relu2(h @ W[p + "up"].T) @ W[p + "down"].T


def routed_experts(h, W, ml):
    """softmax router over all experts; the `top` largest scores weigh their experts as they are (earlier expert first among equals)."""
    top = ml["router"]["top"]
    z = h @ W["router"].T
    s = np.exp(z - z.max(axis=1, keepdims=True))
    s = s / s.sum(axis=1, keepdims=True)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in np.argsort(-s[t], kind="stable")[:top]:
            out[t] += s[t, e] * ff_unit(h[t], W, "e%d." % e)
    if "shared.up" in W:
        out += ff_unit(h, W, "shared.") * sigmoid(h @ W["shared.sg"].T)
    return out


class Lupolorn:
    def __init__(self, config, weights):
        self.cfg = config
        self.w = {k: np.asarray(v, F) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        return {"pos": 0, "layers": [dict() for _ in self.cfg["layers"]]}

    def forward(self, tokens, state=None, trace=None):
        """tokens [T] of ONE sequence, appended to what `state` holds (None: a new sequence).  Returns logits [T, vocab] (float64).
        trace: a list that receives the stream after every layer."""
        cfg, w, eps = self.cfg, self.w, self.eps
        if state is None:
            state = self.new_state()
        tokens = np.asarray(tokens, np.int64)
        x = w["embed"][tokens] * float(cfg.get("embedding", {}).get("scale", 1.0))
        pos0 = state["pos"]
        for l, ly in enumerate(cfg["layers"]):
            st, p = state["layers"][l], "l%d." % l
            h = rms_norm(x, w[p + "norm1"], eps)
            W = self.sub(p + "mix.")
            if ly["type"] == "mingru":
                y = mingru_mixer(h, W, st)
            elif ly["type"] == "latent_attention":
                y = latent_attention_mixer(h, W, ly["mixer"], eps, st, pos0)
            elif ly["type"] == "attention":
                y = attention_mixer(h, W, ly["mixer"], eps, st, pos0)
            else:
                raise ValueError(ly["type"])
            x = x + rms_norm(y, w[p + "norm1b"], eps)
            if ly.get("mlp"):
                h = rms_norm(x, w[p + "norm2"], eps)
                W = self.sub(p + "mlp.")
                y = ff_unit(h, W) if ly["mlp"]["kind"] == "dense" else routed_experts(h, W, ly["mlp"])
                x = x + rms_norm(y, w[p + "norm2b"], eps)
            if trace is not None:
                trace.append(x.copy())
        state["pos"] = pos0 + len(tokens)
        return rms_norm(x, w["final.norm"], eps) @ w["embed"].T

    def greedy(self, prompt, n):
        """n tokens of greedy decoding after `prompt` (the first of equal maxima wins)."""
        st = self.new_state()
        lg = self.forward(prompt, st)[-1]
        out = []
        for _ in range(n):
            out.append(int(np.argmax(lg.astype(np.float32))))
            lg = self.forward([out[-1]], st)[-1]
        return out
