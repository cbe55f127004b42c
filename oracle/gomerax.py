"""Plain numpy restatement of the Gomerax decoder (float64 arithmetic on the checkpoint's values): test infrastructure only.

A Gomerax model is a list of layers read from config["layers"]; a span of them ("loop") may run several times in a row with the same
weights, every pass with caches of its own, and the embedding output is added to the stream again before every pass but the first.
The embedding is the scaled table row plus a learned vector of the token's position.  A layer is PARALLEL: one RMS norm whose gain is
stored as an offset from one,

    h = x / rms(x) * (1 + w),      x += mixer(h) + ff(h),

with both sublayers reading the same h.  The mixer is windowed latent attention: queries through a normed latent of their own, one
normed latent plus one rotated key part per token shared by all heads, rotary positions on interleaved pairs, and a softmax whose
denominator holds exp(sink) of a learned number per head.  Feed-forwards: dense (silu gate, biases everywhere) or routed experts
(clamped gate / up with a sigmoid-weighted gate; softmax router with a choice correction, expert groups, weights renormalised over
the chosen experts and scaled) plus a shared expert.  The unscaled embedding table is the output projection.
One function per mechanism; `Gomerax.forward` carries a per-sequence state so that a prompt may be fed in portions.
"""
import numpy as np

F = np.float64
GLU_SLOPE = 1.702       # the experts' gate is g * sigmoid(GLU_SLOPE * g)
WEIGHT_FLOOR = 1e-20    # added to the sum of the chosen scores before the division


def sigmoid(z):
    return 0.5 * (1.0 + np.tanh(0.5 * np.asarray(z, F)))


def silu(z):
    return z * sigmoid(z)


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_plain(x, w, eps):
    """gain stored as it is applied"""
    return rms_unit(x, eps) * w


def norm_offset(x, w, eps):
    """gain stored around zero"""
    return rms_unit(x, eps) * (1.0 + w)


def embed_rows(tokens, pos, table, pos_table, scale):
    return table[tokens] * scale + pos_table[pos]


def rotary_frequencies(base, dims):
    return np.array([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], F)


def rotate_pairs(x, pos, freqs):
    """x [T, ..., n]: coordinates (2i, 2i + 1) of the first 2 len(freqs) turn by pos * f_i, the rest pass."""
    out = x.copy()
    n = 2 * len(freqs)
    ang = pos.astype(F)[:, None] * freqs[None, :]
    c, s = np.cos(ang), np.sin(ang)
    while c.ndim < x.ndim:
        c, s = c[:, None], s[:, None]
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def sink_softmax(s, visible, sink):
    """rows of s over the visible entries; the denominator also holds exp(sink)"""
    s = np.where(visible, s, -np.inf)
    m = np.maximum(s.max(axis=1, keepdims=True), sink)
    p = np.exp(s - m)
    return p / (p.sum(axis=1, keepdims=True) + np.exp(sink - m))


def latent_attention_mixer(h, W, mx, eps, st, pos0):
    H, D, R, Dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    window = mx["mask"]["size"]
    T = h.shape[0]
    pos = pos0 + np.arange(T)
    freqs = rotary_frequencies(mx["rot"]["base"], mx["rot"]["dims"])
    q = (norm_plain(h @ W["dq"].T, W["dq.norm"], eps) @ W["uq"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, freqs)
    dkv = h @ W["dkv"].T
    c = norm_plain(dkv[:, :rank], W["dkv.norm"], eps)
    k_rot = rotate_pairs(dkv[:, rank:], pos, freqs)
    if "c" in st:
        c, k_rot = np.concatenate([st["c"], c]), np.concatenate([st["kr"], k_rot])
    st["c"], st["kr"] = c, k_rot
    S = c.shape[0]
    k = (c @ W["uk"].T).reshape(S, H, D)
    v = (c @ W["uv"].T).reshape(S, H, Dv)
    j = np.arange(S)[None, :]
    visible = (j <= pos[:, None]) & (pos[:, None] - j < window)
    o = np.zeros((T, H, Dv), F)
    for hd in range(H):
        s = (q_plain[:, hd] @ k[:, hd].T + q_rot[:, hd] @ k_rot.T) * mx["scale"]
        o[:, hd] = sink_softmax(s, visible, W["sink"][hd]) @ v[:, hd]
    return o.reshape(T, H * Dv) @ W["o"].T


def dense_ff(h, W):
    g = h @ W["gate"].T + W["gate.b"]
    u = h @ W["up"].T + W["up.b"]
    return (silu(g) * u) @ W["down"].T + W["down.b"]


def clamped_expert(h, W, p, limit):
    g = np.minimum(h @ W[p + "gate"].T, limit)
    u = np.clip(h @ W[p + "up"].T, -limit, limit)
    return (g * sigmoid(GLU_SLOPE * g) * (u + 1.0)) @ W[p + "down"].T


def route(z, correction, router):
    """z [experts] router logits of one token -> (chosen experts, their weights)"""
    E, top = router["experts"], router["top"]
    s = np.exp(z - z.max())
    s = s / s.sum()
    choice = s + correction
    groups = router.get("groups")
    if groups:
        n = E // groups["count"]
        best = choice.reshape(groups["count"], n).max(axis=1)
        kept = np.argsort(-best, kind="stable")[:groups["keep"]]
        allowed = np.zeros(E, bool)
        for g in kept:
            allowed[g * n:(g + 1) * n] = True
        choice = np.where(allowed, choice, -np.inf)
    chosen = np.argsort(-choice, kind="stable")[:top]
    w = s[chosen] / (s[chosen].sum() + WEIGHT_FLOOR) * router["scale"]
    return chosen, w


def routed_experts(h, W, ml):
    z = h @ W["router"].T
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, w = route(z[t], W["correction"], ml["router"])
        for e, we in zip(chosen, w):
            out[t] += we * clamped_expert(h[t], W, "e%d." % e, ml["expert"]["limit"])
    if ml.get("shared"):
        out += clamped_expert(h, W, "shared.", ml["shared"]["limit"])
    return out


def layer_runs(cfg):
    """(layer, opens a pass after the first) for every layer run, in order"""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(l, False) for l in range(lp["start"])]
    for t in range(lp["times"] if lp["stop"] > lp["start"] else 0):
        runs += [(l, t > 0 and l == lp["start"]) for l in range(lp["start"], lp["stop"])]
    return runs + [(l, False) for l in range(lp["stop"], n)]


class Gomerax:
    def __init__(self, config, weights):
        self.cfg = config
        self.w = {k: np.asarray(v, F) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])
        self.runs = layer_runs(config)

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        return {"pos": 0, "runs": [dict() for _ in self.runs]}

    def forward(self, tokens, state=None, trace=None):
        """tokens [T] of ONE sequence, appended to what `state` holds (None: a new sequence).  Returns logits [T, vocab] (float64).
        trace: a list that receives the stream after every layer run."""
        cfg, w, eps = self.cfg, self.w, self.eps
        if state is None:
            state = self.new_state()
        tokens = np.asarray(tokens, np.int64)
        pos0 = state["pos"]
        x0 = embed_rows(tokens, pos0 + np.arange(len(tokens)), w["embed"], w["pos"], float(cfg["embedding"]["scale"]))
        x = x0.copy()
        for r, (l, again) in enumerate(self.runs):
            ly, p = cfg["layers"][l], "l%d." % l
            if again:
                x = x + x0
            h = norm_offset(x, w[p + "norm1"], eps)
            assert ly["type"] == "latent_attention", ly["type"]
            y = latent_attention_mixer(h, self.sub(p + "mix."), ly["mixer"], eps, state["runs"][r], pos0)
            if ly.get("mlp"):
                W = self.sub(p + "mlp.")
                y = y + (dense_ff(h, W) if ly["mlp"]["kind"] == "dense" else routed_experts(h, W, ly["mlp"]))
            x = x + y
            if trace is not None:
                trace.append(x.copy())
        state["pos"] = pos0 + len(tokens)
        return norm_offset(x, w["final.norm"], eps) @ w["embed"].T

    def greedy(self, prompt, n):
        """n tokens of greedy decoding after `prompt` (the first of equal maxima wins)."""
        st = self.new_state()
        lg = self.forward(prompt, st)[-1]
        out = []
        for _ in range(n):
            out.append(int(np.argmax(lg.astype(np.float32))))
            lg = self.forward([out[-1]], st)[-1]
        return out
