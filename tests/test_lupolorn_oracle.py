"""The plain Lupolorn restatement (oracle/lupolorn.py) checked against closed forms, and the host-side pieces that need no GPU:
synthetic checkpoints through the safetensors reader, the choice of the executor by config.json."""
import json
import math
import os

import numpy as np

from aha_b200 import synth
from oracle import lupolorn as Z


def test_mingru_candidate_is_continuous_and_the_recurrence_has_closed_forms():
    assert Z.mingru_candidate(np.array([0.0]))[0] == 0.5 and abs(Z.mingru_candidate(np.array([-1e-9]))[0] - 0.5) < 1e-9
    assert np.allclose(Z.mingru_candidate(np.array([2.0, -2.0])), [2.5, 1.0 / (1.0 + math.e ** 2)])
    # identity projections: the gate reads channel pairs of h directly.  A constant gate z and candidate c give S_t = c (1 - (1 - z)^t)
    n, T = 3, 12
    eye = np.eye(n)
    W = {"z": eye, "z.b": np.zeros(n), "x": eye * 0.0, "x.b": np.array([1.5, -0.7, 0.0]), "g": eye * 0.0, "o": eye}
    h = np.tile(np.array([0.0, 2.0, -3.0]), (T, 1))
    st = {}
    y = Z.mingru_mixer(h, W, st)
    z, c = Z.sigmoid(h[0]), Z.mingru_candidate(W["x.b"])
    assert np.allclose(st["S"], c * (1.0 - (1.0 - z) ** T))
    assert np.allclose(y, 0.0)                                  # silu(0) = 0 closes the output gate
    W["g"] = eye
    st2, parts = {}, []
    for a, b in [(0, 1), (1, 3), (3, 4), (4, 12)]:              # fed in portions: the state carries over
        parts.append(Z.mingru_mixer(h[a:b], W, st2))
    assert np.allclose(np.concatenate(parts), Z.mingru_mixer(h, W, {})) and np.allclose(st2["S"], st["S"])


def test_sink_softmax_leaves_room_for_nothing():
    s = np.array([[0.0, 0.0, 0.0], [50.0, -50.0, 0.0], [-60.0, -60.0, -60.0]])
    vis = np.ones_like(s, bool)
    p = Z.softmax_rows(s, vis, sink=True)
    assert np.allclose(p[0], 0.25) and np.allclose(p[0].sum(), 0.75)
    assert np.allclose(p[1], [1.0, 0.0, 0.0], atol=1e-20)       # a large score: the sink does not matter
    assert p[2].sum() < 1e-25                                    # very negative scores: the head attends to (almost) nothing
    q = Z.softmax_rows(s, vis)
    assert np.allclose(q.sum(axis=1), 1.0)
    vis[0, 2] = False
    assert np.allclose(Z.softmax_rows(s, vis, sink=True)[0], [1 / 3, 1 / 3, 0.0])


def test_banded_frequencies_keep_short_waves_and_stretch_long_ones():
    rot = {"base": 100.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}}
    plain = Z.banded_frequencies({"base": 100.0, "dims": 16})
    f = Z.banded_frequencies(rot)
    assert np.allclose(plain, [100.0 ** (-2.0 * i / 16) for i in range(8)])
    wl = 2 * math.pi / plain
    assert np.allclose(f[wl < 10.0], plain[wl < 10.0]) and (wl < 10.0).any()
    assert np.allclose(f[wl > 40.0], plain[wl > 40.0] / 4.0) and (wl > 40.0).any()
    mid = (wl >= 10.0) & (wl <= 40.0)
    assert mid.any() and ((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 4.0)).all()
    s = (40.0 / wl[mid] - 1.0) / 3.0
    assert np.allclose(f[mid], (1 - s) * plain[mid] / 4.0 + s * plain[mid])


def test_rotation_turns_interleaved_pairs_and_keeps_the_rest():
    x = np.random.default_rng(0).standard_normal((5, 2, 10))
    pos = np.array([0, 1, 2, 7, 30])
    fr = np.array([1.0, 0.1, 0.01])
    y = Z.rotate_pairs(x, pos, fr)
    assert np.allclose(y[0], x[0]) and np.allclose(y[..., 6:], x[..., 6:])
    for t in range(5):
        for i in range(3):
            a = pos[t] * fr[i]
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            assert np.allclose(y[t, :, 2 * i], u * math.cos(a) - v * math.sin(a)) and np.allclose(y[t, :, 2 * i + 1], v * math.cos(a) + u * math.sin(a))
    # a dot product of two rotated vectors depends on the distance only
    q, k = x[0, 0], x[1, 0]
    d = [Z.rotate_pairs(q[None, None], np.array([p + 4]), fr)[0, 0] @ Z.rotate_pairs(k[None, None], np.array([p]), fr)[0, 0] for p in (0, 9, 100)]
    assert np.allclose(d, d[0])


def _attention_weights(T=9, H=4, G=2, D=6, Dv=5, W=7, seed=1):
    rng = np.random.default_rng(seed)
    return {"q": rng.standard_normal((H * D, W)), "k": rng.standard_normal((G * D, W)), "v": rng.standard_normal((G * Dv, W)),
            "g": rng.standard_normal((H, W)), "o": rng.standard_normal((W, H * Dv))}, rng.standard_normal((T, W))


def test_attention_is_causal_grouped_gated_and_unit_normed():
    mx = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.7, "rot": {"base": 50.0, "dims": 4}}
    W, h = _attention_weights()
    y = Z.attention_mixer(h, W, mx, 1e-6, {}, 0)
    h2 = h.copy(); h2[6:] += 1.0
    assert np.allclose(Z.attention_mixer(h2, W, mx, 1e-6, {}, 0)[:6], y[:6])            # later tokens do not reach back
    st, parts = {}, []
    for a, b in [(0, 2), (2, 3), (3, 9)]:
        parts.append(Z.attention_mixer(h[a:b], W, mx, 1e-6, st, a))
    assert np.allclose(np.concatenate(parts), y)
    # unit-norm queries and keys: scaling W_q or W_k changes nothing (eps aside); a closed gate silences its head
    W2 = dict(W); W2["q"] = 3.0 * W["q"]; W2["k"] = 0.5 * W["k"]
    assert np.allclose(Z.attention_mixer(h, W2, mx, 0.0, {}, 0), Z.attention_mixer(h, W, mx, 0.0, {}, 0))
    # one gate number per head: with head 1's gate shut, head 1's columns of W_o no longer matter
    hp = np.abs(h)
    W3 = dict(W); W3["g"] = W["g"].copy(); W3["g"][1] = -100.0
    W4 = dict(W3); W4["o"] = W["o"].copy(); W4["o"][:, 5:10] = 0.0
    assert np.allclose(Z.attention_mixer(hp, W3, mx, 1e-6, {}, 0), Z.attention_mixer(hp, W4, mx, 1e-6, {}, 0))
    # the first token sees only itself and the sink: with q = k (one head, no rotation at position 0) its weight is e^s / (1 + e^s), s = scale * dim
    one = {"heads": 1, "kv_heads": 1, "dim": 6, "vdim": 5, "scale": 0.7, "rot": {"base": 50.0, "dims": 4}}
    W5 = {"q": W["q"][:6], "k": W["q"][:6], "v": W["v"][:5], "g": np.zeros((1, 7)), "o": np.eye(5)}
    s = 0.7 * 6
    assert np.allclose(Z.attention_mixer(h[:1], W5, one, 0.0, {}, 0)[0], 0.5 * math.exp(s) / (1 + math.exp(s)) * (h[0] @ W5["v"].T))


def test_latent_attention_window_is_exact_at_its_edges():
    rng = np.random.default_rng(3)
    H, D, Dv, r, qr, Wd, T, win = 2, 4, 3, 5, 6, 7, 14, 4
    mx = {"heads": H, "dim": D, "vdim": Dv, "kv_rank": r, "q_rank": qr, "mask": {"size": win}, "scale": 0.5}
    W = {"dq": rng.standard_normal((qr, Wd)), "dq.norm": rng.standard_normal(qr), "uq": rng.standard_normal((H * D, qr)), "dkv": rng.standard_normal((r, Wd)),
         "dkv.norm": rng.standard_normal(r), "uk": rng.standard_normal((H * D, r)), "uv": rng.standard_normal((H * Dv, r)), "o": np.eye(H * Dv)}
    h = rng.standard_normal((T, Wd))
    y = Z.latent_attention_mixer(h, W, mx, 1e-6, {}, 0)
    for j, moved in [(10 - win, False), (10 - win + 1, True), (10, True), (11, False)]:      # position 10 sees 7 .. 10
        h2 = h.copy(); h2[j] += 2.0
        y2 = Z.latent_attention_mixer(h2, W, mx, 1e-6, {}, 0)
        assert (not np.allclose(y2[10], y[10])) == moved, j
    st, parts = {}, []
    for a, b in [(0, 1), (1, 6), (6, 8), (8, 14)]:
        parts.append(Z.latent_attention_mixer(h[a:b], W, mx, 1e-6, st, a))
    assert np.allclose(np.concatenate(parts), y)
    wide = dict(mx); wide["mask"] = {"size": 100}
    assert np.allclose(Z.latent_attention_mixer(h[:win], W, wide, 1e-6, {}, 0), y[:win])      # the first tokens see everything before them


def test_routed_experts_use_the_best_scores_unrenormalised():
    rng = np.random.default_rng(4)
    Wd, E, ff, T = 6, 5, 4, 8
    W = {"router": rng.standard_normal((E, Wd)) * 2}
    for e in range(E):
        W["e%d.up" % e] = rng.standard_normal((ff, Wd)); W["e%d.down" % e] = rng.standard_normal((Wd, ff))
    h = rng.standard_normal((T, Wd))
    ml = {"router": {"experts": E, "top": 2}}
    y = Z.routed_experts(h, W, ml)
    z = h @ W["router"].T
    s = np.exp(z) / np.exp(z).sum(axis=1, keepdims=True)
    for t in range(T):
        best = np.argsort(-s[t])[:2]
        want = sum(s[t, e] * (np.maximum(h[t] @ W["e%d.up" % e].T, 0) ** 2) @ W["e%d.down" % e].T for e in best)
        assert np.allclose(y[t], want) and s[t, best].sum() < 1.0
    allE = Z.routed_experts(h, W, {"router": {"experts": E, "top": E}})
    assert np.allclose(allE, sum(s[:, e:e + 1] * Z.ff_unit(h, W, "e%d." % e) for e in range(E)))
    W["shared.up"] = rng.standard_normal((3, Wd)); W["shared.down"] = rng.standard_normal((Wd, 3)); W["shared.sg"] = rng.standard_normal((1, Wd))
    assert np.allclose(Z.routed_experts(h, W, ml) - y, Z.ff_unit(h, W, "shared.") * Z.sigmoid(h @ W["shared.sg"].T))


LAYERS = [{"type": "attention", "heads": 4, "kv_heads": 2, "dim": 6, "vdim": 4, "rot_dims": 4, "base": 30.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 16}, "ff": 20},
          {"type": "mingru", "width": 10, "ff": {"experts": 4, "top": 2, "ff": 8, "shared": 6}},
          {"type": "latent_attention", "heads": 3, "dim": 4, "vdim": 6, "kv_rank": 5, "q_rank": 7, "window": 9, "ff": None}]


def test_portions_equal_the_whole_prompt_and_the_head_is_the_embedding():
    cfg = synth.lupolorn_config(LAYERS, width=12, vocab=31, embed_scale=2.5)
    w = {k: synth.bf16_to_f32(v) for k, v in synth.make_lupolorn(cfg, 1).items()}
    assert "head" not in w and cfg["layers"][2]["mlp"] is None
    m = Z.Lupolorn(cfg, w)
    ids = np.random.default_rng(2).integers(0, 31, 40)
    trace = []
    want = m.forward(ids, None, trace)
    assert len(trace) == 3 and want.shape == (40, 31)
    st, parts = m.new_state(), []
    for a, b in [(0, 1), (1, 3), (3, 4), (4, 20), (20, 22), (22, 40)]:
        parts.append(m.forward(ids[a:b], st))
    assert np.allclose(np.concatenate(parts), want)
    w2 = dict(w); w2["embed"] = w["embed"] * 2.0            # the table is used twice: as the (scaled) input and, unscaled, as the output projection
    m2 = Z.Lupolorn({**cfg, "embedding": {"scale": 1.25}}, w2)
    assert np.allclose(m2.forward(ids), 2.0 * want)
    g = m.greedy(ids[:5], 6)
    assert len(g) == 6 and all(0 <= t < 31 for t in g)


def test_safetensors_roundtrip_and_kind(tmp_path):
    from aha_b200.checkpoint import model_kind, read_safetensors, write_safetensors
    cfg = synth.lupolorn_config(LAYERS, width=12, vocab=31)
    w = synth.make_lupolorn(cfg, 3)
    write_safetensors(os.path.join(tmp_path, "model.safetensors"), w)
    back = read_safetensors(os.path.join(tmp_path, "model.safetensors"))
    assert set(back) == set(w)
    for k in w:
        assert np.array_equal(np.asarray(back[k]).view(np.ndarray), np.asarray(w[k]).view(np.ndarray)), k
    assert model_kind(json.loads(json.dumps(cfg))) == "lupolorn"
    big = synth.lupolorn_shape(width=256, n_layers=4, heads=4, kv_heads=2, head_dim=64, ff=512, experts=4, top=2, expert_ff=128, vocab=100, kv_rank=64, q_rank=128, window=128)
    assert [ly["type"] for ly in big["layers"]] == ["attention", "mingru", "latent_attention", "attention"]
    assert [ly["mlp"]["kind"] for ly in big["layers"]] == ["dense", "moe", "dense", "moe"]
