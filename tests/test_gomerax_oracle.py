"""The plain Gomerax restatement (oracle/gomerax.py) checked against closed forms, and the host-side pieces that need no GPU:
synthetic checkpoints through the safetensors reader, the choice of the executor by config.json."""
import json
import math
import os

import numpy as np

from aha_b200 import synth
from oracle import gomerax as Z


def test_offset_norm_and_embedding_with_positions():
    x = np.array([[3.0, -4.0, 0.0, 0.0]])
    assert np.allclose(Z.norm_offset(x, np.zeros(4), 0.0), x / 2.5)                     # a stored gain of zero is the identity gain
    assert np.allclose(Z.norm_offset(x, np.array([1.0, 0.0, -1.0, 2.0]), 0.0), x / 2.5 * [2.0, 1.0, 0.0, 3.0])
    assert np.allclose(Z.norm_plain(x, np.full(4, 0.5), 0.0), x / 5.0)
    assert np.allclose(Z.rms_unit(np.zeros((1, 4)), 1e-4), 0.0)                        # eps sits inside the root
    table, pos = np.arange(12.0).reshape(4, 3), 100.0 + np.arange(15.0).reshape(5, 3)
    e = Z.embed_rows(np.array([2, 2, 0]), np.array([3, 4, 0]), table, pos, 2.0)
    assert np.allclose(e, [table[2] * 2 + pos[3], table[2] * 2 + pos[4], table[0] * 2 + pos[0]])     # the position row is not scaled


def test_rotation_turns_interleaved_pairs_and_depends_on_distance_only():
    fr = Z.rotary_frequencies(50.0, 6)
    assert np.allclose(fr, [1.0, 50.0 ** (-2 / 6), 50.0 ** (-4 / 6)])
    x = np.random.default_rng(0).standard_normal((5, 2, 8))
    pos = np.array([0, 1, 2, 7, 30])
    y = Z.rotate_pairs(x, pos, fr)
    assert np.allclose(y[0], x[0]) and np.allclose(y[..., 6:], x[..., 6:])
    for t in range(5):
        for i in range(3):
            a = pos[t] * fr[i]
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            assert np.allclose(y[t, :, 2 * i], u * math.cos(a) - v * math.sin(a)) and np.allclose(y[t, :, 2 * i + 1], v * math.cos(a) + u * math.sin(a))
    q, k = x[0, 0, :6], x[1, 0, :6]
    d = [Z.rotate_pairs(q[None], np.array([p + 4]), fr)[0] @ Z.rotate_pairs(k[None], np.array([p]), fr)[0] for p in (0, 9, 100)]
    assert np.allclose(d, d[0])


def test_sink_softmax_counts_the_sink_once_and_unscaled():
    s = np.array([[0.0, 0.0, 0.0], [50.0, -50.0, 0.0], [-60.0, -60.0, -60.0]])
    vis = np.ones_like(s, bool)
    p = Z.sink_softmax(s, vis, 0.0)
    assert np.allclose(p[0], 0.25) and p[2].sum() < 1e-25
    p = Z.sink_softmax(s, vis, math.log(5.0))
    assert np.allclose(p[0], 1.0 / 8.0)                                                # exp(sink) = 5 beside three ones
    assert np.allclose(Z.sink_softmax(s, vis, -1e3).sum(axis=1), 1.0)                  # a very negative sink: an ordinary softmax
    vis[0, 2] = False
    assert np.allclose(Z.sink_softmax(s, vis, 0.0)[0], [1 / 3, 1 / 3, 0.0])
    assert np.allclose(Z.sink_softmax(s + 700.0, np.ones_like(s, bool), 700.0), Z.sink_softmax(s, np.ones_like(s, bool), 0.0))      # no overflow


def _latent_weights(H, D, R, Dv, r, qr, Wd, seed=3):
    rng = np.random.default_rng(seed)
    return {"dq": rng.standard_normal((qr, Wd)), "dq.norm": rng.standard_normal(qr), "uq": rng.standard_normal((H * (D + R), qr)),
            "dkv": rng.standard_normal((r + R, Wd)), "dkv.norm": rng.standard_normal(r), "uk": rng.standard_normal((H * D, r)),
            "uv": rng.standard_normal((H * Dv, r)), "sink": rng.standard_normal(H), "o": np.eye(H * Dv)}


def test_latent_attention_window_cache_and_rotated_part():
    H, D, R, Dv, r, qr, Wd, T, win = 2, 4, 6, 3, 5, 7, 8, 14, 4
    mx = {"heads": H, "dim": D, "rot_dim": R, "vdim": Dv, "kv_rank": r, "q_rank": qr, "mask": {"size": win}, "scale": 0.5, "rot": {"base": 30.0, "dims": R}}
    W = _latent_weights(H, D, R, Dv, r, qr, Wd)
    h = np.random.default_rng(5).standard_normal((T, Wd))
    y = Z.latent_attention_mixer(h, W, mx, 1e-6, {}, 0)
    for j, moved in [(10 - win, False), (10 - win + 1, True), (10, True), (11, False)]:      # position 10 sees 7 .. 10
        h2 = h.copy(); h2[j] += 2.0
        assert (not np.allclose(Z.latent_attention_mixer(h2, W, mx, 1e-6, {}, 0)[10], y[10])) == moved, j
    st, parts = {}, []
    for a, b in [(0, 1), (1, 6), (6, 8), (8, 14)]:
        parts.append(Z.latent_attention_mixer(h[a:b], W, mx, 1e-6, st, a))
    assert np.allclose(np.concatenate(parts), y)
    assert st["c"].shape == (T, r) and st["kr"].shape == (T, R)                       # one latent and one rotated part per token is all that is kept
    # the rotated key part is not normed: scaling its rows of W_dkv changes the result, scaling the latent rows does not (eps = 0)
    W2 = dict(W); W2["dkv"] = W["dkv"].copy(); W2["dkv"][:r] *= 3.0
    assert np.allclose(Z.latent_attention_mixer(h, W2, mx, 0.0, {}, 0), Z.latent_attention_mixer(h, W, mx, 0.0, {}, 0))
    W3 = dict(W); W3["dkv"] = W["dkv"].copy(); W3["dkv"][r:] *= 3.0
    assert not np.allclose(Z.latent_attention_mixer(h, W3, mx, 0.0, {}, 0), y)
    # positions enter through the rotated part only: with the rotated query rows zero the rotary base does not matter, otherwise it does
    W4 = dict(W); W4["uq"] = W["uq"].copy()
    for hd in range(H):
        W4["uq"][hd * (D + R) + D:(hd + 1) * (D + R)] = 0.0
    other = dict(mx, rot={"base": 7.0, "dims": R})
    assert np.allclose(Z.latent_attention_mixer(h, W4, mx, 1e-6, {}, 0), Z.latent_attention_mixer(h, W4, other, 1e-6, {}, 0))
    assert not np.allclose(y, Z.latent_attention_mixer(h, W, other, 1e-6, {}, 0))
    # the first token sees itself and the sink: weight e^s / (e^s + e^sink)
    one = dict(mx, heads=1)
    W5 = _latent_weights(1, D, R, Dv, r, qr, Wd, seed=9)
    o = Z.latent_attention_mixer(h[:1], W5, one, 1e-6, {}, 0)[0]
    q = (Z.norm_plain(h[:1] @ W5["dq"].T, W5["dq.norm"], 1e-6) @ W5["uq"].T)[0]
    dkv = (h[:1] @ W5["dkv"].T)[0]
    c = Z.norm_plain(dkv[None, :r], W5["dkv.norm"], 1e-6)[0]
    s = (q[:D] @ (W5["uk"] @ c) + q[D:] @ dkv[r:]) * 0.5
    assert np.allclose(o, math.exp(s) / (math.exp(s) + math.exp(W5["sink"][0])) * (W5["uv"] @ c))


def test_dense_and_clamped_units():
    rng = np.random.default_rng(1)
    W = {"gate": rng.standard_normal((5, 4)), "gate.b": rng.standard_normal(5), "up": rng.standard_normal((5, 4)), "up.b": rng.standard_normal(5),
         "down": rng.standard_normal((4, 5)), "down.b": rng.standard_normal(4)}
    assert np.allclose(Z.dense_ff(np.zeros((1, 4)), W), (Z.silu(W["gate.b"]) * W["up.b"]) @ W["down"].T + W["down.b"])
    eye = np.eye(3)
    E = {"x.gate": eye, "x.up": eye, "x.down": eye}
    h = np.array([[10.0, -10.0, 0.5]])
    y = Z.clamped_expert(h, E, "x.", 2.0)[0]
    sg = lambda g: g / (1.0 + math.exp(-Z.GLU_SLOPE * g))
    assert np.allclose(y, [sg(2.0) * 3.0, sg(-10.0) * (-2.0 + 1.0), sg(0.5) * 1.5])       # the gate is cut above only, the other input on both sides
    assert Z.GLU_SLOPE == 1.702


def test_router_correction_groups_and_weights():
    rt = {"experts": 8, "top": 2, "scale": 2.5, "groups": {"count": 4, "keep": 2}}
    z = np.log(np.array([0.05, 0.05, 0.30, 0.02, 0.20, 0.01, 0.17, 0.20]))
    s = np.exp(z) / np.exp(z).sum()
    ch, w = Z.route(z, np.zeros(8), rt)
    assert list(ch) == [2, 4] and np.allclose(w, s[[2, 4]] / s[[2, 4]].sum() * 2.5)       # groups (2,3) and (4,5) win; 7 ties with 4 but its group is out
    ch, w = Z.route(z, np.zeros(8), dict(rt, groups={"count": 4, "keep": 3}))
    assert list(ch) == [2, 4]                                                           # the earlier expert wins among equal scores
    ch, w = Z.route(z, np.array([0, 0, 0, 0, 0, 0, 0, 0.01]), dict(rt, groups={"count": 4, "keep": 3}))
    assert list(ch) == [2, 7] and np.allclose(w, s[[2, 7]] / s[[2, 7]].sum() * 2.5)       # the correction decides the choice, not the weight
    ch, w = Z.route(z, np.array([0, 0, -5.0, -5.0, 0, 0, 0, 0]), dict(rt, groups={"count": 4, "keep": 1}))
    assert list(ch) == [4, 5]                                                           # one group: the earlier of the two best, although expert 5 is weak
    ch, w = Z.route(z, np.full(8, -3.0), rt)
    assert list(ch) == [2, 4]                                                           # negative choice scores still beat a group that is out
    ch, w = Z.route(z, np.zeros(8), {"experts": 8, "top": 8, "scale": 1.0})
    assert np.allclose(w.sum(), 1.0)


def test_routed_experts_add_the_shared_expert_ungated():
    rng = np.random.default_rng(4)
    Wd, E, ff, T = 6, 6, 4, 8
    W = {"router": rng.standard_normal((E, Wd)) * 2, "correction": rng.standard_normal(E) * 0.05}
    for e in range(E):
        W["e%d.gate" % e] = rng.standard_normal((ff, Wd)); W["e%d.up" % e] = rng.standard_normal((ff, Wd)); W["e%d.down" % e] = rng.standard_normal((Wd, ff))
    h = rng.standard_normal((T, Wd))
    ml = {"router": {"experts": E, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}, "expert": {"ff": ff, "limit": 1.0}}
    y = Z.routed_experts(h, W, ml)
    for t in range(T):
        ch, w = Z.route(h[t] @ W["router"].T, W["correction"], ml["router"])
        assert np.allclose(w.sum(), 1.5)
        assert np.allclose(y[t], sum(wk * Z.clamped_expert(h[t], W, "e%d." % e, 1.0) for e, wk in zip(ch, w)))
    W["shared.gate"] = rng.standard_normal((3, Wd)); W["shared.up"] = rng.standard_normal((3, Wd)); W["shared.down"] = rng.standard_normal((Wd, 3))
    ml2 = dict(ml, shared={"ff": 3, "limit": 0.25})
    assert np.allclose(Z.routed_experts(h, W, ml2) - y, Z.clamped_expert(h, W, "shared.", 0.25))
    assert not np.allclose(Z.clamped_expert(h, W, "shared.", 0.25), Z.clamped_expert(h, W, "shared.", 1.0))      # the shared expert has a limit of its own


def L(heads=3, dim=4, rot_dim=2, vdim=6, kv_rank=5, q_rank=7, window=9, ff=None, **kw):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, window=window, ff=ff, **kw)


LAYERS = [L(ff=20), L(heads=2, rot_dim=4, ff={"experts": 6, "top": 2, "ff": 8, "limit": 1.5, "scale": 2.0, "groups": (3, 2), "shared": (6, 0.75)}), L(window=3), L(ff=12)]


def test_layer_runs_and_portions_and_the_tied_head():
    assert Z.layer_runs({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False), (4, False)]
    assert Z.layer_runs({"layers": [0] * 2}) == [(0, False), (1, False)]
    assert Z.layer_runs({"layers": [0] * 2, "loop": {"start": 0, "stop": 2, "times": 1}}) == [(0, False), (1, False)]
    cfg = synth.gomerax_config(LAYERS, width=12, vocab=31, embed_scale=2.5, max_positions=64, loop=(1, 3, 3))
    w = {k: synth.bf16_to_f32(v) for k, v in synth.make_gomerax(cfg, 1).items()}
    assert "head" not in w and cfg["layers"][2]["mlp"] is None
    m = Z.Gomerax(cfg, w)
    ids = np.random.default_rng(2).integers(0, 31, 40)
    trace = []
    want = m.forward(ids, None, trace)
    assert len(trace) == 8 and want.shape == (40, 31)
    st, parts = m.new_state(), []
    for a, b in [(0, 1), (1, 3), (3, 4), (4, 20), (20, 22), (22, 40)]:
        parts.append(m.forward(ids[a:b], st))
    assert np.allclose(np.concatenate(parts), want)
    assert len(st["runs"]) == 8 and st["runs"][1]["c"] is not st["runs"][3]["c"]       # every pass has a cache of its own
    # the embedding output comes back before the later passes: without it the result differs, and the position rows matter
    once = Z.Gomerax(dict(cfg, loop={"start": 1, "stop": 3, "times": 1}), w).forward(ids)
    assert not np.allclose(once, want)
    w2 = dict(w); w2["pos"] = w["pos"] * 0.0
    assert not np.allclose(Z.Gomerax(cfg, w2).forward(ids), want)
    g = m.greedy(ids[:5], 6)
    assert len(g) == 6 and all(0 <= t < 31 for t in g)


def test_safetensors_roundtrip_and_kind(tmp_path):
    from aha_b200.checkpoint import model_kind, read_safetensors, write_safetensors
    cfg = synth.gomerax_config(LAYERS, width=12, vocab=31, loop=(0, 2, 2))
    w = synth.make_gomerax(cfg, 3)
    write_safetensors(os.path.join(tmp_path, "model.safetensors"), w)
    back = read_safetensors(os.path.join(tmp_path, "model.safetensors"))
    assert set(back) == set(w)
    for k in w:
        assert np.array_equal(np.asarray(back[k]).view(np.ndarray), np.asarray(w[k]).view(np.ndarray)), k
    assert model_kind(json.loads(json.dumps(cfg))) == "gomerax"
    big = synth.gomerax_shape(width=256, n_layers=3, heads=4, head_dim=64, ff=512, experts=8, top=2, expert_ff=128, vocab=100, kv_rank=64, q_rank=128, window=128)
    assert [ly["mlp"]["kind"] for ly in big["layers"]] == ["dense", "moe", "moe"] and big["layers"][1]["mlp"]["router"]["groups"] == {"count": 4, "keep": 3}
