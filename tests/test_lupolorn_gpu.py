"""The Lupolorn design of the layered engine on a B200 against the plain restatement (oracle/lupolorn.py): every mechanism alone,
prompts cut into portions, decoding through the caches and the state slots, mixed batches, pages and slots that are used again, keys
far away / at page borders / just inside and just outside the sliding window made visible by a token whose embedding is scaled up,
other sizes (also values that a model may happen to make equal or 1), the tensor-core paths, and greedy generation through the
library's own entries."""
import numpy as np
import pytest

from aha_b200 import synth
from conftest import has_gpu

pytestmark = pytest.mark.gpu
if not has_gpu():
    pytest.skip("needs a GPU", allow_module_level=True)

from aha_b200 import B200Model            # noqa: E402
from oracle.lupolorn import Lupolorn      # noqa: E402

TOL32 = 2e-4     # exact mode: fp32 everywhere against float64
TOL16 = 6e-2     # serving mode: bf16 products

BANDS = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}


def R(width=24, ff=None):
    return {"type": "mingru", "width": width, "ff": ff}


def A(heads=4, kv_heads=2, dim=8, vdim=12, rot_dims=6, base=100.0, scaling=BANDS, scale=None, ff=None):
    d = {"type": "attention", "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot_dims": rot_dims, "base": base, "scaling": scaling, "ff": ff}
    if scale is not None:
        d["scale"] = scale
    return d


def Lt(heads=3, dim=8, vdim=12, kv_rank=16, q_rank=20, window=40, scale=None, ff=None):
    d = {"type": "latent_attention", "heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "window": window, "ff": ff}
    if scale is not None:
        d["scale"] = scale
    return d


def E(experts=5, top=2, ff=24, shared=16):
    return {"experts": experts, "top": top, "ff": ff, "shared": shared}


TINY = dict(layers=[A(heads=4, kv_heads=2, dim=8, vdim=6, rot_dims=4, ff=40), R(width=28, ff=E(6, 2, 20, 12)), Lt(heads=3, dim=8, vdim=10, kv_rank=12, q_rank=14, window=37, ff=36),
                    A(heads=2, kv_heads=2, dim=12, vdim=12, rot_dims=12, scaling=None, ff=E(4, 3, 16, None)), R(width=20)],
            width=48, vocab=83, embed_scale=3.0)


class Pair:
    """The library's handle and the oracle on the same random checkpoint."""

    def __init__(self, cfg, seed=0, exact=True, max_ctx=1024, max_seqs=4, step_tokens=512, boost=None, plain=False, edit=None):
        self.cfg = cfg
        w = synth.make_lupolorn(cfg, seed)
        f = {k: synth.bf16_to_f32(v) for k, v in w.items()}
        if boost is not None:       # one token's embedding scaled up (still bf16-exact): its key / value stand out wherever it is visible
            f["embed"] = f["embed"].copy()
            f["embed"][boost] *= 8.0
            w["embed"] = synth._bf16_round(f["embed"])
        if edit is not None:        # edit(name, values) -> new values or None, for every tensor
            for k in list(f):
                a = edit(k, f[k])
                if a is not None:
                    w[k] = synth._bf16_round(np.asarray(a, np.float32))
                    f[k] = synth.bf16_to_f32(w[k])
        self.m = B200Model("lupolorn", cfg, w, max_ctx=max_ctx, max_prefill=step_tokens, max_seqs=max_seqs, exact_fp32=exact, attn_impl=1 if plain else 0)
        self.o = Lupolorn(cfg, f)
        self.tol = TOL32 if exact else TOL16
        self.V = cfg["vocab"]

    def ids(self, n, seed=0, avoid=None):
        r = np.random.default_rng(seed).integers(0, self.V, n)
        if avoid is not None:
            r[r == avoid] = (avoid + 1) % self.V
        return r.astype(np.uint32)

    def check(self, got, want, what=""):
        want = np.asarray(want, np.float64)
        err = np.abs(got - want).max() / max(1.0, want.std())
        assert err <= self.tol, f"{what}: logits differ from the plain implementation by {err:.3e} (row {int(np.abs(got - want).max(axis=1).argmax())})"

    def run_cuts(self, ids, cuts):
        """One sequence fed in portions ending at `cuts`; all logits."""
        s = self.m.seq_open()
        out, a = [], 0
        for b in list(cuts) + [len(ids)]:
            if b > a:
                out.append(self.m.feed([(s, ids[a:b], range(b - a))]))
                a = b
        self.m.seq_close(s)
        return np.concatenate(out)

    def close(self):
        self.m.close()


def cfg_of(layers, **kw):
    base = dict(width=40, vocab=77, embed_scale=2.0)
    base.update(kw)
    return synth.lupolorn_config(layers, **base)


MECHANISMS = {
    "mingru": cfg_of([R(width=56)]),
    "mingru_narrow": cfg_of([R(width=1)], width=8),
    "mingru_wider_than_the_stream": cfg_of([R(width=100)], width=24),
    "attention_grouped": cfg_of([A(heads=6, kv_heads=2, dim=8, vdim=12, rot_dims=6)]),
    "attention_one_kv_head": cfg_of([A(heads=5, kv_heads=1, dim=10, vdim=4, rot_dims=10, scaling=None, scale=0.9)]),
    "attention_one_head_no_rotation": cfg_of([A(heads=1, kv_heads=1, dim=16, vdim=16, rot_dims=0, scaling=None, scale=0.4)], embed_scale=1.0),
    "attention_two_rotated_coordinates": cfg_of([A(heads=3, kv_heads=3, dim=6, vdim=20, rot_dims=2, base=3.0, scaling={"factor": 2.0, "low": 2.0, "high": 8.0, "original": 6})]),
    "latent": cfg_of([Lt(heads=4, dim=8, vdim=16, kv_rank=24, q_rank=12, window=21)]),
    "latent_window_one": cfg_of([Lt(heads=2, dim=6, vdim=6, kv_rank=6, q_rank=6, window=1)]),
    "latent_window_beyond_the_prompt": cfg_of([Lt(heads=1, dim=20, vdim=5, kv_rank=9, q_rank=30, window=500, scale=0.3)]),
    "dense": cfg_of([R(width=16, ff=72)]),
    "experts": cfg_of([R(width=16, ff=E(7, 2, 20, 12))]),
    "experts_top1_no_shared": cfg_of([R(width=16, ff=E(3, 1, 36, None))]),
    "experts_all_chosen": cfg_of([A(ff=E(3, 3, 12, 12))]),
    "experts_one_expert": cfg_of([Lt(ff=E(1, 1, 8, 40))]),
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name):
    p = Pair(MECHANISMS[name], seed=5)
    ids = p.ids(45, 1)
    trace = []
    want = p.o.forward(ids, None, trace)
    p.m.set_trace(True)
    s = p.m.seq_open()
    got = p.m.feed([(s, ids, range(len(ids)))])
    p.check(got, want, name)
    for l, x in enumerate(trace):       # the residual stream after every layer
        h = p.m.debug_read("hidden", l, x.size).reshape(x.shape)
        assert np.abs(h - x).max() <= TOL32 * max(1.0, np.abs(x).max()), f"{name}: layer {l}"
    p.m.seq_close(s)
    p.m.set_trace(False)
    # the same tokens one by one, and in portions
    p.check(p.run_cuts(ids, range(1, len(ids))), want, name + " token by token")
    p.check(p.run_cuts(ids, [2, 4, 9, 10, 31, 33]), want, name + " in portions")
    p.close()


@pytest.mark.parametrize("exact", [True, False])
def test_whole_model_portions_and_decoding(exact):
    p = Pair(synth.lupolorn_config(**TINY), seed=2, exact=exact)
    ids = p.ids(150, 3)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, []), want, "whole")
    p.check(p.run_cuts(ids, [2, 4, 5, 8, 15, 31, 32, 33, 64, 96, 97, 127, 129]), want, "portions of 1, 2, 3, 7 and more tokens, at page borders")
    p.check(p.run_cuts(ids, list(range(60, 150))), want, "prompt then 90 decoded tokens")
    p.check(p.run_cuts(ids, list(range(1, 12))), want, "the first tokens one by one")
    p.check(p.run_cuts(ids, list(range(2, 150, 2))), want, "two tokens at a time")
    p.close()


def test_tensor_core_paths_in_serving_mode():
    # sizes that tile (K % 64 == 0, N % 32 == 0, head size 64): portions of 32 tokens and more run their Linear layers, the experts' grouped
    # products and both attentions on the tcgen05 kernels, shorter ones and decode steps on the CUDA cores; both must agree with the plain
    # implementation, and the marked token (far back, at a page's last place) must be seen by the rows that can see it
    mark = 3
    layers = [A(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, base=1e4, scaling={"factor": 4.0, "low": 1.0, "high": 4.0, "original": 128}, ff=E(4, 2, 64, 64)),
              R(width=128, ff=256), Lt(heads=3, dim=64, vdim=64, kv_rank=64, q_rank=64, window=150, ff=E(3, 1, 128, 64))]
    cfg = cfg_of(layers, width=128, vocab=160, embed_scale=4.0)
    p = Pair(cfg, seed=21, exact=False, max_ctx=2048, step_tokens=2048, boost=mark)
    ids = p.ids(700, 4, avoid=mark)
    ids[[31, 200, 455]] = mark
    want = p.o.forward(ids)
    for cuts in ([], [40, 45, 300, 333, 429, 461, 600], [130, 131, 194, 195, 259] + list(range(640, 700))):
        got = p.run_cuts(ids, cuts)
        err = np.abs(got - want).max() / want.std()
        assert err < 3e-3, (cuts[:4], err, int(np.abs(got - want).max(axis=1).argmax()))          # bf16 hi + lo operands: far inside the bf16 budget
    plain = ids.copy(); plain[455] = (mark + 2) % 160
    assert np.abs(p.o.forward(plain)[461] - want[461]).max() / want.std() > 0.03      # ten times the budget above: the marked key is seen
    assert p.m.stats()["kernel_launches"] > 0
    p.close()


@pytest.mark.parametrize("dims", [(64, 64, 64), (128, 128, 128), (32, 64, 64), (128, 64, 128), (160, 128, 64)])
def test_tensor_core_attention_head_sizes(dims):
    # (latent dim, latent vdim, attention head size): value sizes 64 / 128 with keys of up to 128 / 192 run on the tcgen05 flash kernel, windowed for
    # the latent layer, with sink and head gates for the other; keys shorter than values are zero-padded
    dim, vdim, hd = dims
    mark = 5
    cfg = cfg_of([Lt(heads=2, dim=dim, vdim=vdim, kv_rank=64, q_rank=64, window=100, ff=64), A(heads=4, kv_heads=1, dim=hd, vdim=hd, rot_dims=hd // 2, base=1e4, scaling=BANDS)], width=64, vocab=90)
    p = Pair(cfg, seed=31, exact=False, max_ctx=1024, step_tokens=1024, boost=mark)
    ids = p.ids(420, 6, avoid=mark)
    ids[[7, 200, 263]] = mark
    want = p.o.forward(ids)
    for cuts in ([], [40, 45, 300, 333], [130, 131, 194, 195, 259] + list(range(400, 420))):
        got = p.run_cuts(ids, cuts)
        err = np.abs(got - want).max() / want.std()
        assert err < 3e-3, (cuts[:4], err, int(np.abs(got - want).max(axis=1).argmax()))
    p.close()


def test_plain_kernels_agree_with_the_fast_ones():
    cfg = synth.lupolorn_config(**TINY)
    ids = np.random.default_rng(3).integers(0, cfg["vocab"], 300).astype(np.uint32)
    out = []
    for plain in (False, True):
        p = Pair(cfg, seed=17, plain=plain)
        out.append(p.run_cuts(ids, [70, 71, 200] + list(range(250, 300))))
        p.check(out[-1], p.o.forward(ids), "plain kernels" if plain else "fast kernels")
        p.close()
    assert np.abs(out[0] - out[1]).max() < 1e-3


def test_long_portions_of_the_recurrence_run_side_by_side():
    # an entry of more than 64 tokens is walked by sixteen token lanes per channel whose composites are joined; gates near 0 and near 1 (a state
    # that barely moves, a state that is overwritten) must survive the join, and a second portion must continue from the slot's state
    def edit(name, a):
        if name.endswith("mix.z.b"):
            b = a.copy(); b[::3] = -9.0; b[1::3] = 9.0
            return b
        return None
    cfg = cfg_of([R(width=70, ff=32), R(width=33)], width=32, vocab=50)
    p = Pair(cfg, seed=9, max_ctx=2048, step_tokens=2048, edit=edit)
    ids = p.ids(1100, 2)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, []), want, "one portion of 1100 tokens")
    p.check(p.run_cuts(ids, [257, 258, 300, 317, 829]), want, "portions of 257, 1, 42, 17, 512 and 271 tokens")
    p.close()


def test_launches_shorter_than_a_step_are_cut_by_the_scheduler():
    p = Pair(synth.lupolorn_config(**TINY), seed=4, step_tokens=24)      # the engine itself cuts a 100-token entry into 24-token launches
    ids = p.ids(100, 7)
    p.check(p.run_cuts(ids, []), p.o.forward(ids), "launch size 24")
    p.close()


def test_mixed_batches_equal_each_request_alone():
    p = Pair(synth.lupolorn_config(**TINY), seed=6, max_ctx=1024, max_seqs=4)
    reqs = [p.ids(n, 10 + i) for i, n in enumerate([70, 3, 41, 129])]
    want = [p.o.forward(r) for r in reqs]
    slots = [p.m.seq_open() for _ in reqs]
    at = [0] * len(reqs)
    got = [[] for _ in reqs]
    plan = [[16, 1, 2, 40], [1, 1, 30, 1], [30, 1, 0, 64], [1, 0, 1, 1], [2, 0, 2, 2], [20, 0, 6, 21]]     # portions beside single tokens
    for step in plan:
        ent, who = [], []
        for i, n in enumerate(step):
            n = min(n, len(reqs[i]) - at[i])
            if n > 0:
                ent.append((slots[i], reqs[i][at[i]:at[i] + n], range(n))); who.append((i, n)); at[i] += n
        lg = p.m.feed(ent)
        r = 0
        for i, n in who:
            got[i].append(lg[r:r + n]); r += n
    for i in range(len(reqs)):
        assert at[i] == len(reqs[i])
        p.check(np.concatenate(got[i]), want[i], f"request {i} in a mixed batch")
    p.close()


def test_pages_and_slots_are_used_again():
    p = Pair(synth.lupolorn_config(**TINY), seed=8, max_ctx=256, max_seqs=2)
    a, b, c, d = p.ids(120, 1), p.ids(100, 2), p.ids(130, 3), p.ids(90, 4)
    sa = p.m.seq_open(); sb = p.m.seq_open()
    with pytest.raises(Exception):
        p.m.seq_open()                                   # both slots are live
    ga = p.m.feed([(sa, a[:100], range(100)), (sb, b[:60], range(60))])
    gb2 = p.m.feed([(sb, b[60:], range(40)), (sa, a[100:], range(20))])
    p.check(np.concatenate([ga[:100], gb2[40:]]), p.o.forward(a), "a")
    p.check(np.concatenate([ga[100:], gb2[:40]]), p.o.forward(b), "b")
    assert p.m.seq_info()["free_tokens"] == 256 - 128 - 128
    with pytest.raises(Exception):
        p.m.feed([(sa, a[:40], [])])                     # the pool is exhausted
    p.m.seq_close(sa)                                    # a's pages and slot (recurrent states) go to c while b is still live
    sc = p.m.seq_open()
    assert sc == sa
    gc = p.m.feed([(sc, c[:128], range(128))])
    p.m.seq_close(sb)
    sd = p.m.seq_open()
    g2 = p.m.feed([(sc, c[128:], range(2)), (sd, d, range(90))])
    p.check(np.concatenate([gc, g2[:2]]), p.o.forward(c), "c in a's slot and pages")
    p.check(g2[2:], p.o.forward(d), "d in b's slot and pages")
    p.close()


def test_far_key_among_hundreds_and_page_borders():
    mark = 7
    cfg = cfg_of([A(heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=8, ff=E(4, 2, 24, 8))], width=48, vocab=60)
    p = Pair(cfg, seed=11, boost=mark, max_ctx=1024, step_tokens=1024)
    ids = p.ids(420, 5, avoid=mark)
    ids[31] = mark                                         # the last token of the first page
    want = p.o.forward(ids)
    plain = ids.copy(); plain[31] = (mark + 2) % 60
    assert np.abs(p.o.forward(plain)[-1] - want[-1]).max() > 50 * p.tol       # the far key matters at the last position
    s = p.m.seq_open()
    g1 = p.m.feed([(s, ids[:380], [31, 32, 63, 64, 379])])
    g2 = [p.m.feed([(s, ids[t:t + 1], [0])]) for t in range(380, 420)]      # decoding across page borders, keys split over several blocks
    p.m.seq_close(s)
    p.check(g1, want[[31, 32, 63, 64, 379]], "prompt rows at page borders")
    p.check(np.concatenate(g2), want[380:], "decoded rows that still see position 31")
    p.close()


@pytest.mark.parametrize("window", [1, 2, 31, 32, 33, 64, 100, 129])
def test_window_edges_in_prompts_and_in_decoding(window):
    # a single latent layer: the marked token at position m is seen by rows m .. m + window - 1 and by no other.  The oracle says so, and the
    # engine must agree with it whether the row is part of a long portion (expanded keys), a short one or decoded alone (absorbed form)
    mark, m = 9, 70
    cfg = cfg_of([Lt(heads=3, dim=12, vdim=8, kv_rank=16, q_rank=10, window=window, ff=24)], width=32, vocab=50)
    p = Pair(cfg, seed=19, boost=mark, max_ctx=1024, step_tokens=512)
    ids = p.ids(m + window + 40, 3, avoid=mark)
    ids[m] = mark
    want = p.o.forward(ids)
    plain = ids.copy(); plain[m] = (mark + 2) % 50
    other = p.o.forward(plain)
    last_in, first_out = m + window - 1, m + window
    assert np.abs(other[last_in] - want[last_in]).max() > 50 * p.tol and np.abs(other[first_out] - want[first_out]).max() == 0.0
    p.check(p.run_cuts(ids, []), want, "one portion")
    p.check(p.run_cuts(ids, [m - 3, last_in, first_out]), want, "portions that end at the edge")
    p.check(p.run_cuts(ids, [m + 1] + list(range(m + 2, len(ids)))), want, "the window passes over decoded tokens")
    p.check(p.run_cuts(ids, [last_in - 1, last_in + 1, last_in + 35]), want, "a two-token portion across the edge, then a long one behind it")
    p.close()


def test_latent_and_attention_layers_of_other_head_sizes():
    # portions of 32 tokens and more expand keys and values and run the tiled kernels (odd sizes leave partial tiles), shorter ones and decoded
    # tokens the absorbed form; both continue one another's cache (18 heads: the decode kernel serves sixteen heads at a time, then the other two)
    for layers in ([Lt(heads=2, dim=20, vdim=136, kv_rank=24, q_rank=7, window=90), A(heads=3, kv_heads=3, dim=34, vdim=5, rot_dims=10)],
                   [Lt(heads=3, dim=6, vdim=5, kv_rank=9, q_rank=40, window=64), A(heads=8, kv_heads=2, dim=4, vdim=70, rot_dims=4, scaling=None)],
                   [Lt(heads=18, dim=8, vdim=8, kv_rank=20, q_rank=16, window=33), A(heads=1, kv_heads=1, dim=130, vdim=24, rot_dims=64)]):
        p = Pair(cfg_of(layers, width=32, vocab=50), seed=27, max_ctx=1024, max_seqs=3, step_tokens=512)
        ids = p.ids(330, 3)
        want = p.o.forward(ids)
        p.check(p.run_cuts(ids, [70, 75, 140, 141, 205, 269, 300] + list(range(301, 330))), want, "long and short portions in turn")
        a, b = p.ids(200, 4), p.ids(90, 5)
        sa, sb = p.m.seq_open(), p.m.seq_open()
        g1 = p.m.feed([(sa, a[:100], range(100)), (sb, b[:3], range(3))])
        g2 = p.m.feed([(sb, b[3:80], range(77)), (sa, a[100:165], range(65))])          # two long entries, both continuing
        g3 = p.m.feed([(sa, a[165:], range(35)), (sb, b[80:], range(10))])
        p.check(np.concatenate([g1[:100], g2[77:], g3[:35]]), p.o.forward(a), "a")
        p.check(np.concatenate([g1[100:], g2[:77], g3[35:]]), p.o.forward(b), "b")
        p.close()


def test_sink_and_head_gate_show():
    # keys that point away from every query (scores near -scale * dim): the sink takes most of the weight, so a softmax without it differs grossly;
    # one head's gate shut: the head's part of W_o must not matter
    def edit(name, a):
        if name.endswith("mix.k"):
            return -np.abs(a) * 2.0
        if name.endswith("mix.q"):
            return np.abs(a) * 2.0
        if name.endswith("mix.g"):
            b = a.copy(); b[1] = -60.0
            return b
        if name == "embed":
            return np.abs(a) + 0.05
        if name.endswith("norm1"):
            return np.abs(a)
        return None
    cfg = cfg_of([A(heads=3, kv_heads=1, dim=8, vdim=8, rot_dims=0, scaling=None, scale=1.0)], width=24, vocab=40)
    p = Pair(cfg, seed=23, edit=edit)
    ids = p.ids(90, 1)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, [50, 52] + list(range(60, 90))), want, "sink and gates")
    w2 = dict(p.o.w); w2["l0.mix.o"] = p.o.w["l0.mix.o"].copy(); w2["l0.mix.o"][:, 8:16] = 0.0
    assert np.abs(Lupolorn(cfg, w2).forward(ids) - want).max() < 1e-9                 # the shut head adds nothing
    from oracle import lupolorn as Z
    keep = Z.softmax_rows
    try:                                                                              # the same model with an ordinary softmax is far away
        Z.softmax_rows = lambda s, vis, sink=False: keep(s, vis, False)
        assert np.abs(Lupolorn(cfg, p.o.w).forward(ids) - want).max() > 1000 * p.tol
    finally:
        Z.softmax_rows = keep
    p.close()


def test_rotary_bands_show_far_beyond_the_original_length():
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 16}
    layer = A(heads=2, kv_heads=1, dim=16, vdim=8, rot_dims=16, base=50.0, scaling=sc)
    cfg = cfg_of([layer], width=32, vocab=40)
    p = Pair(cfg, seed=15)
    ids = p.ids(300, 8)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, [290] + list(range(291, 300))), want, "banded rotary")
    for other_sc in (None, dict(sc, factor=7.0), dict(sc, original=32), dict(sc, high=2.0)):
        other = Lupolorn(cfg_of([dict(layer, scaling=other_sc)], width=32, vocab=40), p.o.w).forward(ids)
        assert np.abs(other[-1] - want[-1]).max() > 50 * p.tol
    p.close()


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes_and_layer_orders(seed):
    # sizes, head counts, layer order and constants drawn at random (odd sizes included): nothing may rest on one model's values
    r = np.random.default_rng(200 + seed)
    pick = lambda *xs: xs[int(r.integers(0, len(xs)))]
    width = pick(6, 10, 16, 20, 36, 64)

    def ff():
        n = pick(2, 3, 5, 9)
        return pick(None, pick(8, 24, 50), E(n, int(r.integers(1, n + 1)), pick(6, 16, 24), pick(None, 6, 16, 30)))

    def layer():
        t = pick("mingru", "attention", "latent")
        if t == "mingru":
            return R(width=pick(1, 7, 32, 50, 96), ff=ff())
        if t == "attention":
            g = pick(1, 2, 3)
            d = pick(4, 6, 16, 24, 64)
            sc = pick(None, {"factor": pick(2.0, 6.0, 16.0), "low": pick(0.5, 1.0, 2.0), "high": pick(3.0, 4.0, 8.0), "original": pick(8, 32, 128)})
            return A(heads=g * pick(1, 2, 4), kv_heads=g, dim=d, vdim=pick(4, 6, 16, 36, 64), rot_dims=2 * int(r.integers(0, d // 2 + 1)), base=pick(10.0, 1e3, 1e6), scaling=sc,
                     scale=pick(None, 0.2, 0.5), ff=ff())
        return Lt(heads=pick(1, 2, 3, 7), dim=pick(4, 6, 16, 24), vdim=pick(4, 6, 16, 36), kv_rank=pick(4, 10, 16, 48), q_rank=pick(3, 8, 32), window=pick(1, 5, 32, 60, 200),
                  scale=pick(None, 0.2, 0.5), ff=ff())

    layers = [layer() for _ in range(int(r.integers(1, 6)))]
    cfg = synth.lupolorn_config(layers, width=width, vocab=pick(17, 50, 131), eps=pick(1e-6, 1e-5, 1e-3), embed_scale=pick(0.25, 1.0, 8.0))
    p = Pair(cfg, seed=seed, exact=seed % 3 != 0, max_ctx=512, max_seqs=3, step_tokens=pick(48, 200, 512))      # (every third one in serving mode)
    ids = p.ids(170, seed)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, []), want, "whole")
    p.check(p.run_cuts(ids, [1, 3, 40, 41, 100, 133] + list(range(140, 170))), want, "portions and decoding")
    p.close()


def test_long_decoding_keeps_states_and_caches():
    cfg = cfg_of([R(width=24, ff=E(3, 2, 8, 8)), Lt(heads=2, dim=8, vdim=8, kv_rank=8, q_rank=8, window=50), A(heads=2, kv_heads=1, dim=8, vdim=8, rot_dims=8, ff=16)], width=24, vocab=40)
    p = Pair(cfg, seed=12)
    ids = p.ids(400, 9)
    p.check(p.run_cuts(ids, list(range(3, 400))), p.o.forward(ids), "397 decoded tokens")
    p.close()


def test_greedy_generation_through_the_entry_points():
    cfg = synth.lupolorn_config(**TINY)
    p = Pair(cfg, seed=13, max_seqs=4)
    prompts = [p.ids(n, 20 + i) for i, n in enumerate([9, 40, 1])]
    want = [p.o.greedy(list(pr), 10) for pr in prompts]
    for pr, w in zip(prompts, want):
        toks, usage = p.m.generate(pr, max_tokens=10)          # decoded tokens are fed back on the device
        assert toks == w and usage["completion_tokens"] == 10
    out = p.m.generate_batch([dict(input_ids=pr, max_tokens=10) for pr in prompts])
    assert [o[0] for o in out] == want
    # the batch session: requests join while others decode, a finished one frees its slot
    p.m.batch_open()
    s0, t0, fin = p.m.batch_add(prompts[0], max_tokens=10)
    got = {s0: [t0]}
    for _ in range(3):
        got[s0].append(p.m.batch_step()[s0][0])
    s1, t1, fin = p.m.batch_add(prompts[1], max_tokens=10)
    assert s1 != s0
    got[s1] = [t1]
    live = {s0, s1}
    while live:
        res = p.m.batch_step()
        assert set(res) == live
        for s, (tok, finished) in res.items():
            got[s].append(tok)
            if finished:
                live.discard(s)
    p.m.batch_close()
    assert got[s0] == want[0] and got[s1] == want[1]
    lg = p.m.forward_initial(prompts[1], 0)[0, 0]
    p.check(lg[None], p.o.forward(prompts[1])[-1:], "forward_initial")
    p.close()


def test_sampler_runs_on_the_engine():
    cfg = synth.lupolorn_config(**TINY)
    p = Pair(cfg, seed=14)
    pr = p.ids(12, 1)
    a, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=5)
    b, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=5)
    assert a == b and len(a) == 8 and all(0 <= t < cfg["vocab"] for t in a)
    p.close()


@pytest.mark.parametrize("seed", range(6))
def test_random_shapes_that_tile_for_the_tensor_cores(seed):
    # widths, head sizes and feed-forward sizes that the tcgen05 kernels take (multiples of 64; head size 64 / 128), everything else drawn at random:
    # group counts, windows that end inside a tile, expert counts, layer order; serving mode and exact mode must both agree with the plain implementation
    r = np.random.default_rng(300 + seed)
    pick = lambda *xs: xs[int(r.integers(0, len(xs)))]
    width = pick(64, 128, 192, 320)

    def ff():
        n = pick(2, 3, 6)
        return pick(None, pick(64, 192), E(n, int(r.integers(1, n + 1)), pick(64, 128), pick(None, 64, 96)))

    def layer():
        t = pick("mingru", "attention", "latent")
        if t == "mingru":
            return R(width=pick(64, 96, 160), ff=ff())
        if t == "attention":
            g, d = pick(1, 2, 3), pick(64, 128)
            sc = pick(None, {"factor": pick(2.0, 16.0), "low": pick(1.0, 2.0), "high": pick(4.0, 8.0), "original": pick(32, 128)})
            return A(heads=g * pick(1, 2, 3), kv_heads=g, dim=d, vdim=d, rot_dims=pick(d, d // 2, 2), base=pick(1e3, 1e6), scaling=sc, scale=pick(None, 0.1), ff=ff())
        dv = pick(64, 128)
        return Lt(heads=pick(1, 2, 5), dim=pick(32, 64, 128), vdim=dv, kv_rank=pick(32, 64, 80), q_rank=pick(24, 64, 128), window=pick(1, 33, 64, 150, 257, 1000), scale=pick(None, 0.1), ff=ff())

    layers = [layer() for _ in range(int(r.integers(2, 5)))]
    cfg = synth.lupolorn_config(layers, width=width, vocab=pick(64, 100, 160), eps=pick(1e-6, 1e-5), embed_scale=pick(1.0, 8.0))
    exact = seed % 2 == 1
    p = Pair(cfg, seed=seed, exact=exact, max_ctx=1024, max_seqs=3, step_tokens=pick(256, 1024))
    ids = p.ids(600, seed)
    want = p.o.forward(ids)
    for cuts in ([], [33, 35, 100, 164, 300, 333, 560] + list(range(580, 600))):
        got = p.run_cuts(ids, cuts)
        err = np.abs(got - want).max() / max(1.0, want.std())
        assert err < (TOL32 if exact else 3e-3), (cuts[:3], err, int(np.abs(got - want).max(axis=1).argmax()))
    p.close()
