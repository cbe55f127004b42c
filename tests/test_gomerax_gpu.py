"""The Gomerax design of the layered engine on a B200 against the plain restatement (oracle/gomerax.py): every mechanism alone,
prompts cut into portions, decoding through the caches, mixed batches, pages and slots that are used again, keys far away / at
page borders / just inside and just outside the sliding window made visible by a token whose embedding is scaled up, the sink,
the clamps, the router's correction and groups made to show, other sizes (also values that a model may happen to make equal or 1),
the tensor-core paths, and greedy generation through the library's own entries."""
import numpy as np
import pytest

from aha_b200 import synth
from conftest import has_gpu

pytestmark = pytest.mark.gpu
if not has_gpu():
    pytest.skip("needs a GPU", allow_module_level=True)

from aha_b200 import B200Model            # noqa: E402
from oracle.gomerax import Gomerax        # noqa: E402
from oracle import gomerax as Z           # noqa: E402

TOL32 = 2e-4     # exact mode: fp32 everywhere against float64
TOL16 = 6e-2     # serving mode: bf16 products


def Lt(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=16, q_rank=20, window=40, scale=None, base=100.0, ff=None):
    d = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, window=window, base=base, ff=ff)
    if scale is not None:
        d["scale"] = scale
    return d


def E(experts=6, top=2, ff=24, limit=1.5, scale=2.0, groups=(3, 2), shared=(16, 0.75)):
    return {"experts": experts, "top": top, "ff": ff, "limit": limit, "scale": scale, "groups": groups, "shared": shared}


TINY = dict(layers=[Lt(heads=4, dim=8, rot_dim=4, vdim=6, kv_rank=12, q_rank=14, window=37, ff=40), Lt(heads=3, dim=6, rot_dim=6, vdim=10, window=50, ff=E(8, 3, 20, 1.0, 2.5, (4, 3), (12, 0.5))),
                    Lt(heads=2, dim=12, rot_dim=2, vdim=12, kv_rank=10, q_rank=9, window=19), Lt(heads=5, dim=4, rot_dim=8, vdim=4, window=64, ff=E(5, 2, 16, 2.0, 1.0, None, None))],
            width=48, vocab=83, embed_scale=3.0, max_positions=640, loop=(1, 3, 2))


class Pair:
    """The library's handle and the oracle on the same random checkpoint."""

    def __init__(self, cfg, seed=0, exact=True, max_ctx=1024, max_seqs=4, step_tokens=512, boost=None, plain=False, edit=None):
        self.cfg = cfg
        w = synth.make_gomerax(cfg, seed)
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
        self.w = w
        self.m = B200Model("gomerax", cfg, w, max_ctx=max_ctx, max_prefill=step_tokens, max_seqs=max_seqs, exact_fp32=exact, attn_impl=1 if plain else 0)
        self.o = Gomerax(cfg, f)
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
    base = dict(width=40, vocab=77, embed_scale=2.0, max_positions=1200)
    base.update(kw)
    return synth.gomerax_config(layers, **base)


def spotlight(cfg, mark, gain=8.0):
    """An edit that makes the key of token `mark` stand out for head 0 of layer 0: channel 0 of the stream is zero for every token but `mark`,
    channel 1 is the same positive number for all; the latent's channel 0 reads the one, the query latent's channel 0 the other, and the head's
    first unrotated coordinate multiplies the two, times gain^2.  Every query that can see `mark` gives it nearly all of head 0's weight."""
    mx = cfg["layers"][0]["mixer"]
    s = cfg["embedding"]["scale"]

    def edit(name, a):
        b = a.copy()
        if name == "embed":
            b[:, 0] = 0.0; b[mark, 0] = 4.0 / s; b[:, 1] = 1.0 / s
        elif name == "pos":
            b[:, :2] = 0.0
        elif name == "l0.norm1":
            b[:2] = 0.0
        elif name == "l0.mix.dkv":
            b[0] = 0.0; b[0, 0] = 1.0; b[1:, 0] = 0.0
        elif name == "l0.mix.dq":
            b[0] = 0.0; b[0, 1] = 1.0
        elif name in ("l0.mix.dkv.norm", "l0.mix.dq.norm"):
            b[0] = 1.0
        elif name == "l0.mix.uk":
            b[0] = 0.0; b[:, 0] = 0.0; b[0, 0] = gain
        elif name == "l0.mix.uq":
            b[0] = 0.0; b[0, 0] = gain
        else:
            return None
        return b
    assert mx["dim"] >= 1
    return edit


MECHANISMS = {
    "latent_no_ff": cfg_of([Lt(heads=4, dim=8, rot_dim=6, vdim=16, kv_rank=24, q_rank=12, window=21)]),
    "latent_window_one": cfg_of([Lt(heads=2, dim=6, rot_dim=2, vdim=6, kv_rank=6, q_rank=6, window=1)]),
    "latent_window_beyond_the_prompt": cfg_of([Lt(heads=1, dim=20, rot_dim=10, vdim=5, kv_rank=9, q_rank=30, window=500, scale=0.3)]),
    "latent_one_rotated_pair": cfg_of([Lt(heads=3, dim=1, rot_dim=2, vdim=1, kv_rank=1, q_rank=1, window=8, base=3.0)], width=8),
    "latent_seventeen_heads": cfg_of([Lt(heads=17, dim=4, rot_dim=4, vdim=4, kv_rank=8, q_rank=8, window=30)]),
    "dense": cfg_of([Lt(ff=72)]),
    "dense_one_unit": cfg_of([Lt(ff=1)]),
    "experts": cfg_of([Lt(ff=E(8, 2, 20, 1.5, 2.5, (4, 2), (12, 0.5)))]),
    "experts_top1_no_shared_no_groups": cfg_of([Lt(ff=E(3, 1, 36, 0.7, 1.0, None, None))]),
    "experts_all_groups_kept": cfg_of([Lt(ff=E(6, 4, 12, 3.0, 0.5, (3, 3), (12, 3.0)))]),
    "experts_groups_of_one": cfg_of([Lt(ff=E(5, 2, 12, 3.0, 1.0, (5, 2), None))]),
    "experts_one_group_kept": cfg_of([Lt(ff=E(40, 3, 8, 2.0, 2.0, (8, 1), (8, 9.0)))]),
    "experts_one_expert": cfg_of([Lt(ff=E(1, 1, 8, 2.0, 3.0, None, (40, 1.0)))]),
    "loop_whole_model": cfg_of([Lt(ff=24), Lt(ff=E())], loop=(0, 2, 3)),
    "loop_one_layer_in_the_middle": cfg_of([Lt(ff=24), Lt(window=7), Lt(ff=E())], loop=(1, 2, 4)),
    "loop_once": cfg_of([Lt(ff=24), Lt(ff=16)], loop=(0, 1, 1)),
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
    for l, x in enumerate(trace):       # the residual stream after every layer run (before the embedding output comes back for the next pass)
        h = p.m.debug_read("hidden", l, x.size).reshape(x.shape)
        assert np.abs(h - x).max() <= TOL32 * max(1.0, np.abs(x).max()), f"{name}: layer run {l}"
    p.m.seq_close(s)
    p.m.set_trace(False)
    # the same tokens one by one, and in portions
    p.check(p.run_cuts(ids, range(1, len(ids))), want, name + " token by token")
    p.check(p.run_cuts(ids, [2, 4, 9, 10, 31, 33]), want, name + " in portions")
    p.close()


@pytest.mark.parametrize("exact", [True, False])
def test_whole_model_portions_and_decoding(exact):
    p = Pair(synth.gomerax_config(**TINY), seed=2, exact=exact)
    ids = p.ids(150, 3)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, []), want, "whole")
    p.check(p.run_cuts(ids, [2, 4, 5, 8, 15, 31, 32, 33, 64, 96, 97, 127, 129]), want, "portions of 1, 2, 3, 7 and more tokens, at page borders")
    p.check(p.run_cuts(ids, list(range(60, 150))), want, "prompt then 90 decoded tokens")
    p.check(p.run_cuts(ids, list(range(1, 12))), want, "the first tokens one by one")
    p.check(p.run_cuts(ids, list(range(2, 150, 2))), want, "two tokens at a time")
    p.close()


def test_tensor_core_paths_in_serving_mode():
    # sizes that tile (K % 64 == 0, N % 32 == 0, value size 64): portions of 32 tokens and more run their Linear layers, the experts' grouped
    # products with the clamped unit as their epilogue and the latent attention (windowed, with the sink) on the tcgen05 kernels, shorter ones
    # and decode steps on the CUDA cores; both must agree with the plain implementation, and the marked token (far back, at a page's last
    # place) must be seen by the rows that can see it
    mark = 3
    layers = [Lt(heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=64, q_rank=96, window=150, base=1e4, ff=256),
              Lt(heads=3, dim=32, rot_dim=32, vdim=64, kv_rank=96, q_rank=64, window=70, base=1e4, ff=E(8, 2, 64, 1.5, 2.5, (4, 3), (64, 0.75))),
              Lt(heads=2, dim=128, rot_dim=64, vdim=128, kv_rank=64, q_rank=64, window=300, base=1e4, ff=E(3, 1, 128, 1.0, 1.0, None, None))]
    cfg = cfg_of(layers, width=128, vocab=160, embed_scale=4.0, loop=(0, 2, 2))
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


@pytest.mark.parametrize("dims", [(64, 0, 64), (32, 32, 64), (96, 32, 64), (64, 64, 128), (128, 64, 128), (16, 16, 128), (160, 32, 64)])
def test_tensor_core_attention_head_sizes(dims):
    # (dim, rot_dim, vdim): value sizes 64 / 128 with keys of up to 128 / 192 run on the tcgen05 flash kernel, windowed and with the sink; keys
    # shorter than values are zero-padded; the last one is too long for it and stays on the CUDA cores
    dim, rot, vdim = dims
    mark = 5
    cfg = cfg_of([Lt(heads=2, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=64, q_rank=64, window=100, base=1e4, ff=64)], width=64, vocab=90)
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
    cfg = synth.gomerax_config(**TINY)
    ids = np.random.default_rng(3).integers(0, cfg["vocab"], 300).astype(np.uint32)
    out = []
    for plain in (False, True):
        p = Pair(cfg, seed=17, plain=plain)
        out.append(p.run_cuts(ids, [70, 71, 200] + list(range(250, 300))))
        p.check(out[-1], p.o.forward(ids), "plain kernels" if plain else "fast kernels")
        p.close()
    assert np.abs(out[0] - out[1]).max() < 1e-3


def test_launches_shorter_than_a_step_are_cut_by_the_scheduler():
    p = Pair(synth.gomerax_config(**TINY), seed=4, step_tokens=24)      # the engine itself cuts a 100-token entry into 24-token launches
    ids = p.ids(100, 7)
    p.check(p.run_cuts(ids, []), p.o.forward(ids), "launch size 24")
    p.close()


def test_mixed_batches_equal_each_request_alone():
    p = Pair(synth.gomerax_config(**TINY), seed=6, max_ctx=1024, max_seqs=4)
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
    p = Pair(synth.gomerax_config(**TINY), seed=8, max_ctx=256, max_seqs=2)
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
    p.m.seq_close(sa)                                    # a's pages and slot go to c while b is still live
    sc = p.m.seq_open()
    assert sc == sa
    gc = p.m.feed([(sc, c[:128], range(128))])
    p.m.seq_close(sb)
    sd = p.m.seq_open()
    g2 = p.m.feed([(sc, c[128:], range(2)), (sd, d, range(90))])
    p.check(np.concatenate([gc, g2[:2]]), p.o.forward(c), "c in a's slot and pages")
    p.check(g2[2:], p.o.forward(d), "d in b's slot and pages")
    p.close()


def test_learned_positions_end_where_the_table_ends():
    cfg = cfg_of([Lt(ff=16)], max_positions=50)
    p = Pair(cfg, seed=3)
    ids = p.ids(50, 2)
    p.check(p.run_cuts(ids, [20, 49]), p.o.forward(ids), "up to the last learned position")
    s = p.m.seq_open()
    p.m.feed([(s, ids, [])])
    with pytest.raises(Exception):
        p.m.feed([(s, ids[:1], [0])])                    # position 50 has no row
    p.close()


def test_far_information_travels_through_the_layers_and_page_borders():
    # one layer sees `window` tokens back, a stack of layer runs several windows: the marked token at a page's last place still shows at a position
    # that no single window reaches, in a long portion, in short ones and in tokens decoded alone
    mark = 7
    cfg = cfg_of([Lt(heads=4, dim=16, rot_dim=8, vdim=16, window=96, ff=E(4, 2, 24, 1.5, 2.0, (2, 1), (8, 1.0))), Lt(heads=2, window=96, ff=24)], width=48, vocab=60, loop=(0, 2, 3))
    p = Pair(cfg, seed=11, boost=mark, max_ctx=1024, step_tokens=1024)
    ids = p.ids(420, 5, avoid=mark)
    ids[31] = mark                                         # the last token of the first page
    want = p.o.forward(ids)
    plain = ids.copy(); plain[31] = (mark + 2) % 60
    other = p.o.forward(plain)
    felt = np.where(np.abs(other - want).max(axis=1) > 50 * p.tol)[0]
    assert felt.max() > 31 + 96 + 16                               # further back than one window: through the stack of layer runs
    s = p.m.seq_open()
    g1 = p.m.feed([(s, ids[:280], [31, 32, 63, 64, 126, 127, 128, 279])])
    g2 = [p.m.feed([(s, ids[t:t + 1], [0])]) for t in range(280, 320)]      # decoding across page borders, keys split over several blocks
    g3 = p.m.feed([(s, ids[320:322], [0, 1])])
    g4 = p.m.feed([(s, ids[322:], range(98))])
    p.m.seq_close(s)
    p.check(g1, want[[31, 32, 63, 64, 126, 127, 128, 279]], "prompt rows at page borders and window edges")
    p.check(np.concatenate(g2 + [g3, g4]), want[280:], "decoded rows and later portions that still feel position 31")
    p.close()


@pytest.mark.parametrize("window", [1, 2, 31, 32, 33, 64, 100, 129])
def test_window_edges_in_prompts_and_in_decoding(window):
    # a single layer: the marked token at position m is seen by rows m .. m + window - 1 and by no other.  The oracle says so, and the engine
    # must agree with it whether the row is part of a long portion (expanded keys), a short one or decoded alone (absorbed form)
    mark, m = 9, 70
    cfg = cfg_of([Lt(heads=3, dim=12, rot_dim=6, vdim=8, kv_rank=16, q_rank=10, window=window, ff=24)], width=32, vocab=50)
    p = Pair(cfg, seed=19, edit=spotlight(cfg, mark), max_ctx=1024, step_tokens=512)
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


def test_window_edges_on_the_tensor_cores():
    # the same on the tcgen05 flash kernel (serving mode): windows that end inside a 64-key tile, at its border and beyond two tiles
    mark, m = 9, 70
    for window in (33, 64, 129):
        cfg = cfg_of([Lt(heads=2, dim=32, rot_dim=32, vdim=64, kv_rank=64, q_rank=64, window=window, base=1e4, ff=64)], width=64, vocab=50)
        p = Pair(cfg, seed=19, exact=False, edit=spotlight(cfg, mark), max_ctx=1024, step_tokens=512)
        ids = p.ids(m + window + 70, 3, avoid=mark)
        ids[m] = mark
        want = p.o.forward(ids)
        plain = ids.copy(); plain[m] = (mark + 2) % 50
        other = p.o.forward(plain)
        last_in, first_out = m + window - 1, m + window
        assert np.abs(other[last_in] - want[last_in]).max() / want.std() > 0.03 and np.abs(other[first_out] - want[first_out]).max() == 0.0
        for cuts in ([], [m - 3, last_in, first_out + 40], [first_out - 33, first_out + 33]):
            got = p.run_cuts(ids, cuts)
            assert np.abs(got - want).max() / want.std() < 3e-3, (window, cuts)
        p.close()


def test_other_head_sizes_and_unequal_portions():
    # portions of 32 tokens and more expand keys and values and run the tiled kernels (odd sizes leave partial tiles), shorter ones and decoded
    # tokens the absorbed form; both continue one another's cache (18 heads: the decode kernel serves sixteen heads at a time, then the other two)
    for layers in ([Lt(heads=2, dim=20, rot_dim=14, vdim=136, kv_rank=24, q_rank=7, window=90), Lt(heads=3, dim=34, rot_dim=2, vdim=5, kv_rank=7, q_rank=33, window=200, ff=9)],
                   [Lt(heads=3, dim=6, rot_dim=10, vdim=5, kv_rank=9, q_rank=40, window=64, ff=E(7, 3, 5, 0.5, 1.5, None, (3, 0.25)))],
                   [Lt(heads=18, dim=8, rot_dim=8, vdim=8, kv_rank=20, q_rank=16, window=33), Lt(heads=1, dim=130, rot_dim=64, vdim=24, kv_rank=50, q_rank=16, window=150)]):
        p = Pair(cfg_of(layers, width=30, vocab=50), seed=27, max_ctx=1024, max_seqs=3, step_tokens=512)
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


def test_sink_shows_and_is_not_scaled():
    # a small attention scale makes every score nearly 0, so a row's six visible keys weigh about one each and the sink exp(sink): leaving it out,
    # counting it as exp(0) or scaling it like a score differs grossly
    def edit(name, a):
        return np.array([2.0, -1.0, 0.5]) if name.endswith("mix.sink") else None
    cfg = cfg_of([Lt(heads=3, dim=8, rot_dim=4, vdim=8, kv_rank=8, q_rank=8, window=6, scale=0.01)], width=24, vocab=40)
    p = Pair(cfg, seed=23, edit=edit)
    ids = p.ids(90, 1)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, [50, 52] + list(range(60, 90))), want, "sink")
    keep = Z.sink_softmax
    try:
        for variant in (lambda s, vis, sink: keep(s, vis, -1e9), lambda s, vis, sink: keep(s, vis, 0.0), lambda s, vis, sink: keep(s, vis, sink * 0.01)):
            Z.sink_softmax = variant
            assert np.abs(Gomerax(cfg, p.o.w).forward(ids) - want).max() > 300 * p.tol
    finally:
        Z.sink_softmax = keep
    p.close()


def test_router_correction_groups_and_clamps_show():
    # a correction that reverses the choice, groups that shut out the best expert, clamps that cut most values: each changes the result grossly,
    # so an engine that ignored one of them would be far from the plain implementation
    def edit(name, a):
        if name.endswith("mlp.correction"):
            return np.array([0.9, -0.9, 0.5, -0.5, 0.7, -0.7, 0.3, -0.3], np.float32)
        return None
    ff = E(8, 2, 20, 0.5, 2.5, (4, 1), (12, 0.25))      # (one group kept: both experts of a token are neighbours)
    cfg = cfg_of([Lt(ff=ff)], width=32, vocab=64)
    p = Pair(cfg, seed=29, edit=edit)
    ids = p.ids(120, 2)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, [40, 42, 90] + list(range(91, 120))), want, "router rule and clamps")
    w = p.o.w
    no_corr = dict(w); no_corr["l0.mlp.correction"] = w["l0.mlp.correction"] * 0.0
    assert np.abs(Gomerax(cfg, no_corr).forward(ids) - want).max() > 100 * p.tol
    for other in (dict(ff, groups=None), dict(ff, groups=(2, 1)), dict(ff, limit=5.0), dict(ff, shared=(12, 5.0)), dict(ff, scale=1.0)):
        assert np.abs(Gomerax(cfg_of([Lt(ff=other)], width=32, vocab=64), w).forward(ids) - want).max() > 100 * p.tol, other
    keep = Z.route
    try:        # weights taken from the corrected scores, or not renormalised: far away as well
        def corrected(z, corr, rt):
            ch, _ = keep(z, corr, rt)
            s = np.exp(z - z.max()); s = s / s.sum() + corr
            return ch, s[ch] / (s[ch].sum() + 1e-20) * rt["scale"]
        def raw(z, corr, rt):
            ch, _ = keep(z, corr, rt)
            s = np.exp(z - z.max()); s = s / s.sum()
            return ch, s[ch] * rt["scale"]
        for variant in (corrected, raw):
            Z.route = variant
            assert np.abs(Gomerax(cfg, w).forward(ids) - want).max() > 100 * p.tol
    finally:
        Z.route = keep
    p.close()


def test_loop_passes_have_their_own_caches_and_get_the_embedding_again():
    cfg = cfg_of([Lt(window=25, ff=24), Lt(window=11, ff=E())], loop=(0, 2, 3), width=32, vocab=50)
    p = Pair(cfg, seed=33)
    ids = p.ids(140, 4)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, [33, 35, 100] + list(range(101, 140))), want, "three passes")
    one_pass = Gomerax(dict(cfg, loop={"start": 0, "stop": 2, "times": 1}), p.o.w).forward(ids)
    assert np.abs(one_pass - want).max() > 100 * p.tol                        # (the passes matter)
    w = p.o.w
    no_pos = dict(w); no_pos["pos"] = w["pos"] * 0.0
    assert np.abs(Gomerax(cfg, no_pos).forward(ids) - want).max() > 100 * p.tol
    keep = Z.layer_runs
    try:        # without the embedding output before the later passes the result is far away
        Z.layer_runs = lambda c: [(l, False) for l, _ in keep(c)]
        assert np.abs(Gomerax(cfg, w).forward(ids) - want).max() > 100 * p.tol
    finally:
        Z.layer_runs = keep
    p.close()


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes_and_layer_orders(seed):
    # sizes, head counts, layer order, loops and constants drawn at random (odd sizes included): nothing may rest on one model's values
    r = np.random.default_rng(400 + seed)
    pick = lambda *xs: xs[int(r.integers(0, len(xs)))]
    width = pick(6, 10, 16, 20, 36, 64)

    def ff():
        g = pick(None, (1, 1), (2, 1), (3, 2), (4, 4))
        per = pick(1, 2, 3)
        n = (g[0] if g else pick(2, 3, 5)) * per
        most = (g[1] * per) if g else n
        return pick(None, pick(8, 24, 50), E(n, int(r.integers(1, most + 1)), pick(6, 16, 24), pick(0.3, 1.0, 7.0), pick(0.5, 1.0, 2.5), g, pick(None, (6, 0.4), (16, 2.0), (30, 7.0))))

    def layer():
        return Lt(heads=pick(1, 2, 3, 7), dim=pick(4, 6, 16, 24), rot_dim=pick(0, 2, 6, 16), vdim=pick(4, 6, 16, 36), kv_rank=pick(4, 10, 16, 48), q_rank=pick(3, 8, 32),
                  window=pick(1, 5, 32, 60, 200), scale=pick(None, 0.2, 0.5), base=pick(10.0, 1e3, 1e6), ff=ff())

    n = int(r.integers(1, 5))
    layers = [layer() for _ in range(n)]
    a = int(r.integers(0, n)); b = int(r.integers(a, n + 1))
    loop = pick(None, (a, b, int(r.integers(1, 4))))
    cfg = synth.gomerax_config(layers, width=width, vocab=pick(17, 50, 131), eps=pick(1e-6, 1e-5, 1e-3), embed_scale=pick(0.25, 1.0, 8.0), max_positions=pick(170, 300), loop=loop)
    p = Pair(cfg, seed=seed, exact=seed % 3 != 0, max_ctx=512, max_seqs=3, step_tokens=pick(48, 200, 512))      # (every third one in serving mode)
    ids = p.ids(170, seed)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, []), want, "whole")
    p.check(p.run_cuts(ids, [1, 3, 40, 41, 100, 133] + list(range(140, 170))), want, "portions and decoding")
    p.close()


@pytest.mark.parametrize("seed", range(6))
def test_random_shapes_that_tile_for_the_tensor_cores(seed):
    # widths, head sizes and feed-forward sizes that the tcgen05 kernels take (multiples of 64; value size 64 / 128), everything else drawn at random
    r = np.random.default_rng(500 + seed)
    pick = lambda *xs: xs[int(r.integers(0, len(xs)))]
    width = pick(64, 128, 192, 320)

    def ff():
        g = pick(None, (2, 1), (4, 3))
        n = (g[0] if g else pick(2, 3)) * pick(1, 2)
        most = g[1] * (n // g[0]) if g else n
        return pick(None, pick(64, 192), E(n, int(r.integers(1, most + 1)), pick(64, 128), pick(0.5, 2.0, 7.0), pick(1.0, 2.5), g, pick(None, (64, 1.0), (96, 7.0))))

    def layer():
        dv = pick(64, 128)
        return Lt(heads=pick(1, 2, 5), dim=pick(32, 64, 96), rot_dim=pick(0, 32, 64), vdim=dv, kv_rank=pick(32, 64, 80), q_rank=pick(24, 64, 128), window=pick(1, 33, 64, 150, 257, 1000),
                  scale=pick(None, 0.1), base=pick(1e3, 2e4), ff=ff())

    n = int(r.integers(2, 5))
    layers = [layer() for _ in range(n)]
    cfg = synth.gomerax_config(layers, width=width, vocab=pick(64, 100, 160), eps=pick(1e-6, 1e-5), embed_scale=pick(1.0, 8.0), max_positions=640, loop=pick(None, (0, n - 1, 2), (1, n, 2)))
    exact = seed % 2 == 1
    p = Pair(cfg, seed=seed, exact=exact, max_ctx=1024, max_seqs=3, step_tokens=pick(256, 1024))
    ids = p.ids(600, seed)
    want = p.o.forward(ids)
    for cuts in ([], [33, 35, 100, 164, 300, 333, 560] + list(range(580, 600))):
        got = p.run_cuts(ids, cuts)
        err = np.abs(got - want).max() / max(1.0, want.std())
        assert err < (TOL32 if exact else 3e-3), (cuts[:3], err, int(np.abs(got - want).max(axis=1).argmax()))
    p.close()


def test_long_decoding_keeps_the_caches():
    cfg = cfg_of([Lt(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=8, q_rank=8, window=50, ff=E(4, 2, 8, 1.0, 2.0, (2, 1), (8, 1.0))), Lt(window=130, ff=16)], width=24, vocab=40, loop=(0, 1, 2))
    p = Pair(cfg, seed=12)
    ids = p.ids(400, 9)
    p.check(p.run_cuts(ids, list(range(3, 400))), p.o.forward(ids), "397 decoded tokens")
    p.close()


def test_greedy_generation_through_the_entry_points():
    cfg = synth.gomerax_config(**TINY)
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
    cfg = synth.gomerax_config(**TINY)
    p = Pair(cfg, seed=14)
    pr = p.ids(12, 1)
    a, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=5)
    b, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=5)
    assert a == b and len(a) == 8 and all(0 <= t < cfg["vocab"] for t in a)
    p.close()


def test_a_checkpoint_folder_is_served_by_the_one_loader(tmp_path):
    import json
    import os
    from aha_b200.checkpoint import load_model, write_safetensors
    cfg = synth.gomerax_config(**TINY)
    w = synth.make_gomerax(cfg, 40)
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(tmp_path, "model.safetensors"), w)
    m = load_model(str(tmp_path), max_ctx=256, max_prefill=128, max_seqs=2, exact_fp32=True)
    assert m.kind == "gomerax"
    ids = np.random.default_rng(1).integers(0, cfg["vocab"], 60).astype(np.uint32)
    s = m.seq_open()
    got = m.feed([(s, ids, range(60))])
    want = Gomerax(cfg, {k: synth.bf16_to_f32(v) for k, v in w.items()}).forward(ids)
    assert np.abs(got - want).max() / max(1.0, want.std()) < TOL32
    m.close()
