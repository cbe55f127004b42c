"""Synthetic checkpoints: seeded random-init weights with the REAL tensor names and shapes the
reference's loaders read (`vb.pp(...)` calls at /root/reference/src/models/qwen3/model.rs:28-62,105-125,
qwen3vl/model.rs:54,61,129-132,201-202,291-313,389-410,848-860, qwen3_asr/model.rs:43-61,104-151,239-247,
317-326,375).  There is no network for real checkpoints; values are N(0, 0.02) (norm gains 1 + N(0, 0.02))
rounded to fp16 so that fp16 storage is lossless for both the CUDA path and the fp32 oracle.

Config dicts follow the HF `config.json` layout that the reference deserialises
(qwen3/config.rs, qwen3vl/config.rs, qwen3_asr/config.rs)."""
import copy
import numpy as np

# ----------------------------------------------------------------------------- configs
_TEXT_06 = dict(attention_bias=False, head_dim=128, hidden_act="silu", hidden_size=1024, intermediate_size=3072,
                num_attention_heads=16, num_hidden_layers=28, num_key_value_heads=8, rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=True, vocab_size=151936, eos_token_id=151645)
_TEXT_TINY = dict(attention_bias=False, head_dim=128, hidden_act="silu", hidden_size=256, intermediate_size=512,
                  num_attention_heads=4, num_hidden_layers=2, num_key_value_heads=2, rms_norm_eps=1e-6,
                  rope_theta=1000000.0, tie_word_embeddings=True, vocab_size=1024, eos_token_id=1023)
_MROPE = dict(rope_type="default", mrope_section=[24, 20, 20], mrope_interleaved=True)

QWEN3 = {
    "tiny": dict(_TEXT_TINY),
    # Qwen3-VL-2B text-stack row shapes (H=2048, I=6144, 16/8 heads) with 2 layers and a small vocabulary: exercises the
    # production code paths of the decode kernels (4-row K=2048 stages, 1-row K=6144 stages) at test cost
    "mid": dict(_TEXT_06, hidden_size=2048, intermediate_size=6144, num_hidden_layers=2, vocab_size=4096, rope_theta=5000000.0,
                eos_token_id=4095),
    "tiny-untied": dict(_TEXT_TINY, tie_word_embeddings=False),
    # GQA groups other than 2 (every shipped Qwen3 size the fused kernel accepts has nh / nkv = 2): MHA and a group of 4
    "tiny-g1": dict(_TEXT_TINY, num_attention_heads=2, num_key_value_heads=2),
    "tiny-g4": dict(_TEXT_TINY, num_attention_heads=4, num_key_value_heads=1),
    "q0.6": dict(_TEXT_06),
}

_VIS_2B = dict(deepstack_visual_indexes=[5, 11, 17], depth=24, hidden_act="gelu_pytorch_tanh", hidden_size=1024,
               in_channels=3, intermediate_size=4096, num_heads=16, num_position_embeddings=2304,
               out_hidden_size=2048, patch_size=16, spatial_merge_size=2, temporal_patch_size=2)
_VIS_TINY = dict(deepstack_visual_indexes=[0, 2], depth=4, hidden_act="gelu_pytorch_tanh", hidden_size=128,
                 in_channels=3, intermediate_size=256, num_heads=2, num_position_embeddings=64,
                 out_hidden_size=256, patch_size=16, spatial_merge_size=2, temporal_patch_size=2)
# the Qwen3-VL-8B / 32B tower: hidden 1152 over 16 heads = head_dim 72, intermediate 4304 (neither tiles the tensor-core kernels: the
# library pads head slots to 128 and the intermediate to 4352 at upload, vision_model.cuh)
_VIS_8B = dict(_VIS_2B, depth=27, deepstack_visual_indexes=[8, 16, 24], hidden_size=1152, intermediate_size=4304, out_hidden_size=4096)
_VL_IDS = dict(image_token_id=151655, video_token_id=151656, vision_start_token_id=151652, vision_end_token_id=151653)

QWEN3VL = {
    "tiny": dict(image_token_id=1001, video_token_id=1002, vision_start_token_id=1003, vision_end_token_id=1004,
                 tie_word_embeddings=True,
                 text_config=dict(_TEXT_TINY, rope_theta=5000000.0, rope_scaling=dict(_MROPE)),
                 vision_config=dict(_VIS_TINY)),
    # head_dim 72 and an intermediate size that is not a multiple of 64, at test cost (K = 576 and the padded shapes tile the tcgen05 GEMM)
    "tiny-hd72": dict(image_token_id=1001, video_token_id=1002, vision_start_token_id=1003, vision_end_token_id=1004,
                      tie_word_embeddings=True,
                      text_config=dict(_TEXT_TINY, rope_theta=5000000.0, rope_scaling=dict(_MROPE)),
                      vision_config=dict(_VIS_TINY, depth=2, deepstack_visual_indexes=[0], hidden_size=576, num_heads=8,
                                         intermediate_size=1080)),
    "vl2": dict(_VL_IDS, tie_word_embeddings=True,
                text_config=dict(_TEXT_06, hidden_size=2048, intermediate_size=6144, rope_theta=5000000.0,
                                 rope_scaling=dict(_MROPE)),
                vision_config=dict(_VIS_2B)),
    # BASELINE.json config 5 says "7B"; the reference registry has 2B/4B/8B/32B only (model_mapping.rs:57-64) -> Qwen3-VL-8B: text stack
    # H 4096, 36 layers, 32 / 8 heads, I 12288; vision tower 27 blocks of hidden 1152 / 16 heads (head_dim 72), intermediate 4304.
    "vl8": dict(_VL_IDS, tie_word_embeddings=False,
                text_config=dict(_TEXT_06, hidden_size=4096, intermediate_size=12288, num_attention_heads=32,
                                 num_hidden_layers=36, rope_theta=5000000.0, rope_scaling=dict(_MROPE)),
                vision_config=dict(_VIS_8B)),
}

_AUD_06 = dict(activation_function="gelu", conv_chunksize=500, d_model=896, downsample_hidden_size=480,
               encoder_attention_heads=14, encoder_ffn_dim=3584, encoder_layers=18, n_window=50, n_window_infer=800,
               num_mel_bins=128, output_dim=1024, max_source_positions=1500)
_AUD_TINY = dict(activation_function="gelu", conv_chunksize=2, d_model=128, downsample_hidden_size=32,
                 encoder_attention_heads=2, encoder_ffn_dim=256, encoder_layers=2, n_window=50, n_window_infer=800,
                 num_mel_bins=128, output_dim=256, max_source_positions=1500)

QWEN3_ASR = {
    "tiny": dict(thinker_config=dict(audio_token_id=1001, audio_start_token_id=1002, audio_end_token_id=1003,
                                     audio_config=dict(_AUD_TINY),
                                     text_config=dict(_TEXT_TINY, rope_scaling=dict(_MROPE)))),
    "asr0.6": dict(thinker_config=dict(audio_token_id=151676, audio_start_token_id=151669, audio_end_token_id=151670,
                                       audio_config=dict(_AUD_06),
                                       text_config=dict(_TEXT_06, rope_scaling=dict(_MROPE)))),
}


def get_config(kind, preset):
    return copy.deepcopy({"qwen3": QWEN3, "qwen3vl": QWEN3VL, "qwen3_asr": QWEN3_ASR, "malasun": MALASUN}[kind][preset])


# ----------------------------------------------------------------------------- weights
class _Gen:
    def __init__(self, seed, std=0.02, fast=False):
        self.rng = np.random.default_rng(seed)
        self.std = std
        self.fast = fast       # uniform with the same std instead of normal: 3x faster to draw (the 8-billion-parameter timing preset)
        self.w = {}

    def mat(self, name, *shape):
        n = int(np.prod(shape))
        if self.fast:
            a = self.rng.random(n, dtype=np.float32)
            a -= np.float32(0.5)
            a *= np.float32(self.std * 3.4641016)
        else:
            a = self.rng.standard_normal(n, dtype=np.float32)
            a *= np.float32(self.std)
        self.w[name] = a.astype(np.float16).reshape(shape)

    def gain(self, name, n):
        self.w[name] = (1.0 + self.std * self.rng.standard_normal(n, dtype=np.float32)).astype(np.float16)

    def bias(self, name, n):
        self.w[name] = (self.std * self.rng.standard_normal(n, dtype=np.float32)).astype(np.float16)

    def linear(self, prefix, out_f, in_f, bias):
        self.mat(prefix + ".weight", out_f, in_f)
        if bias:
            self.bias(prefix + ".bias", out_f)

    def lnorm(self, prefix, n):
        self.gain(prefix + ".weight", n)
        self.bias(prefix + ".bias", n)


def _text_layers(g, p, tc):
    H, I = tc["hidden_size"], tc["intermediate_size"]
    nh, nkv, hd = tc["num_attention_heads"], tc["num_key_value_heads"], tc["head_dim"]
    b = tc.get("attention_bias", False)
    g.mat(p + "embed_tokens.weight", tc["vocab_size"], H)
    for i in range(tc["num_hidden_layers"]):
        lp = f"{p}layers.{i}."
        g.linear(lp + "self_attn.q_proj", nh * hd, H, b)
        g.linear(lp + "self_attn.k_proj", nkv * hd, H, b)
        g.linear(lp + "self_attn.v_proj", nkv * hd, H, b)
        g.linear(lp + "self_attn.o_proj", H, nh * hd, b)
        g.gain(lp + "self_attn.q_norm.weight", hd)
        g.gain(lp + "self_attn.k_norm.weight", hd)
        g.linear(lp + "mlp.gate_proj", I, H, False)
        g.linear(lp + "mlp.up_proj", I, H, False)
        g.linear(lp + "mlp.down_proj", H, I, False)
        g.gain(lp + "input_layernorm.weight", H)
        g.gain(lp + "post_attention_layernorm.weight", H)
    g.gain(p + "norm.weight", H)


def make_qwen3(cfg, seed=0, fast=False):
    g = _Gen(seed, fast=fast)
    _text_layers(g, "model.", cfg)
    if not cfg.get("tie_word_embeddings", False):
        g.mat("lm_head.weight", cfg["vocab_size"], cfg["hidden_size"])
    return g.w


def make_qwen3vl(cfg, seed=0):
    g = _Gen(seed, fast=cfg["text_config"]["hidden_size"] >= 4096)
    vc, tc = cfg["vision_config"], cfg["text_config"]
    Hv, Iv, p = vc["hidden_size"], vc["intermediate_size"], "model.visual."
    ps, tp, m = vc["patch_size"], vc["temporal_patch_size"], vc["spatial_merge_size"]
    g.mat(p + "patch_embed.proj.weight", Hv, vc["in_channels"], tp, ps, ps)
    g.bias(p + "patch_embed.proj.bias", Hv)
    g.mat(p + "pos_embed.weight", vc["num_position_embeddings"], Hv)
    for i in range(vc["depth"]):
        bp = f"{p}blocks.{i}."
        g.lnorm(bp + "norm1", Hv)
        g.lnorm(bp + "norm2", Hv)
        g.linear(bp + "attn.qkv", 3 * Hv, Hv, True)
        g.linear(bp + "attn.proj", Hv, Hv, True)
        g.linear(bp + "mlp.linear_fc1", Iv, Hv, True)
        g.linear(bp + "mlp.linear_fc2", Hv, Iv, True)

    def merger(mp, post):
        Hm = Hv * m * m
        g.lnorm(mp + "norm", Hm if post else Hv)
        g.linear(mp + "linear_fc1", Hm, Hm, True)
        g.linear(mp + "linear_fc2", vc["out_hidden_size"], Hm, True)

    merger(p + "merger.", False)
    for i in range(len(vc["deepstack_visual_indexes"])):
        merger(f"{p}deepstack_merger_list.{i}.", True)
    _text_layers(g, "model.language_model.", tc)
    if not cfg.get("tie_word_embeddings", False):
        g.mat("lm_head.weight", tc["vocab_size"], tc["hidden_size"])
    return g.w


def make_qwen3_asr(cfg, seed=0):
    g = _Gen(seed)
    tk = cfg["thinker_config"]
    ac, tc = tk["audio_config"], tk["text_config"]
    p, D, C = "thinker.audio_tower.", ac["d_model"], ac["downsample_hidden_size"]
    g.mat(p + "conv2d1.weight", C, 1, 3, 3); g.bias(p + "conv2d1.bias", C)
    g.mat(p + "conv2d2.weight", C, C, 3, 3); g.bias(p + "conv2d2.bias", C)
    g.mat(p + "conv2d3.weight", C, C, 3, 3); g.bias(p + "conv2d3.bias", C)
    fdim = ((((ac["num_mel_bins"] + 1) // 2 + 1) // 2 + 1) // 2)
    g.mat(p + "conv_out.weight", D, C * fdim)
    for i in range(ac["encoder_layers"]):
        lp = f"{p}layers.{i}."
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            g.linear(lp + "self_attn." + n, D, D, True)
        g.lnorm(lp + "self_attn_layer_norm", D)
        g.linear(lp + "fc1", ac["encoder_ffn_dim"], D, True)
        g.linear(lp + "fc2", D, ac["encoder_ffn_dim"], True)
        g.lnorm(lp + "final_layer_norm", D)
    g.lnorm(p + "ln_post", D)
    g.linear(p + "proj1", D, D, True)
    g.linear(p + "proj2", ac["output_dim"], D, True)
    _text_layers(g, "thinker.model.", tc)
    if not tc.get("tie_word_embeddings", False):
        g.mat("thinker.lm_head.weight", tc["vocab_size"], tc["hidden_size"])
    return g.w


# ----------------------------------------------------------------------------- Malasun (layered engine)
def malasun_config(layers, width=64, vocab=96, eps=1e-5):
    """config.json of a Malasun model.  layers: list of dicts, each
         {"type": "hgrn2", "heads", "dim", "vdim", "ff": None | int}
         {"type": "attention", "heads", "kv_heads", "dim", "vdim", "window": None | int, "conv": None | taps, "scale": float,
          "kv_from": None | layer index, "ff": None | int}"""
    out = []
    for ly in layers:
        if ly["type"] == "hgrn2":
            mx = {"heads": ly["heads"], "dim": ly["dim"], "vdim": ly["vdim"]}
        else:
            mx = {"heads": ly["heads"], "kv_heads": ly["kv_heads"], "dim": ly["dim"], "vdim": ly["vdim"],
                  "scale": ly.get("scale", float(ly["dim"]) ** -0.5)}
            if ly.get("window"):
                mx["mask"] = {"size": ly["window"]}
            if ly.get("conv"):
                mx["conv"] = ly["conv"]
            if ly.get("kv_from") is not None:
                mx["kv_from"] = ly["kv_from"]
        out.append({"type": ly["type"], "mixer": mx, "mlp": {"kind": "dense", "ff": ly["ff"]} if ly.get("ff") else None})
    return {"architecture": "Malasun", "layers": out, "norm": {"eps": eps}, "vocab": vocab, "width": width}


MALASUN = {
    # every branch once, with sizes that differ from one another: attention first, a feed-forward on a recurrent layer, two kv heads,
    # dim != vdim, a shared cache read through a narrower window, an attention layer without window / convolution
    "tiny": malasun_config([
        {"type": "attention", "heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "window": 40, "conv": 3, "ff": 80},
        {"type": "hgrn2", "heads": 3, "dim": 16, "vdim": 8, "ff": 48},
        {"type": "attention", "heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "window": 17, "conv": 2, "kv_from": 0, "ff": None},
        {"type": "hgrn2", "heads": 2, "dim": 24, "vdim": 40, "ff": None},
        {"type": "attention", "heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "window": None, "conv": None, "ff": 64},
    ], width=72, vocab=101),
}


def malasun_shape(width, n_layers, heads, kv_heads, head_dim, window, ff, rec_heads, rec_dim, vocab=32000, taps=4, share_every=2):
    """A layer list of the sizes a served model would have: recurrent and attention layers alternate, every `share_every`-th attention
    layer reads the cache of the attention layer before it."""
    layers, last_kv, n_att = [], None, 0
    for i in range(n_layers):
        if i % 2 == 0:
            layers.append({"type": "hgrn2", "heads": rec_heads, "dim": rec_dim, "vdim": rec_dim, "ff": None})
        else:
            share = last_kv is not None and share_every and n_att % share_every == share_every - 1
            layers.append({"type": "attention", "heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "window": window,
                           "conv": taps, "kv_from": last_kv if share else None, "ff": ff})
            if not share:
                last_kv = i
            n_att += 1
    return malasun_config(layers, width=width, vocab=vocab, eps=1e-6)


def _bf16_round(a):
    from ._lib import to_bf16
    a = np.asarray(a, np.float32)
    return to_bf16(a).reshape(a.shape)


def bf16_to_f32(a):
    """Values of a `_lib.BF16`-tagged array as float32."""
    return (np.asarray(a).view(np.ndarray).astype(np.uint32) << 16).view(np.float32)


def make_malasun(cfg, seed=0, fast=False):
    """Random weights under the checkpoint's tensor names, all bfloat16 (`_lib.BF16`-tagged bit patterns)."""
    rng = np.random.default_rng(seed)
    w = {}

    def rnd(*shape, std=1.0):
        if fast:
            a = rng.random(int(np.prod(shape)), dtype=np.float32)
            a -= np.float32(0.5)
            a *= np.float32(std * 3.4641016)
        else:
            a = rng.standard_normal(int(np.prod(shape)), dtype=np.float32) * np.float32(std)
        return a.reshape(shape)

    def put(name, a):
        w[name] = _bf16_round(a)

    def lin(name, out_f, in_f, gain=1.0):
        put(name, rnd(out_f, in_f, std=gain / np.sqrt(in_f)))

    W, V = cfg["width"], cfg["vocab"]
    put("embed", rnd(V, W))
    lin("head", V, W)
    put("final.norm", np.float32(1.0 + 0.2 * rng.standard_normal()))
    for i, ly in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, ly["mixer"]
        put(p + "norm1", np.float32(1.0 + 0.2 * rng.standard_normal()))
        if ly["type"] == "hgrn2":
            H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
            lin(p + "mix.q", H * D, W); lin(p + "mix.f", H * D, W, 2.0); lin(p + "mix.v", H * Dv, W)
            put(p + "mix.f.b", rnd(H * D, std=1.0))
            put(p + "mix.lower", 1.0 / (1.0 + np.exp(-rnd(H * D, std=1.5))))
            put(p + "mix.norm", 1.0 + 0.2 * rnd(Dv))
            lin(p + "mix.o", W, H * Dv)
        else:
            H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            own = "kv_from" not in mx
            parts = [("q", H * D)] + ([("k", G * D), ("v", G * Dv)] if own else [])
            for nm, n in parts:
                lin(p + "mix." + nm, n, W)
                put(p + "mix." + nm + ".b", rnd(n, std=0.3))
                if "conv" in mx:
                    put(p + "mix." + nm + ".conv", rnd(n, mx["conv"], std=0.6))
            put(p + "mix.q.norm", 1.0 + 0.3 * rnd(H * D))
            if own:
                put(p + "mix.k.norm", 1.0 + 0.3 * rnd(G * D))
            lin(p + "mix.g", H * Dv, W)
            lin(p + "mix.o", W, H * Dv)
        if ly.get("mlp"):
            ff = ly["mlp"]["ff"]
            put(p + "norm2", np.float32(1.0 + 0.2 * rng.standard_normal()))
            lin(p + "mlp.up", ff, W); lin(p + "mlp.down", W, ff)
            put(p + "mlp.act", rnd(2, std=0.7))
    return w



def gomerax_config(layers, width=64, vocab=96, eps=1e-5, embed_scale=1.0, max_positions=512, loop=None):
    """config.json of a Gomerax model.  layers: list of dicts
         {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "window", "scale", "base"}
       each with "ff": None | int (dense) | {"experts", "top", "ff", "limit", "scale", "groups": None | (count, keep), "shared": None | (ff, limit)}.
       loop: None | (start, stop, times)."""
    out = []
    for ly in layers:
        R = ly["rot_dim"]
        mx = {"heads": ly["heads"], "dim": ly["dim"], "rot_dim": R, "vdim": ly["vdim"], "kv_rank": ly["kv_rank"], "q_rank": ly["q_rank"],
              "mask": {"size": ly["window"]}, "rot": {"base": float(ly.get("base", 10000.0)), "dims": R},
              "scale": float(ly.get("scale", (ly["dim"] + R) ** -0.5))}
        ff = ly.get("ff")
        if ff is None:
            mlp = None
        elif isinstance(ff, dict):
            router = {"experts": ff["experts"], "top": ff["top"], "scale": float(ff.get("scale", 1.0))}
            if ff.get("groups"):
                router["groups"] = {"count": ff["groups"][0], "keep": ff["groups"][1]}
            mlp = {"kind": "moe", "expert": {"ff": ff["ff"], "limit": float(ff.get("limit", 7.0))}, "router": router}
            if ff.get("shared"):
                mlp["shared"] = {"ff": ff["shared"][0], "limit": float(ff["shared"][1])}
        else:
            mlp = {"kind": "dense", "ff": int(ff)}
        out.append({"type": "latent_attention", "mixer": mx, "mlp": mlp})
    cfg = {"architecture": "Gomerax", "layers": out, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "max_positions": max_positions,
           "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def gomerax_shape(width, n_layers, heads, head_dim, ff, experts, top, expert_ff, vocab=32000, kv_rank=256, q_rank=512, rot_dim=32, window=1024, max_positions=4096,
                  loop=None):
    """A layer list of the sizes a served model would have: a dense feed-forward on the first layer, routed experts (groups of four, three kept) with a
    shared expert on the others."""
    layers = []
    for i in range(n_layers):
        f = ff if i == 0 else {"experts": experts, "top": top, "ff": expert_ff, "limit": 7.0, "scale": 2.5, "groups": (4, 3) if experts % 4 == 0 and experts >= 8 else None,
                               "shared": (expert_ff, 7.0)}
        layers.append({"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank, "q_rank": q_rank, "window": window, "ff": f})
    return gomerax_config(layers, width=width, vocab=vocab, eps=1e-6, embed_scale=float(np.sqrt(width)), max_positions=max_positions, loop=loop)


def make_gomerax(cfg, seed=0, fast=False):
    """Random weights under the checkpoint's tensor names, all bfloat16 (`_lib.BF16`-tagged bit patterns).  Norm gains are stored around zero."""
    rng = np.random.default_rng(seed)
    w = {}

    def rnd(*shape, std=1.0):
        if fast:
            a = rng.random(int(np.prod(shape)), dtype=np.float32)
            a -= np.float32(0.5)
            a *= np.float32(std * 3.4641016)
        else:
            a = rng.standard_normal(int(np.prod(shape)), dtype=np.float32) * np.float32(std)
        return a.reshape(shape)

    def put(name, a):
        w[name] = _bf16_round(a)

    def lin(name, out_f, in_f, gain=1.0):
        put(name, rnd(out_f, in_f, std=gain / np.sqrt(in_f)))

    W, V = cfg["width"], cfg["vocab"]
    put("embed", rnd(V, W, std=1.0 / max(1.0, cfg["embedding"]["scale"])))
    put("pos", rnd(cfg["max_positions"], W, std=0.5))
    put("final.norm", 0.2 * rnd(W))
    for i, ly in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, ly["mixer"]
        put(p + "norm1", 0.2 * rnd(W))
        H, D, R, Dv, rank, qr = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
        lin(p + "mix.dq", qr, W); put(p + "mix.dq.norm", 1.0 + 0.2 * rnd(qr)); lin(p + "mix.uq", H * (D + R), qr, 2.0)
        lin(p + "mix.dkv", rank + R, W, 1.5); put(p + "mix.dkv.norm", 1.0 + 0.2 * rnd(rank))
        lin(p + "mix.uk", H * D, rank, 2.0); lin(p + "mix.uv", H * Dv, rank); lin(p + "mix.o", W, H * Dv, 0.7)
        put(p + "mix.sink", rnd(H, std=1.5))
        ml = ly.get("mlp")
        if not ml:
            continue
        if ml["kind"] == "dense":
            ff = ml["ff"]
            lin(p + "mlp.gate", ff, W, 1.5); lin(p + "mlp.up", ff, W); lin(p + "mlp.down", W, ff, 0.7)
            put(p + "mlp.gate.b", rnd(ff, std=0.3)); put(p + "mlp.up.b", rnd(ff, std=0.3)); put(p + "mlp.down.b", rnd(W, std=0.1))
        else:
            ff, E = ml["expert"]["ff"], ml["router"]["experts"]
            lim = ml["expert"]["limit"]
            for e in range(E):      # (gains chosen so that the clamp cuts some of the values)
                lin(p + "mlp.e%d.gate" % e, ff, W, 0.6 * lim); lin(p + "mlp.e%d.up" % e, ff, W, 0.6 * lim); lin(p + "mlp.e%d.down" % e, W, ff, 0.7 / max(1.0, lim))
            lin(p + "mlp.router", E, W, 3.0)
            put(p + "mlp.correction", rnd(E, std=0.1))
            if ml.get("shared"):
                fs, ls = ml["shared"]["ff"], ml["shared"]["limit"]
                lin(p + "mlp.shared.gate", fs, W, 0.6 * ls); lin(p + "mlp.shared.up", fs, W, 0.6 * ls); lin(p + "mlp.shared.down", W, fs, 0.7 / max(1.0, ls))
    return w


def make_weights(kind, cfg, seed=0):
    return {"qwen3": make_qwen3, "qwen3vl": make_qwen3vl, "qwen3_asr": make_qwen3_asr, "malasun": make_malasun, "gatuzen": make_gatuzen, "lupolorn": make_lupolorn, "gomerax": make_gomerax}[kind](cfg, seed)


# ----------------------------------------------------------------------------- synthetic inputs
# BASELINE.json's full-size workloads (configs 3, 2, 4); tests/golden/make_golden_full.py, tests/test_fullsize_gpu.py and
# bench.py all build their inputs from these
FULL_VL2_IMAGE = (1088, 1920)    # img_smart_resize(1080, 1920, 32, ...) -- SURVEY 8c known answer
FULL_VL2_TEXT = 512
FULL_Q06_PROMPT = 1920
FULL_ASR_SECONDS = 30.0


def synth_text_ids(n, vocab, seed, avoid=()):
    """Uniform ids in [0, vocab) avoiding the given special ids."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, size=n, dtype=np.int64)
    avoid = set(int(a) for a in avoid)
    for i in range(n):
        while int(ids[i]) in avoid:
            ids[i] = (ids[i] + 7) % vocab
    return ids.astype(np.uint32)


def synth_image(h, w, seed=1):
    """Uniform-noise uint8 HWC image (already a multiple of 32 so the reference's resize is the identity)."""
    return np.random.default_rng(seed).integers(0, 256, size=(h, w, 3), dtype=np.uint8)


def synth_audio(seconds, sr=16000, seed=2):
    """Sum of 5 sines + N(0, 0.01) noise, peak 0.9."""
    rng = np.random.default_rng(seed)
    n = int(seconds * sr)
    t = np.arange(n, dtype=np.float64) / sr
    x = sum(np.sin(2 * np.pi * f * t + ph) for f, ph in zip((220.0, 440.0, 880.0, 1760.0, 3520.0), rng.uniform(0, 6.28, 5)))
    x = x + 0.01 * rng.standard_normal(n)
    x = 0.9 * x / np.max(np.abs(x))
    return x.astype(np.float32)


def vl_prompt_ids(cfg, grid_thw, n_text, seed=3):
    """<|vision_start|> + (t*h*w/merge^2) x <|image_pad|> + <|vision_end|> per image, then n_text synthetic ids."""
    m2 = cfg["vision_config"]["spatial_merge_size"] ** 2
    special = (cfg["image_token_id"], cfg["video_token_id"], cfg["vision_start_token_id"], cfg["vision_end_token_id"])
    ids = []
    for t, h, w in np.asarray(grid_thw).tolist():
        ids += [cfg["vision_start_token_id"]] + [cfg["image_token_id"]] * (t * h * w // m2) + [cfg["vision_end_token_id"]]
    V = cfg["text_config"]["vocab_size"]
    ids += synth_text_ids(n_text, min(V, 151000), seed, avoid=special).tolist()
    return np.asarray(ids, dtype=np.uint32)


def vl_video_prompt_ids(cfg, video_grid_thw, n_stamp=3, seed=5):
    """One video the way Qwen3VLProcessor lays it out (qwen3vl/processor.rs:447-571): per temporal grid step a few timestamp text ids,
    then <|vision_start|> + (h*w/merge^2) x <|video_pad|> + <|vision_end|>."""
    m2 = cfg["vision_config"]["spatial_merge_size"] ** 2
    special = (cfg["image_token_id"], cfg["video_token_id"], cfg["vision_start_token_id"], cfg["vision_end_token_id"])
    V = cfg["text_config"]["vocab_size"]
    ids = []
    k = 0
    for t, h, w in np.asarray(video_grid_thw).tolist():
        for _ in range(t):
            ids += synth_text_ids(n_stamp, min(V, 151000), seed + k, avoid=special).tolist()
            ids += [cfg["vision_start_token_id"]] + [cfg["video_token_id"]] * (h * w // m2) + [cfg["vision_end_token_id"]]
            k += 1
    return np.asarray(ids, dtype=np.uint32)


def asr_audio_tokens(n_frames):
    """Audio tokens of `n_frames` log-mel frames: 13 per full 100-frame chunk + three stride-2 convolutions over the rest
    (get_feat_extract_output_lengths, /root/reference/src/models/qwen3_asr/processor.rs:187-195)."""
    leave = n_frames % 100
    tail = ((((leave - 1) // 2 + 1) - 1) // 2 + 1 - 1) // 2 + 1 if leave > 0 else 0
    return tail + (n_frames // 100) * 13


def asr_prompt_ids(cfg, n_audio_tokens, n_text=8, seed=4):
    tk = cfg["thinker_config"]
    special = (tk["audio_token_id"], tk["audio_start_token_id"], tk["audio_end_token_id"])
    V = tk["text_config"]["vocab_size"]
    pre = synth_text_ids(n_text // 2, min(V, 151000), seed, avoid=special).tolist()
    post = synth_text_ids(n_text - n_text // 2, min(V, 151000), seed + 1, avoid=special).tolist()
    ids = pre + [tk["audio_start_token_id"]] + [tk["audio_token_id"]] * n_audio_tokens + [tk["audio_end_token_id"]] + post
    return np.asarray(ids, dtype=np.uint32)


# ----------------------------------------------------------------------------- Gatuzen (layered engine, sandwich template)
def gatuzen_config(layers, width=64, vocab=96, eps=1e-5, groups=2, taps=3, residual_mult=0.5, embed_scale=1.0, logit_scale=1.0, loop=None):
    """config.json of a Gatuzen model.  layers: list of dicts with "type" and the mixer's sizes,
         {"type": "gla", "heads", "dim", "vdim", "tau", "rank"}          (rank: rows of the low-rank decay projection, a tensor shape only)
         {"type": "mamba2", "heads", "vdim", "state", "groups", "norm_groups", "conv"}
         {"type": "latent_attention", "heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "base", "scaling": None | dict}
       each with "moe": None | {"experts", "top", "ff"}.  loop: None | (start, stop, times)."""
    out = []
    for ly in layers:
        t = ly["type"]
        if t == "gla":
            mx = {"heads": ly["heads"], "dim": ly["dim"], "vdim": ly["vdim"], "tau": float(ly.get("tau", 16.0))}
        elif t == "mamba2":
            mx = {"heads": ly["heads"], "vdim": ly["vdim"], "state": ly["state"], "groups": ly.get("groups", 1), "norm_groups": ly.get("norm_groups", 1),
                  "conv": ly.get("conv", 4)}
        elif t == "latent_attention":
            rot = {"base": float(ly.get("base", 10000.0)), "dims": ly["rot_dim"]}
            if ly.get("scaling"):
                rot["scaling"] = dict(ly["scaling"])
            mx = {"heads": ly["heads"], "dim": ly["dim"], "rot_dim": ly["rot_dim"], "vdim": ly["vdim"], "kv_rank": ly["kv_rank"], "rot": rot,
                  "scale": float(ly.get("scale", (ly["dim"] + ly["rot_dim"]) ** -0.5))}
        else:
            raise ValueError(t)
        moe = ly.get("moe")
        out.append({"type": t, "mixer": mx, "_rank": ly.get("rank", 8),
                    "mlp": {"kind": "moe", "expert": {"ff": moe["ff"]}, "router": {"experts": moe["experts"], "top": moe["top"]}} if moe else None})
    cfg = {"architecture": "Gatuzen", "layers": out, "norm": {"eps": eps, "groups": groups}, "canon": {"taps": taps}, "residual_mult": residual_mult,
           "embedding": {"scale": embed_scale}, "logit_scale": logit_scale, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def gatuzen_shape(width, n_layers, heads, head_dim, ff, experts, top, vocab=32000, state=64, kv_rank=256, rot_dim=32, taps=4, loop=None):
    """A layer list of the sizes a served model would have: gla, mamba2 and latent-attention layers in turn, every layer with experts."""
    layers = []
    moe = {"experts": experts, "top": top, "ff": ff}
    for i in range(n_layers):
        k = i % 3
        if k == 0:
            layers.append({"type": "gla", "heads": heads, "dim": head_dim, "vdim": head_dim, "tau": 8.0, "rank": 32, "moe": moe})
        elif k == 1:
            layers.append({"type": "mamba2", "heads": heads, "vdim": head_dim, "state": state, "groups": max(1, heads // 8), "norm_groups": 2, "conv": 4, "moe": moe})
        else:
            layers.append({"type": "latent_attention", "heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank, "base": 5e5,
                           "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}, "moe": moe})
    return gatuzen_config(layers, width=width, vocab=vocab, eps=1e-6, groups=2, taps=taps, residual_mult=0.5, embed_scale=0.75, logit_scale=1.5, loop=loop)


def make_gatuzen(cfg, seed=0, fast=False):
    """Random weights under the checkpoint's tensor names: bfloat16 (`_lib.BF16`-tagged bit patterns), the expert tables as float32 integers."""
    rng = np.random.default_rng(seed)
    w = {}

    def rnd(*shape, std=1.0):
        if fast:
            a = rng.random(int(np.prod(shape)), dtype=np.float32)
            a -= np.float32(0.5)
            a *= np.float32(std * 3.4641016)
        else:
            a = rng.standard_normal(int(np.prod(shape)), dtype=np.float32) * np.float32(std)
        return a.reshape(shape)

    def put(name, a):
        w[name] = _bf16_round(a)

    def lin(name, out_f, in_f, gain=1.0):
        put(name, rnd(out_f, in_f, std=gain / np.sqrt(in_f)))

    W, V, taps = cfg["width"], cfg["vocab"], cfg.get("canon", {}).get("taps", 0)
    put("embed", rnd(V, W))
    lin("head", V, W)
    put("final.norm", 1.0 + 0.2 * rnd(W))
    if cfg.get("loop"):
        put("loop.step", rnd(cfg["loop"]["times"], W, std=0.3))
    for i, ly in enumerate(cfg["layers"]):
        p, mx, t = "l%d." % i, ly["mixer"], ly["type"]
        for nm in ("norm1", "norm1b"):
            put(p + nm, 1.0 + 0.2 * rnd(W))
        if taps:
            put(p + "canon1", rnd(W, taps, std=0.4))
        if t == "gla":
            H, D, Dv, r = mx["heads"], mx["dim"], mx["vdim"], ly.get("_rank", 8)
            lin(p + "mix.q", H * D, W); lin(p + "mix.k", H * D, W); lin(p + "mix.v", H * Dv, W); lin(p + "mix.g", H * Dv, W)
            lin(p + "mix.a1", r, W); lin(p + "mix.a2", H * D, r, 2.0)
            put(p + "mix.a2.b", 1.0 + rnd(H * D, std=1.0))
            put(p + "mix.norm", 1.0 + 0.2 * rnd(Dv))
            lin(p + "mix.o", W, H * Dv)
        elif t == "mamba2":
            H, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
            inner, Cc = H * P, H * P + 2 * G * N
            lin(p + "mix.in", 2 * inner + 2 * G * N + H, W)
            put(p + "mix.conv", rnd(Cc, mx["conv"], std=0.5)); put(p + "mix.conv.b", rnd(Cc, std=0.2))
            put(p + "mix.dt_bias", rnd(H, std=1.0)); put(p + "mix.A_log", rnd(H, std=0.7)); put(p + "mix.D", rnd(H, std=1.0))
            put(p + "mix.norm", 1.0 + 0.2 * rnd(inner))
            lin(p + "mix.o", W, inner)
        else:
            H, D, R, Dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
            lin(p + "mix.q", H * (D + R), W, 2.0); lin(p + "mix.dkv", rank + R, W, 2.0)
            put(p + "mix.dkv.norm", 1.0 + 0.2 * rnd(rank))
            lin(p + "mix.uk", H * D, rank, 2.0); lin(p + "mix.uv", H * Dv, rank)
            lin(p + "mix.g", H * Dv, W); lin(p + "mix.o", W, H * Dv)
        if ly.get("mlp"):
            ml = ly["mlp"]
            ff, E, top = ml["expert"]["ff"], ml["router"]["experts"], ml["router"]["top"]
            for nm in ("norm2", "norm2b"):
                put(p + nm, 1.0 + 0.2 * rnd(W))
            if taps:
                put(p + "canon2", rnd(W, taps, std=0.4))
            for e in range(E):
                q = p + "mlp.e%d." % e
                lin(q + "gate", ff, W); lin(q + "up", ff, W); lin(q + "down", W, ff)
            tb = np.stack([rng.permutation(E)[:top] for _ in range(V)]).astype(np.float32)
            w[p + "mlp.table"] = tb
    return w


# ----------------------------------------------------------------------------- Lupolorn (layered engine, sandwich template without groups / convolution)
def lupolorn_config(layers, width=64, vocab=96, eps=1e-5, embed_scale=1.0):
    """config.json of a Lupolorn model.  layers: list of dicts with "type" and the mixer's sizes,
         {"type": "mingru", "width"}
         {"type": "attention", "heads", "kv_heads", "dim", "vdim", "scale", "rot_dims", "base", "scaling": None | {"factor", "low", "high", "original"}}
         {"type": "latent_attention", "heads", "dim", "vdim", "kv_rank", "q_rank", "window", "scale"}
       each with "ff": None | int (dense) | {"experts", "top", "ff", "shared": None | int}."""
    out = []
    for ly in layers:
        t = ly["type"]
        if t == "mingru":
            mx = {"width": ly["width"]}
        elif t == "attention":
            rot = {"base": float(ly.get("base", 10000.0)), "dims": ly.get("rot_dims", ly["dim"])}
            if ly.get("scaling"):
                rot["scaling"] = dict(ly["scaling"])
            mx = {"heads": ly["heads"], "kv_heads": ly.get("kv_heads", ly["heads"]), "dim": ly["dim"], "vdim": ly.get("vdim", ly["dim"]), "rot": rot,
                  "scale": float(ly.get("scale", ly["dim"] ** -0.5))}
        elif t == "latent_attention":
            mx = {"heads": ly["heads"], "dim": ly["dim"], "vdim": ly["vdim"], "kv_rank": ly["kv_rank"], "q_rank": ly["q_rank"], "mask": {"size": ly["window"]},
                  "scale": float(ly.get("scale", ly["dim"] ** -0.5))}
        else:
            raise ValueError(t)
        ff = ly.get("ff")
        if ff is None:
            mlp = None
        elif isinstance(ff, dict):
            mlp = {"kind": "moe", "expert": {"ff": ff["ff"]}, "router": {"experts": ff["experts"], "top": ff["top"]}}
            if ff.get("shared"):
                mlp["shared"] = {"ff": ff["shared"]}
        else:
            mlp = {"kind": "dense", "ff": int(ff)}
        out.append({"type": t, "mixer": mx, "mlp": mlp})
    return {"architecture": "Lupolorn", "layers": out, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "vocab": vocab, "width": width}


def lupolorn_shape(width, n_layers, heads, kv_heads, head_dim, ff, experts, top, expert_ff, vocab=32000, kv_rank=256, q_rank=512, window=1024):
    """A layer list of the sizes a served model would have: attention, minGRU, latent-attention and attention layers in turn, a dense feed-forward
    on the even layers and routed experts with a shared expert on the odd ones."""
    layers = []
    for i in range(n_layers):
        k = i % 4
        f = ff if i % 2 == 0 else {"experts": experts, "top": top, "ff": expert_ff, "shared": expert_ff}
        if k == 1:
            layers.append({"type": "mingru", "width": width, "ff": f})
        elif k == 2:
            layers.append({"type": "latent_attention", "heads": heads, "dim": head_dim, "vdim": head_dim, "kv_rank": kv_rank, "q_rank": q_rank, "window": window, "ff": f})
        else:
            layers.append({"type": "attention", "heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "rot_dims": head_dim, "base": 5e5,
                           "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 8192}, "ff": f})
    return lupolorn_config(layers, width=width, vocab=vocab, eps=1e-6, embed_scale=float(np.sqrt(width)))


def make_lupolorn(cfg, seed=0, fast=False):
    """Random weights under the checkpoint's tensor names, all bfloat16 (`_lib.BF16`-tagged bit patterns)."""
    rng = np.random.default_rng(seed)
    w = {}

    def rnd(*shape, std=1.0):
        if fast:
            a = rng.random(int(np.prod(shape)), dtype=np.float32)
            a -= np.float32(0.5)
            a *= np.float32(std * 3.4641016)
        else:
            a = rng.standard_normal(int(np.prod(shape)), dtype=np.float32) * np.float32(std)
        return a.reshape(shape)

    def put(name, a):
        w[name] = _bf16_round(a)

    def lin(name, out_f, in_f, gain=1.0):
        put(name, rnd(out_f, in_f, std=gain / np.sqrt(in_f)))

    W, V = cfg["width"], cfg["vocab"]
    put("embed", rnd(V, W, std=1.0 / max(1.0, cfg["embedding"]["scale"])))
    put("final.norm", 1.0 + 0.2 * rnd(W))
    for i, ly in enumerate(cfg["layers"]):
        p, mx, t = "l%d." % i, ly["mixer"], ly["type"]
        for nm in ("norm1", "norm1b"):
            put(p + nm, 1.0 + 0.2 * rnd(W))
        if t == "mingru":
            n = mx["width"]
            lin(p + "mix.z", n, W, 2.0); lin(p + "mix.x", n, W, 2.0); lin(p + "mix.g", n, W); lin(p + "mix.o", W, n)
            put(p + "mix.z.b", rnd(n, std=1.0)); put(p + "mix.x.b", rnd(n, std=0.5))
        elif t == "attention":
            H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            lin(p + "mix.q", H * D, W, 2.0); lin(p + "mix.k", G * D, W, 2.0); lin(p + "mix.v", G * Dv, W)
            lin(p + "mix.g", H, W, 2.0); lin(p + "mix.o", W, H * Dv)
        else:
            H, D, Dv, rank, qr = mx["heads"], mx["dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            lin(p + "mix.dq", qr, W); put(p + "mix.dq.norm", 1.0 + 0.2 * rnd(qr)); lin(p + "mix.uq", H * D, qr, 2.0)
            lin(p + "mix.dkv", rank, W); put(p + "mix.dkv.norm", 1.0 + 0.2 * rnd(rank))
            lin(p + "mix.uk", H * D, rank, 2.0); lin(p + "mix.uv", H * Dv, rank); lin(p + "mix.o", W, H * Dv)
        ml = ly.get("mlp")
        if ml:
            for nm in ("norm2", "norm2b"):
                put(p + nm, 1.0 + 0.2 * rnd(W))
            if ml["kind"] == "dense":
                lin(p + "mlp.up", ml["ff"], W); lin(p + "mlp.down", W, ml["ff"])
            else:
                ff, E = ml["expert"]["ff"], ml["router"]["experts"]
                for e in range(E):
                    lin(p + "mlp.e%d.up" % e, ff, W); lin(p + "mlp.e%d.down" % e, W, ff)
                lin(p + "mlp.router", E, W, 3.0)
                if ml.get("shared"):
                    fs = ml["shared"]["ff"]
                    lin(p + "mlp.shared.up", fs, W); lin(p + "mlp.shared.down", W, fs); lin(p + "mlp.shared.sg", 1, W, 2.0)
    return w
