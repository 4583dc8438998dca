"""Known shapes of the Qwen2 dense decoder, for the random-weights mode (``cima random``), and shapes of the
Vunovik decoder at the same widths, heads, feed-forward sizes and vocabularies (no trained model of that design
exists; they serve measurements beside the Qwen2 shape of equal size), and shapes of the Gisirax decoder at those
widths: two delta-rule layers, then one layer of softmax attention beside a decay recurrence, every layer with routed
experts of which a token uses as many values of a feed-forward's middle as the Qwen2 shape has, and shapes of the
Lipizen decoder at those widths: of every four layers one runs the gate recurrence and three differential attention (the
last of them on the keys and values of the one before it), every layer with the dense feed-forward of the Qwen2 shape.
And shapes of the Netezen decoder at those widths: two copies of the stream; layers alternate between latent attention
(a position keeps 96 + 32 values) and grouped-query attention with the Qwen2 shape's heads behind a window that keeps first
positions; the first layer's feed-forward is the ungated one, the others route 3 of 16 clamped experts beside a shared
one, a token using as many values of a middle as the Qwen2 shape has.
Every entry is a complete config.json; nothing here is read by the model code."""


def _qwen2(layers, hidden, heads, kv_heads, head_dim, inter, vocab, theta, eps, tied, max_pos):
    return dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=layers, hidden_size=hidden,
                num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
                vocab_size=vocab, rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=tied,
                use_sliding_window=False, max_position_embeddings=max_pos, hidden_act="silu")


def _vunovik(layers, width, heads, dim, rank, ff, vocab, taps=4):
    """Every second layer makes latents, the one after it reads them; keys and values of ``dim`` per head."""
    out = []
    for i in range(layers):
        mixer = {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": rank, "scale": dim ** -0.5}
        if i % 2:
            mixer["kv_from"] = i - 1
        out.append({"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Vunovik", "vocab": vocab, "width": width, "canon": {"taps": taps},
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "layers": out}


def _gisirax(layers, width, heads, kv_heads, dim, ff, vocab, experts=16, top=4, groups=4, keep=2, taps=4, rank=64):
    """Layers 0, 1 of every three run the gated delta rule, layer 2 the two attentions side by side; ``top`` experts of
    ``ff / top`` values each stand for the dense feed-forward of ``ff`` values."""
    per = -(-ff // top // 64) * 64
    mlp = {"kind": "moe", "expert": {"ff": per}, "router": {"experts": experts, "top": top, "scale": 1.0,
                                                             "groups": {"count": groups, "keep": keep}}}
    out = []
    for i in range(layers):
        if i % 3 == 2:
            left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                    "rot": {"dims": dim, "base": 1000000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
            right = {"heads": heads, "dim": dim, "vdim": dim, "decay": [1.0 - 2.0 ** (-5.0 - 5.0 * h / max(1, heads - 1)) for h in range(heads)]}
            out.append({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp})
        else:
            out.append({"type": "channel_delta", "mlp": mlp,
                        "mixer": {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "conv": taps, "a_rank": rank, "g_rank": rank}})
    return {"architecture": "Gisirax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
            "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 8191, "mul_cur": 127}}, "layers": out}


def _lipizen(layers, width, heads, kv_heads, dim, ff, vocab, taps=4, window=1024, keep_first=64, groups=2):
    """Layers 0 and 2 of every four run differential attention with keys of their own, layer 1 the gate recurrence, layer 3
    differential attention on layer 2's keys and values.  A head has two maps of ``dim / 2`` and values of ``dim``, so the
    projections have the Qwen2 shape's sizes."""
    out = []
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    for i in range(layers):
        if i % 4 == 1:
            out.append({"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": dim}, "mlp": mlp})
            continue
        mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim // 2, "vdim": dim, "scale": (dim // 2) ** -0.5, "diff": 0.8,
                 "conv": taps, "rot": {"dims": dim // 2, "base": 1000000.0, "scaling": {"factor": 4.0}},
                 "mask": {"size": window, "keep_first": keep_first}}
        if i % 4 == 3:
            mixer["kv_from"] = i - 1
        out.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Lipizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": groups}, "postln_alpha": 1.0,
            "logit_softcap": 30.0, "layers": out}


def _netezen(layers, width, heads, kv_heads, dim, ff, vocab, experts=16, top=3, window=1024, keep_first=64, rank=96, rot=32, streams=2):
    """Even layers: latent attention with ``heads`` heads of ``dim - rot`` plain and ``rot`` rotated values; odd layers:
    grouped-query attention.  ``top`` routed experts and the shared one have ``ff / (top + 1)`` values each."""
    per = -(-ff // (top + 1) // 64) * 64
    moe = {"kind": "moe", "expert": {"ff": per, "limit": 7.0}, "router": {"experts": experts, "top": top}, "shared": {"ff": per, "limit": 7.0}}
    out = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": -(-(3 * ff // 2) // 64) * 64} if i == 0 else moe
        if i % 2 == 0:
            mixer = {"heads": heads, "dim": dim - rot, "rot_dim": rot, "vdim": dim, "kv_rank": rank, "q_rank": max(64, width // 4 // 64 * 64),
                     "scale": dim ** -0.5, "rot": {"dims": rot, "base": 10000.0}, "mask": {"size": window}}
            out.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
        else:
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                     "rot": {"dims": dim // 2, "base": 1000000.0, "scaling": {"factor": 4.0, "original": 8192, "fast": 32.0, "slow": 1.0}},
                     "mask": {"size": window, "keep_first": keep_first}}
            out.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Netezen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "streams": streams,
            "layers": out}


# the Qwen2 shape that a Vunovik, Gisirax, Lipizen or Netezen shape is measured beside
TWINS = {"netezen-0.5b": "qwen2.5-0.5b", "netezen-1.5b": "qwen2.5-1.5b", "netezen-3b": "qwen2.5-3b", "netezen-7b": "qwen2.5-7b",
         "lipizen-0.5b": "qwen2.5-0.5b", "lipizen-1.5b": "qwen2.5-1.5b", "lipizen-3b": "qwen2.5-3b", "lipizen-7b": "qwen2.5-7b",
         "gisirax-0.5b": "qwen2.5-0.5b", "gisirax-1.5b": "qwen2.5-1.5b", "gisirax-3b": "qwen2.5-3b", "gisirax-7b": "qwen2.5-7b",
         "vunovik-0.5b": "qwen2.5-0.5b", "vunovik-1.5b": "qwen2.5-1.5b", "vunovik-3b": "qwen2.5-3b", "vunovik-7b": "qwen2.5-7b"}

SHAPES = {
    "netezen-tiny": _netezen(4, 128, 4, 2, 32, 256, 512, experts=6, top=2, window=96, keep_first=4, rank=48, rot=16),
    "netezen-0.5b": _netezen(24, 896, 14, 2, 64, 4864, 151936, rank=96, rot=32),
    "netezen-1.5b": _netezen(28, 1536, 12, 2, 128, 8960, 151936),
    "netezen-3b": _netezen(36, 2048, 16, 2, 128, 11008, 151936),
    "netezen-7b": _netezen(28, 3584, 28, 4, 128, 18944, 152064),
    "lipizen-tiny": _lipizen(4, 128, 4, 2, 32, 256, 512, taps=3, window=96, keep_first=4),
    "lipizen-0.5b": _lipizen(24, 896, 14, 2, 64, 4864, 151936),
    "lipizen-1.5b": _lipizen(28, 1536, 12, 2, 128, 8960, 151936),
    "lipizen-3b": _lipizen(36, 2048, 16, 2, 128, 11008, 151936),
    "lipizen-7b": _lipizen(28, 3584, 28, 4, 128, 18944, 152064),
    "gisirax-tiny": _gisirax(3, 128, 4, 2, 32, 256, 512, experts=8, top=2, groups=2, keep=1, taps=3, rank=16),
    "gisirax-0.5b": _gisirax(24, 896, 14, 2, 64, 4864, 151936),
    "gisirax-1.5b": _gisirax(28, 1536, 12, 2, 128, 8960, 151936),
    "gisirax-3b": _gisirax(36, 2048, 16, 2, 128, 11008, 151936),
    "gisirax-7b": _gisirax(28, 3584, 28, 4, 128, 18944, 152064),
    "vunovik-tiny": _vunovik(3, 128, 4, 32, 64, 256, 512, taps=3),
    "vunovik-0.5b": _vunovik(24, 896, 14, 64, 64, 4864, 151936),
    "vunovik-1.5b": _vunovik(28, 1536, 12, 128, 128, 8960, 151936),
    "vunovik-3b": _vunovik(36, 2048, 16, 128, 128, 11008, 151936),
    "vunovik-7b": _vunovik(28, 3584, 28, 128, 128, 18944, 152064),
    "tiny-a": _qwen2(2, 128, 4, 2, 32, 256, 512, 10000.0, 1e-6, True, 128),
    "tiny-b": _qwen2(3, 192, 3, 1, 64, 448, 1000, 1000000.0, 1e-5, False, 256),
    "qwen2.5-0.5b": _qwen2(24, 896, 14, 2, 64, 4864, 151936, 1000000.0, 1e-6, True, 32768),
    "qwen2.5-1.5b": _qwen2(28, 1536, 12, 2, 128, 8960, 151936, 1000000.0, 1e-6, True, 32768),
    "qwen2.5-3b": _qwen2(36, 2048, 16, 2, 128, 11008, 151936, 1000000.0, 1e-6, True, 32768),
    "qwen2.5-7b": _qwen2(28, 3584, 28, 4, 128, 18944, 152064, 1000000.0, 1e-6, False, 32768),
    "qwen2.5-14b": _qwen2(48, 5120, 40, 8, 128, 13824, 152064, 1000000.0, 1e-6, False, 32768),
    "qwen2.5-32b": _qwen2(64, 5120, 40, 8, 128, 27648, 152064, 1000000.0, 1e-6, False, 32768),
}
