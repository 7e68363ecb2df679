"""Known shapes of the Qwen2 dense decoder, for the random-weights mode (``cima random``), and shapes of the
Vunovik decoder at the same widths, heads, feed-forward sizes and vocabularies (no trained model of that design
exists; they serve measurements beside the Qwen2 shape of equal size).
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


# the Qwen2 shape that a Vunovik shape is measured beside
TWINS = {"vunovik-0.5b": "qwen2.5-0.5b", "vunovik-1.5b": "qwen2.5-1.5b", "vunovik-3b": "qwen2.5-3b", "vunovik-7b": "qwen2.5-7b"}

SHAPES = {
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
