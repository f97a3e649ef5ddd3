"""Known shapes of the Qwen2 dense decoder, for the random-weights mode (``cima random``).
Every entry is a complete config.json; nothing here is read by the model code."""


def _qwen2(layers, hidden, heads, kv_heads, head_dim, inter, vocab, theta, eps, tied, max_pos):
    return dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], num_hidden_layers=layers, hidden_size=hidden,
                num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
                vocab_size=vocab, rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=tied,
                use_sliding_window=False, max_position_embeddings=max_pos, hidden_act="silu")


SHAPES = {
    "tiny-a": _qwen2(2, 128, 4, 2, 32, 256, 512, 10000.0, 1e-6, True, 128),
    "tiny-b": _qwen2(3, 192, 3, 1, 64, 448, 1000, 1000000.0, 1e-5, False, 256),
    "qwen2.5-0.5b": _qwen2(24, 896, 14, 2, 64, 4864, 151936, 1000000.0, 1e-6, True, 32768),
    "qwen2.5-1.5b": _qwen2(28, 1536, 12, 2, 128, 8960, 151936, 1000000.0, 1e-6, True, 32768),
    "qwen2.5-3b": _qwen2(36, 2048, 16, 2, 128, 11008, 151936, 1000000.0, 1e-6, True, 32768),
    "qwen2.5-7b": _qwen2(28, 3584, 28, 4, 128, 18944, 152064, 1000000.0, 1e-6, False, 32768),
    "qwen2.5-14b": _qwen2(48, 5120, 40, 8, 128, 13824, 152064, 1000000.0, 1e-6, False, 32768),
    "qwen2.5-32b": _qwen2(64, 5120, 40, 8, 128, 27648, 152064, 1000000.0, 1e-6, False, 32768),
}
