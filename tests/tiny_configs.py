"""Tiny configurations of the dense Qwen3 decoder for tests.  They differ in every size and
option: layers, width, heads and groups, head size, feed-forward width, vocabulary, rotary
base, norm eps, context, tied or separate head, and (C) windows per layer, a rotated width
below the head size and an explicit attention scale.  Several sizes are no powers of two."""

# "D" is not tiny in its head size: 128, the size the tensor-memory (tcgen05) attention and product
# kernels serve, so that those kernels are also compared with the plain implementation inside a
# whole model and in every way of cutting the work.
TINY = {
    "D": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1000, hidden_size=512,
              num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
              intermediate_size=1536, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=1024,
              tie_word_embeddings=False, eos_token_id=999),
    "A": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=128, rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=128,
              tie_word_embeddings=True, eos_token_id=255),
    "B": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=384, hidden_size=96,
              num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=32,
              intermediate_size=224, rope_theta=1000000.0, rms_norm_eps=1e-5, max_position_embeddings=256,
              tie_word_embeddings=False, eos_token_id=[380, 381]),
    "C": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=300, hidden_size=80,
              num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
              intermediate_size=172, rope_theta=500000.0, rms_norm_eps=3e-6, max_position_embeddings=512,
              tie_word_embeddings=False, eos_token_id=7, partial_rotary_factor=0.5,
              query_pre_attn_scalar=32.0, use_sliding_window=True, sliding_window=40,
              layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"]),
}
