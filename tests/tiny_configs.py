"""The tiny Qwen3 configurations of the tests.  A and B differ in every size and
option: layers, width, heads and groups, head size (B's heads x head size is not
the width), feed-forward width, vocabulary, rope base, norm eps, tied or separate
output matrix, stored dtype of the weights.  C has larger heads and several
pages per sequence for the cache tests."""

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 128,
}
TINY_A_STORED = "float32"

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 160, "vocab_size": 512, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "eos_token_id": [7, 300],
}
TINY_B_STORED = "bfloat16"

TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 1000, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "max_position_embeddings": 2048,
}
TINY_C_STORED = "bfloat16"

# the head size of the large models (128: the tcgen05 prefill and the streaming decode attention), three query
# heads per kv head, a width that is no multiple of 64
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 168, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 328, "vocab_size": 777, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 2048,
}
TINY_D_STORED = "bfloat16"

ALL = {"A": (TINY_A, TINY_A_STORED), "B": (TINY_B, TINY_B_STORED), "C": (TINY_C, TINY_C_STORED),
       "D": (TINY_D, TINY_D_STORED)}
