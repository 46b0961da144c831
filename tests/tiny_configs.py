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

# Further odd sizes, each through the whole engine (tests/test_replay_gpu.py::test_odd_sizes):
#  E: a width that is no multiple of 8 (the bfloat16 weight-streaming linear does not take it: the library product
#     stands in), as many kv heads as heads, head size 80, an odd vocabulary, tied output matrix
#  F: 20 query heads on one kv head (more than the 16 rows of one pass of the decode attention), head size 16
#  G: head size 256 (the largest of the tensor-core attention kernels), a feed-forward width that is no multiple of 8
#     (gate and up rows are then not interleaved)
#  H: head size 24 (no multiple of 16: the attention of the float32 path serves bfloat16 too), rope base 500
def _odd(layers, hidden, heads, kv, head_dim, inter, vocab, theta, eps, tied):
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
            "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": head_dim,
            "intermediate_size": inter, "vocab_size": vocab, "rope_theta": theta, "rms_norm_eps": eps,
            "tie_word_embeddings": tied, "max_position_embeddings": 512}


ODD = {
    "E": (_odd(2, 100, 5, 5, 80, 136, 1001, 10000.0, 1e-6, True), "bfloat16"),
    "F": (_odd(2, 64, 20, 1, 16, 96, 300, 1000000.0, 1e-5, False), "float32"),
    "G": (_odd(1, 72, 2, 1, 256, 100, 513, 50000.0, 1e-6, False), "bfloat16"),
    "H": (_odd(2, 88, 4, 2, 24, 120, 777, 500.0, 2e-6, True), "bfloat16"),
}
