"""Two tiny Llama configurations that differ in every size and option, and a third that is
the shape of the reference's own test fixture (tests/conftest.py:15-37 there)."""

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 192, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 256, "eos_token_id": 1, "bos_token_id": 0,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 320, "vocab_size": 512,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 512,
    "eos_token_id": [2, 3],
}

TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 5,
    "num_key_value_heads": 5, "head_dim": 48, "intermediate_size": 112, "vocab_size": 331,
    "rope_theta": 250000.0,
    "rope_scaling": {"type": "llama3", "factor": 4.0, "low_freq_factor": 2.0,
                     "high_freq_factor": 6.0, "original_max_position_embeddings": 32},
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "max_position_embeddings": 384,
}

# A fourth that takes the ways around the fast paths: head size 80 (no tcgen05 attention), a width
# and a feed-forward size that are no multiples of 16 (the gate and up rows cannot alternate in
# blocks, the few-row product's inner dimension is no multiple of 64), pages of 32 tokens.
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 80, "intermediate_size": 200, "vocab_size": 1000,
    "rope_theta": 1000000.0, "rms_norm_eps": 2e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 320,
}

PAGE_SIZE = {"A": 16, "B": 8, "C": 4, "D": 32}
