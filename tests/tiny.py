"""The two tiny Qwen3 configurations of the tests.  They differ in every size and option: layers,
hidden size (96 is no power of two), heads and group size, head_dim (heads * head_dim == hidden in
A, != in B), intermediate size, vocabulary (1000 is no power of two), rope_theta, the norms' eps,
tied or untied head, attention bias, sliding window (A: none; B: layers 1 and 2 see 40 keys), and
the cache page size they are run with."""

import copy

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 128,
    "vocab_size": 512,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "max_position_embeddings": 256,
    "tie_word_embeddings": True,
    "hidden_act": "silu",
    "attention_bias": False,
    "use_sliding_window": False,
    "eos_token_id": 3,
}
PAGE_A = 16

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "intermediate_size": 160,
    "vocab_size": 1000,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5,
    "max_position_embeddings": 512,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": True,
    "use_sliding_window": True,
    "sliding_window": 40,
    "max_window_layers": 1,
    "eos_token_id": [7, 9],
}
PAGE_B = 32

# A third, small configuration with the head shape of the benchmark model (head_dim 128, groups of four q-heads,
# an intermediate size that is a multiple of 64): the sizes at which the tcgen05 attention kernel and the fused
# epilogues of the decode GEMM run.  Layer 1 sees a window of 48 keys.
SMALL_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 512,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 128,
    "intermediate_size": 1152,
    "vocab_size": 1536,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "max_position_embeddings": 1024,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": False,
    "use_sliding_window": True,
    "sliding_window": 48,
    "max_window_layers": 1,
    "eos_token_id": 2,
}
PAGE_C = 16

CONFIGS = {"A": (TINY_A, PAGE_A), "B": (TINY_B, PAGE_B), "C": (SMALL_C, PAGE_C)}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name][0])
