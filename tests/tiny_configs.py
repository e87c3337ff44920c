"""Small configurations of the architecture for the tests.  They differ in every
size and option: layer count, width, heads and groups (GQA 2:1, MQA, MHA), head
size (16, 32, 48 = not H/heads), feed-forward width and vocabulary that are no
power of two, theta, rope scaling on/off, eps, tied or untied head, window, page
size, and how the norm weights are drawn."""
import copy

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "intermediate_size": 192, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 128, "hidden_act": "silu", "eos_token_id": 2, "bos_token_id": 1,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 352, "vocab_size": 320,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256,
    "hidden_act": "silu", "eos_token_id": [3, 7],
}
# head_dim 48 is not hidden/heads; odd vocabulary; full MHA; every other layer has a window
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 4, "hidden_size": 120, "num_attention_heads": 5,
    "num_key_value_heads": 5, "head_dim": 48, "intermediate_size": 200, "vocab_size": 301,
    "rope_theta": 25000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 512, "hidden_act": "silu",
    "sliding_window": 24,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
}

# head size 64 and 128 in turn take the tensor-core attention kernels of the bfloat16 mode;
# widths that are multiples of 8 take the weight-streaming and tcgen05 products
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 328, "vocab_size": 500,
    "rope_theta": 100000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 1024, "hidden_act": "silu",
    "rope_scaling": {"rope_type": "linear", "factor": 2.0},
}
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 264, "vocab_size": 384,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 1024, "hidden_act": "silu", "sliding_window": 80,
    "layer_types": ["full_attention", "sliding_attention"],
}

# name -> (config, page size, std of matrices, jitter of norm weights)
TINY = {
    "tiny_a": (TINY_A, 16, 0.12, 0.0),
    "tiny_b": (TINY_B, 8, 0.09, 0.1),
    "tiny_c": (TINY_C, 32, 0.10, 0.05),
    "tiny_d": (TINY_D, 16, 0.07, 0.05),
    "tiny_e": (TINY_E, 16, 0.06, 0.0),
}


def get(name):
    cfg, page, std, jitter = TINY[name]
    return copy.deepcopy(cfg), page, std, jitter
