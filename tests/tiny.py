"""The tiny configurations the tests build models from.  They differ in every size and
option: head counts and grouping, head size, sizes that are no power of two, number of
layers, vocabulary, the norms' eps, rotary base and scaling, tied or untied head, window,
storage type."""
import json
import os

TINY_A = {   # float32 storage, untied, multi-head, ragged feed-forward width
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 4, "head_dim": 16, "intermediate_size": 172, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 128, "tie_word_embeddings": False,
    "torch_dtype": "float32", "eos_token_id": 7,
}
TINY_B = {   # bfloat16 storage, tied, grouped 3:1, llama3 scaling
    "architectures": ["LlamaForCausalLM"], "hidden_size": 192, "num_hidden_layers": 3, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 512, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "tie_word_embeddings": True, "torch_dtype": "bfloat16",
    "eos_token_id": [3, 5],
}
TINY_C = {   # head size 48 (a step of 16, no power of two), hidden != heads*head_dim, window, linear scaling, 5:1
    "architectures": ["LlamaForCausalLM"], "hidden_size": 200, "num_hidden_layers": 2, "num_attention_heads": 5,
    "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 328, "vocab_size": 301, "rope_theta": 25000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 2.0}, "rms_norm_eps": 3e-6, "max_position_embeddings": 512,
    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "sliding_window": 40, "use_sliding_window": True,
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def make_model_dir(tmp_path, cfg, seed=1, dtype=None):
    from ithaca_b200.weights import write_random_model
    d = os.path.join(str(tmp_path), f"model_{abs(hash(json.dumps(cfg, sort_keys=True))) % 10**8}_{seed}_{dtype}")
    if not os.path.isdir(d):
        write_random_model(d, cfg, seed, dtype)
    return d
