"""Two tiny Llama configurations that differ in every size and option, and helpers to make their
model folders with random weights in a temporary place."""

from __future__ import annotations

import os

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "max_position_embeddings": 128, "tie_word_embeddings": True, "bos_token_id": 1,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 384,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "max_position_embeddings": 256, "tie_word_embeddings": False,
}

# A third one with sizes that are no power of two anywhere (width 80, vocabulary 301, 5 heads in
# a group of 5 over one key/value head pair, head size 48).
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 80, "intermediate_size": 176, "num_hidden_layers": 2,
    "num_attention_heads": 10, "num_key_value_heads": 2, "head_dim": 48, "vocab_size": 301,
    "rms_norm_eps": 3e-6, "rope_theta": 25000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
    "max_position_embeddings": 512, "tie_word_embeddings": True,
}

# Head size 64 with query heads in pairs, widths that are multiples of 128: in bfloat16 this one runs
# the kernels that the large models run (tcgen05 prefill attention, tensor-core decode attention with
# keys by bulk tensor copies and its own rotation, the tcgen05 gate|up product with the gating in its
# epilogue, the streaming products with the norms in their epilogues, decode steps from graphs).
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 256, "intermediate_size": 384, "num_hidden_layers": 2,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 1000,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "max_position_embeddings": 1024, "tie_word_embeddings": True,
}

# Head size 128 in groups of three (the mma.sync flash kernel and the 128-wide decode kernel).
TINY_E = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 320, "intermediate_size": 448, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 777,
    "rms_norm_eps": 2e-6, "rope_theta": 100000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 96},
    "max_position_embeddings": 1024, "tie_word_embeddings": False,
}

# The layer sizes of Llama 3.2 1B with two layers (the sizes the benchmark runs at).
ONE_B_2L = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True,
}

# The layer sizes of Llama 3.2 3B with two layers: heads of 128 in groups of three.
THREE_B_2L = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 3072, "intermediate_size": 8192, "num_hidden_layers": 2,
    "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True,
}

SEEDS = {"A": 0, "B": 2, "C": 7, "D": 11, "E": 13, "1B2L": 4, "3B2L": 5}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "1B2L": ONE_B_2L, "3B2L": THREE_B_2L}


def make_model_dir(tmp_root: str, which: str, store_dtype: str = "bfloat16") -> str:
    from rust_llm_inference_server_b200.weights import write_random_model
    out = os.path.join(tmp_root, f"tiny_{which}_{store_dtype}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_random_model(CONFIGS[which], out, SEEDS[which], store_dtype)
    return out


def load_plain_weights(model_dir: str) -> dict:
    """Reads the folder with the `safetensors` package (not with the engine's reader)."""
    from safetensors.torch import load_file
    import torch
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: v.to(torch.float32) for k, v in w.items()}
