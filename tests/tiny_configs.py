"""The tiny configurations the tests run on: they differ in every size and option.

tiny-A and tiny-B are the two that the build's baseline names; tiny-C adds what
they leave out: biases, a head size of 48 (a multiple of 16 that is no power of
two), a group of one (as many KV heads as heads), linear rope scaling and the
tanh GELU.
"""

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 512, "hidden_size": 64, "intermediate_size": 176,
    "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": True, "max_position_embeddings": 256,
    "hidden_act": "silu",
}
TINY_A_SEED, TINY_A_PAGE = 0, 16

TINY_B = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 1000, "hidden_size": 96, "intermediate_size": 320,
    "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 16,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "tie_word_embeddings": False, "max_position_embeddings": 512, "hidden_act": "silu",
}
TINY_B_SEED, TINY_B_PAGE = 1, 8

TINY_C = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 777, "hidden_size": 120, "intermediate_size": 112,
    "num_hidden_layers": 1, "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 48,
    "rms_norm_eps": 1e-4, "rope_theta": 1000.0, "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "tie_word_embeddings": False, "max_position_embeddings": 512, "hidden_act": "gelu_pytorch_tanh",
    "attention_bias": True, "mlp_bias": True,
}
TINY_C_SEED, TINY_C_PAGE = 2, 4

# Head size 64 and groups of two: what the tensor-core attention kernel takes, at toy width.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 300, "hidden_size": 128, "intermediate_size": 96,
    "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128},
    "tie_word_embeddings": True, "max_position_embeddings": 1024, "hidden_act": "silu",
}
TINY_D_SEED, TINY_D_PAGE = 3, 16

# Head size 128 in groups of three (the 3B shape's grouping), projections wider than the model (6 x 128 = 768
# against 384), untied head: the <128> instantiations of the tensor-core, TMA and tcgen05 attention kernels.
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 411, "hidden_size": 384, "intermediate_size": 272,
    "num_hidden_layers": 2, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128,
    "rms_norm_eps": 3e-6, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
    "tie_word_embeddings": False, "max_position_embeddings": 2048, "hidden_act": "silu",
}
TINY_E_SEED, TINY_E_PAGE = 5, 16

ALL = {"tiny_a": (TINY_A, TINY_A_SEED, TINY_A_PAGE), "tiny_b": (TINY_B, TINY_B_SEED, TINY_B_PAGE),
       "tiny_c": (TINY_C, TINY_C_SEED, TINY_C_PAGE), "tiny_d": (TINY_D, TINY_D_SEED, TINY_D_PAGE),
       "tiny_e": (TINY_E, TINY_E_SEED, TINY_E_PAGE)}


def prompt(vocab: int, length: int, seed: int) -> list[int]:
    """`length` uniform token ids, the same on every machine."""
    import torch

    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()
