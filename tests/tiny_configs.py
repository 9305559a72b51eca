"""Tiny configurations of the architecture for the tests.  They differ in every
size and option: layers, width, head counts and groups, head size, feed-forward
width, vocabulary (a power of two, not a multiple of 64, odd), rotary base and
pairing, eps, bias, tied or untied head, and the page size they are run with."""

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 512, "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 512,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "use_sliding_window": False, "hidden_act": "silu",
}
TINY_A_PAGE = 16

TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 1000, "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "max_position_embeddings": 640,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "use_sliding_window": False, "hidden_act": "silu",
}
TINY_B_PAGE = 8

# head size given in the file and not hidden / heads; five query heads per group;
# no bias; half-split rotary pairs; odd vocabulary
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 777, "hidden_size": 80, "intermediate_size": 112, "num_hidden_layers": 1,
    "num_attention_heads": 10, "num_key_value_heads": 2, "head_dim": 48, "max_position_embeddings": 384,
    "rope_theta": 50000.0, "rms_norm_eps": 1e-3, "tie_word_embeddings": False, "attention_bias": False,
    "rope_pairing": "half", "use_sliding_window": False, "hidden_act": "silu",
}
TINY_C_PAGE = 32

# head sizes 64 and 128: the tensor-core attention kernels run in bfloat16
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 320, "hidden_size": 112, "intermediate_size": 96, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "max_position_embeddings": 512,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
}
TINY_D_PAGE = 16

TINY_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 411, "hidden_size": 72, "intermediate_size": 200, "num_hidden_layers": 1,
    "num_attention_heads": 7, "num_key_value_heads": 1, "head_dim": 128, "max_position_embeddings": 512,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "rope_pairing": "half",
}
TINY_E_PAGE = 8

ALL = {"A": (TINY_A, TINY_A_PAGE, 0), "B": (TINY_B, TINY_B_PAGE, 1), "C": (TINY_C, TINY_C_PAGE, 2),
       "D": (TINY_D, TINY_D_PAGE, 3), "E": (TINY_E, TINY_E_PAGE, 4)}

# Not one of the five above (the suites that run over ALL would take too long on it): a long context limit, five
# query heads on one key/value head of 128 (the grouping of the Qwen2.5-14B shape), for the long-context replay.
TINY_LONG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 300, "hidden_size": 48, "intermediate_size": 80, "num_hidden_layers": 1,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 128, "max_position_embeddings": 8192,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
EXTRA = {"L": (TINY_LONG, 16, 6), "L2": (dict(TINY_LONG, max_position_embeddings=8448), 16, 6)}
