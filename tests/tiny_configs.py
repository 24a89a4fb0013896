"""Tiny Gemma 2 configurations for the tests.  A and B differ in every size and option;
C switches the options off (no window, no soft-caps) and has sizes that are no power of two;
D has a head size of 64, the smallest the tensor-memory prefill attention and the decode kernel's
fixed-size form take, so that those run inside a whole model."""
import copy

TINY_A = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0, "sliding_window": 8, "query_pre_attn_scalar": 16,
    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "max_position_embeddings": 512,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True,
    "bos_token_id": 2, "eos_token_id": 1,
}

TINY_B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 160, "vocab_size": 384, "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0, "sliding_window": 16, "query_pre_attn_scalar": 24,
    "attn_logit_softcapping": 20.0, "final_logit_softcapping": 15.0, "max_position_embeddings": 1024,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True,
    "bos_token_id": 0, "eos_token_id": [5, 7],
}

TINY_C = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 1, "hidden_size": 80, "num_attention_heads": 3, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 112, "vocab_size": 131, "rms_norm_eps": 1e-4,
    "rope_theta": 500.0, "sliding_window": None, "query_pre_attn_scalar": 100,
    "attn_logit_softcapping": None, "final_logit_softcapping": None, "max_position_embeddings": 256,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True,
    "eos_token_id": 3,
}

TINY_D = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 136, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 200, "vocab_size": 301, "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0, "sliding_window": 100, "query_pre_attn_scalar": 50,
    "attn_logit_softcapping": 30.0, "final_logit_softcapping": 20.0, "max_position_embeddings": 1024,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True,
    "bos_token_id": 2, "eos_token_id": 1,
}

# awkward sizes: a head size that is no multiple of 16 (the fast attention kernels do not take it), widths
# that are no multiple of 8 (the tensor-core products do not take them), a window shorter than a page row
TINY_E = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 50, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 24, "intermediate_size": 70, "vocab_size": 97, "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0, "sliding_window": 5, "query_pre_attn_scalar": 24,
    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "max_position_embeddings": 256,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": False,
    "bos_token_id": 2, "eos_token_id": 1,
}

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4)}


def config(name):
    cfg, seed = CONFIGS[name]
    return copy.deepcopy(cfg), seed
