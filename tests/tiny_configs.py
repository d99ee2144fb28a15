"""Small configurations of the architecture for the tests.  They differ from one another in every
size and option: head counts and groups, head size, rotary share, theta, q/k norm on and off, experts
and top-k, expert width, vocabulary (one is prime), eps, tied head, and the spread of the weights."""
import json
import os

import torch

from fieldrun_b200 import RandomInit

ARCH = "MiniMaxM2ForCausalLM"

CONFIG_A = dict(
    architectures=[ARCH], model_type="minimax_m2", num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, rotary_dim=8, rope_theta=10000.0, use_qk_norm=True, num_local_experts=4,
    num_experts_per_tok=2, intermediate_size=32, vocab_size=256, rms_norm_eps=1e-6, tie_word_embeddings=False,
    eos_token_id=255)
INIT_A = RandomInit(seed=0, matrix_std=0.02, norm_std=0.1, bias_std=0.0)

CONFIG_B = dict(
    architectures=[ARCH], model_type="minimax_m2", num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
    num_key_value_heads=2, head_dim=32, rotary_dim=32, rope_theta=1000000.0, use_qk_norm=False, num_local_experts=8,
    num_experts_per_tok=3, intermediate_size=48, vocab_size=389, rms_norm_eps=1e-5, tie_word_embeddings=False,
    eos_token_id=[7, 11])
INIT_B = RandomInit(seed=1, matrix_std=0.03, norm_std=0.05, bias_std=0.1)

# a head size that is no multiple of 16, a group of 4, a tied head, no eos
CONFIG_C = dict(
    architectures=[ARCH], model_type="minimax_m2", num_hidden_layers=1, hidden_size=40, num_attention_heads=8,
    num_key_value_heads=2, head_dim=12, partial_rotary_factor=0.5, rope_theta=500.0, use_qk_norm=True,
    num_experts=5, num_experts_per_tok=1, intermediate_size=24, vocab_size=131, rms_norm_eps=1e-4,
    tie_word_embeddings=True)
INIT_C = RandomInit(seed=2, matrix_std=0.05, norm_std=0.2, bias_std=0.05, stored_dtype=torch.float32)

# sizes that the tcgen05 kernels take (widths in steps of 128, head size 64), so that prompts of a few dozen
# tokens run on them inside the engine
CONFIG_D = dict(
    architectures=[ARCH], model_type="minimax_m2", num_hidden_layers=2, hidden_size=128, num_attention_heads=4,
    num_key_value_heads=2, head_dim=64, rotary_dim=32, rope_theta=50000.0, use_qk_norm=True, num_local_experts=4,
    num_experts_per_tok=2, intermediate_size=128, vocab_size=300, rms_norm_eps=1e-6, tie_word_embeddings=False)
INIT_D = RandomInit(seed=3, matrix_std=0.04, norm_std=0.1, bias_std=0.05)

# the tiny model of the reference's own gate (scripts/gemma3_ref.py:61-77: vocab 64, hidden 32, 3 layers, 4 heads
# over 2, head size 8, 8 experts, 2 per token, width 16), its config.json in the form the architecture's writer
# emits (theta and the rotary share under rope_parameters, a stop token outside the vocabulary), and the gate's
# recipe for the weights: norm weights N(0, 0.1) around ZERO and a routing bias N(0, 0.2) (:223-247)
with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures", "written_config_tiny.json")) as _handle:
    CONFIG_E = json.load(_handle)
INIT_E = RandomInit(seed=4, matrix_std=0.02, norm_std=0.1, norm_mean=0.0, bias_std=0.2, stored_dtype=torch.float32)
# folders of these configurations keep the config.json as it is written here, key for key
WRITTEN_AS_IS = {"e": CONFIG_E}

ALL = {"e": (CONFIG_E, INIT_E), "a": (CONFIG_A, INIT_A), "b": (CONFIG_B, INIT_B), "c": (CONFIG_C, INIT_C), "d": (CONFIG_D, INIT_D)}
