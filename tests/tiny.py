"""The tiny configurations that the tests use, and helpers to make their model folders.

A and B are the two tiny shapes of the benchmark description (they differ in
every size: layers, width, heads, groups, head size, intermediate size,
vocabulary, theta, eps, tied or untied head).  C adds what neither has: a
sliding window on the upper layers, an explicit head_dim that is not
hidden/heads, and sizes that are no power of two.  D has head size 128 and is
run with sequences of a few hundred tokens.
"""

from __future__ import annotations

import os

import torch

from somi_inference_b200.config import Qwen2Config
from somi_inference_b200.weights import write_random_model

TINY_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
              hidden_size=64, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=128, use_sliding_window=False, hidden_act="silu")
TINY_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3,
              hidden_size=192, num_attention_heads=3, num_key_value_heads=1, intermediate_size=320,
              vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=256, use_sliding_window=False, hidden_act="silu")
TINY_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=4,
              hidden_size=80, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
              intermediate_size=176, vocab_size=517, rope_theta=50000.0, rms_norm_eps=3e-6,
              tie_word_embeddings=False, max_position_embeddings=320, use_sliding_window=True,
              sliding_window=24, max_window_layers=1, hidden_act="silu")
# D has the head size of the large models (128) and room for sequences of several key tiles and
# several 128-row query tiles; its upper layer has a window that is longer than a key tile.
TINY_D = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
              hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
              intermediate_size=384, vocab_size=700, rope_theta=1000000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=512, use_sliding_window=True,
              sliding_window=160, max_window_layers=1, hidden_act="silu")
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3}
PAGE_SIZES = {"A": 16, "B": 8, "C": 16, "D": 16}


def make_model(name: str, root: str, dtype=torch.float32, std: float = 0.02) -> str:
    out = os.path.join(root, f"tiny_{name}_{str(dtype).split('.')[-1]}_std{std}")
    if not os.path.isdir(out):
        write_random_model(Qwen2Config.from_dict(TINY[name]), SEEDS[name], out, dtype=dtype, std=std)
    return out


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
