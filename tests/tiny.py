"""The two tiny configurations of the tests (they differ in every size and option) and
helpers that write their model folders into a temporary directory."""
from __future__ import annotations

import numpy as np
import torch

from coheryn_ai_studio_b200.config import Qwen2Config
from coheryn_ai_studio_b200.engine import write_random_model
from coheryn_ai_studio_b200.weights import InitPolicy

TINY_A = Qwen2Config(
    vocab_size=512, hidden_size=64, intermediate_size=176, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=256,
    rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True)
POLICY_A = InitPolicy(matrix_std=0.02, bias_std=0.02, norm_jitter=0.01)

TINY_B = Qwen2Config(
    vocab_size=1000, hidden_size=96, intermediate_size=256, num_hidden_layers=3,
    num_attention_heads=3, num_key_value_heads=1, head_dim=32, max_position_embeddings=512,
    rms_norm_eps=1e-5, rope_theta=1e6, tie_word_embeddings=False)
POLICY_B = InitPolicy(matrix_std=0.02, bias_std=0.1, norm_jitter=0.01)

# Larger deviations make the logits spread enough that a wrong key or a wrong page
# changes them visibly.
POLICY_LOUD = InitPolicy(matrix_std=0.08, bias_std=0.2, norm_jitter=0.05)

CONFIGS = {"A": (TINY_A, POLICY_A, 0), "B": (TINY_B, POLICY_B, 1),
           "A_loud": (TINY_A, POLICY_LOUD, 0), "B_loud": (TINY_B, POLICY_LOUD, 1)}


def make_folder(tmp_path, name: str, policy=None, store=torch.bfloat16) -> str:
    cfg, pol, seed = CONFIGS[name]
    d = str(tmp_path / f"tiny_{name}")
    write_random_model(d, cfg, seed, policy or pol, store=store)
    return d


def prompt(seed: int, length: int, vocab: int):
    return np.random.default_rng(seed).integers(0, vocab, size=length).tolist()
