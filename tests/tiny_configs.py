"""The two tiny Qwen3 configurations of the tests, differing in every size and option,
and helpers that write them as model folders with random weights."""
from __future__ import annotations


import torch

CONFIG_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, vocab_size=256, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=10000.0,
    tie_word_embeddings=True, hidden_act="silu", attention_bias=False,
)
PAGE_A = 4

CONFIG_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2,
    head_dim=32, vocab_size=384, max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=1000000.0,
    tie_word_embeddings=False, use_sliding_window=True, sliding_window=16, max_window_layers=1,
    hidden_act="silu", attention_bias=False, rope_scaling=None,
)
PAGE_B = 8

TINY = {"A": (CONFIG_A, PAGE_A, 0), "B": (CONFIG_B, PAGE_B, 1)}  # name -> (config, page size, seed)


def write_tiny_model(folder: str, name: str) -> dict:
    """Writes tiny model ``name`` into ``folder`` through the framework's random-weights mode."""
    import kirai_b200  # noqa: F401
    from kirai_b200.registry import config_from_dict
    from kirai_b200.weights import write_random_model

    raw, _, seed = TINY[name]
    write_random_model(folder, config_from_dict(raw), seed, std=0.02, norm_jitter=0.1, dtype=torch.bfloat16)
    return raw


def random_tokens(count: int, vocab: int, seed: int):
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()
