"""The plain implementation against the closed-form values of the reference's own unit tests
(crates/llm-backend/src/core/tests/cpu_ops.rs, crates/llm-sampler/src/lib.rs) and against itself in 64-bit."""
import math

import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import random_tokens, write_tiny_model


def test_rms_norm_closed_form():
    # cpu_ops.rs:27-31: rms_norm([3,4],[1,2], eps 0) = [0.84852815, 2.2627418]
    out = plain.rms_norm(torch.tensor([3.0, 4.0]), torch.tensor([1.0, 2.0]), 0.0)
    assert torch.allclose(out, torch.tensor([0.84852815, 2.2627418]), atol=1e-6)
    assert torch.equal(plain.rms_norm(torch.zeros(4), torch.ones(4), 0.0), torch.zeros(4))


def test_silu_closed_form():
    # cpu_ops.rs:236-242
    out = plain.silu(torch.tensor([0.0, 2.0, -2.0]))
    assert torch.allclose(out, torch.tensor([0.0, 1.761594, -0.23840584]), atol=1e-6)


def test_rope_and_causal_scores_two_tokens():
    # cpu_ops.rs:526-573: head_dim 2, theta such that inv_freq_0 = 1: the key [sqrt2, 0] at position 0 stays,
    # at position 1 it turns by 1 radian; a query [sqrt2, 0] at position 1 scores sqrt2*cos(1)*... against key 0.
    x = torch.tensor([[[math.sqrt(2.0), 0.0]], [[math.sqrt(2.0), 0.0]]])
    rotated = plain.rope(x, [0, 1], theta=10000.0)
    assert torch.allclose(rotated[0, 0], torch.tensor([math.sqrt(2.0), 0.0]), atol=1e-6)  # cpu_ops.rs:631
    assert torch.allclose(rotated[1, 0], torch.tensor([math.sqrt(2.0) * math.cos(1.0), math.sqrt(2.0) * math.sin(1.0)]), atol=1e-6)
    # scores of the second token: q1.k0 * d^-1/2 = sqrt2 * cos 1, q1.k1 * d^-1/2 = sqrt2
    scale = 2 ** -0.5
    s0 = float(rotated[1, 0] @ rotated[0, 0]) * scale
    s1 = float(rotated[1, 0] @ rotated[1, 0]) * scale
    assert abs(s0 - math.sqrt(2.0) * math.cos(1.0)) < 1e-6 and abs(s1 - math.sqrt(2.0)) < 1e-6
    v = torch.tensor([[[1.0, 0.0]], [[0.0, 2.0]]])
    out = plain.causal_attention(rotated, rotated, v, None)
    w0 = math.exp(s0) / (math.exp(s0) + math.exp(s1))
    assert torch.allclose(out[0, 0], torch.tensor([1.0, 0.0]))
    assert torch.allclose(out[1, 0], torch.tensor([w0, 2.0 * (1.0 - w0)]), atol=1e-6)


def test_sliding_window_keeps_last_rows():
    # cpu_ops.rs:638-685: a window of 2 over 3 tokens: the last token sees tokens 1 and 2 only
    torch.manual_seed(0)
    q, k, v = torch.randn(3, 1, 4), torch.randn(3, 1, 4), torch.randn(3, 1, 4)
    windowed = plain.causal_attention(q, k, v, 2)
    tail = plain.causal_attention(q[1:], k[1:], v[1:], None)
    assert torch.allclose(windowed[2], tail[1], atol=1e-6)
    assert not torch.allclose(windowed[2], plain.causal_attention(q, k, v, None)[2], atol=1e-4)


def test_grouped_heads_read_their_kv_head():
    torch.manual_seed(1)
    q, k, v = torch.randn(5, 6, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    out = plain.causal_attention(q, k, v, None)
    for head in range(6):
        single = plain.causal_attention(q[:, head : head + 1], k[:, head // 3 : head // 3 + 1], v[:, head // 3 : head // 3 + 1], None)
        assert torch.allclose(out[:, head], single[:, 0], atol=1e-6)


def test_argmax_ties_take_lowest_index():
    # llm-sampler/src/lib.rs:234-238
    assert plain.argmax_first(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1


def test_top_p_draws():
    # llm-sampler/src/lib.rs:255-294 in spirit: probabilities 0.5, 0.3, 0.2 with top_p 0.75 keep two entries (sum 0.8)
    logits = torch.log(torch.tensor([0.2, 0.5, 0.3]))
    assert plain.sample_top_p(logits, 1.0, 0.75, 0.0) == 1
    assert plain.sample_top_p(logits, 1.0, 0.75, 0.62) == 1   # 0.62 * 0.8 = 0.496 <= 0.5
    assert plain.sample_top_p(logits, 1.0, 0.75, 0.63) == 2   # 0.504 > 0.5
    assert plain.sample_top_p(logits, 1.0, 0.75, 0.999) == 2
    assert plain.sample_top_p(logits, 1.0, 1.0, 0.95) == 0
    assert plain.sample_top_p(logits, 0.01, 1.0, 0.9999) == 1  # a low temperature concentrates on the maximum


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_agrees_with_float64(name, tmp_path):
    write_tiny_model(str(tmp_path), name)
    config, w32 = plain.read_model_folder(str(tmp_path), torch.float32)
    _, w64 = plain.read_model_folder(str(tmp_path), torch.float64)
    tokens = random_tokens(48, config["vocab_size"], 5)
    l32 = plain.forward_logits(config, w32, tokens)
    l64 = plain.forward_logits(config, w64, tokens)
    assert float((l32.double() - l64).abs().max()) < 2e-5


def test_prefix_logits_do_not_depend_on_what_follows(tmp_path):
    write_tiny_model(str(tmp_path), "B")
    config, weights = plain.read_model_folder(str(tmp_path))
    tokens = random_tokens(40, config["vocab_size"], 9)
    whole = plain.forward_logits(config, weights, tokens)
    part = plain.forward_logits(config, weights, tokens[:23])
    assert torch.allclose(whole[:23], part, atol=1e-6)
