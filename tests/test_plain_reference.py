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


# The reference's attention tests below run its gated, one-centred variant (q_projection_gate and
# one_centered_rms_norm true: the q projection carries a gate of zeros, whose sigmoid halves the mixed output, and a
# norm weight w stands for 1 + w, so its zero weights are ones).  The dense model has neither
# (crates/llm-backend/src/core/qwen/ops/attention_full.rs:521-522, both flags are ``!spec.is_qwen3_dense()``): the plain
# functions are composed here as attention_full.rs:240-309 composes them, with a weight of ones, and the reference's
# expected numbers are what they give times GATE = sigmoid(0) = 0.5.
GATE = 0.5


def reference_attention(q_rows, k_rows, v_rows, norm_weight, eps, theta, rotate, window):
    """Projected rows in, mixed rows out (one head of width 2, identity output projection): per-head norm, rotation at
    positions 0.., attention over the visible rows."""
    T = len(q_rows)
    q = plain.rms_norm(torch.tensor(q_rows).reshape(T, 1, 2), torch.tensor(norm_weight), eps)
    k = plain.rms_norm(torch.tensor(k_rows).reshape(T, 1, 2), torch.tensor(norm_weight), eps)
    if rotate:
        q, k = plain.rope(q, range(T), theta), plain.rope(k, range(T), theta)
    v = torch.tensor(v_rows).reshape(T, 1, 2)
    return q, k, plain.causal_attention(q, k, v, window).reshape(T, 2)


def test_first_token_sees_only_itself():
    # cpu_ops.rs:504-524: width 1, q projection 0 (and a gate of 0), v = 8, o_proj = 3: output 12.0.
    # A first token's softmax has one entry, so the mixed row is v; 8 * 3 = 24 without the gate, 12 with it.
    q = k = torch.zeros(1, 1, 1)
    mixed = plain.causal_attention(q, k, torch.tensor([[[8.0]]]), None).reshape(1, 1)
    out = mixed @ torch.tensor([[3.0]]).T
    assert float(out) == 24.0 and float(out) * GATE == 12.0


def test_norm_then_rope_then_causal_softmax_two_tokens():
    # cpu_ops.rs:526-573, every number as there: q and k rows [1, 0] at both tokens, v rows [2, 0] and [0, 4],
    # eps 0, theta 10000, identity o_proj.  The norm comes first: [1, 0] has mean square 1/2, so it becomes
    # [sqrt 2, 0] (cpu_ops.rs:631 checks exactly this key in the cache), and only then is it turned by
    # position * theta^0 = 1 radian at the second token.
    q, k, mixed = reference_attention([[1.0, 0.0]] * 2, [[1.0, 0.0]] * 2, [[2.0, 0.0], [0.0, 4.0]], [1.0, 1.0], 0.0, 10_000.0, True, None)
    assert torch.allclose(k[0, 0], torch.tensor([math.sqrt(2.0), 0.0]), atol=1e-6)
    assert torch.allclose(k[1, 0], torch.tensor([math.sqrt(2.0) * math.cos(1.0), math.sqrt(2.0) * math.sin(1.0)]), atol=1e-6)
    score0 = math.sqrt(2.0) * math.cos(1.0)  # the reference's own expectation, cpu_ops.rs:562-569
    score1 = math.sqrt(2.0)
    top = max(score0, score1)
    exp0, exp1 = math.exp(score0 - top), math.exp(score1 - top)
    w0, w1 = exp0 / (exp0 + exp1), exp1 / (exp0 + exp1)
    assert torch.allclose(mixed[0] * GATE, torch.tensor([1.0, 0.0]), atol=1e-6)          # cpu_ops.rs:571
    assert torch.allclose(mixed[1] * GATE, torch.tensor([w0, 2.0 * w1]), atol=1e-6)      # cpu_ops.rs:572


def test_window_of_two_over_three_tokens():
    # cpu_ops.rs:638-685 (whole sequence into a cache of 2 rows) and :688-747 (two tokens, then one step): no rotation
    # (partial_rotary_factor 0), q and k rows [1, 0] everywhere, v rows [2, 0], [0, 4], [8, 0].  The third token sees
    # the last two rows with equal scores: (0, 4)/2 + (8, 0)/2 = [4, 2]; the reference expects [2.0, 1.0] = [4, 2] * GATE.
    # The plain implementation keeps no cache, so both cases are the same computation here.
    _, _, mixed = reference_attention([[1.0, 0.0]] * 3, [[1.0, 0.0]] * 3, [[2.0, 0.0], [0.0, 4.0], [8.0, 0.0]], [1.0, 1.0], 0.0,
                                      10_000.0, False, 2)
    assert torch.allclose(mixed[2], torch.tensor([4.0, 2.0]), atol=1e-6)
    assert torch.allclose(mixed[2] * GATE, torch.tensor([2.0, 1.0]), atol=1e-6)
    # without the window the first row would count too: (2, 0)/3 + (0, 4)/3 + (8, 0)/3
    _, _, unwindowed = reference_attention([[1.0, 0.0]] * 3, [[1.0, 0.0]] * 3, [[2.0, 0.0], [0.0, 4.0], [8.0, 0.0]], [1.0, 1.0],
                                           0.0, 10_000.0, False, None)
    assert torch.allclose(unwindowed[2], torch.tensor([10.0 / 3.0, 4.0 / 3.0]), atol=1e-6)


def test_swiglu_mlp_closed_form():
    # cpu_ops.rs:1146-1151: input [1, 2], gate row [1, 0], up row [0, 1], down column [1, 2]:
    # silu(1) * 2 = 1.4621172, then [1, 2] times that.
    out = plain.swiglu_mlp(torch.tensor([[1.0, 2.0]]), torch.tensor([[1.0, 0.0]]), torch.tensor([[0.0, 1.0]]), torch.tensor([[1.0], [2.0]]))
    assert torch.allclose(out[0], torch.tensor([1.4621172, 2.9242344]), atol=1e-6)


def test_order_of_norm_and_rotation_and_the_kv_head_of_a_query_head():
    """A case worked by hand, with numbers that no other reading of the formulas gives.

    Six query heads over two kv heads (groups of 3), width 2, two tokens, eps 0, theta anything (the only frequency
    is theta^0 = 1, so the angle is the position).  The q and k norms share the NON-uniform weight [1, 3].
    Projected rows, the same at both tokens: every query head [1, 0]; kv head 0 has k = [1, 0], kv head 1 has k = [0, 1].
    Values: kv head 0 has v = [1, 0] then [0, 1]; kv head 1 has v = [10, 0] then [0, 10].

    Norm first (mean square 1/2, scale sqrt 2, then the weight): q = [sqrt 2, 0]; k of kv head 0 = [sqrt 2, 0];
    k of kv head 1 = [0, 3 sqrt 2].  Then the rotation by 1 radian at the second token:
    q1 = sqrt 2 [cos 1, sin 1]; kv 0: k0 = [sqrt 2, 0], k1 = sqrt 2 [cos 1, sin 1]; kv 1: k0 = [0, 3 sqrt 2],
    k1 = 3 sqrt 2 [-sin 1, cos 1].  Scores of the second token (times 2^-1/2):
      against kv 0: s0 = sqrt 2 cos 1 = 0.7641050, s1 = sqrt 2 = 1.4142136  ->  weights 0.3429646, 0.6570354
      against kv 1: s0 = 3 sqrt 2 sin 1 = 3.5700579, s1 = 0                 ->  weights 0.9726168, 0.0273832
    so a head on kv 0 gives [0.3429646, 0.6570354] and a head on kv 1 gives [9.7261676, 0.2738324].
    Heads 0, 1, 2 read kv 0 and heads 3, 4, 5 read kv 1 (h // 3).  Had heads been dealt round-robin (h % 2), head 1
    would give the kv 1 row and head 4 the kv 0 row.  Had the rotation come before the norm, the second component
    would carry the weight 3 after turning: kv 0's s1 would be (2 cos^2 1 + 18 sin^2 1) / sqrt 2 = 9.4251 and its
    first weight 0.000173 instead of 0.3429646.
    """
    T, weight = 2, torch.tensor([1.0, 3.0])
    q = torch.tensor([1.0, 0.0]).repeat(T, 6, 1)
    k = torch.tensor([[1.0, 0.0], [0.0, 1.0]]).repeat(T, 1, 1)
    v = torch.tensor([[[1.0, 0.0], [10.0, 0.0]], [[0.0, 1.0], [0.0, 10.0]]])
    qn, kn = plain.rms_norm(q, weight, 0.0), plain.rms_norm(k, weight, 0.0)
    qr, kr = plain.rope(qn, [0, 1], 123.0), plain.rope(kn, [0, 1], 123.0)
    out = plain.causal_attention(qr, kr, v, None)
    on_kv0, on_kv1 = torch.tensor([0.3429646, 0.6570354]), torch.tensor([9.7261676, 0.2738324])
    for head in range(6):
        assert torch.allclose(out[0, head], v[0, head // 3], atol=1e-6)  # the first token sees itself only
        assert torch.allclose(out[1, head], on_kv0 if head < 3 else on_kv1, atol=2e-6), head
    # the same numbers through the plain attention block, with the projections as identity-like selections:
    # hidden 2, q_proj stacks six copies of [[1, 0], [0, 1]] (so q = x per head), k_proj/v_proj pick per kv head
    cfg = dict(num_attention_heads=6, num_key_value_heads=2, head_dim=2, rms_norm_eps=0.0, rope_theta=123.0)
    eye = torch.eye(2)
    weights = {"a.q_proj.weight": eye.repeat(6, 1), "a.k_proj.weight": torch.cat([eye, eye.flip(0)]),
               "a.v_proj.weight": torch.cat([eye, 10.0 * eye]), "a.q_norm.weight": weight, "a.k_norm.weight": weight,
               "a.o_proj.weight": torch.eye(12)}
    # x = [1, 0] at both tokens gives q = [1, 0] per head, k = [1, 0] / [0, 1]; v = [1, 0] / [10, 0] at both tokens
    block = plain.attention_block(torch.tensor([[1.0, 0.0], [1.0, 0.0]]), weights, "a.", cfg, [0, 1], None).reshape(2, 6, 2)
    assert torch.allclose(block[1, 0], torch.tensor([1.0, 0.0]), atol=1e-6) and torch.allclose(block[1, 5], torch.tensor([10.0, 0.0]), atol=1e-6)
    # with v equal at both tokens only the head-to-kv mapping shows: heads 0-2 sum to 1, heads 3-5 to 10
    assert [round(float(block[1, h].sum())) for h in range(6)] == [1, 1, 1, 10, 10, 10]


def test_grouped_heads_read_their_kv_head():
    torch.manual_seed(1)
    q, k, v = torch.randn(5, 6, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    out = plain.causal_attention(q, k, v, None)
    for head in range(6):
        single = plain.causal_attention(q[:, head : head + 1], k[:, head // 3 : head // 3 + 1], v[:, head // 3 : head // 3 + 1], None)
        assert torch.allclose(out[:, head], single[:, 0], atol=1e-6)


def test_argmax_as_the_reference_tests_it():
    # llm-sampler/src/lib.rs:222-239: greedy over [-1, 0.25, 3.5, 3] is 2; the first of two equal maxima wins
    assert plain.argmax_first(torch.tensor([-1.0, 0.25, 3.5, 3.0])) == 2
    assert plain.argmax_first(torch.tensor([1.0, 2.0, 2.0])) == 1
    assert plain.argmax_first(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1


# (logits, temperature, top_p, draw, token) exactly as llm-sampler/src/lib.rs:255-294 has them
REFERENCE_TOP_P_CASES = [
    ([2.0, 1.0, 0.0], 1.0, 0.9, 0.0, 0),          # :262-267 low draw samples top token
    ([2.0, 1.0, 0.0], 1.0, 0.9, 0.8, 1),          # :268-273 high draw samples second nucleus token
    ([2.0, 2.0, 2.0, 0.0], 1.0, 0.6, 0.0, 0),     # :283-288 low draw samples first tied token
    ([2.0, 2.0, 2.0, 0.0], 1.0, 0.6, 0.99, 1),    # :289-294 high draw samples second tied token (ties in index order)
]


def test_top_p_cases_of_the_reference():
    for logits, temperature, top_p, draw, token in REFERENCE_TOP_P_CASES:
        assert plain.sample_top_p(torch.tensor(logits), temperature, top_p, draw) == token
    # why: softmax([2, 1, 0]) = 0.6652410, 0.2447285, 0.0900306; the nucleus for 0.9 is the first two (0.9099695);
    # 0.8 * 0.9099695 = 0.7279756 > 0.6652410, so the second.  softmax([2, 2, 2, 0]) = 0.3189 x 3, 0.0432; two of the
    # tied entries reach 0.6 (0.6379); 0.99 * 0.6379 = 0.6315 > 0.3189, so the second of them, index 1.


def test_top_p_draws():
    # more of the same kind, own numbers: probabilities 0.5, 0.3, 0.2 with top_p 0.75 keep two entries (sum 0.8)
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
