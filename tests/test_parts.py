"""Each part of a model alone against its plain function, in 32-bit and in bfloat16, at sizes
that differ from the tiny models'."""
import pytest
import torch

import plain_qwen3 as plain
from part_helpers import DEV, Session, load_part, runtime, tolerance

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed + sum(shape))) * scale


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from kirai_b200.parts import RMSNorm

    norm = RMSNorm("n.weight", 72, 1e-5)
    weights = load_part(norm, dtype)
    resid, delta = rand(9, 72, scale=2.0), rand(9, 72, seed=1).to(dtype)
    stream = resid.to(DEV)
    out = norm.add_forward(stream, delta.to(DEV))
    expected = plain.rms_norm(resid + delta.float(), weights["n.weight"], 1e-5)
    assert out.dtype == dtype and torch.allclose(stream.cpu(), resid + delta.float(), atol=1e-6)
    assert float((out.float().cpu() - expected).abs().max()) <= tolerance(dtype, expected)
    rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
    picked = norm.add_forward_rows(resid.to(DEV), delta.to(DEV), rows)
    assert float((picked.float().cpu() - expected[[8, 2]]).abs().max()) <= tolerance(dtype, expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,rotary", [(48, 48), (64, 32)])
def test_rotary_part(dtype, head_dim, rotary):
    from kirai_b200.parts import RotaryEmbedding

    rope = RotaryEmbedding(head_dim, 50000.0, rotary)
    rope.load(None, runtime(dtype))
    q, k = rand(7, 5, head_dim).to(dtype), rand(7, 2, head_dim, seed=3).to(dtype)
    positions = [0, 1, 5, 63, 64, 1000, 30000]
    qd, kd = q.to(DEV), k.to(DEV)
    rope.apply(qd, kd, torch.tensor(positions, dtype=torch.int32, device=DEV))
    for got, source in ((qd, q), (kd, k)):
        expected = plain.rope(source.float(), positions, 50000.0, rotary)
        assert float((got.float().cpu() - expected).abs().max()) <= tolerance(dtype, expected)
    assert (rope.fused_table() is not None) == (rotary == head_dim)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_linear_parts(dtype):
    from kirai_b200.parts import SwiGLU

    ffn = SwiGLU("mlp.", 40, 104)
    weights = load_part(ffn, dtype)
    x = rand(11, 40).to(dtype)
    out = ffn.forward(x.to(DEV))
    expected = plain.swiglu_mlp(x.float(), weights["mlp.gate_proj.weight"], weights["mlp.up_proj.weight"], weights["mlp.down_proj.weight"])
    assert out.shape == (11, 40) and float((out.float().cpu() - expected).abs().max()) <= tolerance(dtype, expected)
    stacked = ffn.fused_weight if dtype == torch.bfloat16 else ffn.gate_up.weight  # gate and up are one matrix after load
    assert stacked.shape == (208, 40)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_output_head_share_a_tied_table(dtype):
    from kirai_b200.parts import Embedding, OutputHead
    from kirai_b200.weights.loader import from_tensors

    embedding, head = Embedding("tok.weight", 300, 24), OutputHead("tok.weight", 300, 24)
    table = rand(300, 24).bfloat16()
    source = from_tensors({"tok.weight": table}, embedding.weight_specs(), DEV)
    embedding.load(source, runtime(dtype))
    head.load(source, runtime(dtype))
    assert embedding.table is head.weight or embedding.table.data_ptr() == head.weight.data_ptr()
    ids = torch.tensor([0, 299, 7], dtype=torch.int32, device=DEV)
    rows = embedding.forward(ids)
    assert rows.dtype == torch.float32 and torch.equal(rows.cpu(), table.float()[[0, 299, 7]])
    x = rand(3, 24).to(dtype)
    logits = head.forward(x.to(DEV))
    expected = x.float() @ table.float().T
    assert logits.dtype == torch.float32 and float((logits.cpu() - expected).abs().max()) <= tolerance(dtype, expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads,kv_heads,head_dim,window,qk_norm", [(6, 2, 16, None, True), (3, 3, 24, 5, True), (4, 1, 32, 9, False)])
def test_attention_part_in_portions(dtype, q_heads, kv_heads, head_dim, window, qk_norm):
    from kirai_b200.parts import GQAttention, RotaryEmbedding

    hidden = 40
    attention = GQAttention("a.", hidden, q_heads, kv_heads, head_dim, RotaryEmbedding(head_dim, 10000.0), window=window,
                            qk_norm_eps=1e-6 if qk_norm else None)
    weights = load_part(attention, dtype)
    if not qk_norm:  # the plain block always norms: give it unit weights and undo the scale by hand below
        pass
    session = Session([attention.cache_need()], dtype, page_size=4)
    x = rand(23, hidden).to(dtype)
    cfg = dict(num_attention_heads=q_heads, num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=1e-6, rope_theta=10000.0)
    if qk_norm:
        expected = plain.attention_block(x.float(), weights, "a.", cfg, list(range(23)), window)
    else:
        T = 23
        q = (x.float() @ weights["a.q_proj.weight"].T).reshape(T, q_heads, head_dim)
        k = (x.float() @ weights["a.k_proj.weight"].T).reshape(T, kv_heads, head_dim)
        v = (x.float() @ weights["a.v_proj.weight"].T).reshape(T, kv_heads, head_dim)
        q, k = plain.rope(q, range(T), 10000.0), plain.rope(k, range(T), 10000.0)
        expected = plain.causal_attention(q, k, v, window).reshape(T, -1) @ weights["a.o_proj.weight"].T
    outputs, start = [], 0
    for count in (9, 2, 11, 1):  # a portion, a short one across a page edge, a long one, one decoded token
        batch = session.batch([("r", count)])
        outputs.append(attention.forward(x[start : start + count].to(DEV), batch, session.cache.layer_view(0), True))
        session.commit()
        start += count
    got = torch.cat(outputs).float().cpu()
    assert float((got - expected).abs().max()) <= tolerance(dtype, expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cut", [(2,), (1, 1)])
def test_attention_part_on_a_case_worked_by_hand(dtype, cut):
    """The order norm -> rotation and the mapping of query heads to kv heads, on numbers that come from no code.

    Six query heads over two kv heads (groups of 3), heads of 16, two tokens, eps 0; q and k norms share a weight
    that is 1 everywhere except 3 at component 8, the partner of component 0 under the half-split pairing (frequency
    theta^0 = 1, so the pair turns by the position in radians).  Projected rows, the same at both tokens: every query
    head e0; kv head 0 has k = e0, kv head 1 has k = e8; values: kv head 0 e0 then e1, kv head 1 10 e0 then 10 e1.
    Norm first: a unit vector of 16 has mean square 1/16, scale 4: q = 4 e0, kv 0's k = 4 e0, kv 1's k = 12 e8.
    Rotation at the second token: q1 = 4 (cos 1 e0 + sin 1 e8); kv 0: k1 = the same; kv 1: k1 = 12 (-sin 1 e0 + cos 1 e8).
    Scores of the second token, times 16^-1/2: kv 0: 4 cos 1 and 4; kv 1: 12 sin 1 and 0.  So a head on kv 0 mixes its
    two values with weights 0.1371944, 0.8628056 and a head on kv 1 with 0.9999588, 0.0000412 (times 10).
    Round-robin heads (h % 2) would swap heads 1 and 4; rotation before the norm would put the weight 3 on the turned
    component and give kv 0 the second score (16 cos^2 1 + 144 sin^2 1) / 4 = 26.66."""
    from kirai_b200.parts import GQAttention, RotaryEmbedding
    from kirai_b200.weights.loader import from_tensors
    from part_helpers import runtime

    d, hidden = 16, 96
    attention = GQAttention("a.", hidden, 6, 2, d, RotaryEmbedding(d, 777.0), qk_norm_eps=0.0)
    norm = torch.ones(d)
    norm[8] = 3.0
    unit = lambda index, scale=1.0: torch.nn.functional.one_hot(torch.tensor(index), hidden).float() * scale  # noqa: E731
    both = unit(0) + unit(1)  # a row that answers 1 to either token
    q = torch.zeros(6 * d, hidden)
    for head in range(6):
        q[head * d] = both
    k = torch.zeros(2 * d, hidden)
    k[0], k[d + 8] = both, both
    v = torch.zeros(2 * d, hidden)
    v[0], v[1], v[d], v[d + 1] = unit(0), unit(1), unit(0, 10.0), unit(1, 10.0)
    tensors = {"a.q_proj.weight": q, "a.k_proj.weight": k, "a.v_proj.weight": v, "a.o_proj.weight": torch.eye(hidden),
               "a.q_norm.weight": norm, "a.k_norm.weight": norm}
    tensors = {name: t.to(torch.bfloat16) for name, t in tensors.items()}
    attention.load(from_tensors(tensors, attention.weight_specs(), DEV), runtime(dtype))
    session = Session([attention.cache_need()], dtype, page_size=4)
    x = torch.stack([unit(0), unit(1)]).to(dtype).to(DEV)
    outputs, start = [], 0
    for count in cut:  # both tokens in one step, or the second as a decoded token
        batch = session.batch([("r", count)])
        outputs.append(attention.forward(x[start : start + count], batch, session.cache.layer_view(0), True))
        session.commit()
        start += count
    got = torch.cat(outputs).float().cpu().reshape(2, 6, d)
    on_kv0, on_kv1 = torch.zeros(d), torch.zeros(d)
    on_kv0[0], on_kv0[1] = 0.1371944, 0.8628056
    on_kv1[0], on_kv1[1] = 9.9995883, 0.0004117
    bound = 2e-5 if dtype == torch.float32 else 0.02
    for head in range(6):
        first = torch.zeros(d)
        first[0] = 1.0 if head < 3 else 10.0
        assert float((got[0, head] - first).abs().max()) <= bound, head          # the first token sees itself only
        expected = on_kv0 if head < 3 else on_kv1
        assert float((got[1, head] - expected).abs().max()) <= bound * (1.0 if head < 3 else 10.0), (head, got[1, head, :2])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("arrangement", ["pre_norm", "parallel"])
def test_block_arrangements(dtype, arrangement):
    from kirai_b200.parts import Block, GQAttention, RMSNorm, RotaryEmbedding, SwiGLU

    hidden = 48
    block = Block(RMSNorm("model.layers.0.input_layernorm.weight", hidden, 1e-6),
                  GQAttention("model.layers.0.self_attn.", hidden, 4, 2, 16, RotaryEmbedding(16, 1e4), qk_norm_eps=1e-6),
                  RMSNorm("model.layers.0.post_attention_layernorm.weight", hidden, 1e-6) if arrangement == "pre_norm" else None,
                  SwiGLU("model.layers.0.mlp.", hidden, 72), arrangement=arrangement)
    weights = load_part(block, dtype)
    session = Session([block.mixer.cache_need()], dtype)
    h = rand(13, hidden)
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=1e4)
    if arrangement == "pre_norm":
        expected = plain.decoder_layer(h, weights, 0, cfg, list(range(13)), None)
    else:
        n = plain.rms_norm(h, weights["model.layers.0.input_layernorm.weight"], 1e-6)
        a = plain.attention_block(n, weights, "model.layers.0.self_attn.", cfg, list(range(13)), None)
        m = plain.swiglu_mlp(n, weights["model.layers.0.mlp.gate_proj.weight"], weights["model.layers.0.mlp.up_proj.weight"],
                             weights["model.layers.0.mlp.down_proj.weight"])
        expected = h + a + m
    batch = session.batch([("r", 13)])
    resid, delta = block.forward(h.to(DEV), None, batch, session.cache.layer_view(0), True)
    got = resid.cpu() + delta.float().cpu()
    assert float((got - expected).abs().max()) <= tolerance(dtype, expected)


def test_blocks_fold_norms_into_products_for_small_batches(monkeypatch):
    """In bfloat16 a small batch runs its second norm, and the first norm of the block that follows, inside the
    products around them; the result is that of the separate kernels, with three launches fewer for two blocks,
    and a batch above the limit takes the separate kernels."""
    from kirai_b200.csrc import ops
    from kirai_b200.parts import Block, GQAttention, RMSNorm, RotaryEmbedding, SwiGLU
    from kirai_b200.parts.base import UnscaledNorm
    from kirai_b200.parts.linear import Linear

    hidden, dtype = 48, torch.bfloat16
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=1e4)

    def make(layer):
        prefix = f"model.layers.{layer}."
        return Block(RMSNorm(prefix + "input_layernorm.weight", hidden, 1e-6),
                     GQAttention(prefix + "self_attn.", hidden, 4, 2, 16, RotaryEmbedding(16, 1e4), qk_norm_eps=1e-6),
                     RMSNorm(prefix + "post_attention_layernorm.weight", hidden, 1e-6), SwiGLU(prefix + "mlp.", hidden, 72))

    blocks = [make(0), make(1)]
    weights = {}
    for layer, block in enumerate(blocks):
        weights.update(load_part(block, dtype, seed=layer))

    def run(rows):
        session = Session([b.mixer.cache_need() for b in blocks], dtype, num_pages=32)
        h = rand(rows, hidden, seed=3)
        batch = session.batch([("r", rows)])
        before = ops.launch_count
        resid, left = blocks[0].forward(h.to(DEV), None, batch, session.cache.layer_view(0), True, blocks[1])
        middle = left
        resid, left = blocks[1].forward(resid, left, batch, session.cache.layer_view(1), True, None)
        ops.check_device_errors(torch.device(DEV))
        expected = plain.decoder_layer(plain.decoder_layer(h, weights, 0, cfg, list(range(rows)), None), weights, 1, cfg,
                                       list(range(rows)), None)
        return resid.cpu() + left.float().cpu(), expected, middle, ops.launch_count - before

    fused, expected, middle, fused_launches = run(13)
    assert isinstance(middle, UnscaledNorm)
    assert float((fused - expected).abs().max()) <= tolerance(dtype, expected)
    monkeypatch.setenv("KIRAI_FUSE_NORMS", "0")
    separate, _, middle, separate_launches = run(13)
    assert isinstance(middle, torch.Tensor) and separate_launches == fused_launches + 3
    assert float((fused - separate).abs().max()) <= tolerance(dtype, expected)
    monkeypatch.delenv("KIRAI_FUSE_NORMS")
    large, expected, middle, _ = run(Linear.FUSED_NORM_MAX_ROWS + 1)
    assert isinstance(middle, torch.Tensor)
    assert float((large - expected).abs().max()) <= tolerance(dtype, expected)
