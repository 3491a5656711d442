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
