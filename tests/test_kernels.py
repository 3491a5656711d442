"""Each kernel alone against plain torch arithmetic, at sizes other than the engine's tiny models:
head sizes in steps of 16, head counts and groups that are no power of two, widths and
vocabularies that are no power of two."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    import kirai_b200  # noqa: F401
    from kirai_b200.csrc import ops as module

    module.library()
    return module


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    generator = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=generator) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,hidden", [(1000, 72), (257, 200), (130, 4104)])
def test_embedding(ops, dtype, vocab, hidden):
    table = rand(vocab, hidden, dtype=dtype)
    ids = torch.tensor([0, vocab - 1, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = ops.embedding(table, ids)
    assert out.dtype == torch.float32 and torch.equal(out, table.float()[ids.long()])
    ops.embedding(table, torch.tensor([vocab], dtype=torch.int32, device=DEV))
    with pytest.raises(ops.KernelError):
        ops.check_device_errors(torch.device(DEV))
    if dtype == torch.bfloat16:  # the gather from the tensor-core product's box layout
        boxes = ops.tile_weight(table)
        assert torch.equal(ops.embedding(boxes, ids), out)
        ops.embedding(boxes, torch.tensor([-1], dtype=torch.int32, device=DEV))
        with pytest.raises(ops.KernelError):
            ops.check_device_errors(torch.device(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,eps", [(7, 200, 1e-5), (33, 4104, 1e-6), (1, 48, 0.0)])
def test_add_rmsnorm(ops, dtype, rows, hidden, eps):
    resid = rand(rows, hidden, scale=2.0)
    delta = rand(rows, hidden, dtype=dtype, seed=1)
    weight = 1.0 + 0.1 * rand(hidden, seed=2)
    expected_sum = resid + delta.float()
    expected = expected_sum * torch.rsqrt((expected_sum ** 2).mean(-1, keepdim=True) + eps) * weight
    stream = resid.clone()
    out = ops.add_rmsnorm(stream, delta, weight, eps, dtype)
    assert torch.allclose(stream, expected_sum, atol=1e-6)
    assert float((out.float() - expected).abs().max()) <= tol(dtype, float(expected.abs().max()))
    # chosen rows only: the stream stays as it is
    index = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    stream2 = resid.clone()
    out_rows, summed = ops.add_rmsnorm(stream2, delta, weight, eps, dtype, row_index=index)
    assert torch.equal(stream2, resid) and torch.allclose(summed, expected_sum[index.long()], atol=1e-6)
    assert float((out_rows.float() - expected[index.long()]).abs().max()) <= tol(dtype, float(expected.abs().max()))
    zero = ops.add_rmsnorm(torch.zeros(2, hidden, device=DEV), None, weight, 0.0, dtype)
    assert torch.equal(zero.float(), torch.zeros(2, hidden, device=DEV))  # mean + eps == 0 gives scale 0


def rope_reference(x, positions, inv_freq, rotary_dim):
    half = rotary_dim // 2
    angle = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(angle.double()).float()[:, None, :], torch.sin(angle.double()).float()[:, None, :]
    out = x.clone().float()
    first, second = x[..., :half].float(), x[..., half:rotary_dim].float()
    out[..., :half] = first * cos - second * sin
    out[..., half:rotary_dim] = second * cos + first * sin
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,width,rotary", [(3, 48, 48), (5, 80, 32), (2, 256, 256)])
def test_rope_and_head_rmsnorm(ops, dtype, heads, width, rotary):
    rows = 19
    buffer = rand(rows, heads * width + 24, dtype=dtype)  # heads live inside a wider row
    x = buffer[:, : heads * width].unflatten(1, (heads, width))
    positions = torch.tensor([0, 1, 2, 3, 100, 4095, 40959, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 31], dtype=torch.int32, device=DEV)
    inv_freq = torch.pow(torch.tensor(1e6), -(2.0 * torch.arange(rotary // 2)) / rotary).to(DEV)
    expected = rope_reference(x, positions, inv_freq, rotary)
    before_tail = buffer[:, heads * width :].clone()
    ops.rope_(x, positions, inv_freq, rotary)
    assert float((x.float() - expected).abs().max()) <= tol(dtype, float(expected.abs().max()))
    assert torch.equal(buffer[:, heads * width :], before_tail)
    weight = 1.0 + 0.1 * rand(width, seed=5)
    y = x.clone()
    expected = y.float() * torch.rsqrt((y.float() ** 2).mean(-1, keepdim=True) + 1e-5) * weight
    ops.head_rmsnorm_(y, weight, 1e-5)
    assert float((y.float() - expected).abs().max()) <= tol(dtype, float(expected.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(5, 200), (130, 1000)])
def test_swiglu(ops, dtype, rows, inter):
    gate_up = rand(rows, 2 * inter, dtype=dtype, scale=3.0)
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    expected = g / (1.0 + torch.exp(-g)) * u
    out = ops.swiglu(gate_up)
    assert float((out.float() - expected).abs().max()) <= tol(dtype, float(expected.abs().max()))


@pytest.mark.parametrize("m,n,k", [(1, 40, 24), (7, 130, 200), (70, 257, 72), (129, 64, 1000)])
def test_linear_plain_float32_is_exact_enough(ops, m, n, k):
    x, w = rand(m, k), rand(n, k, seed=3)
    expected = (x.double() @ w.double().T).float()
    out = ops.linear_plain(x, w)
    assert float((out - expected).abs().max()) <= 1e-5 * math.sqrt(k)


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (3, 200, 136), (16, 1000, 512), (48, 520, 1032), (64, 4096, 264),
                                   (65, 264, 192), (100, 1000, 2080), (128, 4096, 4096), (129, 520, 1032),
                                   (200, 96, 64), (256, 4096, 2112), (257, 264, 192), (300, 1000, 520), (1024, 768, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_tcgen05_against_plain(ops, m, n, k, out_dtype):
    x, w = rand(m, k, dtype=torch.bfloat16, scale=0.5), rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=3)
    expected = x.float() @ w.float().T
    out = ops.linear_tcgen05(x, w, out_dtype)
    plain = ops.linear_plain(x, w, out_dtype)
    ops.check_device_errors(torch.device(DEV))
    bound = (2e-5 * math.sqrt(k) if out_dtype == torch.float32 else 1e-2) * float(expected.abs().max())
    assert float((out.float() - expected).abs().max()) <= bound
    assert float((out.float() - plain.float()).abs().max()) <= bound
    if m <= 256:  # split along K between the CTAs of a cluster (up to 64 rows: slots beside the ring; up to 256: in it)
        split = ops.linear_tcgen05(x, w, out_dtype, splits=3)
        assert float((split.float() - expected).abs().max()) <= bound
        two = ops.linear_tcgen05(x, w, out_dtype, splits=2)
        assert float((two.float() - expected).abs().max()) <= bound
    if m <= 64:
        eight = ops.linear_tcgen05(x, w, out_dtype, splits=8)  # the largest cluster
        assert float((eight.float() - expected).abs().max()) <= bound
    # a row-strided input (a slice of a wider buffer)
    wide = torch.zeros(m, k + 16, dtype=torch.bfloat16, device=DEV)
    wide[:, :k] = x
    strided = ops.linear_tcgen05(wide[:, :k], w, out_dtype)
    assert torch.equal(strided, out)
    # the same weights cut into boxes at load: the same products in the same order, bit for bit
    tiled = ops.tile_weight(w)
    assert tiled.shape == (n, k) and torch.equal(tiled.row_major(), w)
    assert torch.equal(ops.linear_tcgen05(x, tiled, out_dtype), out)
    if m <= 256:
        assert torch.equal(ops.linear_tcgen05(x, tiled, out_dtype, splits=3), split)
    assert torch.equal(ops.linear(wide[:, :k], tiled, out_dtype), out)
    ops.check_device_errors(torch.device(DEV))


def test_linear_refuses_rows_that_tma_cannot_read(ops):
    x, w = rand(4, 70, dtype=torch.bfloat16), rand(32, 70, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError):
        ops.linear_tcgen05(x, w)
    out = ops.linear(x, w)  # the product path takes the CUDA-core kernel for such a K
    expected = x.float() @ w.float().T
    assert float((out.float() - expected).abs().max()) <= 1e-2 * float(expected.abs().max())


def paged_setup(dtype, lengths, kv_heads, head_dim, page_size, seed=0):
    """Random keys and values for requests of the given lengths, scattered over shuffled pages."""
    generator = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page_size) for n in lengths]
    num_pages = sum(pages_per) + 3
    order = torch.randperm(num_pages, generator=generator).tolist()
    cache = torch.zeros(num_pages, 2, kv_heads, page_size, head_dim, dtype=dtype, device=DEV)
    width = max(pages_per)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    keys, values = [], []
    cursor = 0
    for r, n in enumerate(lengths):
        k = (torch.randn(n, kv_heads, head_dim, generator=generator)).to(dtype)
        v = (torch.randn(n, kv_heads, head_dim, generator=generator)).to(dtype)
        keys.append(k)
        values.append(v)
        for p in range(pages_per[r]):
            table[r, p] = order[cursor]
            cursor += 1
    return cache, table.to(DEV), keys, values


def attention_reference(q, k, v, positions, window, scale):
    """q [T, nq, d] at absolute positions of one request; k, v [n, nkv, d] all its rows."""
    nq, nkv = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape, dtype=torch.float32)
    for t, pos in enumerate(positions):
        lo = 0 if not window else max(0, pos - window + 1)
        for h in range(nq):
            kv = h // (nq // nkv)
            s = (k[lo : pos + 1, kv].float() @ q[t, h].float()) * scale
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[lo : pos + 1, kv].float()
    return out


@pytest.mark.parametrize("rows", [1, 8, 16, 23, 64])
@pytest.mark.parametrize("hidden,q_width,inter,qkv_width", [(200, 136, 328, 264), (4096, 4096, 1536, 6144), (128, 64, 16, 96)])
def test_products_held_back_and_launched_as_one_kernel(ops, monkeypatch, rows, hidden, q_width, inter, qkv_width):
    """A layer's products (output projection with the residual and the next norm, gate/up with SwiGLU, down with the
    residual and the norm, the next q/k/v) through ``chained_products`` as one persistent kernel, against the same
    calls launched one by one and against 32-bit arithmetic; twice in a row, since the kernel leaves its counters for
    its next launch."""
    eps = 1e-6
    bf = torch.bfloat16
    monkeypatch.setattr(ops, "chain_products", True)
    w_o, w_gate, w_up = rand(hidden, q_width, dtype=bf, scale=0.05), rand(inter, hidden, dtype=bf, scale=0.05, seed=1), rand(inter, hidden, dtype=bf, scale=0.05, seed=2)
    w_down, w_qkv = rand(hidden, inter, dtype=bf, scale=0.05, seed=3), rand(qkv_width, hidden, dtype=bf, scale=0.05, seed=4)
    norm1, norm2 = 1.0 + 0.1 * rand(hidden, seed=5), 1.0 + 0.1 * rand(hidden, seed=6)
    tiled = {name: ops.tile_weight(w) for name, w in (("o", w_o), ("down", w_down), ("qkv", w_qkv))}
    tiled["gate_up"] = ops.tile_weight(ops.interleave_gate_up(w_gate, w_up))
    x = rand(rows, q_width, dtype=bf, seed=7)
    stream0 = rand(rows, hidden, scale=2.0, seed=8)

    def layer(stream):
        rows1, sumsq1 = ops.linear_residual_norm(x, tiled["o"], stream, norm1)
        act = ops.linear_tcgen05(rows1, tiled["gate_up"], swiglu=True, row_scale=(sumsq1, hidden, eps))
        rows2, sumsq2 = ops.linear_residual_norm(act, tiled["down"], stream, norm2)
        return ops.linear_tcgen05(rows2, tiled["qkv"], row_scale=(sumsq2, hidden, eps))

    single_stream = stream0.clone()
    single = layer(single_stream)
    before = ops.launch_count
    for attempt in range(2):
        chained_stream = stream0.clone()
        with ops.chained_products():
            chained = layer(chained_stream)
            assert ops.chaining()
        ops.check_device_errors(torch.device(DEV))
        assert not ops.chaining()
        # 32-bit arithmetic on the same bf16 inputs, with the roundings to bf16 where the kernels round
        r1 = stream0 + x.float() @ w_o.float().T
        n1 = (r1 * norm1).to(bf).float() * torch.rsqrt((r1 ** 2).mean(-1, keepdim=True) + eps)
        gate, up = n1 @ w_gate.float().T, n1 @ w_up.float().T
        a = (gate / (1.0 + torch.exp(-gate)) * up).to(bf).float()
        r2 = r1 + a @ w_down.float().T
        n2 = (r2 * norm2).to(bf).float() * torch.rsqrt((r2 ** 2).mean(-1, keepdim=True) + eps)
        expected = n2 @ w_qkv.float().T
        scale = float(expected.abs().max())
        assert float((chained.float() - expected).abs().max()) <= tol(bf, scale)
        assert float((chained_stream - r2).abs().max()) <= tol(bf, float(r2.abs().max()))
        assert float((chained.float() - single.float()).abs().max()) <= tol(bf, scale)
        assert float((chained_stream - single_stream).abs().max()) <= tol(bf, float(r2.abs().max()))
    assert ops.launch_count - before == 2  # four products, one launch, each time


def test_products_held_back_go_out_before_any_other_kernel(ops, monkeypatch):
    """Launch order is kept: a kernel of another kind, asked for while products are held back, sees their results."""
    bf = torch.bfloat16
    monkeypatch.setattr(ops, "chain_products", True)
    w1, w2 = ops.tile_weight(rand(256, 128, dtype=bf, scale=0.1)), ops.tile_weight(rand(128, 256, dtype=bf, scale=0.1, seed=1))
    x = rand(5, 128, dtype=bf, seed=2)
    stream = torch.zeros(5, 128, device=DEV)
    with ops.chained_products():
        y = ops.linear_tcgen05(ops.linear_tcgen05(x, w1), w2)
        ops.add_into_residual(stream, y)  # not a product: the two held back are launched first
        z = ops.linear_tcgen05(y, w1)     # held back until the block ends
    expected = (x.float() @ w1.row_major().float().T).to(bf).float() @ w2.row_major().float().T
    assert float((stream - expected).abs().max()) <= tol(bf, float(expected.abs().max()))
    assert float((z.float() - y.float() @ w1.row_major().float().T).abs().max()) <= tol(bf, float(z.float().abs().max()))
    with pytest.raises(RuntimeError, match="boom"):
        with ops.chained_products():
            ops.linear_tcgen05(x, w1)
            raise RuntimeError("boom")
    assert not ops.chaining() and ops.linear_tcgen05(x, w1).shape == (5, 256)  # nothing stayed behind
    ops.check_device_errors(torch.device(DEV))


def test_a_bounded_wait_that_runs_out_is_reported_and_the_device_stays_usable(ops):
    """Every barrier wait in the kernels gives up after a number of polls, sets the device error word and lets the
    kernel return.  The self-test kernel waits for a barrier that nothing completes: the host must read "a bounded
    wait ... ran out", and the launches after it must run as if nothing had happened."""
    device = torch.device(DEV)
    assert ops.wait_selftest(device, limit=10_000, arrive=True) == 0   # the control: an answered wait is no error
    ops.check_device_errors(device)
    assert ops.wait_selftest(device, limit=10_000) == 10_000
    with pytest.raises(ops.KernelError, match="bounded wait inside a kernel ran out"):
        ops.check_device_errors(device)
    ops.check_device_errors(device)  # reading the word cleared it
    x = rand(5, 64, dtype=torch.bfloat16)
    w = rand(24, 64, dtype=torch.bfloat16, seed=1)
    out = ops.linear(x, w)  # a tensor-core product with its own barrier waits, right after
    assert float((out.float() - x.float() @ w.float().T).abs().max()) <= tol(torch.bfloat16, 8.0)
    ops.check_device_errors(device)
    with pytest.raises(ops.KernelError, match="refused"):
        ops.wait_selftest(device, limit=1 << 21)


@pytest.mark.parametrize("balanced", ["0", "1"])
@pytest.mark.parametrize("q_heads,kv_heads,head_dim,page_size,window,lengths",
                         [(32, 8, 128, 16, None, [700, 33, 512, 129, 1]), (6, 2, 64, 4, 9, [40, 7, 16]), (4, 4, 256, 64, None, [300, 65]),
                          (16, 1, 128, 8, 100, [260, 1, 17, 16, 130]), (8, 2, 128, 16, None, [4100])])
def test_decode_attention_that_prepares_its_queries_and_keys(ops, monkeypatch, balanced, q_heads, kv_heads, head_dim, page_size, window, lengths):
    """One kernel (per-head norm of q and k, rotation, the new token appended to its page, attention) against the two
    that it replaces, on the same inputs: the attention rows and every byte of the cache must be equal, with either
    way of cutting the keys (equal ranges per request, merged through a buffer; one range per
    SM), heads of 64, 128 and 256, groups of 1 to 16, a window, pages smaller and larger than a key tile."""
    from types import SimpleNamespace

    monkeypatch.setenv("KIRAI_DECODE_BALANCED", balanced)
    dtype = torch.bfloat16
    requests = len(lengths)
    cache, table, keys, values = paged_setup(dtype, lengths, kv_heads, head_dim, page_size, seed=11)
    for r, n in enumerate(lengths):  # the tokens before the new one are in the pages already
        if n > 1:
            pos = torch.arange(n - 1, dtype=torch.int32, device=DEV)
            ops.kv_write(keys[r][: n - 1].to(DEV).contiguous(), values[r][: n - 1].to(DEV).contiguous(), cache, table,
                         torch.full((n - 1,), r, dtype=torch.int32, device=DEV), pos)
    width = (q_heads + 2 * kv_heads) * head_dim
    qkv = rand(requests, width, dtype=dtype, seed=5)
    q_weight, k_weight = 1.0 + 0.1 * rand(head_dim, seed=6), 1.0 + 0.1 * rand(head_dim, seed=7)
    inv_freq = torch.pow(torch.tensor(10000.0), -torch.arange(head_dim // 2, dtype=torch.float32) * 2.0 / head_dim).to(DEV)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    context_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    rows = torch.arange(requests, dtype=torch.int32, device=DEV)
    batch = SimpleNamespace(decode_only=True, num_requests=requests, context_len=context_len, max_context_len=max(lengths),
                            start_positions=[n - 1 for n in lengths], query_lens=[1] * requests, decode_balanced=None,
                            request_of_token=rows, positions=positions, num_decode=requests)
    scale = head_dim ** -0.5
    for weights in ((q_weight, k_weight, inv_freq), (None, None, inv_freq), (q_weight, k_weight, None)):
        qw, kw, freq = weights
        separate_cache, separate_qkv = cache.clone(), qkv.clone()
        ops.qk_norm_rope_kv_write_(separate_qkv, q_heads, kv_heads, head_dim, qw, kw, freq, 1e-6, separate_cache, table, rows, positions, True)
        q = separate_qkv[:, : q_heads * head_dim].unflatten(1, (q_heads, head_dim))
        expected = ops.paged_attention(q, separate_cache, table, batch, window, scale)
        fused_cache, fused_qkv = cache.clone(), qkv.clone()
        assert ops.decode_prepares_qk(fused_qkv, fused_cache, batch, q_heads, kv_heads, head_dim)
        crowd = SimpleNamespace(decode_only=True, num_requests=1 + ops.sm_count(torch.device(DEV)) // kv_heads)
        assert not ops.decode_prepares_qk(fused_qkv.expand(crowd.num_requests, -1) if requests == 1 else fused_qkv, fused_cache, crowd, q_heads, kv_heads, head_dim)
        got = ops.attention_decode_qk(fused_qkv, q_heads, kv_heads, head_dim, qw, kw, freq, 1e-6, fused_cache, table, batch, window, scale)
        ops.check_device_errors(torch.device(DEV))
        assert torch.equal(fused_qkv, qkv)                      # the product's rows are left as they were
        assert torch.equal(fused_cache, separate_cache)         # the same key and value rows, in the same places
        assert torch.equal(got, expected)
        assert float(got.float().abs().max()) > 0.01


def test_read_only_stream_kernel_runs_and_reports_nothing(ops):
    """The kernel that measures what a read-only stream reaches: whole 16 KB boxes only, no error word."""
    data = torch.zeros(37 * 16384, dtype=torch.uint8, device=DEV)  # fewer boxes than SMs: some CTAs have nothing to read
    ops.stream_read(data)
    ops.stream_read(torch.zeros(1000 * 16384, dtype=torch.uint8, device=DEV))
    ops.check_device_errors(torch.device(DEV))
    with pytest.raises(AssertionError):
        ops.stream_read(torch.zeros(1000, dtype=torch.uint8, device=DEV))


def test_sampler_on_the_cases_of_the_reference(ops):
    """crates/llm-sampler/src/lib.rs:222-294 through the device sampler, all rows in one launch: greedy, the first of
    equal maxima, a draw inside the nucleus, and ties inside the nucleus taken in index order."""
    from test_plain_reference import REFERENCE_TOP_P_CASES

    width = 4
    rows = [([-1.0, 0.25, 3.5, 3.0], 0.0, 1.0, 0.0, 2), ([1.0, 2.0, 2.0, -1e30], 0.0, 1.0, 0.0, 1)]
    rows += [(logits + [-1e30] * (width - len(logits)), t, p, draw, token) for logits, t, p, draw, token in REFERENCE_TOP_P_CASES]
    logits = torch.tensor([r[0] for r in rows], device=DEV)
    column = lambda i: torch.tensor([r[i] for r in rows], dtype=torch.float32, device=DEV)  # noqa: E731
    got = ops.sample_rows(logits, column(1), column(2), column(3)).tolist()
    assert got == [r[4] for r in rows]
    assert ops.argmax_rows(logits).tolist()[:2] == [2, 1]
    ops.check_device_errors(torch.device(DEV))


def test_a_row_without_a_maximum_sets_the_error_word_and_stays_in_bounds(ops):
    """All NaN or all -inf: no entry is greater than -inf.  Token 0 is written (nothing is read at a made-up index)
    and the device error word says so; rows beside it are sampled as usual."""
    logits = torch.randn(4, 300, device=DEV)
    logits[1] = float("nan")
    logits[2] = float("-inf")
    zeros, ones = torch.zeros(4, device=DEV), torch.ones(4, device=DEV)
    for temperature in (zeros, ones):
        got = ops.sample_rows(logits, temperature, ones, zeros + 0.5).tolist()
        assert got[1] == 0 and got[2] == 0 and 0 <= got[0] < 300 and 0 <= got[3] < 300
        with pytest.raises(ops.KernelError, match="no maximum"):
            ops.check_device_errors(torch.device(DEV))
    assert ops.argmax_rows(logits).tolist()[1:3] == [0, 0]
    with pytest.raises(ops.KernelError, match="no maximum"):
        ops.check_device_errors(torch.device(DEV))
    assert ops.argmax_rows(logits[:1]).tolist() == [int(logits[0].argmax())]
    ops.check_device_errors(torch.device(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads,kv_heads,head_dim,page_size,window",
                         [(6, 2, 48, 8, None), (5, 5, 16, 4, 7), (8, 1, 128, 16, 40), (3, 1, 80, 1, None)])
def test_kv_write_and_paged_attention(ops, dtype, q_heads, kv_heads, head_dim, page_size, window):
    lengths = [37, 5, 64]
    cache, table, keys, values = paged_setup(dtype, lengths, kv_heads, head_dim, page_size)
    # write every row through the kernel, in two uneven portions per request
    for cut in (0, 1):
        rows_k, rows_v, req, pos = [], [], [], []
        for r, n in enumerate(lengths):
            lo, hi = (0, n // 3) if cut == 0 else (n // 3, n)
            rows_k.append(keys[r][lo:hi]); rows_v.append(values[r][lo:hi])
            req += [r] * (hi - lo); pos += list(range(lo, hi))
        k_rows, v_rows = torch.cat(rows_k).to(DEV).contiguous(), torch.cat(rows_v).to(DEV).contiguous()
        ops.kv_write(k_rows, v_rows, cache, table, torch.tensor(req, dtype=torch.int32, device=DEV),
                     torch.tensor(pos, dtype=torch.int32, device=DEV))
    for r, n in enumerate(lengths):
        for p in (0, n - 1):
            page = int(table[r, p // page_size])
            assert torch.equal(cache[page, 0, :, p % page_size].cpu(), keys[r][p])
            assert torch.equal(cache[page, 1, :, p % page_size].cpu(), values[r][p])
    # queries: the last 9 positions of request 0, one of request 1, the last 2 of request 2
    spans = [(0, list(range(28, 37))), (1, [4]), (2, [62, 63])]
    generator = torch.Generator().manual_seed(9)
    q = torch.randn(sum(len(s[1]) for s in spans), q_heads, head_dim, generator=generator).to(dtype)
    req = [r for r, ps in spans for _ in ps]
    pos = [p for _, ps in spans for p in ps]
    scale = head_dim ** -0.5
    out = ops.paged_attention_plain(q.to(DEV), cache, table, torch.tensor(req, dtype=torch.int32, device=DEV),
                                    torch.tensor(pos, dtype=torch.int32, device=DEV), window, scale)
    ops.check_device_errors(torch.device(DEV))
    row = 0
    for r, ps in spans:
        expected = attention_reference(q[row : row + len(ps)], keys[r], values[r], ps, window, scale)
        got = out[row : row + len(ps)].float().cpu().unflatten(1, (q_heads, head_dim))
        assert float((got - expected).abs().max()) <= tol(dtype, 4.0)
        row += len(ps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads,kv_heads,head_dim", [(6, 2, 48), (4, 4, 16), (8, 2, 128), (2, 1, 512), (3, 1, 64), (5, 2, 256), (32, 8, 128)])
def test_fused_norm_rope_cache_write_equals_the_separate_kernels(ops, dtype, q_heads, kv_heads, head_dim):
    page_size, lengths = 8, [11, 30]
    cache_a, table, _, _ = paged_setup(dtype, lengths, kv_heads, head_dim, page_size)
    cache_b = cache_a.clone()
    rows = sum(lengths)
    qkv = rand(rows, (q_heads + 2 * kv_heads) * head_dim, dtype=dtype)
    req = torch.tensor([0] * 11 + [1] * 30, dtype=torch.int32, device=DEV)
    pos = torch.tensor(list(range(11)) + list(range(30)), dtype=torch.int32, device=DEV)
    qw, kw = 1.0 + 0.1 * rand(head_dim, seed=1), 1.0 + 0.1 * rand(head_dim, seed=2)
    inv_freq = torch.pow(torch.tensor(1e4), -(2.0 * torch.arange(head_dim // 2)) / head_dim).to(DEV)
    fused = qkv.clone()
    ops.qk_norm_rope_kv_write_(fused, q_heads, kv_heads, head_dim, qw, kw, inv_freq, 1e-6, cache_a, table, req, pos)
    separate = qkv.clone()
    nq, nkv, d = q_heads, kv_heads, head_dim
    q = separate[:, : nq * d].unflatten(1, (nq, d))
    k = separate[:, nq * d : (nq + nkv) * d].unflatten(1, (nkv, d))
    v = separate[:, (nq + nkv) * d :].unflatten(1, (nkv, d))
    ops.head_rmsnorm_(q, qw, 1e-6); ops.head_rmsnorm_(k, kw, 1e-6)
    ops.rope_(q, pos, inv_freq, d); ops.rope_(k, pos, inv_freq, d)
    ops.kv_write(k, v, cache_b, table, req, pos)
    ops.check_device_errors(torch.device(DEV))
    # the fused kernel keeps the normed value in 32-bit where the separate kernels round in between
    bound = 0.0 if dtype == torch.float32 else 0.05
    assert float((fused.float() - separate.float()).abs().max()) <= bound + 1e-6
    assert float((cache_a.float() - cache_b.float()).abs().max()) <= bound + 1e-6
    # against the formulas in 32-bit
    x = qkv.float()[:, : nq * d].unflatten(1, (nq, d))
    normed = x * torch.rsqrt((x ** 2).mean(-1, keepdim=True) + 1e-6) * qw
    expected = rope_reference(normed, pos, inv_freq, d)
    assert float((fused[:, : nq * d].float().unflatten(1, (nq, d)) - expected).abs().max()) <= tol(dtype, float(expected.abs().max()))


@pytest.mark.parametrize("vocab", [130, 257, 1000, 151936])  # 130: one block per row; the others: a row over a cluster of CTAs
def test_argmax_and_sampling(ops, vocab):
    import plain_qwen3 as plain

    generator = torch.Generator().manual_seed(vocab)
    logits = torch.randn(6, vocab, generator=generator) * 3.0
    logits[0, 5] = logits[0, 77] = 50.0        # a tie: the lower index wins
    logits[1, vocab - 1] = 60.0                # the last entry
    dev = logits.to(DEV)
    assert ops.argmax_rows(dev).tolist() == [plain.argmax_first(row) for row in logits]
    temperatures = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.7, 2.0])
    top_ps = torch.tensor([1.0, 1.0, 0.9, 0.5, 0.05, 1.0])
    # Exact bookkeeping in 64-bit: the order, the running sums and the nucleus of every sampled row.
    exact = {}
    for row in range(1, 6):
        probs = torch.softmax(logits[row].double() / float(temperatures[row]), 0)
        order = torch.argsort(-probs, stable=True)
        running = torch.cumsum(probs[order], 0)
        top_p = float(top_ps[row])
        last = int(torch.searchsorted(running, torch.tensor(top_p, dtype=torch.float64))) if top_p < 1.0 else vocab - 1
        last = min(last, vocab - 1)
        rank = torch.empty(vocab, dtype=torch.long)
        rank[order] = torch.arange(vocab)
        exact[row] = (running, float(running[last]), rank)
    # 32-bit sums over a whole vocabulary carry about sqrt(V) * 2^-24 of rounding, whatever their order
    slack = 1e-4
    for draw in (0.0, 0.25, 0.5, 0.83, 0.999999):
        draws = torch.full((6,), draw)
        got = ops.sample_rows(dev, temperatures.to(DEV), top_ps.to(DEV), draws.to(DEV)).tolist()
        assert got[0] == plain.argmax_first(logits[0])
        for row in range(1, 6):
            running, total, rank = exact[row]
            place = int(rank[got[row]])
            threshold = draw * total
            before = float(running[place - 1]) if place > 0 else 0.0
            assert before - slack <= threshold <= float(running[place]) + slack, (row, draw, got[row])
            if vocab <= 1000:  # small enough that the sequential 32-bit walk of the plain implementation is exact too
                expected = plain.sample_top_p(logits[row], float(temperatures[row]), float(top_ps[row]), draw)
                assert abs(place - int(rank[expected])) <= 1, (row, draw, got[row], expected)


@pytest.mark.parametrize("vocab", [200, 1024, 4104])  # 200: one block per row; the others: a row over a cluster of CTAs
def test_sampling_among_many_equal_probabilities(ops, vocab):
    """Logits that take four values only: most entries tie with hundreds of others, inside the nucleus and at its
    edge.  Equal probabilities are ordered by index.  For every draw the sampled entry's stretch of the exact running
    sum in that order must hold the threshold, up to the rounding of 32-bit sums (ties enter the kernel's sum one by
    one, as the reference's sequential walk adds them, and a thousand additions of one small value round the same
    way each time); with top-p the entry must lie inside the exact nucleus, up to the same rounding."""
    generator = torch.Generator().manual_seed(vocab)
    logits = torch.randint(0, 4, (4, vocab), generator=generator).float()
    temperatures = torch.tensor([1.0, 0.5, 1.0, 2.0])
    top_ps = torch.tensor([1.0, 1.0, 0.6, 0.3])
    dev = logits.to(DEV)
    for draw in (0.0, 0.1, 0.37, 0.5, 0.75, 0.93, 0.999999):
        got = ops.sample_rows(dev, temperatures.to(DEV), top_ps.to(DEV), torch.full((4,), draw).to(DEV)).tolist()
        for row in range(4):
            probs = torch.softmax(logits[row].double() / float(temperatures[row]), 0)
            order = torch.argsort(-probs, stable=True)  # ties by index
            running = torch.cumsum(probs[order], 0)
            top_p = float(top_ps[row])
            last = vocab - 1 if top_p >= 1.0 else min(int(torch.searchsorted(running, torch.tensor(top_p, dtype=torch.float64))), vocab - 1)
            threshold = draw * float(running[last])
            rank = torch.empty(vocab, dtype=torch.long)
            rank[order] = torch.arange(vocab)
            place = int(rank[got[row]])
            before = float(running[place - 1]) if place > 0 else 0.0
            slack = 1e-4
            assert before - slack <= threshold <= float(running[place]) + slack, (row, draw, got[row], place)
            assert before <= float(running[last]) + slack, (row, draw, got[row], place, last)  # inside the nucleus
    ops.check_device_errors(torch.device(DEV))


@pytest.mark.parametrize("q_heads,kv_heads,head_dim,page_size,window",
                         [(6, 2, 48, 8, None), (5, 5, 16, 4, 7), (8, 2, 128, 16, 40), (32, 8, 128, 16, None),
                          (3, 1, 80, 1, None), (4, 2, 256, 64, 33), (16, 1, 64, 16, None),
                          # how the tcgen05 kernel fetches a page: whole rows in one request (head sizes 64 and 128,
                          # pages of 8 tokens and more, up to more than a tile), else panel by panel, 8 rows at most
                          (4, 2, 96, 32, None), (8, 4, 80, 4, 9), (8, 2, 128, 64, None), (4, 1, 128, 128, 50),
                          (2, 2, 64, 8, None), (2, 1, 192, 16, None)])
def test_tensor_core_attention_against_plain(ops, q_heads, kv_heads, head_dim, page_size, window):
    """Prompt portions that start in the middle of a context, and single decoded tokens, through the
    tensor-core kernels and through the plain kernel, against 32-bit arithmetic."""
    dtype = torch.bfloat16
    lengths = [150, 5, 64, 300]
    cache, table, keys, values = paged_setup(dtype, lengths, kv_heads, head_dim, page_size, seed=3)
    for r, n in enumerate(lengths):
        pos = torch.arange(n, dtype=torch.int32, device=DEV)
        ops.kv_write(keys[r].to(DEV).contiguous(), values[r].to(DEV).contiguous(), cache, table,
                     torch.full((n,), r, dtype=torch.int32, device=DEV), pos)
    scale = head_dim ** -0.5
    generator = torch.Generator().manual_seed(4)
    # mixed: the last 71 tokens of request 0, the whole of 1, one token of 2, the last 130 of 3
    spans = [(0, 150 - 71, 71), (1, 0, 5), (2, 63, 1), (3, 170, 130)]
    total = sum(s[2] for s in spans)
    q = (torch.randn(total, q_heads, head_dim, generator=generator) * 2.0).to(dtype).to(DEV)
    query_start = torch.tensor([0] + list(torch.tensor([s[2] for s in spans]).cumsum(0)), dtype=torch.int32, device=DEV)
    context_len = torch.tensor([s[1] + s[2] for s in spans], dtype=torch.int32, device=DEV)
    req = torch.tensor([i for i, s in enumerate(spans) for _ in range(s[2])], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for s in spans for p in range(s[1], s[1] + s[2])], dtype=torch.int32, device=DEV)
    # only the keys up to each request's context length count: later rows are in the pages but masked
    plain = ops.paged_attention_plain(q, cache, table, req, pos, window, scale)
    kernels = [False] + ([True] if ops.attention_prefill_takes_tcgen05(q_heads, kv_heads, head_dim, page_size) else [])
    for use_tcgen05 in kernels:  # the warp-level mma.sync kernel, and the tcgen05 kernel where it takes the shape
        fast = ops.attention_prefill(q, cache, table, query_start, context_len, max(s[2] for s in spans), window, scale,
                                     tcgen05=use_tcgen05)
        ops.check_device_errors(torch.device(DEV))
        row = 0
        for r, first, count in spans:
            expected = attention_reference(q[row : row + count].cpu(), keys[r], values[r], list(range(first, first + count)), window, scale)
            got = fast[row : row + count].float().cpu().unflatten(1, (q_heads, head_dim))
            assert float((got - expected).abs().max()) <= 2.5e-2, (use_tcgen05, r, first, count)
            row += count
        assert float((fast.float() - plain.float()).abs().max()) <= 2.5e-2
    # decode: one token per request at the end of each context, with 1, 2 and 5 splits
    if q_heads // kv_heads <= 16:
        ends = [n - 1 for n in lengths]
        qd = (torch.randn(len(lengths), q_heads, head_dim, generator=generator) * 2.0).to(dtype).to(DEV)
        ctx = torch.tensor(lengths, dtype=torch.int32, device=DEV)
        for splits in (1, 2, 5):
            got = ops.attention_decode(qd, cache, table, ctx, window, scale, splits).float().cpu().unflatten(1, (q_heads, head_dim))
            ops.check_device_errors(torch.device(DEV))
            for r, end in enumerate(ends):
                expected = attention_reference(qd[r : r + 1].cpu(), keys[r], values[r], [end], window, scale)
                assert float((got[r : r + 1] - expected).abs().max()) <= 2.5e-2, (r, splits)
        # the same with the keys of all (request, kv head) pairs cut into equal ranges: one CTA that walks through
        # every pair, a few CTAs whose borders cut pairs in two or more pieces, more CTAs than there are tiles
        for ctas in (1, 3, 7, 148, 1000):
            got = ops.attention_decode_balanced(qd, cache, table, ctx, window, scale, ctas).float().cpu().unflatten(1, (q_heads, head_dim))
            ops.check_device_errors(torch.device(DEV))
            for r, end in enumerate(ends):
                expected = attention_reference(qd[r : r + 1].cpu(), keys[r], values[r], [end], window, scale)
                assert float((got[r : r + 1] - expected).abs().max()) <= 2.5e-2, (r, ctas)


def test_prompt_attention_of_thousands_of_tokens_with_both_kernels(ops):
    """A prompt long enough that hundreds of CTAs each walk dozens of key tiles: the pipelines' barriers go through
    many phases (a wait that skipped a phase once stalled only at this size), and the two kernels must agree."""
    dtype, q_heads, kv_heads, head_dim, page_size, tokens = torch.bfloat16, 8, 2, 128, 16, 4096
    pages = tokens // page_size + 1
    generator = torch.Generator().manual_seed(9)
    cache = (torch.randn(pages, 2, kv_heads, page_size, head_dim, generator=generator) * 0.5).to(dtype).to(DEV)
    table = torch.arange(pages, dtype=torch.int32, device=DEV)[None, :].contiguous()
    q = (torch.randn(tokens, q_heads, head_dim, generator=generator)).to(dtype).to(DEV)
    qs = torch.tensor([0, tokens], dtype=torch.int32, device=DEV)
    ctx = torch.tensor([tokens], dtype=torch.int32, device=DEV)
    scale = head_dim ** -0.5
    for _ in range(3):  # the stall was a matter of timing: several launches
        fast = ops.attention_prefill(q, cache, table, qs, ctx, tokens, None, scale, tcgen05=True)
        ops.check_device_errors(torch.device(DEV))
    slow = ops.attention_prefill(q, cache, table, qs, ctx, tokens, None, scale, tcgen05=False)
    ops.check_device_errors(torch.device(DEV))
    assert float((fast.float() - slow.float()).abs().max()) <= 2.5e-2
    # a few rows against 32-bit arithmetic
    keys = cache[:, 0].permute(0, 2, 1, 3).reshape(-1, kv_heads, head_dim)[:tokens].float().cpu()
    values = cache[:, 1].permute(0, 2, 1, 3).reshape(-1, kv_heads, head_dim)[:tokens].float().cpu()
    for row in (0, 63, 64, 2047, 4095):
        expected = attention_reference(q[row : row + 1].cpu(), keys.to(dtype), values.to(dtype), [row], None, scale)
        got = fast[row : row + 1].float().cpu().unflatten(1, (q_heads, head_dim))
        assert float((got - expected).abs().max()) <= 2.5e-2, row


def test_tensor_core_attention_finds_a_far_key(ops):
    """One key among hundreds, far back and on a page edge, is made to dominate: the output must be its value."""
    dtype, q_heads, kv_heads, head_dim, page_size = torch.bfloat16, 8, 2, 128, 16
    lengths = [777]
    cache, table, keys, values = paged_setup(dtype, lengths, kv_heads, head_dim, page_size, seed=8)
    far = 16 * 3  # first row of the fourth page
    direction = torch.randn(head_dim, generator=torch.Generator().manual_seed(1))
    direction = direction / direction.norm()
    keys[0][far] = (direction * 30.0).to(dtype)
    ops.kv_write(keys[0].to(DEV).contiguous(), values[0].to(DEV).contiguous(), cache, table,
                 torch.zeros(777, dtype=torch.int32, device=DEV), torch.arange(777, dtype=torch.int32, device=DEV))
    q = (direction * 30.0).to(dtype).repeat(1, q_heads, 1).to(DEV)
    ctx = torch.tensor([777], dtype=torch.int32, device=DEV)
    for splits in (1, 4):
        out = ops.attention_decode(q, cache, table, ctx, None, head_dim ** -0.5, splits).float().cpu().unflatten(1, (q_heads, head_dim))
        for head in range(q_heads):
            assert float((out[0, head] - values[0][far, head // 4].float()).abs().max()) <= 2e-2
    for ctas in (2, 5, 148):
        out = ops.attention_decode_balanced(q, cache, table, ctx, None, head_dim ** -0.5, ctas).float().cpu().unflatten(1, (q_heads, head_dim))
        for head in range(q_heads):
            assert float((out[0, head] - values[0][far, head // 4].float()).abs().max()) <= 2e-2, ctas
    qs = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    out = ops.attention_prefill(q, cache, table, qs, ctx, 1, None, head_dim ** -0.5).float().cpu().unflatten(1, (q_heads, head_dim))
    assert float((out[0, 0] - values[0][far, 0].float()).abs().max()) <= 2e-2
    # with a window that ends one short of the far key it must vanish from the result
    out = ops.attention_decode(q, cache, table, ctx, 777 - far - 1, head_dim ** -0.5, 2).float().cpu().unflatten(1, (q_heads, head_dim))
    assert float((out[0, 0] - values[0][far, 0].float()).abs().max()) > 0.5
    out = ops.attention_decode(q, cache, table, ctx, 777 - far, head_dim ** -0.5, 2).float().cpu().unflatten(1, (q_heads, head_dim))
    assert float((out[0, 0] - values[0][far, 0].float()).abs().max()) <= 2e-2


@pytest.mark.parametrize("q_heads,kv_heads,head_dim", [(8, 2, 128), (32, 2, 64), (3, 1, 256)])
def test_decode_attention_cut_into_any_number_of_ranges(ops, q_heads, kv_heads, head_dim):
    """Every number of ranges from 2 to 18 and some beyond (more ranges than key tiles too: the empty ones must not
    count) against one range, whose result needs no merge: the merge may differ from it by rounding only."""
    dtype, page_size, length = torch.bfloat16, 16, 1500
    cache, table, keys, values = paged_setup(dtype, [length], kv_heads, head_dim, page_size, seed=21)
    ops.kv_write(keys[0].to(DEV).contiguous(), values[0].to(DEV).contiguous(), cache, table,
                 torch.zeros(length, dtype=torch.int32, device=DEV), torch.arange(length, dtype=torch.int32, device=DEV))
    q = rand(1, q_heads, head_dim, dtype=dtype, seed=22)
    ctx = torch.tensor([length], dtype=torch.int32, device=DEV)
    scale = head_dim ** -0.5
    one = ops.attention_decode(q, cache, table, ctx, None, scale, 1).float()
    plain = ops.paged_attention_plain(q, cache, table, torch.zeros(1, dtype=torch.int32, device=DEV),
                                      torch.tensor([length - 1], dtype=torch.int32, device=DEV), None, scale).float()
    assert float((one - plain).abs().max()) <= 2.5e-2
    for splits in list(range(2, 19)) + [33, 64, 100]:
        got = ops.attention_decode(q, cache, table, ctx, None, scale, splits)
        assert float((got.float() - one).abs().max()) <= 1e-2, splits
    ops.check_device_errors(q.device)


@pytest.mark.parametrize("m,inter,k,splits", [(1, 128, 64, 0), (5, 200, 136, 0), (16, 1000, 512, 3), (64, 1536, 1032, 8),
                                              (65, 264, 192, 0), (128, 1536, 1032, 0), (100, 6144, 1024, 3), (250, 1536, 2048, 2),
                                              (300, 1000, 520, 0), (1024, 768, 256, 0)])
def test_linear_swiglu_epilogue(ops, m, inter, k, splits):
    x = rand(m, k, dtype=torch.bfloat16, scale=0.5)
    gate, up = rand(inter, k, dtype=torch.bfloat16, scale=0.1, seed=3), rand(inter, k, dtype=torch.bfloat16, scale=0.1, seed=4)
    weight = ops.interleave_gate_up(gate, up)
    assert torch.equal(weight[:8], gate[:8]) and torch.equal(weight[8:16], up[:8]) and torch.equal(weight[16:24], gate[8:16])
    g, u = x.float() @ gate.float().T, x.float() @ up.float().T
    expected = g / (1.0 + torch.exp(-g)) * u
    out = ops.linear_tcgen05(x, weight, splits=splits, swiglu=True)
    ops.check_device_errors(torch.device(DEV))
    assert out.shape == (m, inter)
    assert float((out.float() - expected).abs().max()) <= 1e-2 * float(expected.abs().max())
    separate = ops.swiglu(ops.linear_tcgen05(x, torch.cat([gate, up])))  # rounds gate and up to bf16 in between
    assert float((out.float() - separate.float()).abs().max()) <= 2e-2 * float(expected.abs().max())
    assert torch.equal(ops.linear_tcgen05(x, ops.tile_weight(weight), splits=splits, swiglu=True), out)
    ops.check_device_errors(torch.device(DEV))


@pytest.mark.parametrize("m,n,k,splits", [(1, 128, 64, 0), (5, 200, 136, 0), (16, 1000, 512, 3), (40, 520, 1032, 4),
                                          (64, 1536, 264, 0), (65, 264, 192, 0), (128, 4096, 1032, 3), (70, 520, 2048, 2),
                                          (256, 1024, 2048, 3), (180, 520, 520, 0), (300, 1000, 520, 0), (1024, 768, 256, 0)])
def test_linear_residual_norm_epilogue_and_row_scaled_products(ops, m, n, k, splits):
    """The product whose epilogue adds into the 32-bit stream and leaves the next norm's rows without their
    1 / rms factor, and the products that apply that factor to their result, against the formulas."""
    eps = 1e-5
    x, w = rand(m, k, dtype=torch.bfloat16, scale=0.5), rand(n, k, dtype=torch.bfloat16, scale=0.1, seed=3)
    before = rand(m, n, scale=2.0, seed=5)
    norm_weight = (1.0 + 0.3 * rand(n, seed=6)).contiguous()
    resid = before.clone()
    rows, sumsq = ops.linear_residual_norm(x, w, resid, norm_weight, splits)
    ops.check_device_errors(torch.device(DEV))
    stream = before.double() + x.double() @ w.double().T
    assert float((resid.double() - stream).abs().max()) <= 1e-5 * float(stream.abs().max())
    unscaled = stream * norm_weight.double()
    assert float((rows.double() - unscaled).abs().max()) <= 5e-3 * float(unscaled.abs().max())
    assert sumsq.shape[1] == m
    total = (stream ** 2).sum(1)
    assert float(((sumsq.double().sum(0) - total) / total).abs().max()) <= 1e-5
    again = before.clone()
    rows_tiled, sumsq_tiled = ops.linear_residual_norm(x, ops.tile_weight(w), again, norm_weight, splits)
    assert torch.equal(rows_tiled, rows) and torch.equal(sumsq_tiled, sumsq) and torch.equal(again, resid)
    # the products that follow: plain (both output types) and with the SwiGLU epilogue
    normed = unscaled * torch.rsqrt((stream ** 2).mean(1, keepdim=True) + eps)
    width = 272
    w2 = rand(width, n, dtype=torch.bfloat16, scale=0.1, seed=7)
    expected = (normed @ w2.double().T).float()
    bound = 1e-2 * float(expected.abs().max())
    for out_dtype in (torch.bfloat16, torch.float32):
        out = ops.linear_tcgen05(rows, w2, out_dtype, row_scale=(sumsq, n, eps))
        assert out.dtype == out_dtype and float((out.float() - expected).abs().max()) <= bound
    gate, up = w2[: width // 2].contiguous(), w2[width // 2:].contiguous()
    g, u = expected[:, : width // 2], expected[:, width // 2:]
    expected_act = g / (1.0 + torch.exp(-g)) * u
    act = ops.linear_tcgen05(rows, ops.interleave_gate_up(gate, up), swiglu=True, row_scale=(sumsq, n, eps))
    assert float((act.float() - expected_act).abs().max()) <= 1e-2 * float(expected_act.abs().max())
    # and against the separate kernels of the same path: add + norm, then the product
    separate_stream = before.clone()
    delta = ops.linear_tcgen05(x, w)
    separate = ops.linear_tcgen05(ops.add_rmsnorm(separate_stream, delta, norm_weight, eps, torch.bfloat16), w2, torch.float32)
    ops.check_device_errors(torch.device(DEV))
    assert float((separate - expected).abs().max()) <= 2 * bound


def test_row_scaled_product_of_a_zero_row_is_zero(ops):
    """A row whose variance plus eps is 0 gets the scale 0, as the norm kernel gives it, not a NaN."""
    m, n, k = 3, 64, 32
    x, w = torch.zeros(m, k, dtype=torch.bfloat16, device=DEV), rand(n, k, dtype=torch.bfloat16)
    resid = torch.zeros(m, n, device=DEV)
    resid[1] = 1.0
    rows, sumsq = ops.linear_residual_norm(x, w, resid, torch.ones(n, device=DEV))
    out = ops.linear_tcgen05(rows, rand(16, n, dtype=torch.bfloat16, seed=2), torch.float32, row_scale=(sumsq, n, 0.0))
    assert torch.isfinite(out).all() and float(out[0].abs().max()) == 0.0 and float(out[2].abs().max()) == 0.0
    assert float(out[1].abs().max()) > 0.0


def test_attention_with_block_tables_longer_than_the_shared_copy(ops):
    """Contexts whose block tables exceed what the kernels keep in shared memory (1,024 entries) read
    the table from global memory instead; a key near the start and one near the end must both be found."""
    dtype, q_heads, kv_heads, head_dim, page_size = torch.bfloat16, 4, 1, 64, 4
    length = 4 * 1100 + 3  # 1,101 pages
    cache, table, keys, values = paged_setup(dtype, [length], kv_heads, head_dim, page_size, seed=11)
    direction = torch.randn(head_dim, generator=torch.Generator().manual_seed(2))
    direction = direction / direction.norm()
    for marked in (5, length - 9):
        keys[0][marked] = (direction * 40.0).to(dtype)
    ops.kv_write(keys[0].to(DEV).contiguous(), values[0].to(DEV).contiguous(), cache, table,
                 torch.zeros(length, dtype=torch.int32, device=DEV), torch.arange(length, dtype=torch.int32, device=DEV))
    expected = 0.5 * (values[0][5, 0].float() + values[0][length - 9, 0].float())  # two equal scores dominate
    q = (direction * 40.0).to(dtype).repeat(1, q_heads, 1).to(DEV)
    ctx = torch.tensor([length], dtype=torch.int32, device=DEV)
    scale = head_dim ** -0.5
    for splits in (1, 3):
        out = ops.attention_decode(q, cache, table, ctx, None, scale, splits).float().cpu().unflatten(1, (q_heads, head_dim))
        assert float((out[0, 0] - expected).abs().max()) <= 3e-2, splits
    for ctas in (1, 2):  # ranges of more than 1,024 pages
        out = ops.attention_decode_balanced(q, cache, table, ctx, None, scale, ctas).float().cpu().unflatten(1, (q_heads, head_dim))
        assert float((out[0, 0] - expected).abs().max()) <= 3e-2, ctas
    qs = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    for use_tcgen05 in (False, True):
        out = ops.attention_prefill(q, cache, table, qs, ctx, 1, None, scale, tcgen05=use_tcgen05).float().cpu().unflatten(1, (q_heads, head_dim))
        assert float((out[0, 0] - expected).abs().max()) <= 3e-2, use_tcgen05
    ops.check_device_errors(torch.device(DEV))
