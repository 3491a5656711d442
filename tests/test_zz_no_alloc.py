"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called through
its exported C symbol and compared with the ordinary entry point.

The ordinary entry point takes a scratch buffer for the splits' partial results from its
caller; this one keeps the scratch in a fixed array inside the library, for callers that
cannot allocate device memory while they run (no allocator of their own and a device whose
memory is already handed out, or a rule against allocating after start-up).  The test makes
every buffer itself, so the only memory the call under test could add would be its own.
Two calls in a row, of different sizes, share the array: the second must not be disturbed by
what the first left there.  This file sorts last on purpose, so that a run that stops at the
first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_case(requests, q_heads, kv_heads, head_dim, page_size, lengths, seed):
    generator = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page_size) for n in lengths]
    num_pages = sum(pages_per) + 2
    order = torch.randperm(num_pages, generator=generator).tolist()
    cache = torch.randn(num_pages, 2, kv_heads, page_size, head_dim, generator=generator).to(torch.bfloat16).to(DEV)
    table = torch.full((requests, max(pages_per)), -1, dtype=torch.int32)
    cursor = 0
    for r in range(requests):
        for p in range(pages_per[r]):
            table[r, p] = order[cursor]
            cursor += 1
    q = (torch.randn(requests, q_heads, head_dim, generator=generator) * 2.0).to(torch.bfloat16).to(DEV)
    return q, cache, table.to(DEV), torch.tensor(lengths, dtype=torch.int32, device=DEV)


def call(lib, name, q, cache, table, ctx, splits, partial=None, with_partial=False):
    requests, q_heads, head_dim = q.shape
    num_pages, _, kv_heads, page_size, _ = cache.shape
    out = torch.zeros(requests, q_heads * head_dim, dtype=torch.bfloat16, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    p = ctypes.c_void_p
    args = [p(q.data_ptr()), p(cache.data_ptr()), p(out.data_ptr())]
    if with_partial:
        args.append(p(partial.data_ptr() if partial is not None else 0))
    args += [p(table.data_ptr()), p(ctx.data_ptr()), ctypes.c_int(requests), ctypes.c_int(q_heads), ctypes.c_int(kv_heads),
             ctypes.c_int(head_dim), ctypes.c_long(q.stride(0)), ctypes.c_int(page_size), ctypes.c_int(table.shape[1]),
             ctypes.c_int(num_pages), ctypes.c_int(0), ctypes.c_float(head_dim ** -0.5), ctypes.c_int(splits),
             p(flag.data_ptr()), p(torch.cuda.current_stream().cuda_stream)]
    fn = getattr(lib, name)
    fn.restype = ctypes.c_int
    status = fn(*args)
    torch.cuda.synchronize()
    return status, out, int(flag.item())


def test_static_scratch_entry_point_matches_the_allocating_one():
    import kirai_b200  # noqa: F401
    from kirai_b200.csrc import ops

    lib = ops.library()
    lib.kirai_static_scratch_capacity_floats.restype = ctypes.c_uint
    capacity = lib.kirai_static_scratch_capacity_floats()
    assert capacity == 1 << 20
    cases = [  # two calls in a row on the shared array: the second is smaller and must not see the first's leftovers
        dict(requests=5, q_heads=8, kv_heads=2, head_dim=128, page_size=16, lengths=[700, 33, 512, 129, 1], splits=4, seed=1),
        dict(requests=2, q_heads=6, kv_heads=2, head_dim=48, page_size=8, lengths=[90, 300], splits=3, seed=2),
    ]
    for case in cases:
        splits = case.pop("splits")
        q, cache, table, ctx = make_case(**case)
        requests, q_heads, head_dim = q.shape
        assert requests * q_heads * splits * (head_dim + 2) <= capacity
        partial = torch.empty(requests, q_heads, splits, head_dim + 2, dtype=torch.float32, device=DEV)
        status_a, expected, flag_a = call(lib, "kirai_attention_decode_bf16", q, cache, table, ctx, splits, partial, True)
        status_b, got, flag_b = call(lib, "kirai_attention_decode_bf16_static_scratch", q, cache, table, ctx, splits)
        assert (status_a, flag_a) == (0, 0) and (status_b, flag_b) == (0, 0)
        assert float(expected.float().abs().max()) > 0.1  # the kernels did write something
        # same kernels, same split boundaries, same order of additions: equal bit for bit
        assert torch.equal(got, expected)
        # and against the single-split run, which uses no scratch at all
        _, single, _ = call(lib, "kirai_attention_decode_bf16_static_scratch", q, cache, table, ctx, 1)
        assert float((got.float() - single.float()).abs().max()) <= 2.5e-2


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    import kirai_b200  # noqa: F401
    from kirai_b200.csrc import ops

    lib = ops.library()
    q, cache, table, ctx = make_case(requests=64, q_heads=32, kv_heads=8, head_dim=128, page_size=16, lengths=[40] * 64, seed=3)
    # 64 * 32 * 5 * 130 floats exceed the 2^20 of the array: refused before any launch
    status, out, flag = call(lib, "kirai_attention_decode_bf16_static_scratch", q, cache, table, ctx, 5)
    assert status == -5 and flag == 0 and float(out.float().abs().max()) == 0.0
    status, out, flag = call(lib, "kirai_attention_decode_bf16_static_scratch", q, cache, table, ctx, 3)
    assert status == 0 and flag == 0 and float(out.float().abs().max()) > 0.1
