"""Python bindings of the hand-written CUDA kernels.

Every function takes torch tensors that live on a CUDA device, checks dtypes,
shapes and strides on the host, and launches on torch's current stream through
the library's ``extern "C"`` entry points.  There is no CPU fallback: a tensor
on another device, or a missing library, is an error.

Kernels that can meet a bad index (a token id outside the vocabulary, a block
table entry without a page) do not fault: they skip the access and set a device
flag that ``check_device_errors`` reads.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_lib = None
_error_flags = {}

_ERROR_NAMES = {
    1: "a token id is outside the vocabulary",
    2: "a token's position has no page in its request's block table (cache write)",
    3: "a key position has no page in its request's block table (attention read)",
    4: "a bounded wait inside a kernel ran out",
    5: "a row of logits has no maximum (every entry is NaN or -inf); token 0 was written for it",
}

_REFUSALS = {
    -2: "a size is outside what the kernel takes",
    -3: "a pointer or stride is not aligned as the kernel needs",
    -4: "this combination of options is not built",
}


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The shared library, built on first use."""
    global _lib
    if _lib is None:
        path = _build.build()
        _lib = ctypes.CDLL(path)
    return _lib


def _check(status: int, name: str) -> None:
    if status == 0:
        return
    if status in _REFUSALS:
        raise KernelError(f"{name}: refused: {_REFUSALS[status]}")
    raise KernelError(f"{name}: CUDA error {status} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current device's current stream.  Asked of the library's C entry points where it has them: the public
    call builds a stream object on the way and took 5 us of the 25 us that a launch cost the host."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"kernels take float32 or bfloat16 activations, got {dtype}")


launch_count = 0  # entry points called so far (each launches one to three kernels); read by measurements
launch_counts: dict = {}  # the same by entry point: which kernels a step used, and how often (Engine.stats reports it)


def _call(name: str, *args) -> None:
    """Launches one entry point on the current stream.  Products that were held back to be launched together
    (see ``chained_products``) go first: launches keep the order in which they were asked for."""
    if _pending:
        flush_products()
    _launch(name, *args)


def _launch(name: str, *args) -> None:
    global launch_count
    fn = getattr(library(), name)
    fn.restype = ctypes.c_int
    _check(fn(*args), name)
    launch_count += 1
    launch_counts[name] = launch_counts.get(name, 0) + 1


_i = ctypes.c_int
_l = ctypes.c_long
_f = ctypes.c_float


def error_flag(device: torch.device) -> torch.Tensor:
    """The int32 device word that kernels set instead of faulting."""
    key = torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _error_flags[key]


def check_device_errors(device: torch.device) -> None:
    """Reads the device flag (synchronises) and raises if a kernel set it."""
    flag = error_flag(device)
    value = int(flag.item())
    if value != 0:
        flag.zero_()
        if value == 4:  # a kernel gave up in mid-work: counters that it shares with its next launch start from zero again
            for workspace in _chain_workspaces.values():
                workspace.zero_()
        raise KernelError(f"a kernel reported: {_ERROR_NAMES.get(value, f'error {value}')}")


def wait_selftest(device: torch.device, limit: int = 10_000, arrive: bool = False) -> int:
    """Launches the self-test of the bounded waits: a kernel that waits, at most ``limit`` polls, for a barrier on
    which nothing arrives (or, with ``arrive``, on which another thread does).  A wait that runs out sets the device
    error word, which ``check_device_errors`` turns into a KernelError; the kernel returns either way.  Returns the
    number of polls after which the wait gave up (0 if it was answered)."""
    polls = torch.zeros(1, dtype=torch.int32, device=device)
    _call("kirai_wait_selftest", ctypes.c_uint(limit), _i(1 if arrive else 0), _ptr(error_flag(device)), _ptr(polls), _stream())
    return int(polls.item())


def stream_read(data: torch.Tensor) -> None:
    """Reads ``data`` (a multiple of 16 KB) once, one CTA per SM, with bulk copies into shared memory, and drops it: a
    measurement of what a read-only stream reaches on this device (time it with CUDA events)."""
    _need_cuda(data)
    assert data.is_contiguous() and (data.numel() * data.element_size()) % 16384 == 0
    _call("kirai_stream_read", _ptr(data), _l(data.numel() * data.element_size()), _i(sm_count(data.device)),
          _ptr(error_flag(data.device)), _stream())


# ------------------------------------------------------------------- embedding
def embedding(table, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ``ids`` of ``table`` [V, H] (a tensor, or a ``TiledWeight`` shared with the output head) widened to
    the 32-bit residual stream [T, H]."""
    assert ids.dtype == torch.int32 and ids.is_contiguous()
    tokens, hidden = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    if isinstance(table, TiledWeight):
        _need_cuda(table.boxes, ids)
        _call("kirai_embedding_tiled_bf16", _ptr(table.boxes), _ptr(ids), _ptr(out), _i(tokens), _i(hidden),
              _i(table.shape[0]), _ptr(error_flag(table.device)), _stream())
        return out
    _need_cuda(table, ids)
    assert table.dim() == 2 and table.is_contiguous()
    _call(f"kirai_embedding_{_suffix(table.dtype)}", _ptr(table), _ptr(ids), _ptr(out), _i(tokens), _i(hidden),
          _i(table.shape[0]), _ptr(error_flag(table.device)), _stream())
    return out


# --------------------------------------------------------------------- RMSNorm
def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None):
    """``resid += delta`` (32-bit, in place), then RMSNorm of the sum in ``out_dtype``.

    With ``row_index`` only those rows are produced; the residual stream is left as it
    is and the summed rows are returned as the second value.
    """
    _need_cuda(resid, delta, weight, row_index)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == resid.shape[1]
    hidden = resid.shape[1]
    if delta is not None:
        assert delta.shape == resid.shape and delta.dtype == out_dtype and delta.is_contiguous()
    rows = resid.shape[0] if row_index is None else row_index.numel()
    out = torch.empty((rows, hidden), dtype=out_dtype, device=resid.device)
    summed = None
    if row_index is not None:
        assert row_index.dtype == torch.int32 and row_index.is_contiguous()
        summed = torch.empty((rows, hidden), dtype=torch.float32, device=resid.device)
    _call(f"kirai_add_rmsnorm_{_suffix(out_dtype)}", _ptr(resid), _ptr(delta), _ptr(weight), _ptr(out),
          _ptr(row_index), _ptr(summed), _i(rows), _i(hidden), _f(eps), _stream())
    return (out, summed) if row_index is not None else out


def add_into_residual(resid: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """``resid`` (32-bit) += ``delta``, in place."""
    _need_cuda(resid, delta)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and delta.is_contiguous() and delta.shape == resid.shape
    _call(f"kirai_add_residual_{_suffix(delta.dtype)}", _ptr(resid), _ptr(delta), _l(resid.numel()), _stream())
    return resid


def _head_view(x: torch.Tensor):
    """[rows, heads, width] with a dense (heads, width) part; returns the row stride."""
    assert x.dim() == 3 and x.stride(2) == 1 and x.stride(1) == x.shape[2], "heads must be dense within a row"
    return x.shape[0], x.shape[1], x.shape[2], x.stride(0)


def head_rmsnorm_(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last axis of ``x`` [rows, heads, width], in place, one weight [width] for all heads."""
    _need_cuda(x, weight)
    rows, heads, width, stride = _head_view(x)
    assert weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous()
    _call(f"kirai_head_rmsnorm_{_suffix(x.dtype)}", _ptr(x), _ptr(weight), _i(rows), _i(heads), _i(width), _l(stride),
          _f(eps), _stream())
    return x


# ---------------------------------------------------------------------- rotary
def rope_(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Half-split rotary embedding of ``x`` [rows, heads, width] in place."""
    _need_cuda(x, positions, inv_freq)
    rows, heads, width, stride = _head_view(x)
    assert positions.dtype == torch.int32 and positions.numel() == rows and positions.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2 and inv_freq.is_contiguous()
    _call(f"kirai_rope_{_suffix(x.dtype)}", _ptr(x), _ptr(positions), _ptr(inv_freq), _i(rows), _i(heads), _i(width),
          _i(rotary_dim), _l(stride), _stream())
    return x


# ------------------------------------------------------------------- cache write
def _cache_dims(cache: torch.Tensor):
    assert cache.dim() == 5 and cache.shape[1] == 2 and cache.is_contiguous(), "cache layer is [pages, 2, kv_heads, page, d]"
    return cache.shape[0], cache.shape[2], cache.shape[3], cache.shape[4]


def kv_write(k: torch.Tensor, v: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
             request_of_token: torch.Tensor, positions: torch.Tensor) -> None:
    """Writes key rows ``k`` and value rows ``v`` [T, kv_heads, d] to their pages."""
    _need_cuda(k, v, cache, block_table, request_of_token, positions)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, kh, kd, k_stride = _head_view(k)
    rows_v, vh, vd, v_stride = _head_view(v)
    assert (rows, kh, kd) == (rows_v, vh, vd) and (kh, kd) == (kv_heads, head_dim)
    assert k.dtype == cache.dtype == v.dtype
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    _call(f"kirai_kv_write_{_suffix(k.dtype)}", _ptr(k), _ptr(v), _ptr(cache), _ptr(block_table),
          _ptr(request_of_token), _ptr(positions), _i(rows), _i(kv_heads), _i(head_dim), _l(k_stride), _l(v_stride),
          _i(page_size), _i(block_table.shape[1]), _i(num_pages), _ptr(error_flag(k.device)), _stream())


def qk_norm_rope_kv_write_(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
                           q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                           inv_freq: Optional[torch.Tensor], eps: float, cache: Optional[torch.Tensor],
                           block_table: torch.Tensor, request_of_token: torch.Tensor, positions: torch.Tensor,
                           write_cache: bool = True) -> None:
    """Fused per-head q/k RMSNorm, rotation and paged cache write on ``qkv`` [T, (nq + 2 nkv) d], in place."""
    _need_cuda(qkv, q_weight, k_weight, inv_freq, cache, block_table, request_of_token, positions)
    assert qkv.dim() == 2 and qkv.is_contiguous() and qkv.shape[1] == (q_heads + 2 * kv_heads) * head_dim
    num_pages, page_size = 0, 1
    if kv_heads == 0:
        write_cache = False
    if write_cache:
        num_pages, c_heads, page_size, c_dim = _cache_dims(cache)
        assert (c_heads, c_dim) == (kv_heads, head_dim) and cache.dtype == qkv.dtype
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == head_dim and w.is_contiguous())
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2)
    _call(f"kirai_qk_norm_rope_kv_write_{_suffix(qkv.dtype)}", _ptr(qkv), _ptr(q_weight), _ptr(k_weight),
          _ptr(inv_freq), _ptr(cache if write_cache else None), _ptr(block_table), _ptr(request_of_token),
          _ptr(positions), _i(qkv.shape[0]), _i(q_heads), _i(kv_heads), _i(head_dim), _i(head_dim), _f(eps),
          _i(page_size), _i(block_table.shape[1]), _i(num_pages), _i(1 if write_cache else 0),
          _ptr(error_flag(qkv.device)), _stream())


# --------------------------------------------------------------------- attention
def paged_attention_plain(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                          request_of_token: torch.Tensor, positions: torch.Tensor, window: Optional[int],
                          scale: float) -> torch.Tensor:
    """Causal grouped-query attention of ``q`` [T, nq, d] over the paged cache; returns [T, nq * d]."""
    _need_cuda(q, cache, block_table, request_of_token, positions)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, q_heads, qd, q_stride = _head_view(q)
    assert qd == head_dim and q.dtype == cache.dtype
    out = torch.empty((rows, q_heads * head_dim), dtype=q.dtype, device=q.device)
    _call(f"kirai_paged_attention_plain_{_suffix(q.dtype)}", _ptr(q), _ptr(cache), _ptr(out), _ptr(block_table),
          _ptr(request_of_token), _ptr(positions), _i(rows), _i(q_heads), _i(kv_heads), _i(head_dim), _l(q_stride),
          _i(page_size), _i(block_table.shape[1]), _i(num_pages), _i(window or 0), _f(scale),
          _ptr(error_flag(q.device)), _stream())
    return out


def attention_takes_tensor_cores(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether attention over a cache of this dtype and head size runs on the tensor-core kernels (else the
    CUDA-core kernel, which takes any size)."""
    return dtype == torch.bfloat16 and head_dim % 8 == 0 and 0 < head_dim <= 256


def page_size_refusal(dtype: torch.dtype, head_dim: int, page_size: int) -> Optional[str]:
    """Why the attention kernels for this dtype and head size cannot read pages of ``page_size`` tokens, or None.
    The tensor-core kernels fetch keys and values by TMA in boxes of whole page rows that tile their 16- and 64-key
    tiles: a page must be a power of two up to 64 tokens, or a multiple of 64.  The CUDA-core kernel (32-bit, and
    head sizes the others do not take) reads row by row and takes any page size."""
    if page_size < 1:
        return f"a cache page holds at least one token, got {page_size}"
    if not attention_takes_tensor_cores(dtype, head_dim):
        return None
    if page_size <= 64 and page_size & (page_size - 1) == 0:
        return None
    if page_size % 64 == 0:
        return None
    return (f"pages of {page_size} tokens: the bfloat16 attention kernels (head size {head_dim}) take pages of "
            "1, 2, 4, 8, 16, 32 or 64 tokens, or a multiple of 64")


def attention_prefill_takes_tcgen05(q_heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes this shape: head size up to 128, a group size
    that divides its 128 query rows, pages of a power-of-two size."""
    group = q_heads // kv_heads
    return head_dim <= 128 and head_dim % 8 == 0 and 128 % group == 0 and page_size & (page_size - 1) == 0


def attention_prefill(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, query_start: torch.Tensor,
                      context_len: torch.Tensor, max_query_len: int, window: Optional[int], scale: float,
                      tcgen05: Optional[bool] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 tensor-core attention for runs of new tokens (prompt portions, or any mix): q [T, nq, d].
    ``query_start`` holds rows of ``q`` and of the result, so the requests given may be a part of a larger batch
    (``out`` is then the whole batch's result, of which only their rows are written).  ``tcgen05`` picks the kernel (None: the tcgen05 kernel where it takes the shape, else the
    warp-level ``mma.sync`` kernel)."""
    _need_cuda(q, cache, block_table, query_start, context_len)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, q_heads, qd, q_stride = _head_view(q)
    assert qd == head_dim and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
    requests = context_len.numel()
    assert query_start.numel() == requests + 1 and query_start.dtype == torch.int32 and context_len.dtype == torch.int32
    if tcgen05 is None:
        tcgen05 = attention_prefill_takes_tcgen05(q_heads, kv_heads, head_dim, page_size)
    if out is None:
        out = torch.empty((rows, q_heads * head_dim), dtype=q.dtype, device=q.device)
    assert out.shape == (rows, q_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous()
    _call("kirai_attention_prefill_tc_bf16" if tcgen05 else "kirai_attention_prefill_bf16", _ptr(q), _ptr(cache), _ptr(out),
          _ptr(block_table), _ptr(query_start), _ptr(context_len), _i(requests), _i(max_query_len), _i(q_heads), _i(kv_heads),
          _i(head_dim), _l(q_stride), _i(page_size), _i(block_table.shape[1]), _i(num_pages), _i(window or 0), _f(scale),
          _ptr(error_flag(q.device)), _stream())
    return out


DEFAULT_SMS = 148  # for planning on a host without the device (tests); launches ask the device


def decode_splits(requests: int, kv_heads: int, max_context_len: int, tile: int = 16, warps: int = 8,
                  sms: int = DEFAULT_SMS, room=None, head_dim: int = 128, group: int = 4) -> int:
    """How many CTAs share one (request, kv head) in the decode kernel.  A CTA's warps take key tiles in turn, so a
    CTA with n tiles runs ceil(n / warps) rounds plus a fixed cost (set-up, merge); CTAs run in waves of ``sms``; more
    than one range needs the buffer and the second kernel, about three rounds' time (a pair of ranges that merges in
    the kernel, see ``decode_pair_merges``, one round).  A launch that fills all but a
    few SMs pays one round more: the kernel after it finds no SM on which to start early and fetch its weights
    (3.15 against 3.06 ms a step with 144 and with 128 CTAs at two requests of 4,096 tokens, 3.11 against 2.98 at one).
    The split count with the fewest estimated rounds wins."""
    room = room or _default_cluster_room(sms)
    pairs = max(1, requests * kv_heads)
    tiles = max(1, -(-max_context_len // tile))
    best, best_cost = 1, None
    for splits in range(1, min(64, tiles) + 1):
        ctas = pairs * splits
        waves = -(-ctas // sms)
        rounds = -(-(-(-tiles // splits)) // warps) + 3
        merge = 0.0 if splits == 1 else (1.0 if decode_pair_merges(pairs, splits, head_dim, room, group) else 2.75)
        cost = waves * rounds + merge + (1.0 if waves == 1 and ctas > sms - 12 else 0.0)
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    return best


DECODE_CLUSTER_RANGES = 5  # ranges of a (request, kv head) that may merge inside the decode kernel


def _default_cluster_room(sms: int):
    """Clusters of a size that a device of ``sms`` SMs is taken to hold at once when nobody asked it (planning on a
    host without the device): what one B200 said for clusters of one-per-SM CTAs, scaled."""
    return lambda cluster: {1: sms, 2: sms // 2, 3: (sms * 39) // 148, 4: (sms * 33) // 148, 5: (sms * 26) // 148}.get(cluster, 0)


_cluster_rooms: dict = {}


def decode_cluster_room(device: torch.device, head_dim: int, group: int = 1):
    """cluster size -> how many clusters of the decode kernel ``device`` holds at once (0: it refuses the size).  A CTA
    of that kernel fills an SM and a cluster must lie inside one GPC, so the answer is the device's to give: chips of
    one kind differ in the SMs of their GPCs."""
    key = (torch.device(device), head_dim, group <= 8)
    if key not in _cluster_rooms:
        with torch.cuda.device(key[0]):
            fn = getattr(library(), "kirai_attention_decode_resident_clusters")
            fn.restype = ctypes.c_int
            _cluster_rooms[key] = [0] + [int(fn(_i(head_dim), _i(group), _i(c))) for c in range(1, DECODE_CLUSTER_RANGES + 1)]
    counts = _cluster_rooms[key]
    return lambda cluster: counts[cluster] if 0 < cluster < len(counts) else 0


def decode_pair_merges(pairs: int, splits: int, head_dim: int, room, group: int = 4) -> bool:
    """Whether the ranges of every (request, kv head) merge inside the decode kernel, as a cluster of CTAs that write
    their rows into slots in the first one's shared memory: two to five ranges, all clusters running at once (``room``:
    cluster size -> how many the device holds; in a launch of several waves the CTAs that a cluster must place
    together left SMs idle: 6 requests as 48 clusters of 3, of which 39 to 45 fit, 3.92 against 3.44 ms a step), heads
    of up to 128, and the other CTAs' rows (``group`` each) fitting the slots' 16 rows."""
    return (2 <= splits <= DECODE_CLUSTER_RANGES and pairs <= room(splits) and head_dim <= 128
            and (splits - 1) * group <= 16)


def decode_plan(context_lens, kv_heads: int, window: Optional[int] = None, tile: int = 16, warps: int = 8,
                sms: int = DEFAULT_SMS, room=None, head_dim: int = 128, group: int = 4) -> tuple:
    """Which decode attention kernel a batch should take: (balanced, splits).

    The split kernel gives every request the same number of CTAs, so its time is that of the longest request and
    comes in waves of ``sms`` CTAs; the balanced kernel cuts all key tiles into ``sms`` equal ranges, which costs
    it a second start inside most CTAs and a longer merge.  Costs are in rounds of one key tile per warp (about
    1.35 us on the 8B layer sizes); the fixed parts were fitted to measurements of both kernels at batches of 1 to
    64.  Balanced is chosen only when it is expected to be clearly faster: contexts of unequal length, or a batch
    whose CTAs fill the last wave badly."""
    lens = [min(int(n), window) if window else int(n) for n in context_lens]
    if not lens:
        return False, 1
    longest = max(1, max(lens))
    room = room or _default_cluster_room(sms)
    splits = decode_splits(len(lens), kv_heads, longest, tile, warps, sms, room, head_dim, group)
    tiles = [max(1, -(-n // tile)) for n in lens]
    waves = -(-len(lens) * kv_heads * splits // sms)
    rounds_split = -(-(-(-max(tiles) // splits)) // warps)
    cost_split = waves * (rounds_split + 2.5) + (0.0 if splits == 1 else (1.0 if decode_pair_merges(len(lens) * kv_heads, splits, head_dim, room, group) else 2.5))
    rounds_balanced = -(-(-(-kv_heads * sum(tiles) // sms)) // warps)
    cost_balanced = rounds_balanced + 9.5
    return cost_balanced < 0.92 * cost_split, splits


def attention_decode(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, context_len: torch.Tensor,
                     window: Optional[int], scale: float, num_splits: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 tensor-core attention for a batch in which every request brings one token: q [R, nq, d] (row r of ``q``,
    of the tables and of the result belongs to request r; ``out`` may be the head of a larger result)."""
    _need_cuda(q, cache, block_table, context_len)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, q_heads, qd, q_stride = _head_view(q)
    assert qd == head_dim and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
    assert context_len.numel() == rows and context_len.dtype == torch.int32
    if out is None:
        out = torch.empty((rows, q_heads * head_dim), dtype=q.dtype, device=q.device)
    assert out.shape == (rows, q_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous()
    partial = None
    if num_splits > 1 and not decode_pair_merges(rows * kv_heads, num_splits, head_dim, decode_cluster_room(q.device, head_dim, q_heads // kv_heads), q_heads // kv_heads):
        # the ranges' results go through a buffer and a second kernel
        partial = torch.empty((rows, q_heads, num_splits, head_dim + 2), dtype=torch.float32, device=q.device)
    _call("kirai_attention_decode_bf16", _ptr(q), _ptr(cache), _ptr(out), _ptr(partial), _ptr(block_table),
          _ptr(context_len), _i(rows), _i(q_heads), _i(kv_heads), _i(head_dim), _l(q_stride), _i(page_size),
          _i(block_table.shape[1]), _i(num_pages), _i(window or 0), _f(scale), _i(num_splits),
          _ptr(error_flag(q.device)), _stream())
    return out


_sm_counts = {}


def sm_count(device: torch.device) -> int:
    key = torch.device(device)
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_counts[key]


def attention_decode_balanced(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, context_len: torch.Tensor,
                              window: Optional[int], scale: float, ctas: Optional[int] = None,
                              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The decode attention with the key tiles of all (request, kv head) pairs cut into ``ctas`` equal ranges
    (default: one per SM), so that every CTA reads the same number of keys whatever the batch looks like."""
    _need_cuda(q, cache, block_table, context_len)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, q_heads, qd, q_stride = _head_view(q)
    assert qd == head_dim and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
    assert context_len.numel() == rows and context_len.dtype == torch.int32
    ctas = ctas or sm_count(q.device)
    if out is None:
        out = torch.empty((rows, q_heads * head_dim), dtype=q.dtype, device=q.device)
    assert out.shape == (rows, q_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous()
    partial = torch.empty((ctas, 2, 16, head_dim + 2), dtype=torch.float32, device=q.device)
    _call("kirai_attention_decode_balanced_bf16", _ptr(q), _ptr(cache), _ptr(out), _ptr(partial), _ptr(block_table),
          _ptr(context_len), _i(rows), _i(q_heads), _i(kv_heads), _i(head_dim), _l(q_stride), _i(page_size),
          _i(block_table.shape[1]), _i(num_pages), _i(window or 0), _f(scale), _i(ctas),
          _ptr(error_flag(q.device)), _stream())
    return out


def paged_attention(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, batch, window: Optional[int],
                    scale: float) -> torch.Tensor:
    """Attention of the product path over the paged cache for the tokens of ``batch``
    (a kirai_b200.engine.batch.StepBatch).  float32 takes the plain kernel; bfloat16 takes the
    tensor-core kernels (the decode kernel when every request brings one token), or the plain
    kernel for head sizes they do not take (not a multiple of 8, or above 256)."""
    head_dim, q_heads, kv_heads = q.shape[2], q.shape[1], cache.shape[2]
    fast = attention_takes_tensor_cores(q.dtype, head_dim) and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
    if not fast:
        return paged_attention_plain(q, cache, block_table, batch.request_of_token, batch.positions, window, scale)
    decode_rows = batch.num_requests if batch.decode_only else getattr(batch, "num_decode", 0)
    if decode_rows and q_heads // kv_heads <= 16:
        # The requests that bring one token stand first in the batch (the batch builder puts them there) and take the
        # decode kernels, which split a long context over many CTAs; prompt portions take the prompt kernel, and both
        # write their rows of one result.  A prompt kernel alone would give a decoding request one CTA per kv head.
        out = torch.empty((q.shape[0], q_heads * head_dim), dtype=q.dtype, device=q.device)
        _decode_rows(q[:decode_rows], cache, block_table[:decode_rows], batch, decode_rows, window, scale, out[:decode_rows])
        if decode_rows < batch.num_requests:
            attention_prefill(q, cache, block_table[decode_rows:], batch.query_start[decode_rows:], batch.context_len[decode_rows:],
                              batch.max_query_len, window, scale, out=out)
        return out
    return attention_prefill(q, cache, block_table, batch.query_start, batch.context_len, batch.max_query_len, window, scale)


def _decode_rows(q, cache, block_table, batch, rows: int, window: Optional[int], scale: float, out: torch.Tensor) -> None:
    """The decode attention of the first ``rows`` requests of ``batch`` (one token each)."""
    kv_heads = cache.shape[2]
    room = decode_cluster_room(q.device, q.shape[2], q.shape[1] // kv_heads)
    context_len = batch.context_len[:rows]
    # the batch may say which kernel (a captured step does: its lengths change between replays); otherwise
    # the host's copy of the lengths decides; KIRAI_DECODE_BALANCED=0 or 1 overrides both
    balanced = getattr(batch, "decode_balanced", None)
    longest = batch.max_context_len
    if balanced is None:
        lens = [start + count for start, count in zip(batch.start_positions[:rows], batch.query_lens[:rows])]
        balanced, _ = decode_plan(lens, kv_heads, window, sms=sm_count(q.device), room=room, head_dim=q.shape[2],
                                  group=q.shape[1] // kv_heads)
        longest = max(lens)
    forced = os.environ.get("KIRAI_DECODE_BALANCED")
    if forced in ("0", "1"):
        balanced = forced == "1"
    if balanced and rows <= 1024:
        attention_decode_balanced(q, cache, block_table, context_len, window, scale, out=out)
        return
    # (a captured step says how many ranges, planned for its requests' lengths; else the longest context decides)
    splits = getattr(batch, "decode_splits", None) or decode_splits(rows, kv_heads, min(longest, window or longest), sms=sm_count(q.device),
                                                                    room=room, head_dim=q.shape[2], group=q.shape[1] // kv_heads)
    attention_decode(q, cache, block_table, context_len, window, scale, splits, out=out)


def decode_prepares_qk(qkv: torch.Tensor, cache: Optional[torch.Tensor], batch, q_heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether ``attention_decode_qk`` takes this step: every request brings one token, bfloat16, heads of 64, 128 or
    256 in groups of at most 16, rows on 16-byte boundaries, and no more (request, kv head) pairs than SMs: with more,
    every one of the many CTAs repeats the preparation, and the separate kernel, which runs beside the end of the
    product before it, is faster (10.37 against 10.13 ms a step at 64 requests of the 8B shape; 3.29 against 3.31 ms
    at one request)."""
    return (cache is not None and batch.num_requests * kv_heads <= sm_count(qkv.device) and qkv.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and batch.decode_only
            and head_dim in (64, 128, 256) and kv_heads > 0 and q_heads // kv_heads <= 16 and qkv.is_contiguous()
            and qkv.data_ptr() % 16 == 0 and batch.num_requests == qkv.shape[0])


def attention_decode_qk(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, q_weight: Optional[torch.Tensor],
                        k_weight: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], eps: float, cache: torch.Tensor,
                        block_table: torch.Tensor, batch, window: Optional[int], scale: float) -> torch.Tensor:
    """A decode step's attention with its preparation inside the kernel: ``qkv`` [R, (nq + 2 nkv) d] as the q, k, v
    product left it (not modified).  Per-head RMSNorm of q and k, rotation at each request's position, the new token's
    key and value appended to its page, attention over the pages: one kernel, where the separate path runs
    ``qk_norm_rope_kv_write_`` and then the decode kernel.  The result equals that path's bit for bit."""
    _need_cuda(qkv, q_weight, k_weight, inv_freq, cache, block_table, batch.context_len)
    num_pages, c_heads, page_size, c_dim = _cache_dims(cache)
    rows = qkv.shape[0]
    assert (c_heads, c_dim) == (kv_heads, head_dim) and qkv.shape[1] == (q_heads + 2 * kv_heads) * head_dim
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == head_dim and w.is_contiguous())
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2 and inv_freq.is_contiguous())
    context_len = batch.context_len
    out = torch.empty((rows, q_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    balanced = getattr(batch, "decode_balanced", None)
    longest = batch.max_context_len
    room = decode_cluster_room(qkv.device, head_dim, q_heads // kv_heads)
    if balanced is None:
        lens = [start + count for start, count in zip(batch.start_positions, batch.query_lens)]
        balanced, _ = decode_plan(lens, kv_heads, window, sms=sm_count(qkv.device), room=room, head_dim=head_dim,
                                  group=q_heads // kv_heads)
        longest = max(lens)
    forced = os.environ.get("KIRAI_DECODE_BALANCED")
    if forced in ("0", "1"):
        balanced = forced == "1"
    tail = (_ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), _f(eps), _ptr(error_flag(qkv.device)), _stream())
    common = (_ptr(block_table), _ptr(context_len), _i(rows), _i(q_heads), _i(kv_heads), _i(head_dim), _l(qkv.stride(0)),
              _i(page_size), _i(block_table.shape[1]), _i(num_pages), _i(window or 0), _f(scale))
    if balanced and rows <= 1024:
        ctas = sm_count(qkv.device)
        partial = torch.empty((ctas, 2, 16, head_dim + 2), dtype=torch.float32, device=qkv.device)
        _call("kirai_attention_decode_balanced_qk_bf16", _ptr(qkv), _ptr(cache), _ptr(out), _ptr(partial), *common, _i(ctas), *tail)
        return out
    splits = getattr(batch, "decode_splits", None) or decode_splits(rows, kv_heads, min(longest, window or longest), sms=sm_count(qkv.device),
                                                                    room=room, head_dim=head_dim, group=q_heads // kv_heads)
    partial = None
    if splits > 1 and not decode_pair_merges(rows * kv_heads, splits, head_dim, room, q_heads // kv_heads):
        partial = torch.empty((rows, q_heads, splits, head_dim + 2), dtype=torch.float32, device=qkv.device)
    _call("kirai_attention_decode_qk_bf16", _ptr(qkv), _ptr(cache), _ptr(out), _ptr(partial), *common, _i(splits), *tail)
    return out


# ------------------------------------------------------------------------ linear
def linear_plain(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x`` [M, K] times ``weight`` [N, K] transposed on the CUDA cores with 32-bit FMAs."""
    _need_cuda(x, weight)
    assert x.dim() == 2 and x.stride(1) == 1 and weight.dim() == 2 and weight.is_contiguous()
    assert x.shape[1] == weight.shape[1] and x.dtype == weight.dtype
    out_dtype = out_dtype or x.dtype
    m, k, n = x.shape[0], x.shape[1], weight.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32
        name = "kirai_gemm_simt_f32"
    else:
        name = "kirai_gemm_simt_bf16" if out_dtype == torch.bfloat16 else "kirai_gemm_simt_bf16_out_f32"
    _call(name, _ptr(x), _ptr(weight), _ptr(out), _i(m), _i(n), _i(k), _l(x.stride(0)), _l(n), _stream())
    return out


class TiledWeight:
    """A bf16 weight matrix [N, K] in the layout that the tensor-core product streams fastest: boxes of 128 rows
    x 64 columns, each stored as the 16 KB image that the 128-byte swizzle leaves in shared memory (the 16-byte
    chunk c of row r at chunk c ^ (r % 8)), box (row tile, k block) at index row_tile * ceil(K / 64) + k_block,
    zero-padded at the edges.  One box is one contiguous bulk copy."""

    def __init__(self, boxes: torch.Tensor, rows: int, cols: int):
        self.boxes, self.rows, self.cols = boxes, rows, cols

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def device(self):
        return self.boxes.device

    def row_major(self) -> torch.Tensor:
        """The matrix back in rows (for tests and for kernels that do not read boxes)."""
        row_tiles, k_blocks = self.boxes.shape[:2]
        chunks = self.boxes.view(row_tiles, k_blocks, 128, 8, 8)
        plain = chunks[:, :, torch.arange(128, device=self.device)[:, None], _swizzle_index(self.device), :]
        plain = plain.reshape(row_tiles, k_blocks, 128, 64).permute(0, 2, 1, 3).reshape(row_tiles * 128, k_blocks * 64)
        return plain[: self.rows, : self.cols].contiguous()


def _swizzle_index(device) -> torch.Tensor:
    """[128, 8]: where chunk c of row r lies under the 128-byte swizzle (an involution)."""
    rows = torch.arange(128, device=device)[:, None]
    return torch.arange(8, device=device)[None, :] ^ (rows % 8)


def tile_weight(weight: torch.Tensor) -> TiledWeight:
    """Re-packs a bf16 matrix [N, K] on the device into the tiled layout (done once, at load)."""
    _need_cuda(weight)
    assert weight.dim() == 2 and weight.dtype == torch.bfloat16
    n, k = weight.shape
    row_tiles, k_blocks = (n + 127) // 128, (k + 63) // 64
    if row_tiles * 128 != n or k_blocks * 64 != k:
        padded = torch.zeros((row_tiles * 128, k_blocks * 64), dtype=weight.dtype, device=weight.device)
        padded[:n, :k] = weight
    else:
        padded = weight
    boxes = padded.view(row_tiles, 128, k_blocks, 8, 8).permute(0, 2, 1, 3, 4)  # [row tile, k block, row, chunk, 8]
    boxes = boxes[:, :, torch.arange(128, device=weight.device)[:, None], _swizzle_index(weight.device), :]
    boxes = boxes.reshape(row_tiles, k_blocks, 128 * 64).contiguous()
    tiled_bytes = library().kirai_gemm_bf16_tiled_bytes
    tiled_bytes.restype = ctypes.c_long
    assert boxes.numel() * 2 == int(tiled_bytes(_i(n), _i(k)))
    return TiledWeight(boxes, n, k)


# ---- products held back and launched together
# A decode step of a few tokens runs product after product, each bound by its weight stream, and every launch pays a
# ramp of its own.  Inside ``chained_products()`` a product of at most 64 rows with tiled weights is not launched at
# once: it is put on a list, and the list goes out as ONE persistent kernel (csrc/gemm_chain.cu, whose weight stream
# runs on from product to product) as soon as anything else is launched or the block ends.  Results are therefore
# not computed when ``linear_tcgen05`` returns, only when the next kernel of another kind has been asked for: code
# inside such a block must touch activations through the functions of this module only (every one of them sends the
# list out first), never through torch arithmetic or a copy to the host.
chain_stamps = None     # a tensor of sms * 6 * 4 int64: the chain kernel writes its clock stamps there (measurements)
# Off by default: on the 8B layer sizes the chain measured slower than the products launched one by one (see the
# head of csrc/gemm_chain.cu for the figures and the reasons); True lets the model's steps use it.
chain_products = False
_chain_depth = 0
_pending: list = []
_chain_workspaces: dict = {}


class chained_products:
    """``with ops.chained_products(): ...`` holds products back as described above; ``enabled=False`` does nothing."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and chain_products

    def __enter__(self):
        global _chain_depth
        if self.enabled:
            _chain_depth += 1
        return self

    def __exit__(self, kind, value, traceback):
        global _chain_depth
        if self.enabled:
            _chain_depth -= 1
            if _chain_depth == 0:
                if kind is None:
                    flush_products()
                else:
                    _pending.clear()  # an error on the way: nothing half-described is launched
        return False


def chaining() -> bool:
    """Whether products are being held back right now."""
    return _chain_depth > 0 and chain_products


def _chain_workspace(device: torch.device) -> torch.Tensor:
    """One workspace per device (partial tiles and counters, 10 MB): chains on one device run one after the other, as
    everything of a step does; two streams that ran chains at the same time would need one each."""
    key = torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    if key not in _chain_workspaces:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the workspace of chained products must exist before a stream capture begins: "
                              "run the step once outside the capture")
        size = library().kirai_gemm_chain_workspace_bytes
        size.restype = ctypes.c_long
        _chain_workspaces[key] = torch.zeros(int(size()), dtype=torch.uint8, device=device)
    return _chain_workspaces[key]


def _launch_product(item) -> None:
    x, weight, out, n, k, width, splits, form, row_scale, resid, norm_weight, sumsq_out = item
    tiled = isinstance(weight, TiledWeight)
    if row_scale is not None:
        sumsq, count, eps = row_scale
        scale_args = (_ptr(sumsq), _i(sumsq.shape[0]), _f(float(count)), _f(float(eps)))
    else:
        scale_args = (_ptr(None), _i(0), _f(1.0), _f(0.0))
    _launch("kirai_gemm_bf16_general", _ptr(x), _ptr(weight.boxes if tiled else weight), _i(tiled), _ptr(out), _i(x.shape[0]),
            _i(n), _i(k), _l(x.stride(0)), _l(width), _i(splits), _i(form), *scale_args,
            _ptr(resid), _ptr(norm_weight), _ptr(sumsq_out), _ptr(error_flag(x.device)), _stream())


def flush_products() -> None:
    """Launches the products that were held back: one alone through the single-product kernel, several as one chain."""
    global _pending
    items, _pending = _pending, []
    if not items:
        return
    if len(items) > 1:
        count = len(items)
        pointers, longs, ints, floats = ctypes.c_void_p * count, ctypes.c_long * count, ctypes.c_int * count, ctypes.c_float * count

        def ptrs(values):
            return pointers(*[0 if v is None else v.data_ptr() for v in values])

        x0 = items[0][0]
        workspace = _chain_workspace(x0.device)
        scales = [item[8] for item in items]
        fn = library().kirai_gemm_chain_bf16
        fn.restype = ctypes.c_int
        status = fn(
            _i(count), _i(x0.shape[0]), ptrs([item[0] for item in items]), longs(*[item[0].stride(0) for item in items]),
            ptrs([item[1].boxes for item in items]), ptrs([item[2] for item in items]), longs(*[item[5] for item in items]),
            ints(*[item[3] for item in items]), ints(*[item[4] for item in items]), ints(*[item[7] for item in items]),
            ptrs([None if sc is None else sc[0] for sc in scales]), ints(*[0 if sc is None else sc[0].shape[0] for sc in scales]),
            floats(*[1.0 if sc is None else float(sc[1]) for sc in scales]), floats(*[0.0 if sc is None else float(sc[2]) for sc in scales]),
            ptrs([item[9] for item in items]), ptrs([item[10] for item in items]), ptrs([item[11] for item in items]),
            _ptr(workspace), _l(workspace.numel()), _ptr(error_flag(x0.device)), _ptr(chain_stamps), _stream())
        if status == 0:
            global launch_count
            launch_count += 1
            launch_counts["kirai_gemm_chain_bf16"] = launch_counts.get("kirai_gemm_chain_bf16", 0) + 1
            return
        if status not in _REFUSALS:
            _check(status, "kirai_gemm_chain_bf16")
        # refused (a shape the chain does not take): one by one
    for item in items:
        _launch_product(item)


def _gemm(x, weight, out, n: int, k: int, width: int, splits: int, form: int, row_scale, resid, norm_weight, sumsq_out):
    if row_scale is not None:
        sumsq = row_scale[0]
        assert sumsq.dtype == torch.float32 and sumsq.dim() == 2 and sumsq.shape[1] == x.shape[0] and sumsq.is_contiguous()
    item = (x, weight, out, n, k, width, splits, form, row_scale, resid, norm_weight, sumsq_out)
    if chaining() and isinstance(weight, TiledWeight) and x.shape[0] <= 64 and splits == 0:
        if _pending and _pending[0][0].shape[0] != x.shape[0]:
            flush_products()
        _pending.append(item)
        limit = library().kirai_gemm_chain_max_phases
        limit.restype = ctypes.c_int
        if len(_pending) >= int(limit()):
            flush_products()
        return
    if _pending:
        flush_products()
    _launch_product(item)


def _check_product(x, weight) -> tuple:
    if isinstance(weight, TiledWeight):
        _need_cuda(x, weight.boxes)
    else:
        _need_cuda(x, weight)
        assert weight.dim() == 2 and weight.is_contiguous() and weight.dtype == torch.bfloat16
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype == torch.bfloat16 and x.shape[1] == weight.shape[1]
    return x.shape[0], x.shape[1], weight.shape[0]


def linear_tcgen05(x: torch.Tensor, weight, out_dtype: Optional[torch.dtype] = None,
                   splits: int = 0, swiglu: bool = False, row_scale: Optional[tuple] = None) -> torch.Tensor:
    """bf16 ``x`` [M, K] times ``weight`` [N, K] transposed on the tcgen05 tensor cores (32-bit accumulation).

    ``weight`` is a row-major tensor or a ``TiledWeight``.  K and the row stride of ``x`` must be multiples of 8
    (TMA reads rows in 16-byte units).  ``splits`` > 1 cuts K between the CTAs of a cluster (0: chosen from the
    shape, at most 4).  With ``swiglu`` the rows of ``weight`` are 8 gate rows, their 8 up rows, 8 gate rows, ...
    and the result is silu(gate) * up, [M, N / 2].  ``row_scale`` = (sumsq [P, M] float32, count, eps) multiplies
    row m of the product by 1 / sqrt(sum_p sumsq[p, m] / count + eps): ``x`` then holds rows that an RMSNorm left
    unscaled.
    """
    m, k, n = _check_product(x, weight)
    out_dtype = out_dtype or torch.bfloat16
    if swiglu:
        assert out_dtype == torch.bfloat16 and n % 16 == 0
    width = n // 2 if swiglu else n
    out = torch.empty((m, width), dtype=out_dtype, device=x.device)
    form = 2 if swiglu else (0 if out_dtype == torch.bfloat16 else 1)
    _gemm(x, weight, out, n, k, width, splits, form, row_scale, None, None, None)
    return out


def linear_residual_norm(x: torch.Tensor, weight, resid: torch.Tensor, norm_weight: torch.Tensor,
                         splits: int = 0) -> tuple:
    """``resid`` [M, N] (float32, in place) += ``x`` [M, K] times ``weight`` [N, K] transposed, on the tensor cores;
    returns (bf16(resid * norm_weight) [M, N], sumsq [P, M]): the rows of the next RMSNorm without their
    1 / rms factor, and the parts of each row's sum of squares, which ``linear_tcgen05(row_scale=...)`` applies."""
    m, k, n = _check_product(x, weight)
    _need_cuda(resid, norm_weight)
    assert resid.dtype == torch.float32 and resid.shape == (m, n) and resid.is_contiguous()
    assert norm_weight.dtype == torch.float32 and norm_weight.shape == (n,) and norm_weight.is_contiguous()
    parts = int(library().kirai_gemm_bf16_residual_parts(_i(m), _i(n)))
    rows = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty((parts, m), dtype=torch.float32, device=x.device)
    _gemm(x, weight, rows, n, k, n, splits, 3, None, resid, norm_weight, sumsq)
    return rows, sumsq


def tcgen05_takes(x: torch.Tensor) -> bool:
    """Whether the tensor-core GEMM can read ``x`` [M, K] (bf16, 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stacks gate [I, K] and up [I, K] as 8 gate rows, their 8 up rows, ... (I a multiple of 8),
    the row order that the SwiGLU epilogue of the tensor-core GEMM reads."""
    inter, k = gate.shape
    assert up.shape == gate.shape and inter % 8 == 0
    return torch.stack([gate.view(inter // 8, 8, k), up.view(inter // 8, 8, k)], dim=1).reshape(2 * inter, k).contiguous()


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The linear layer of the product path: 32-bit FMAs for float32; for bfloat16 the tcgen05
    kernel, or the CUDA-core kernel when K is not a multiple of 8 (TMA cannot read such rows)."""
    if isinstance(weight, TiledWeight):
        return linear_tcgen05(x if tcgen05_takes(x) else x.contiguous(), weight, out_dtype)
    if tcgen05_takes(x):
        return linear_tcgen05(x, weight, out_dtype)
    return linear_plain(x, weight, out_dtype)


# ------------------------------------------------------------------------ SwiGLU
def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for ``gate_up`` [T, 2 I] (gate half first); returns [T, I]."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _call(f"kirai_swiglu_{_suffix(gate_up.dtype)}", _ptr(gate_up), _ptr(out), _i(rows), _i(inter), _stream())
    return out


def decode_advance(token_ids: torch.Tensor, sampled: torch.Tensor, positions: torch.Tensor, context_len: torch.Tensor) -> None:
    """token_ids <- sampled; positions += 1; context_len += 1 (all int32 [R], on the device)."""
    _need_cuda(token_ids, sampled, positions, context_len)
    for t in (token_ids, sampled, positions, context_len):
        assert t.dtype == torch.int32 and t.is_contiguous() and t.numel() == token_ids.numel()
    _call("kirai_decode_advance", _ptr(token_ids), _ptr(sampled), _ptr(positions), _ptr(context_len),
          _i(token_ids.numel()), _stream())


# ---------------------------------------------------------------------- sampling
def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """Index of the greatest logit of each row, the lowest index on ties."""
    _need_cuda(logits)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.is_contiguous()
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _call("kirai_argmax_rows", _ptr(logits), _ptr(out), _i(logits.shape[0]), _i(logits.shape[1]),
          _ptr(error_flag(logits.device)), _stream())
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, draw: torch.Tensor) -> torch.Tensor:
    """One token per row: greedy where temperature is 0, else nucleus sampling with the row's draw."""
    _need_cuda(logits, temperature, top_p, draw)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.is_contiguous()
    rows = logits.shape[0]
    for t in (temperature, top_p, draw):
        assert t.dtype == torch.float32 and t.numel() == rows and t.is_contiguous()
    needs_scratch = library().kirai_sample_rows_needs_scratch
    needs_scratch.restype = ctypes.c_int
    scratch = torch.empty_like(logits) if needs_scratch(_i(rows), _i(logits.shape[1])) else None
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _call("kirai_sample_rows", _ptr(logits), _ptr(scratch), _ptr(temperature), _ptr(top_p), _ptr(draw), _ptr(out),
          _i(rows), _i(logits.shape[1]), _ptr(error_flag(logits.device)), _stream())
    return out
