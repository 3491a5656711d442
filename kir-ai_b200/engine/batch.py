"""The description of one step's batch, as the kernels read it.

A step runs, for each scheduled request, a contiguous run of new tokens that
starts at the request's current length: a portion of its prompt, or one decoded
token.  The runs are laid end to end into one flat batch of T tokens.  All
index arrays are built on the host, packed into one int32 buffer and sent to
the device in a single copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` and the places among
    them (0-based, within ``tokens``) whose logits are wanted."""

    request: object  # kirai_b200.cache.pages.RequestPages
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepBatch:
    num_tokens: int
    num_requests: int
    # device, int32
    token_ids: torch.Tensor         # [T]
    positions: torch.Tensor         # [T] absolute position of each token in its request
    request_of_token: torch.Tensor  # [T] row of the block tables
    query_start: torch.Tensor       # [R + 1] first token row of each request's run
    context_len: torch.Tensor       # [R] tokens in the cache after this step
    slots: torch.Tensor             # [R] state slot of each request
    block_tables: List[torch.Tensor]  # per cache group [R, width]
    want_rows: Optional[torch.Tensor]  # [n_want] token rows whose logits are wanted
    # host copies, for choosing kernels and for mixers that walk requests on the host
    query_lens: List[int] = field(default_factory=list)
    start_positions: List[int] = field(default_factory=list)
    slot_ids: List[int] = field(default_factory=list)
    max_query_len: int = 0
    max_context_len: int = 0
    num_want: int = 0
    # how many requests at the head of the batch bring exactly one token: the batch builder puts them first, so
    # that kernels made for single tokens can take rows [0, num_decode) and the others the rest
    num_decode: int = 0
    # which decode attention kernel a step of single tokens takes (None: decided from the lengths above)
    decode_balanced: Optional[bool] = None
    # into how many ranges that kernel cuts a request's keys (None or 0: decided from the longest context above)
    decode_splits: Optional[int] = None

    @property
    def decode_only(self) -> bool:
        return self.max_query_len == 1


def build_batch(entries: Sequence[StepEntry], cache, device) -> StepBatch:
    """Packs the entries (whose pages are already reserved) into a StepBatch on ``device``.

    Inside the batch the requests that bring one token come first (in their order), then the others (in theirs);
    ``want_rows`` still lists the wanted places in the order of ``entries`` and of each ``want``, so the caller's
    logits come back in the order it gave."""
    given = list(entries)
    order = [i for i, e in enumerate(given) if len(e.tokens) == 1] + [i for i, e in enumerate(given) if len(e.tokens) != 1]
    num_decode = sum(1 for e in given if len(e.tokens) == 1)
    entries = [given[i] for i in order]
    query_lens = [len(e.tokens) for e in entries]
    starts = [e.request.length for e in entries]
    total = sum(query_lens)
    count = len(entries)
    token_ids = np.empty(total, dtype=np.int32)
    positions = np.empty(total, dtype=np.int32)
    request_of_token = np.empty(total, dtype=np.int32)
    query_start = np.zeros(count + 1, dtype=np.int32)
    first_row = [0] * count  # by place in ``given``
    row = 0
    for index, entry in enumerate(entries):
        n = query_lens[index]
        token_ids[row : row + n] = np.asarray(entry.tokens, dtype=np.int64)
        positions[row : row + n] = np.arange(starts[index], starts[index] + n, dtype=np.int32)
        request_of_token[row : row + n] = index
        first_row[order[index]] = row
        row += n
        query_start[index + 1] = row
    want_rows: List[int] = [first_row[i] + w for i, entry in enumerate(given) for w in entry.want]
    context_len = np.asarray([s + n for s, n in zip(starts, query_lens)], dtype=np.int32)
    slots = np.asarray([e.request.slot for e in entries], dtype=np.int32)
    requests = [e.request for e in entries]
    tables = [cache.block_table_array(requests, g) for g in range(len(cache.groups))]
    want = np.asarray(want_rows, dtype=np.int32)

    pieces = [token_ids, positions, request_of_token, query_start, context_len, slots, want] + [t.reshape(-1) for t in tables]
    # every piece starts on a 16-byte boundary (4 ints) so that vector loads of any piece are aligned
    offsets, cursor = [], 0
    for piece in pieces:
        offsets.append(cursor)
        cursor += -(-piece.size // 4) * 4
    packed = np.zeros(max(cursor, 4), dtype=np.int32)
    for piece, offset in zip(pieces, offsets):
        packed[offset : offset + piece.size] = piece
    host = torch.from_numpy(packed)
    if torch.device(device).type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True)

    def view(i):
        return dev[offsets[i] : offsets[i] + pieces[i].size]

    return StepBatch(
        num_tokens=total,
        num_requests=count,
        token_ids=view(0),
        positions=view(1),
        request_of_token=view(2),
        query_start=view(3),
        context_len=view(4),
        slots=view(5),
        want_rows=view(6) if want.size else None,
        block_tables=[view(7 + g).view(tables[g].shape) for g in range(len(tables))],
        query_lens=query_lens,
        start_positions=starts,
        slot_ids=[int(s) for s in slots],
        max_query_len=max(query_lens) if query_lens else 0,
        max_context_len=int(context_len.max()) if count else 0,
        num_want=int(want.size),
        num_decode=num_decode,
    )
