"""CUDA graphs for decode steps.

A step in which every request brings one token has the same kernel sequence
whenever the number of requests and the width of the block tables are the same,
so it is captured once per (requests, table width) and replayed.  The captured
step reads its inputs from fixed device buffers (token ids, positions, context
lengths, slots, block tables, sampling options and draws), runs the model's own
forward pass, samples, and then feeds itself: the sampled tokens become the next
input and positions move on by one, so a replay needs the host only when a
request's pages, options or membership change.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .batch import StepBatch


class NotOnHost:
    """Stands where a StepBatch has a host list that a captured step cannot have (what it would say changes from
    replay to replay).  Any use raises, so that a part that walks requests on the host is found at capture, not by
    wrong results later."""

    def __init__(self, field: str, instead: str):
        self._message = (f"a captured decode step has no host copy of batch.{field}: read batch.{instead} on the device, "
                         "or leave capture_safe false on the part so that its steps run eagerly")

    def _refuse(self, *args, **kwargs):
        raise RuntimeError(self._message)

    __getitem__ = __iter__ = __len__ = __bool__ = __contains__ = _refuse


class DecodeGraph:
    def __init__(self, runner, num_requests: int, table_width: int, balanced_attention: bool = False, pool=None,
                 attention_splits: int = 0):
        self.runner = runner
        self.pool = pool  # the memory pool that the captures of one runner share for their temporaries (None: its own)
        self.num_requests = B = num_requests
        self.table_width = table_width
        device = runner.rt.device
        groups = len(runner.cache.groups)
        # packed int32 inputs: token_ids, positions, context_len, slots, then one table per group
        self.sections = [B, B, B, B] + [B * table_width] * groups
        offsets, cursor = [], 0
        for size in self.sections:
            offsets.append(cursor)
            cursor += -(-size // 4) * 4
        self.offsets = offsets
        # pinned staging buffers, two of each in turn: a step queued ahead copies from one while the host fills the
        # other for the step after it
        self.host_ints = [torch.zeros(cursor, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.dev_ints = torch.zeros(cursor, dtype=torch.int32, device=device)
        self.host_floats = [torch.zeros(3 * B, dtype=torch.float32).pin_memory() for _ in range(2)]
        self.loads = 0
        self.dev_floats = torch.zeros(3 * B, dtype=torch.float32, device=device)
        self.fixed = torch.arange(B + 1, dtype=torch.int32, device=device)

        def section(i, source):
            return source[offsets[i] : offsets[i] + self.sections[i]]

        self.token_ids, self.positions = section(0, self.dev_ints), section(1, self.dev_ints)
        self.context_len, self.slots = section(2, self.dev_ints), section(3, self.dev_ints)
        self.tables = [section(4 + g, self.dev_ints).view(B, table_width) for g in range(groups)]
        self._host = [[section(i, ints) for i in range(len(self.sections))] for ints in self.host_ints]
        self.batch = StepBatch(
            num_tokens=B, num_requests=B, token_ids=self.token_ids, positions=self.positions,
            request_of_token=self.fixed[:B], query_start=self.fixed, context_len=self.context_len, slots=self.slots,
            block_tables=self.tables, want_rows=self.fixed[:B], query_lens=[1] * B,
            start_positions=NotOnHost("start_positions", "positions"), slot_ids=NotOnHost("slot_ids", "slots"), max_query_len=1, max_context_len=table_width * runner.cache.page_size, num_want=B,
            num_decode=B, decode_balanced=balanced_attention, decode_splits=attention_splits or None,
        )
        self.tokens_out: Optional[torch.Tensor] = None
        self.logits_out: Optional[torch.Tensor] = None  # [B, V] float32 of the last replay (for checks; nothing reads it otherwise)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels_per_replay = 0
        # results of launched steps come back through pinned buffers, two of them in turn: a step's result is
        # read by the host while the step after it is already queued
        self.host_tokens = [torch.zeros(B, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.host_flag = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.launches = 0

    def _body(self) -> None:
        ops = self.runner.rt.ops
        model = self.runner.model
        resid, delta = model.forward(self.batch, self.runner.cache)
        logits = self.logits_out = model.logits(resid, delta, self.batch.want_rows)
        B = self.num_requests
        floats = self.dev_floats
        self.tokens_out = ops.sample_rows(logits, floats[:B], floats[B : 2 * B], floats[2 * B :])
        ops.decode_advance(self.token_ids, self.tokens_out, self.positions, self.context_len)

    def load_inputs(self, token_ids: Optional[Sequence[int]], positions: Sequence[int], slots: Sequence[int],
                    tables: Sequence[np.ndarray], temperatures: Sequence[float], top_ps: Sequence[float],
                    draws: Sequence[float]) -> None:
        """Copies a step's inputs from pinned host memory to the fixed device buffers (two copies).
        ``token_ids`` None leaves the token buffer as the step before left it: the tokens it sampled."""
        B = self.num_requests
        turn = self.loads & 1
        self.loads += 1
        host, host_ints, host_floats = self._host[turn], self.host_ints[turn], self.host_floats[turn]
        if token_ids is not None:
            host[0].copy_(torch.as_tensor(token_ids, dtype=torch.int32))
        position_tensor = torch.as_tensor(positions, dtype=torch.int32)
        host[1].copy_(position_tensor)
        host[2].copy_(position_tensor + 1)
        host[3].copy_(torch.as_tensor(slots, dtype=torch.int32))
        for g, table in enumerate(tables):
            padded = np.full((B, self.table_width), -1, dtype=np.int32)
            padded[:, : table.shape[1]] = table
            host[4 + g].copy_(torch.from_numpy(padded.reshape(-1)))
        host_floats[:B] = torch.as_tensor(temperatures, dtype=torch.float32)
        host_floats[B : 2 * B] = torch.as_tensor(top_ps, dtype=torch.float32)
        host_floats[2 * B :] = torch.as_tensor(draws, dtype=torch.float32)
        first = 0 if token_ids is not None else self.offsets[1]
        self.dev_ints[first:].copy_(host_ints[first:], non_blocking=True)
        self.dev_floats.copy_(host_floats, non_blocking=True)

    @property
    def input_bytes(self) -> int:
        return self.host_ints[0].numel() * 4 + self.host_floats[0].numel() * 4

    @property
    def ahead_input_bytes(self) -> int:
        """What a step copies that takes its tokens from the step before it on the device."""
        return (self.host_ints[0].numel() - self.offsets[1]) * 4 + self.host_floats[0].numel() * 4

    def capture(self) -> None:
        """Runs the step once eagerly (so that everything lazy has happened), then captures it.
        The inputs must describe a valid step; the keys and values that the eager run writes to the pages are
        written again, identically, by the first replay, and the fixed-size state of mixers that keep one is put
        back as it was, so that the first replay advances it once."""
        ops = self.runner.rt.ops
        saved = self.dev_ints.clone()
        state = self.runner.cache.state
        saved_state = {layer: tensor.clone() for layer, tensor in state.items() if tensor is not None}
        stream = torch.cuda.Stream(device=self.runner.rt.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self._body()
        torch.cuda.current_stream().wait_stream(stream)
        # (waiting here for the device is cheaper than capturing beside a busy device: without this wait a run of 64
        # requests with 16 captures took 3.4 to 4.0 s against 3.2 to 3.4 s)
        torch.cuda.synchronize()
        self.dev_ints.copy_(saved)  # undo the eager run's advance
        for layer, tensor in saved_state.items():
            state[layer].copy_(tensor)
        before = ops.launch_count
        # Captured with the graph object's own calls, on the side stream: the context manager of the library also
        # collects garbage and empties the allocator's cache on the way in, 40 to 700 ms in a process with a large
        # heap, against 10 ms for the capture itself; a serving run captures a new batch size every few seconds.
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            self.graph.capture_begin(**({"pool": self.pool} if self.pool is not None else {}))
            try:
                self._body()
            finally:
                self.graph.capture_end()
        torch.cuda.current_stream().wait_stream(stream)
        self.kernels_per_replay = ops.launch_count - before
        self.dev_ints.copy_(saved)  # capture does not run the kernels, but keep the inputs as the caller set them

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.tokens_out

    def launch(self) -> "LaunchedStep":
        """Replays without waiting: the sampled tokens and the device error word are copied to pinned host
        memory behind the step, and an event marks the copies' end."""
        index = self.launches & 1
        self.launches += 1
        self.graph.replay()
        self.host_tokens[index].copy_(self.tokens_out, non_blocking=True)
        self.host_flag[index].copy_(self.runner.rt.ops.error_flag(self.runner.rt.device), non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return LaunchedStep(self, index, event)


class LaunchedStep:
    """A decode step that is queued or running on the device."""

    def __init__(self, graph: DecodeGraph, index: int, event: torch.cuda.Event):
        self.graph, self.index, self.event = graph, index, event

    def wait(self) -> List[int]:
        """Waits for the step; raises if a kernel set the device error word; returns the sampled tokens."""
        self.event.synchronize()
        ops = self.graph.runner.rt.ops
        value = int(self.graph.host_flag[self.index][0])
        if value != 0:
            ops.check_device_errors(self.graph.runner.rt.device)  # reads, clears and raises
        return self.graph.host_tokens[self.index].tolist()


class DecodeGraphs:
    """The captured decode steps of a runner, by (requests, table width bucket, decode attention kernel and its ranges)."""

    def __init__(self, runner):
        self.runner = runner
        self.graphs: Dict[Tuple[int, int, bool, int], DecodeGraph] = {}
        self.pool = None  # made with the first graph: one pool for the temporaries of all captures, which never run at once

    def _plan(self, context_lens: Sequence[int]) -> Tuple[bool, int]:
        """The cheaper decode attention kernel and, for the split kernel, its number of ranges, by the model in
        ops.decode_plan over the layers' cache needs (all of a model's attention layers take the same kernel in one
        captured step: the widest need decides).  The ranges are planned for the lengths that the requests have, not
        for the longest that the block tables' bucket could hold: at 7 requests of 4,100 tokens that is 2 ranges, not
        the 5 that 8,192 tokens would want (3.55 against 3.67 ms a step)."""
        ops = self.runner.rt.ops
        groups = list(self.runner.cache.groups)
        if not groups:
            return False, 0
        need = max(groups, key=lambda g: g.window or (1 << 60))
        device = self.runner.rt.device
        balanced, splits = ops.decode_plan(context_lens, need.kv_heads, need.window, sms=ops.sm_count(device),
                                           room=ops.decode_cluster_room(device, need.head_dim), head_dim=need.head_dim)
        return balanced, (0 if balanced else splits)

    @staticmethod
    def batch_bucket(requests: int) -> int:
        """The batch size whose captured step serves ``requests`` requests: every size up to 8, then four sizes to each
        doubling (10, 12, 14, 16, 20, 24, ...), so that at most a fifth of a step's rows are padding.  (Two sizes to a
        doubling saved 7 of 20 captures of about 16 ms each in a run of 64 requests that ended one by one, and cost
        its decode steps 0.37 s of 1.65 s: rows of padding are not free in the products.)"""
        if requests <= 8:
            return requests
        step = 1 << (max(requests - 1, 1).bit_length() - 3)
        return -(-requests // step) * step

    @staticmethod
    def width_bucket(width: int) -> int:
        bucket = 16
        while bucket < width:
            bucket *= 2
        return bucket

    def get(self, num_requests: int, table_width: int, context_lens: Optional[Sequence[int]] = None
            ) -> Tuple[DecodeGraph, bool]:
        """The graph for this shape and whether it still has to be captured.  ``context_lens`` (the requests'
        lengths after this step) choose between the two decode attention kernels; each has its own capture."""
        balanced, splits = False, 0
        if context_lens is not None:
            balanced, splits = self._plan(context_lens)
        key = (num_requests, self.width_bucket(table_width), balanced, splits)
        graph = self.graphs.get(key)
        if graph is None:
            if self.pool is None or not self.graphs:
                # (a pool whose graphs have all been dropped is gone; its handle must not be used again)
                self.pool = torch.cuda.graph_pool_handle()
            graph = DecodeGraph(self.runner, key[0], key[1], balanced, self.pool, splits)
            self.graphs[key] = graph
        return graph, graph.graph is None


def captured_and_eager_logits(graphs: DecodeGraphs, requests: Sequence[object], tokens: Sequence[int]) -> dict:
    """A check of the captured decode step against the step function, on the same cache state.

    ``requests`` (page handles of live requests) each bring one token of ``tokens``.  The step runs through the
    captured graph, and the step after it is queued behind it the way the engine queues ahead: its input tokens
    are the ones the first step sampled (greedy), taken on the device.  Then the same two steps run through
    ``run_step``, which writes the same keys and values to the same places again and commits them.  Returns the
    four logits tensors [B, V] and the tokens of the first step; the requests end two tokens longer.
    """
    from .batch import StepEntry
    from .step import run_step

    runner = graphs.runner
    cache = runner.cache
    B = len(requests)
    for request in requests:
        if not cache.reserve(request, 2):
            raise RuntimeError("no pages left for the two steps of the check")
    lengths = [request.length for request in requests]
    tables = [cache.block_table_array(requests, g) for g in range(len(cache.groups))]
    width = max([1] + [t.shape[1] for t in tables])
    graph, fresh = graphs.get(B, width, [n + 1 for n in lengths])
    greedy = ([0.0] * B, [1.0] * B, [0.0] * B)
    graph.load_inputs(list(tokens), lengths, [r.slot for r in requests], tables, *greedy)
    if fresh:
        graph.capture()
    first = graph.launch()
    captured_first = graph.logits_out.clone()
    graph.load_inputs(None, [n + 1 for n in lengths], [r.slot for r in requests], tables, *greedy)
    second = graph.launch()
    captured_second = graph.logits_out.clone()
    sampled = first.wait()
    second.wait()
    eager_first = run_step(runner.model, cache, [StepEntry(r, [int(t)], [0]) for r, t in zip(requests, tokens)])
    eager_second = run_step(runner.model, cache, [StepEntry(r, [int(t)], [0]) for r, t in zip(requests, sampled)])
    return {"captured": (captured_first, captured_second), "eager": (eager_first, eager_second), "sampled": sampled,
            "balanced": graph.batch.decode_balanced, "kernels": graph.kernels_per_replay}
