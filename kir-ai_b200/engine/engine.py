"""The Python entry point: ``Engine.generate`` (token ids in, token ids out).

The engine owns a loaded model with its cache (``ModelRunner``), a scheduler and
the sampler, and runs the loop: schedule, step, sample, update.  Option names
and defaults follow the reference's command line where it has them
(crates/llm-engine/src/main.rs:423-475: ``--snapshot``, ``--max-new-tokens`` 256,
``--max-prefill-tokens`` 2048, ``--max-concurrent-requests`` 4); the reference
ignores ``generation_config.json`` and so does this engine.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Union


from ..sampling import rng
from ..sampling.params import SamplingParams
from ..sampling.sampler import sample
from .batch import StepEntry
from .graphs import DecodeGraphs
from .runner import ModelRunner
from .scheduler import FINISHED, RUNNING, NativeScheduler, Request, Scheduled, Scheduler

MAX_NEW_TOKENS_CAP = 65_536       # crates/llm-engine/src/main.rs:25-29
MAX_PREFILL_TOKENS_CAP = 262_144
MAX_CONCURRENT_CAP = 256


@dataclass
class GenerationOutput:
    token_ids: List[int]
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    preemptions: int = 0


class Engine:
    def __init__(self, snapshot: Optional[str] = None, *, config=None, random_weights_seed: Optional[int] = None,
                 dtype: str = "bfloat16", device: str = "cuda:0", max_new_tokens: int = 256,
                 max_prefill_tokens: int = 2048, max_concurrent_requests: int = 4, page_size: int = 16,
                 max_cache_tokens: Optional[int] = None, prefill_chunk: Optional[int] = None,
                 runner: Optional[ModelRunner] = None, cuda_graphs: bool = True, overlap_steps: bool = True):
        if not 1 <= max_new_tokens <= MAX_NEW_TOKENS_CAP:
            raise ValueError(f"--max-new-tokens must be within 1..{MAX_NEW_TOKENS_CAP}")
        if not 1 <= max_prefill_tokens <= MAX_PREFILL_TOKENS_CAP:
            raise ValueError(f"--max-prefill-tokens must be within 1..{MAX_PREFILL_TOKENS_CAP}")
        if not 1 <= max_concurrent_requests <= MAX_CONCURRENT_CAP:
            raise ValueError(f"--max-concurrent-requests must be within 1..{MAX_CONCURRENT_CAP}")
        if runner is None:
            if snapshot is not None and config is None:
                from ..registry import load_config

                config = load_config(snapshot)
            if config is None:
                raise ValueError("give a snapshot folder, or a configuration with random_weights_seed")
            max_positions = getattr(config, "max_position_embeddings", None)
            if max_cache_tokens is None:
                per_request = max(max_prefill_tokens + max_new_tokens, 4096)
                if max_positions:
                    per_request = min(per_request, max_positions)
                max_cache_tokens = max_concurrent_requests * per_request
            # one slot and one page beyond the requests' are for the padding rows of captured decode steps
            common = dict(dtype=dtype, device=device, page_size=page_size, max_tokens=max_cache_tokens + (page_size if cuda_graphs else 0),
                          num_slots=max_concurrent_requests + (1 if cuda_graphs else 0))
            if random_weights_seed is not None:
                runner = ModelRunner.from_random(config, random_weights_seed, **common)
            else:
                runner = ModelRunner.from_folder(snapshot, **common)
        self.runner = runner
        self.max_new_tokens = max_new_tokens
        # the scheduler's decisions run in native code when the cache's page tables do (the default); the Python
        # class decides the same and stays as the readable model
        from ..cache.native_pages import NativePageTables

        scheduler_class = NativeScheduler if isinstance(runner.cache.tables, NativePageTables) else Scheduler
        self.scheduler = scheduler_class(
            runner.cache, max_batched_tokens=max_prefill_tokens, max_running=max_concurrent_requests,
            prefill_chunk=prefill_chunk, max_positions=runner.model.plan.max_positions,
            default_max_new_tokens=max_new_tokens,
        )
        self._next_id = 0
        # None, or a list that receives one entry per step that is launched: [(tokens in the cache before, new tokens)
        # of every request in it] (measurements compute a step's bytes and flops from it)
        self.step_log: Optional[list] = None
        self.counters = {"steps": 0, "graph_steps": 0, "prompt_tokens": 0, "generated_tokens": 0}
        # decode steps are replayed from CUDA graphs only when every part of the model promises that this is safe
        # (Part.capture_safe); a model with a part that does not say so runs every step eagerly
        self.graphs = DecodeGraphs(runner) if cuda_graphs and runner.model.plan.capture_safe() else None
        self.overlap_steps = overlap_steps
        self._in_flight = None  # (scheduled, LaunchedStep) of a decode step that is queued or running
        # Captured decode steps exist for a few batch sizes only (a capture costs tens of milliseconds, and a batch
        # shrinks request by request as requests finish): a step of n requests replays the graph of the next size up,
        # its spare rows filled with a padding request that holds one page and one slot of its own, whose one token
        # at position 0 is computed and thrown away.  Without a spare slot every batch size gets its own graph.
        self._padding = None
        if self.graphs is not None:
            padding = runner.cache.open(("padding rows of captured steps",))
            if padding is not None and runner.cache.reserve(padding, 1):
                self._padding = padding
            elif padding is not None:
                runner.cache.close(padding)

    # ------------------------------------------------------------------ generate
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        params = params or SamplingParams()
        vocab = self.runner.model.plan.vocab_size
        for token in prompt:
            if not 0 <= int(token) < vocab:
                raise ValueError(f"token id {token} outside vocab size {vocab}")
        request = self.scheduler.add(self._next_id, prompt, params)
        self._next_id += 1
        return request

    def step(self) -> List[Request]:
        """One scheduler step; returns the requests that finished in it.

        Decode steps that replay a captured graph are queued one ahead: while the device runs a step, the host
        prepares and queues the next one for the same requests (its input tokens are the ones the running step
        samples, already on the device), and only then waits for the running step's tokens.  A request that turns
        out to have finished (end-of-sequence token) has its token of the step queued ahead dropped."""
        if self._in_flight is None:
            scheduled = self.scheduler.schedule()
            if not (self.graphs is not None and scheduled and all(item.count == 1 for item in scheduled)):
                sampled = self._general_step(scheduled)
                self.runner.rt.ops.check_device_errors(self.runner.rt.device)
                self.counters["steps"] += 1
                return self.scheduler.update(scheduled, sampled)
            self._in_flight = self._launch_decode(scheduled, ahead=False)
        current = self._in_flight
        self._in_flight = self._launch_ahead(current) if self.overlap_steps else None
        return self._retire(current)

    def drain(self) -> List[Request]:
        """Waits for a step that is still queued or running and records it; returns the requests it finished."""
        if self._in_flight is None:
            return []
        current, self._in_flight = self._in_flight, None
        return self._retire(current)

    def abort(self, request: Request) -> List[Request]:
        """Ends a request between steps (finish reason "aborted") and gives back what it holds.  A step that is still
        queued or running is waited for first, so that no kernel in flight reads pages that are handed out again;
        the requests which that step finished are returned.  The reference checks its cancellation tokens at the
        same places, between prompt portions and between decode steps
        (crates/llm-native-runtime/src/native_text/driver.rs:440-454, 801-804)."""
        finished = self.drain()
        if request.state != FINISHED:
            self.scheduler.abort(request)
        return finished

    def _retire(self, flight) -> List[Request]:
        scheduled, launched = flight
        tokens = launched.wait()
        # a request that finished while this step was queued behind its last one: the token is dropped
        live = [(item, token) for item, token in zip(scheduled, tokens) if item.request.state == RUNNING]
        self.counters["steps"] += 1
        return self.scheduler.update([item for item, _ in live], [token for _, token in live])

    def _launch_ahead(self, flight):
        """Queues the decode step after ``flight`` for the same requests, if nothing about the batch can change:
        nobody can be admitted (no one waits, or the running set is full), nobody reaches its token limit in ``flight``, every request gets its page
        without an eviction, and the step replays the same captured graph.  Otherwise None."""
        scheduled, launched = flight
        scheduler = self.scheduler
        if len(scheduled) != len(scheduler.running):
            return None
        if scheduler.waiting and len(scheduler.running) < scheduler.max_running:
            return None  # a waiting request may be admitted into the next step
        for item in scheduled:
            request = item.request
            if request.state != RUNNING or len(request.output) + 2 > request.max_new_tokens:
                return None
        pages = [item.request.pages for item in scheduled]
        cache = self.runner.cache
        if not all(cache.reserve(p, 1) for p in pages):
            return None  # what was reserved stays with its request and is used by its next step
        ahead = [Scheduled(item.request, item.first + 1, 1, True) for item in scheduled]
        return self._launch_decode(ahead, ahead=True, same_graph=launched.graph)

    def _launch_decode(self, scheduled, ahead: bool, same_graph=None):
        """Every request brings one token: queues the captured step for this many requests (the scheduler, or
        ``_launch_ahead``, has reserved the pages) and returns (scheduled, launched step), or None if ``ahead``
        and the step would need another graph."""
        cache = self.runner.cache
        requests = [item.request for item in scheduled]
        pages = [r.pages for r in requests]
        spare = (self.graphs.batch_bucket(len(requests)) - len(requests)) if self._padding is not None else 0
        rows = pages + [self._padding] * spare  # spare rows: the padding request's token at position 0, again and again
        tables = [cache.block_table_array(rows, g) for g in range(len(cache.groups))]
        width = max([1] + [t.shape[1] for t in tables])
        graph, fresh = self.graphs.get(len(rows), width, [p.length + 1 for p in rows])
        if ahead and (fresh or graph is not same_graph):
            return None  # a capture, or another graph's buffers: that step is queued after this one is known
        extra = 1 if ahead else 0  # draws that the step in flight will have used
        graph.load_inputs(
            None if ahead else [r.token_at(item.first) for r, item in zip(requests, scheduled)] + [0] * spare,
            [p.length for p in rows], [p.slot for p in rows], tables, [r.params.temperature for r in requests] + [0.0] * spare,
            [r.params.top_p for r in requests] + [1.0] * spare, [rng.draw(r.seed, r.draws_used + extra) for r in requests] + [0.0] * spare,
        )
        if fresh:
            graph.capture()
        launched = graph.launch()
        if self.step_log is not None:
            self.step_log.append([(p.length, 1) for p in pages])
        for p in pages:
            cache.commit(p, 1)  # bookkeeping only: the step's cache writes are queued in stream order
        self.counters["graph_steps"] += 1
        return scheduled, launched

    def _general_step(self, scheduled) -> List[Optional[int]]:
        entries = []
        if self.step_log is not None:
            self.step_log.append([(item.first, item.count) for item in scheduled])
        for item in scheduled:
            tokens = item.request.token_slice(item.first, item.count)
            entries.append(StepEntry(item.request.pages, tokens, [item.count - 1] if item.sample else []))
        logits = self.runner.step(entries, check_errors=False)
        sampled: List[Optional[int]] = [None] * len(scheduled)
        if logits is not None:
            rows = [i for i, item in enumerate(scheduled) if item.sample]
            requests = [scheduled[i].request for i in rows]
            tokens = sample(
                self.runner.rt.ops, logits,
                [r.params.temperature for r in requests], [r.params.top_p for r in requests],
                [rng.draw(r.seed, r.draws_used) for r in requests],
            ).cpu().tolist()
            for i, token in zip(rows, tokens):
                sampled[i] = token
        return sampled

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[None, SamplingParams, Sequence[SamplingParams]] = None) -> List[GenerationOutput]:
        """Generates a continuation for every prompt (lists of token ids); results in the prompts' order."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        requests = [self.add_request(prompt, p) for prompt, p in zip(prompts, params)]
        while self.scheduler.has_work():
            self.step()
        self.drain()
        outputs = []
        for request in requests:
            self.counters["prompt_tokens"] += len(request.prompt)
            self.counters["generated_tokens"] += len(request.output)
            outputs.append(GenerationOutput(list(request.output), request.finish_reason or "length", len(request.prompt),
                                            len(request.output), request.preemptions))
        return outputs

    def stats(self) -> dict:
        """Counters of the engine, the scheduler and the cache; the cache's figures are those of the requests (the one
        page and slot of the padding rows are taken out)."""
        cache = self.runner.cache.stats()
        if self._padding is not None:
            cache["live_requests"] -= 1
            cache["slots_free"] += 1
            for group in cache["groups"]:
                group["used"] -= 1
            cache["padding_rows"] = {"pages_per_group": 1, "slots": 1}
        return {**self.counters, "scheduler": dict(self.scheduler.stats), "cache": cache,
                "kernel_launches": dict(self.runner.rt.ops.launch_counts)}
