"""The scheduler: which requests run which tokens in the next step.

Every step: (1) each running request that is decoding gets its one token;
(2) what is left of the token budget goes to prompt portions, first of requests
already running, then of waiting requests in arrival order, which are admitted
while a state slot is free and the running set is below its limit.  A prompt is
cut wherever the budget (or ``prefill_chunk``) ends.  The last sampled token of a
request is never run through the model, as in the reference's loop
(crates/llm-native-runtime/src/native_text/driver.rs:439-477).

When pages run out: a prompt portion shrinks to the pages that are free, or
waits (and nobody new is admitted while one waits); a decoding request that
cannot get its next page evicts the most recently admitted other running
request, and so does a step in which nothing at all could run (all running
requests in mid-prompt, all pages held); the evicted request's pages and slot
are freed and it goes back to the front of the waiting queue to be recomputed (its prompt
and the tokens it has generated are prefilled again; its random draws continue
where they were).  A request that could not run even alone is refused when it is
added.  The reference sizes each request's cache up front and refuses what
cannot fit (crates/llm-native-runtime/src/native_text/generation.rs:35-69); its paged pool
evicts the least recently used session (crates/llm-kv-cache/src/block_pool.rs:811-838);
its server admits by a concurrency limit (crates/llm-server/src/engine/scheduler.rs:642-668).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence

from ..sampling.params import SamplingParams
from ..sampling.rng import fresh_seed

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class AdmissionError(ValueError):
    """A request that this engine can never run (too long for the model or the cache)."""


@dataclass(eq=False)  # requests are compared by identity, never by their (long) token lists
class Request:
    request_id: object
    prompt: List[int]
    params: SamplingParams
    max_new_tokens: int
    seed: int
    output: List[int] = field(default_factory=list)
    state: str = WAITING
    finish_reason: Optional[str] = None  # "stop" | "length" | "aborted"
    pages: object = None           # cache handle while running
    computed: int = 0              # tokens whose keys and values are in the cache
    draws_used: int = 0            # random draws consumed so far
    preemptions: int = 0
    key: int = 0                   # the native scheduler's name for the request

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def token_at(self, index: int) -> int:
        n = len(self.prompt)
        return self.prompt[index] if index < n else self.output[index - n]

    def token_slice(self, first: int, count: int) -> List[int]:
        n = len(self.prompt)
        if first + count <= n:
            return self.prompt[first : first + count]
        return [self.token_at(i) for i in range(first, first + count)]

    @property
    def pending(self) -> int:
        """Tokens not yet run: the rest of the prompt, or the one token sampled last."""
        return len(self.prompt) + len(self.output) - self.computed


@dataclass
class Scheduled:
    request: Request
    first: int       # index into request.tokens of the first token run in this step
    count: int
    sample: bool     # the run reaches the end of the request's tokens: sample the next one


class Scheduler:
    def __init__(self, cache, *, max_batched_tokens: int = 2048, max_running: int = 4,
                 prefill_chunk: Optional[int] = None, max_positions: Optional[int] = None,
                 default_max_new_tokens: int = 256):
        if max_batched_tokens < 1 or max_running < 1:
            raise ValueError("max_batched_tokens and max_running must be positive")
        self.cache = cache
        self.max_batched_tokens = max_batched_tokens
        self.max_running = max_running
        self.prefill_chunk = prefill_chunk
        self.max_positions = max_positions
        self.default_max_new_tokens = default_max_new_tokens
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []  # in admission order
        self.stats = {"steps": 0, "preemptions": 0, "scheduled_tokens": 0, "finished": 0}

    # -- admission ----------------------------------------------------------
    def add(self, request_id, prompt: Sequence[int], params: SamplingParams) -> Request:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise AdmissionError("a request needs at least one prompt token")
        max_new = params.max_new_tokens if params.max_new_tokens is not None else self.default_max_new_tokens
        if max_new > self.default_max_new_tokens:
            raise AdmissionError(f"max_tokens {max_new} exceeds the configured maximum {self.default_max_new_tokens}")
        total = len(prompt) + max_new
        if self.max_positions is not None and total > self.max_positions:
            raise AdmissionError(
                f"prompt of {len(prompt)} tokens plus {max_new} new tokens exceeds the model's "
                f"{self.max_positions} positions"
            )
        # the last sampled token is never run, so the cache holds at most total - 1 tokens
        pages = self.cache.pages_for_tokens(total - 1)
        if any(pages > pool.num_pages for pool in self.cache.tables.pools):
            raise AdmissionError(
                f"request needs {pages} cache pages of {self.cache.page_size} tokens; the pool has "
                f"{min(pool.num_pages for pool in self.cache.tables.pools)}"
            )
        request = Request(request_id, prompt, params, max_new, params.seed if params.seed is not None else fresh_seed())
        self.waiting.append(request)
        return request

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- one step -------------------------------------------------------------
    def _portion(self, request: Request, budget: int) -> int:
        count = min(request.pending, budget)
        if self.prefill_chunk is not None and request.pending > 1:
            count = min(count, self.prefill_chunk)
        return count

    def _fit_to_pages(self, request: Request, count: int) -> int:
        """The largest portion <= count whose pages are free (whole pages beyond what it holds)."""
        if self.cache.can_reserve(request.pages, count):
            return count
        free = min(self.cache.free_pages()) if self.cache.free_pages() else 0
        held_capacity = min(len(t) for t in request.pages.tables) * self.cache.page_size if request.pages.tables else 0
        room = held_capacity - request.pages.length + free * self.cache.page_size
        room = min(room, count)
        while room > 0 and not self.cache.can_reserve(request.pages, room):
            room -= 1
        return max(room, 0)

    def _preempt(self, victim: Request) -> None:
        self.cache.close(victim.pages)
        victim.pages = None
        victim.computed = 0
        victim.state = WAITING
        victim.preemptions += 1
        self.running.remove(victim)
        self.waiting.appendleft(victim)
        self.stats["preemptions"] += 1

    def schedule(self) -> List[Scheduled]:
        """Chooses the next step's runs and reserves their pages."""
        budget = self.max_batched_tokens
        chosen: List[Scheduled] = []
        taken = set()

        # (1) decoding requests, oldest first; evict the youngest others when a page is missing
        for request in list(self.running):
            if request.state != RUNNING or request.pending != 1 or budget < 1:
                continue
            while not self.cache.reserve(request.pages, 1):
                victims = [r for r in reversed(self.running) if r is not request and id(r) not in taken]
                if not victims:
                    break
                self._preempt(victims[0])
            else:
                chosen.append(Scheduled(request, request.computed, 1, True))
                taken.add(id(request))
                budget -= 1
                continue
            # nothing left to evict: the request waits for pages (others that were chosen will free some)
        # (2) prompt portions of running requests
        def prompt_portions(budget: int):
            starved = False
            for request in self.running:
                if id(request) in taken or budget < 1 or request.pending < 1:
                    continue
                count = self._fit_to_pages(request, self._portion(request, budget))
                if count < 1:
                    starved = True
                    continue
                ok = self.cache.reserve(request.pages, count)
                assert ok
                chosen.append(Scheduled(request, request.computed, count, count == request.pending))
                taken.add(id(request))
                budget -= count
            return budget, starved

        budget, starved = prompt_portions(budget)
        # (3) admit waiting requests in order, unless a running request already found no page for its prompt
        while not starved and self.waiting and budget >= 1 and len(self.running) < self.max_running:
            request = self.waiting[0]
            pages = self.cache.open(request.request_id)
            if pages is None:
                break  # no state slot
            request.pages = pages
            count = self._fit_to_pages(request, self._portion(request, budget))
            if count < 1:
                self.cache.close(pages)
                request.pages = None
                break
            ok = self.cache.reserve(pages, count)
            assert ok
            self.waiting.popleft()
            request.state = RUNNING
            self.running.append(request)
            chosen.append(Scheduled(request, 0, count, count == request.pending))
            taken.add(id(request))
            budget -= count
        # (4) nothing could run: every running request is in mid-prompt and the pages are all held (a decoding
        # request would have evicted the others in (1)).  The youngest gives its pages to the others until the
        # oldest can go on; a request that is alone always fits (it was refused at admission otherwise).
        while not chosen and len(self.running) > 1:
            self._preempt(self.running[-1])
            budget, starved = prompt_portions(budget)
        if not chosen and self.has_work():
            raise RuntimeError("scheduler made no progress: no request fits the free pages")
        self.stats["steps"] += 1
        self.stats["scheduled_tokens"] += sum(s.count for s in chosen)
        return chosen

    def update(self, scheduled: Sequence[Scheduled], sampled: Sequence[Optional[int]]) -> List[Request]:
        """Records what a step did (``sampled[i]`` is the token of ``scheduled[i]`` if it sampled)
        and returns the requests that finished; their pages and slots are freed at once."""
        finished: List[Request] = []
        for item, token in zip(scheduled, sampled):
            request = item.request
            request.computed += item.count
            if not item.sample:
                continue
            assert token is not None
            request.output.append(int(token))
            request.draws_used += 1
            params = request.params
            if params.eos_token_id is not None and not params.ignore_eos and int(token) == params.eos_token_id:
                request.finish_reason = "stop"
            elif len(request.output) >= request.max_new_tokens:
                request.finish_reason = "length"
            if request.finish_reason:
                self._finish(request)
                finished.append(request)
        return finished

    def _finish(self, request: Request) -> None:
        if request.pages is not None:
            self.cache.close(request.pages)
            request.pages = None
        request.state = FINISHED
        if request in self.running:
            self.running.remove(request)
        self.stats["finished"] += 1

    def abort(self, request: Request) -> None:
        """Ends a request between steps; what it holds is given back."""
        if request.state == FINISHED:
            return
        if request in self.waiting:
            self.waiting.remove(request)
        request.finish_reason = "aborted"
        self._finish(request)


class NativeScheduler(Scheduler):
    """The same scheduler with its decisions made in native code (csrc/scheduler.cpp) on the native page tables.

    The native side knows requests by key and counts; token values, options and stop conditions stay here, and
    the lists ``waiting`` and ``running`` and the requests' fields mirror what the native side decided.  The Python
    class above is the readable model of the same rules; the tests run both on the same random workloads."""

    def __init__(self, cache, **kwargs):
        super().__init__(cache, **kwargs)
        import ctypes

        from ..cache.native_pages import NativePageTables, _library

        if not isinstance(cache.tables, NativePageTables):
            raise ValueError("the native scheduler works on the native page tables")
        self._ctypes = ctypes
        self._lib = lib = _library()
        lib.kirai_sched_create.restype = ctypes.c_void_p
        lib.kirai_sched_create.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_long, ctypes.c_long, ctypes.c_long]
        lib.kirai_sched_destroy.argtypes = [ctypes.c_void_p]
        lib.kirai_sched_add.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_long]
        lib.kirai_sched_abort.argtypes = [ctypes.c_void_p, ctypes.c_long]
        lib.kirai_sched_forget.argtypes = [ctypes.c_void_p, ctypes.c_long]
        lib.kirai_sched_stat.restype = ctypes.c_long
        lib.kirai_sched_stat.argtypes = [ctypes.c_void_p, ctypes.c_int]
        pointer = ctypes.c_void_p
        lib.kirai_sched_schedule.argtypes = [ctypes.c_void_p, pointer, pointer, pointer, pointer, ctypes.c_int, pointer,
                                             pointer, pointer, pointer, pointer]
        lib.kirai_sched_update.argtypes = [ctypes.c_void_p, pointer, pointer, pointer, pointer, ctypes.c_int]
        self._tables = cache.tables
        self._handle = lib.kirai_sched_create(cache.tables._handle, len(cache.tables.groups), cache.page_size,
                                              self.max_batched_tokens, self.max_running, self.prefill_chunk or -1)
        if not self._handle:
            raise ValueError("the native scheduler could not be created")
        self._by_key = {}

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.kirai_sched_destroy(handle)

    def _check(self, code: int, what: str) -> int:
        if code == -7:
            raise RuntimeError("scheduler made no progress: no request fits the free pages")
        if code < 0:
            raise RuntimeError(f"native scheduler: {what} failed with code {code}")
        return code

    def add(self, request_id, prompt: Sequence[int], params: SamplingParams) -> Request:
        request = super().add(request_id, prompt, params)
        request.key = self._tables.new_key()
        self._by_key[request.key] = request
        self._check(self._lib.kirai_sched_add(self._handle, request.key, len(request.prompt)), "add")
        return request

    def schedule(self) -> List[Scheduled]:
        ctypes = self._ctypes
        capacity = len(self.waiting) + len(self.running) + 1
        longs = lambda: (ctypes.c_long * capacity)()  # noqa: E731
        ints = lambda: (ctypes.c_int * capacity)()  # noqa: E731
        keys, first, count, sample = longs(), longs(), longs(), ints()
        preempted, admitted, slots = longs(), longs(), ints()
        num_preempted, num_admitted = ctypes.c_int(0), ctypes.c_int(0)
        runs = self._check(self._lib.kirai_sched_schedule(
            self._handle, keys, first, count, sample, capacity, preempted, ctypes.byref(num_preempted), admitted, slots,
            ctypes.byref(num_admitted)), "schedule")
        for i in range(num_preempted.value):  # mirror the evictions, in the order they happened
            victim = self._by_key[preempted[i]]
            self._tables.disown(victim.pages)
            victim.pages = None
            victim.computed = 0
            victim.state = WAITING
            victim.preemptions += 1
            self.running.remove(victim)
            self.waiting.appendleft(victim)
            self.stats["preemptions"] += 1
        for i in range(num_admitted.value):
            request = self._by_key[admitted[i]]
            assert self.waiting[0] is request
            self.waiting.popleft()
            request.pages = self._tables.adopt(request.request_id, request.key, slots[i])
            for tensor in self.cache.state.values():  # a fresh state slot, as CacheManager.open leaves it
                if tensor is not None:
                    tensor[request.pages.slot].zero_()
            request.state = RUNNING
            self.running.append(request)
        chosen = [Scheduled(self._by_key[keys[i]], first[i], count[i], bool(sample[i])) for i in range(runs)]
        self.stats["steps"] += 1
        self.stats["scheduled_tokens"] += sum(item.count for item in chosen)
        return chosen

    def update(self, scheduled: Sequence[Scheduled], sampled: Sequence[Optional[int]]) -> List[Request]:
        finished = super().update(scheduled, sampled)  # the Python side of it; _finish below does not touch the pages
        ctypes = self._ctypes
        runs = len(scheduled)
        done = {id(request) for request in finished}
        keys = (ctypes.c_long * max(runs, 1))(*[item.request.key for item in scheduled])
        counts = (ctypes.c_long * max(runs, 1))(*[item.count for item in scheduled])
        sampled_flags = (ctypes.c_int * max(runs, 1))(*[1 if item.sample else 0 for item in scheduled])
        finished_flags = (ctypes.c_int * max(runs, 1))(*[1 if id(item.request) in done else 0 for item in scheduled])
        self._check(self._lib.kirai_sched_update(self._handle, keys, counts, sampled_flags, finished_flags, runs), "update")
        for request in finished:
            self._forget(request)
        return finished

    def _finish(self, request: Request) -> None:
        # the native side closes the pages (in update or abort); here only the mirror
        if request.pages is not None:
            self._tables.disown(request.pages)
            request.pages = None
        request.state = FINISHED
        if request in self.running:
            self.running.remove(request)
        self.stats["finished"] += 1

    def _forget(self, request: Request) -> None:
        self._lib.kirai_sched_forget(self._handle, request.key)
        self._by_key.pop(request.key, None)

    def abort(self, request: Request) -> None:
        if request.state == FINISHED:
            return
        self._check(self._lib.kirai_sched_abort(self._handle, request.key), "abort")
        if request in self.waiting:
            self.waiting.remove(request)
        request.finish_reason = "aborted"
        self._finish(request)
        self._forget(request)
