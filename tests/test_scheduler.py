"""The scheduler's decisions, on the host: admission, portions under the token budget, decode
first, finishing and freeing, and what happens when pages run out."""
import pytest

import kirai_b200
from kirai_b200.cache import CacheManager
from kirai_b200.engine.scheduler import AdmissionError, Scheduler
from kirai_b200.parts.base import KVCacheNeed
from kirai_b200.sampling.params import SamplingParams
from kirai_b200.sampling import rng


def make(num_pages=64, page_size=4, num_slots=4, **kwargs):
    cache = CacheManager([KVCacheNeed(1, 8, None), KVCacheNeed(1, 8, 8)], page_size=page_size, num_pages=num_pages,
                         num_slots=num_slots, device=None)
    defaults = dict(max_batched_tokens=16, max_running=4, max_positions=512, default_max_new_tokens=64)
    defaults.update(kwargs)
    return cache, Scheduler(cache, **defaults)


def run(scheduler, cache, token_of=lambda request: 7, max_steps=10_000):
    """Drives the scheduler with a stand-in for the model; returns the trace of steps."""
    trace = []
    while scheduler.has_work():
        chosen = scheduler.schedule()
        assert chosen and sum(item.count for item in chosen) <= scheduler.max_batched_tokens
        for item in chosen:  # what the step function does with the pages
            assert item.first == item.request.pages.length == item.request.computed
            cache.commit(item.request.pages, item.count)
        sampled = [token_of(item.request) if item.sample else None for item in chosen]
        trace.append([(item.request.request_id, item.first, item.count, item.sample) for item in chosen])
        scheduler.update(chosen, sampled)
        cache.tables.check_consistency()
        assert len(trace) < max_steps
    return trace


def test_prompt_is_cut_to_the_budget_then_decodes():
    cache, scheduler = make()
    request = scheduler.add("a", list(range(37)), SamplingParams(temperature=0.0, max_new_tokens=3))
    trace = run(scheduler, cache)
    assert [step[0][1:] for step in trace] == [(0, 16, False), (16, 16, False), (32, 5, True), (37, 1, True), (38, 1, True)]
    assert request.output == [7, 7, 7] and request.finish_reason == "length"
    assert request.computed == 39  # the last sampled token is never run
    assert cache.free_pages() == [64, 64] and cache.tables.slots.free_slots == 4


def test_decode_goes_first_and_prompts_share_the_rest():
    cache, scheduler = make()
    scheduler.add("a", [1, 2, 3], SamplingParams(max_new_tokens=5, seed=1))
    trace_first = scheduler.schedule()
    for item in trace_first:
        cache.commit(item.request.pages, item.count)
    scheduler.update(trace_first, [9])
    scheduler.add("b", list(range(40)), SamplingParams(max_new_tokens=2, seed=1))
    chosen = scheduler.schedule()
    assert [(c.request.request_id, c.count, c.sample) for c in chosen] == [("a", 1, True), ("b", 15, False)]


def test_prefill_chunk_and_concurrency_limit():
    cache, scheduler = make(max_batched_tokens=64, prefill_chunk=8, max_running=2)
    for name in "abc":
        scheduler.add(name, list(range(20)), SamplingParams(max_new_tokens=1, seed=0))
    chosen = scheduler.schedule()
    assert [(c.request.request_id, c.count) for c in chosen] == [("a", 8), ("b", 8)]  # c waits: two may run
    assert len(scheduler.waiting) == 1


def test_stop_token_and_ignore_eos():
    cache, scheduler = make()
    stops = scheduler.add("s", [1, 2], SamplingParams(max_new_tokens=10, eos_token_id=7, seed=0))
    goes_on = scheduler.add("g", [1, 2], SamplingParams(max_new_tokens=4, eos_token_id=7, ignore_eos=True, seed=0))
    run(scheduler, cache)
    assert stops.output == [7] and stops.finish_reason == "stop"
    assert goes_on.output == [7] * 4 and goes_on.finish_reason == "length"


def test_admission_refuses_what_can_never_run():
    cache, scheduler = make(num_pages=8)
    with pytest.raises(AdmissionError):
        scheduler.add("long", list(range(500)), SamplingParams(max_new_tokens=20))  # beyond max_positions
    with pytest.raises(AdmissionError):
        scheduler.add("big", list(range(40)), SamplingParams(max_new_tokens=2))     # 41 tokens > 8 pages of 4
    with pytest.raises(AdmissionError):
        scheduler.add("many", [1], SamplingParams(max_new_tokens=65))               # above the configured maximum
    with pytest.raises(AdmissionError):
        scheduler.add("empty", [], SamplingParams())
    assert scheduler.add("fits", list(range(30)), SamplingParams(max_new_tokens=3)) is not None


def test_pages_run_out_youngest_is_evicted_and_recomputed():
    # 12 pages of 4 tokens.  Two requests of 17 prompt tokens (5 pages each) decode 12 tokens each: they need
    # 8 pages each in the end, 16 in all, so one must give way and come back.
    cache, scheduler = make(num_pages=12, max_batched_tokens=32)
    a = scheduler.add("a", list(range(17)), SamplingParams(max_new_tokens=12, seed=0))
    b = scheduler.add("b", list(range(100, 117)), SamplingParams(max_new_tokens=12, seed=0))
    counter = {"a": 0, "b": 0}

    def token_of(request):
        counter[request.request_id] += 1
        return counter[request.request_id]

    trace = run(scheduler, cache, token_of)
    assert scheduler.stats["preemptions"] >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert a.output == list(range(1, 13)) and b.output == list(range(1, 13))  # nothing lost, nothing sampled twice
    assert b.draws_used == 12
    # after eviction b was run again from position 0 with its prompt and what it had generated
    restarts = [entry for step in trace for entry in step if entry[0] == "b" and entry[1] == 0]
    assert len(restarts) == 1 + b.preemptions and restarts[-1][2] > 17
    assert cache.free_pages() == [12, 12]


def test_portion_shrinks_to_free_pages():
    cache, scheduler = make(num_pages=6, max_batched_tokens=64)
    scheduler.add("a", list(range(14)), SamplingParams(max_new_tokens=1, seed=0))   # 4 pages
    scheduler.add("b", list(range(20)), SamplingParams(max_new_tokens=1, seed=0))   # would need 5, 2 are free
    chosen = scheduler.schedule()
    assert [(c.request.request_id, c.count, c.sample) for c in chosen] == [("a", 14, True), ("b", 8, False)]


@pytest.mark.parametrize("native", [False, True])
def test_two_prompts_that_stall_each_other_in_mid_prompt(native):
    # 100 pages of 16 tokens; two prompts of 1,280 tokens (80 pages each) cut into portions of 256: after three steps
    # both hold pages, neither can finish its prompt and nobody decodes.  The younger one must give way.
    from kirai_b200.engine.scheduler import NativeScheduler

    cache = CacheManager([KVCacheNeed(1, 8, None)], page_size=16, num_pages=100, num_slots=4, device=None)
    scheduler = (NativeScheduler if native else Scheduler)(
        cache, max_batched_tokens=512, max_running=4, prefill_chunk=256, max_positions=4096, default_max_new_tokens=8)
    a = scheduler.add("a", list(range(1280)), SamplingParams(max_new_tokens=4, seed=0))
    b = scheduler.add("b", list(range(1280)), SamplingParams(max_new_tokens=4, seed=0))
    trace = run(scheduler, cache)
    assert a.preemptions == 0 and b.preemptions >= 1 and scheduler.stats["preemptions"] == b.preemptions
    assert len(a.output) == 4 and len(b.output) == 4 and a.finish_reason == b.finish_reason == "length"
    assert cache.free_pages() == [100]
    # while a request waits for pages in mid-prompt nobody new is admitted: b comes back only after a has finished
    # its prompt or freed pages, and is then recomputed from its first token
    restarts = [entry for step in trace for entry in step if entry[0] == "b" and entry[1] == 0]
    assert len(restarts) == 1 + b.preemptions


def test_abort_frees_everything():
    cache, scheduler = make()
    request = scheduler.add("a", list(range(10)), SamplingParams(max_new_tokens=5, seed=0))
    waiting = scheduler.add("b", list(range(10)), SamplingParams(max_new_tokens=5, seed=0))
    chosen = scheduler.schedule()
    for item in chosen:
        cache.commit(item.request.pages, item.count)
    scheduler.update(chosen, [1, 1])
    scheduler.abort(request)
    scheduler.abort(waiting)
    assert request.finish_reason == "aborted" and not scheduler.has_work()
    assert cache.free_pages() == [64, 64] and cache.tables.slots.free_slots == 4


def test_draws_are_a_function_of_seed_and_count():
    values = [rng.draw(5, k) for k in range(1000)]
    assert all(0.0 <= v < 1.0 for v in values) and len(set(values)) > 990
    assert values[:3] == [rng.draw(5, 0), rng.draw(5, 1), rng.draw(5, 2)] and rng.draw(6, 0) != values[0]
    assert 0.45 < sum(values) / len(values) < 0.55


def test_sampling_params_ranges():
    for bad in (dict(temperature=-0.1), dict(temperature=2.5), dict(temperature=float("nan")), dict(top_p=0.0),
                dict(top_p=1.5), dict(max_new_tokens=0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams(temperature=0.0).greedy and SamplingParams().top_p == 1.0 and SamplingParams().temperature == 1.0


def test_decode_plan_prefers_the_balanced_kernel_only_for_uneven_or_badly_filled_batches():
    """The host-side choice between the two decode attention kernels (no GPU needed: it is arithmetic)."""
    import kirai_b200  # noqa: F401
    from kirai_b200.csrc.ops import decode_plan

    assert decode_plan([4096], 8)[0] is False                      # one request: the split kernel has the lower fixed cost
    assert decode_plan([4096] * 8, 8)[0] is False                  # equal lengths that fill one wave
    uneven = [1024, 7168, 2048, 6000, 3000, 5000, 4000, 1500]
    assert decode_plan(uneven, 8)[0] is True                       # the longest request would set the split kernel's time
    assert decode_plan([n for n in uneven], 8, window=512)[0] is False  # a window makes them equal again
    balanced, splits = decode_plan([100_000] + [500] * 15, 8)
    assert balanced is True and splits >= 1
    assert decode_plan([], 8) == (False, 1)


def test_decode_plan_over_random_batches_respects_the_kernels_limits():
    """Whatever the batch, the planner names a split count that the decode kernel takes (1 to 64 ranges, never more
    ranges than key tiles), and ranges are merged inside the kernel only where the device said the clusters fit and
    the other CTAs' rows fit the first one's slots."""
    import random

    import kirai_b200  # noqa: F401
    from kirai_b200.csrc.ops import DECODE_CLUSTER_RANGES, decode_pair_merges, decode_plan, decode_splits

    rnd = random.Random(4)
    for _ in range(300):
        sms = rnd.choice([16, 66, 132, 148])
        counts = {1: sms, 2: sms // 2, 3: rnd.randint(0, sms // 3), 4: rnd.randint(0, sms // 4), 5: rnd.randint(0, sms // 5)}
        room = lambda cluster: counts.get(cluster, 0)  # noqa: E731
        kv_heads, group, head_dim = rnd.choice([1, 2, 8]), rnd.choice([1, 3, 4, 8, 16]), rnd.choice([64, 128, 256])
        lens = [rnd.randint(1, rnd.choice([40, 5000, 40000])) for _ in range(rnd.randint(1, 70))]
        window = rnd.choice([None, None, 512])
        balanced, splits = decode_plan(lens, kv_heads, window, sms=sms, room=room, head_dim=head_dim, group=group)
        longest = max(min(n, window) if window else n for n in lens)
        assert isinstance(balanced, bool) and 1 <= splits <= min(64, -(-longest // 16))
        assert splits == decode_splits(len(lens), kv_heads, longest, sms=sms, room=room, head_dim=head_dim, group=group)
        pairs = len(lens) * kv_heads
        for ranges in range(1, 9):
            merges = decode_pair_merges(pairs, ranges, head_dim, room, group)
            if merges:
                assert 2 <= ranges <= DECODE_CLUSTER_RANGES and pairs <= counts[ranges] and head_dim <= 128
                assert (ranges - 1) * group <= 16


def drive_random_workload(scheduler_class, seed):
    """A random workload (arrivals over time, stop tokens, aborts, few pages and slots) through a scheduler; the
    trace of every decision and of what was left at the end."""
    import random

    rnd = random.Random(seed)
    page_size, num_pages, slots = rnd.choice([2, 4, 8]), rnd.randint(6, 40), rnd.randint(1, 5)
    cache = CacheManager([KVCacheNeed(1, 8, None), KVCacheNeed(1, 8, 8)], page_size=page_size, num_pages=num_pages,
                         num_slots=slots, device=None)
    scheduler = scheduler_class(cache, max_batched_tokens=rnd.choice([4, 16, 33]), max_running=rnd.randint(1, 5), max_positions=512,
                                default_max_new_tokens=64, prefill_chunk=rnd.choice([None, 3, 8]))
    arrivals = [(rnd.randint(1, 40), rnd.randint(1, 12), rnd.randint(0, 30)) for _ in range(rnd.randint(1, 12))]
    trace, step, added = [], 0, 0
    while scheduler.has_work() or added < len(arrivals):
        while added < len(arrivals) and arrivals[added][2] <= step:
            prompt_len, new_tokens, _ = arrivals[added]
            added += 1
            try:
                scheduler.add(f"r{added}", list(range(prompt_len)), SamplingParams(temperature=0.0, max_new_tokens=new_tokens, eos_token_id=5))
            except AdmissionError:
                trace.append(("refused", added))
        step += 1
        if not scheduler.has_work():
            continue
        chosen = scheduler.schedule()  # always finds something to run: it raises if it is stuck
        for item in chosen:
            assert item.first == item.request.pages.length == item.request.computed
            cache.commit(item.request.pages, item.count)
        sampled = [(5 if rnd.random() < 0.05 else 7) if item.sample else None for item in chosen]
        trace.append([(item.request.request_id, item.first, item.count, item.sample) for item in chosen])
        trace.append(("finished", sorted(r.request_id for r in scheduler.update(chosen, sampled))))
        if rnd.random() < 0.03 and scheduler.running:
            victim = rnd.choice(scheduler.running)
            scheduler.abort(victim)
            trace.append(("abort", victim.request_id))
        cache.tables.check_consistency()
        assert step < 5000
    trace.append(("left", cache.free_pages(), cache.tables.slots.free_slots, dict(scheduler.stats)))
    return trace, scheduler.stats["preemptions"]


def test_native_scheduler_decides_as_the_python_model_does():
    """The scheduler in native code (the one the engine uses) against the Python class, step by step, on random
    workloads that admit, cut prompts, evict, recompute, stop, abort and refuse."""
    from kirai_b200.engine.scheduler import NativeScheduler

    evictions = 0
    for seed in range(150):
        expected, preempted = drive_random_workload(Scheduler, seed)
        got, _ = drive_random_workload(NativeScheduler, seed)
        assert got == expected, f"seed {seed}"
        evictions += preempted
    assert evictions > 20  # the workloads do run out of pages
