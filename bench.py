#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen3-8B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers 36]

Prints ONE JSON line.  ``value`` is decoded tokens per second at the default batch with the
requests' caches filled to the context length: K decode steps (forward pass, logits, sampling)
replayed back to back on the device, timed with CUDA events.  ``e2e`` is the same through the
Python entry point (``Engine.step``): every step copies its inputs from pinned host memory and
reads the sampled tokens back to the host.  ``prefill`` is one 2,048-token prompt through the
step function; ``points`` holds decode at batch 1 and 64.  The engine runs on one GPU; for
--gpus > 1 one line says so and the exit code is 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

E2E_SETTLE_STEPS = 24  # untimed engine steps between the prompt phase and the end-to-end warm-up (see measure_decode)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
    max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as handle:
                raw = json.load(handle)
            peaks = dict(FALLBACK_PEAKS)
            for key in peaks:
                if isinstance(raw.get(key), (int, float)):
                    peaks[key] = float(raw[key])
            return peaks, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.process, self.thread = [], None, None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "--id=0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "", 1).isdigit()]
        sm_max = [float(s[1]) for s in self.samples if s[1].replace(".", "", 1).isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [name for i, name in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_numbers(cfg, layers):
    h, i, nq, nkv, d, v = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                           cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"])
    per_layer_weights = (nq + 2 * nkv) * d * h + h * nq * d + 2 * i * h + h * i
    return dict(
        layer_weight_elems=per_layer_weights, head_elems=v * h,
        weight_bytes=2 * (layers * per_layer_weights + v * h),      # every weight a decode step uses, once (bf16)
        kv_bytes_per_token=layers * 2 * nkv * d * 2,
        linear_flops_per_token=2 * layers * per_layer_weights,
        attention_flops=lambda tokens: layers * 2 * nq * d * tokens * tokens,  # causal: 2 products over T^2 / 2 pairs
    )


def ideal_seconds(step_log, numbers, cfg, peaks):
    """The least time the logged steps could take on this GPU: every step reads every weight once and the cache of
    the requests in it (bytes / measured copy bandwidth) and multiplies its tokens through the layers and its queries
    with their keys (flops / measured bf16 rate); a step takes the greater of the two, and the steps add up."""
    nq, d, layers = cfg["num_attention_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    total, byte_steps = 0.0, 0
    for step in step_log:
        tokens = sum(count for _, count in step)
        step_bytes = numbers["weight_bytes"] + sum(first + count for first, count in step) * numbers["kv_bytes_per_token"]
        pairs = sum(count * first + count * (count + 1) // 2 for first, count in step)  # (query, key) pairs
        flops = tokens * numbers["linear_flops_per_token"] + 4 * nq * d * layers * pairs + 2 * numbers["head_elems"] * len(step)
        by_bytes, by_flops = step_bytes / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12)
        total += max(by_bytes, by_flops)
        byte_steps += by_bytes >= by_flops
    return total, byte_steps


def generate_workload(which: str) -> int:
    """The serving-style workloads of the larger configurations, end to end through Engine.generate."""
    import torch

    import kirai_b200  # noqa: F401
    from kirai_b200 import Engine, SamplingParams
    from kirai_b200.registry import config_from_dict

    base = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", head_dim=128, vocab_size=151936,
                max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0)
    if which == "serving-4b":
        raw = dict(base, num_hidden_layers=36, hidden_size=2560, intermediate_size=9728, num_attention_heads=32,
                   num_key_value_heads=8, tie_word_embeddings=True)
        generator = torch.Generator().manual_seed(3)
        lengths = torch.randint(128, 4097, (64,), generator=generator).tolist()
        new_tokens, temperature = 256, 0.0
        # prompts go in portions of 512 tokens, eight of them to a step beside the tokens of the requests that decode
        options = dict(max_new_tokens=256, max_prefill_tokens=4096, prefill_chunk=512, max_concurrent_requests=64,
                       max_cache_tokens=64 * 4400)
        engine = Engine(config=config_from_dict(raw), random_weights_seed=3, dtype="bfloat16", page_size=16, **options)
    else:
        raw = dict(base, num_hidden_layers=64, hidden_size=5120, intermediate_size=25600, num_attention_heads=64,
                   num_key_value_heads=8, tie_word_embeddings=False)
        generator = torch.Generator().manual_seed(4)
        lengths = [8064] * 16
        new_tokens, temperature = 128, 1.0
        options = dict(max_new_tokens=128, max_prefill_tokens=2048, max_concurrent_requests=16, max_cache_tokens=16 * 8256)
        engine = Engine(config=config_from_dict(raw), random_weights_seed=4, dtype="bfloat16", page_size=16, **options)
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=generator).tolist() for n in lengths]
    params = SamplingParams(temperature=temperature, seed=7, max_new_tokens=new_tokens, ignore_eos=True)
    peaks, peak_source = load_peaks()
    engine.step_log = []
    clocks = ClockSampler()
    clocks.start()
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    clock_record = clocks.stop()
    generated = sum(len(o.token_ids) for o in outputs)
    stats = engine.stats()
    numbers = model_numbers(raw, raw["num_hidden_layers"])
    ideal, byte_steps = ideal_seconds(engine.step_log, numbers, raw, peaks)
    print(json.dumps({
        "metric": f"generated tokens/s, {which} workload through Engine.generate", "value": generated / seconds,
        "unit": "tokens/s", "n_gpus": 1, "seconds": seconds, "requests": len(prompts), "prompt_tokens": sum(lengths),
        "generated_tokens": generated, "all_tokens_per_s": (sum(lengths) + generated) / seconds, "dtype": "bf16",
        "data": "synthetic: uniform-random token ids, random weights", "steps": stats["steps"],
        "graph_steps": stats["graph_steps"], "graphs_captured": len(engine.graphs.graphs), "preemptions": stats["scheduler"]["preemptions"],
        "roofline": {"bound": "per step the greater of bytes / hbm and flops / bf16", "ideal_s": ideal, "measured_s": seconds,
                     "frac": ideal / seconds, "steps_bound_by_bytes": byte_steps, "steps_logged": len(engine.step_log), "of": peak_source,
                     "note": "the measured time holds the graph captures and the host's work between steps"},
        "clocks": clock_record,
        "config": {"model": which, "layers": raw["num_hidden_layers"], "hidden": raw["hidden_size"], "page_size": 16,
                   **{k: v for k, v in options.items()}},
    }))
    return 0


def decode_stamps(batch: int, context: int, layers: int) -> int:
    """Clock stamps of the kernels of one captured decode step: every CTA of the weight-streaming products and of the
    decode attention writes %globaltimer at a few places (csrc/gemm_tcgen05.cu::gemm_stamp, csrc/attention_mma.cu::
    decode_stamp) while a buffer is set.  Prints, per kernel of the second layer, first CTA .. last CTA in us after the
    kernel before had finished.  A measurement aid: the stamps cost a little time themselves."""
    import ctypes

    import torch

    import kirai_b200  # noqa: F401
    from kirai_b200 import Engine
    from kirai_b200.csrc import ops
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.registry import config_from_dict

    raw = dict(QWEN3_8B)
    raw["num_hidden_layers"] = layers
    engine = Engine(config=config_from_dict(raw), random_weights_seed=2, dtype="bfloat16", page_size=16, max_new_tokens=512,
                    max_prefill_tokens=2048, max_concurrent_requests=batch, max_cache_tokens=batch * (context + 256))
    runner, cache = engine.runner, engine.runner.cache
    generator = torch.Generator().manual_seed(1)
    requests = [cache.open(i) for i in range(batch)]
    for request in requests:
        prompt = torch.randint(0, raw["vocab_size"], (context - 40,), generator=generator).tolist()
        for first in range(0, len(prompt), 2048):
            runner.step([StepEntry(request, prompt[first : first + 2048], [])], check_errors=False)
    for request in requests:
        assert cache.reserve(request, 32)
    tables = [cache.block_table_array(requests, g) for g in range(len(cache.groups))]
    graph, _ = engine.graphs.get(batch, max(t.shape[1] for t in tables), [r.length + 1 for r in requests])
    graph.load_inputs([1] * batch, [r.length for r in requests], [r.slot for r in requests], tables, [0.0] * batch, [1.0] * batch, [0.0] * batch)
    products = layers * 4 + 1  # per step: q/k/v, o, gate/up, down of every layer, and the output head
    gemm = torch.zeros((2 * products + 2) * 8192, dtype=torch.int64, device="cuda:0")
    attention = torch.zeros((2 * layers + 2) * 8192, dtype=torch.int64, device="cuda:0")
    lib = ops.library()
    lib.kirai_gemm_bf16_set_stamps(ctypes.c_void_p(gemm.data_ptr()))
    lib.kirai_attention_decode_set_stamps(ctypes.c_void_p(attention.data_ptr()))
    graph.capture()  # a warm run, then the capture: the captured launches write to the second half of the buffers
    lib.kirai_gemm_bf16_set_stamps(ctypes.c_void_p(0))
    lib.kirai_attention_decode_set_stamps(ctypes.c_void_p(0))
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    ops.check_device_errors(runner.rt.device)

    def show(name, stamps, columns):
        stamps = stamps[stamps[:, 0] > 0]
        if not len(stamps):
            print(f"{name:10s} no stamps (another kernel variant ran)")
            return
        relative = (stamps - stamps[:, 1].min()) / 1e3
        cells = []
        for index, label in columns:
            seen = relative[:, index][stamps[:, index] > 0]
            if len(seen):
                cells.append(f"{label} {float(seen.min()):6.2f} .. {float(seen.max()):6.2f}")
        print(f"{name:10s} {len(stamps):4d} CTAs | " + " | ".join(cells))

    gemm_columns = [(0, "start"), (2, "first stage"), (3, "products done"), (4, "cluster met"), (6, "tiles summed"), (7, "values stored"), (5, "end")]
    attention_columns = [(0, "start"), (2, "queries in"), (3, "attended"), (4, "merged and stored")]
    per_launch = gemm[products * 8192 :].view(-1, 1024, 8).cpu().double()
    names = ["q/k/v", "o", "gate/up", "down"]
    show("attention", attention[layers * 8192 :].view(-1, 1024, 8).cpu().double()[1], attention_columns)
    for index, name in enumerate(names):
        show(name if index else "q/k/v next", per_launch[4 + (index or 4)], gemm_columns)
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--prefill-tokens", type=int, default=2048)
    parser.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a power of two)")
    parser.add_argument("--points", default="1,64", help="other decode batches to measure (comma separated, '' for none)")
    parser.add_argument("--no-check", action="store_true",
                        help="skip the check of the captured decode step against the step function before each timing")
    parser.add_argument("--workload", default="decode", choices=["decode", "serving-4b", "batch-32b", "decode-stamps"],
                        help="decode: the contract's measurement (default).  serving-4b: 64 requests with prompts of "
                             "128..4096 tokens, 512-token prefill portions mixed with decode, 256 new tokens each, greedy, "
                             "Qwen3-4B shape.  batch-32b: 16 requests of 8,064 prompt tokens, 128 new tokens at temperature 1, "
                             "Qwen3-32B shape.  Both run through Engine.generate and print their own one line.  decode-stamps: "
                             "the kernels' own clock stamps inside one captured decode step (--batch, --context, --layers; "
                             "4 layers are enough), a table instead of the JSON line.")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "michaelasper/kir-ai is a Rust workspace (no setup.py or pyproject.toml, "
                          "pip install refuses it) and its GPU path is Apple Metal; no Rust toolchain or Metal device here"}))
        return 0
    if args.gpus != 1:
        print("bench.py measures one GPU: the engine is a single-GPU engine by design (--gpus 1)")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if args.workload == "decode-stamps":
        return decode_stamps(args.batch, args.context, min(args.layers, 4) if args.layers == QWEN3_8B["num_hidden_layers"] else args.layers)
    if args.workload != "decode":
        return generate_workload(args.workload)

    import torch

    import kirai_b200
    from kirai_b200 import Engine, SamplingParams
    from kirai_b200.csrc import ops
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.registry import config_from_dict

    raw = dict(QWEN3_8B)
    raw["num_hidden_layers"] = args.layers
    config = config_from_dict(raw)
    numbers = model_numbers(raw, args.layers)
    peaks, peak_source = load_peaks()
    batches = [args.batch] + [int(b) for b in args.points.split(",") if b.strip()]
    max_batch = max(batches)
    page_size = args.page_size
    context = args.context
    torch.cuda.set_device(0)
    # what a request may generate while the others are still being filled, and while it is warmed up and timed twice
    new_token_cap = max_batch * -(-context // args.prefill_tokens) + 4 * (warmup + steps) + E2E_SETTLE_STEPS + 64
    engine = Engine(config=config, random_weights_seed=2, dtype="bfloat16", page_size=page_size,
                    max_new_tokens=new_token_cap, max_prefill_tokens=args.prefill_tokens, max_concurrent_requests=max_batch,
                    max_cache_tokens=max_batch * (context + 256))
    runner = engine.runner
    generator = torch.Generator().manual_seed(1234)

    def random_prompt(n):
        return torch.randint(0, raw["vocab_size"], (n,), generator=generator).tolist()

    clocks = ClockSampler()
    clocks.start()

    # ------------------------------------------------------------------ prefill: one prompt through the step function
    T = args.prefill_tokens
    prefill_times = []
    for it in range(warmup + 5):
        pages = runner.cache.open(("prefill", it))
        prompt = random_prompt(T)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry(pages, prompt, [T - 1])], check_errors=False)
        stop.record()
        torch.cuda.synchronize()
        if it >= warmup:
            prefill_times.append(start.elapsed_time(stop))
        runner.cache.close(pages)
    ops.check_device_errors(runner.rt.device)
    prefill_ms = statistics.median(prefill_times)
    prefill_flops = numbers["linear_flops_per_token"] * T + numbers["attention_flops"](T) + 2 * numbers["head_elems"]
    prefill = {"value": T / (prefill_ms / 1e3), "tokens": T, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), "flops": prefill_flops}

    # ------------------------------------------------------------------ decode
    checks = {}

    def check_decode(batch):
        """What is timed below, checked first: on `batch` requests filled to the context length, the captured decode
        step and the step queued behind it give the logits of the step function on the same cache state."""
        from kirai_b200.engine.graphs import captured_and_eager_logits

        cache = runner.cache
        requests = [cache.open(("check", batch, i)) for i in range(batch)]
        filled = context - 8
        for request in requests:
            prompt = random_prompt(filled)
            for first in range(0, filled, args.prefill_tokens):
                runner.step([StepEntry(request, prompt[first : first + args.prefill_tokens], [])], check_errors=False)
        result = captured_and_eager_logits(engine.graphs, requests, random_prompt(batch))
        worst, scale = 0.0, 0.0
        for captured, eager in zip(result["captured"], result["eager"]):
            if not bool(torch.isfinite(captured).all()) or not bool(torch.isfinite(eager).all()):
                raise SystemExit(f"check failed at batch {batch}: logits are not finite")
            worst = max(worst, float((captured - eager).abs().max()))
            scale = max(scale, float(eager.abs().max()))
        for request in requests:
            cache.close(request)
        ops.check_device_errors(runner.rt.device)
        if worst > 0.02 * scale:  # the bound of the bfloat16 tests
            raise SystemExit(f"check failed at batch {batch}: captured and eager logits differ by {worst} (largest logit {scale})")
        checks[batch] = {"max_abs_diff": worst, "largest_logit": scale}

    def measure_decode(batch):
        """Fills `batch` requests' caches through the engine, then times decode steps two ways."""
        if not args.no_check:
            check_decode(batch)
        # Requests that finish their prompt early decode while the others are still being filled, one
        # token per fill step; start them that much lower so that all end near the context length.
        budget = args.prefill_tokens
        fill_steps = batch * -(-context // budget)
        filled = max(16, context - (2 * (warmup + steps) + 4 + E2E_SETTLE_STEPS) - fill_steps)
        params = SamplingParams(temperature=0.0, max_new_tokens=new_token_cap, ignore_eos=True)
        requests = [engine.add_request(random_prompt(filled), params) for _ in range(batch)]
        while any(r.pending > 1 or not r.output for r in requests):
            engine.step()  # prompt portions under the token budget, then the first sampled tokens
        # (a) through the Python entry point: host tokens in and out every step.  The prompt phase just before ran
        # under the power cap; the clocks take about ten decode steps to come back (4.05 falling to 3.65 ms a step
        # at 8 requests), so a fixed number of steps settles them before the warm-up steps that the caller asked for.
        for _ in range(E2E_SETTLE_STEPS + warmup):
            engine.step()
        torch.cuda.synchronize()
        launches_before = engine.counters["graph_steps"]
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        e2e_seconds = time.perf_counter() - t0
        assert engine.counters["graph_steps"] - launches_before == steps
        engine.drain()  # the engine queues decode steps one ahead
        # (b) on the device: the captured step feeds itself; pages for the steps ahead are reserved first
        ahead = warmup + steps
        for r in requests:
            assert runner.cache.reserve(r.pages, ahead + 1)
        cache = runner.cache
        tables = [cache.block_table_array([r.pages for r in requests], g) for g in range(len(cache.groups))]
        # the captured step that the engine itself would replay for these requests (its choice of attention kernel)
        graph, fresh = engine.graphs.get(batch, max(t.shape[1] for t in tables), [r.pages.length + 1 for r in requests])
        graph.load_inputs([r.token_at(r.computed) for r in requests], [r.pages.length for r in requests],
                          [r.pages.slot for r in requests], tables, [0.0] * batch, [1.0] * batch, [0.0] * batch)
        if fresh:
            graph.capture()
        lengths_before = sum(r.pages.length for r in requests) / batch
        for _ in range(warmup):
            graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        device_ms = start.elapsed_time(stop) / steps
        ops.check_device_errors(runner.rt.device)
        mean_context = lengths_before + warmup + steps / 2.0
        step_bytes = numbers["weight_bytes"] + batch * mean_context * numbers["kv_bytes_per_token"]
        result = dict(batch=batch, device_ms=device_ms, tokens_per_s=batch / (device_ms / 1e3),
                      e2e_tokens_per_s=batch * steps / e2e_seconds, e2e_ms=e2e_seconds / steps * 1e3,
                      bytes=step_bytes, gbs=step_bytes / (device_ms / 1e3) / 1e9, context=mean_context,
                      kernels=graph.kernels_per_replay, h2d=graph.ahead_input_bytes, d2h=4 * batch + 4)
        for r in requests:
            engine.scheduler.abort(r)
        return result

    results = {b: measure_decode(b) for b in batches}

    # a second denominator: what a kernel that only reads reaches here (2 GiB, fresh for every pass: above L2)
    ceiling = None
    try:
        scratch = torch.empty(2 << 30, dtype=torch.uint8, device="cuda:0")
        scratch.fill_(1)
        for _ in range(3):
            ops.stream_read(scratch)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(5):
            ops.stream_read(scratch)
        stop.record()
        torch.cuda.synchronize()
        ops.check_device_errors(runner.rt.device)
        ceiling = 5 * scratch.numel() / (start.elapsed_time(stop) / 1e3) / 1e9
        del scratch
    except (RuntimeError, AttributeError):
        pass
    clock_record = clocks.stop()
    main_result = results[args.batch]
    roofline = {"bound": "hbm", "achieved": main_result["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": main_result["gbs"] / peaks["hbm_gbs"], "of": peak_source}
    if ceiling:
        # the copy figure counts a read and a write; a read-only stream goes faster, and the decode step only reads
        roofline["read_only_ceiling"] = ceiling
        roofline["frac_of_read_only_ceiling"] = main_result["gbs"] / ceiling
    line = {
        "metric": "decode tok/s at batch 8 (points: batch 1 and 64); prefill tok/s at 2,048 tokens (Qwen3-8B)",
        "value": main_result["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main_result["device_ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights (seed 2)",
        "config": {
            "model": "Qwen3-8B shape", "layers": args.layers, "layers_of_config": QWEN3_8B["num_hidden_layers"],
            "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
            "global_batch": args.batch, "seq_len": context, "context_at_timing": round(main_result["context"]),
            "page_size": page_size, "prefill_tokens": T, "parallelism": "single GPU",
            "l2": "weights (16 GB) and cache exceed L2; no flush needed", "peaks": peak_source,
        },
        "prefill": {k: prefill[k] for k in ("value", "tokens", "ms", "frac")},
        "roofline": roofline,
        "points": {f"decode_b{b}": results[b]["tokens_per_s"] for b in batches if b != args.batch},
        "points_detail": {f"decode_b{b}": {"ms": results[b]["device_ms"], "gbs": results[b]["gbs"],
                                           "frac": results[b]["gbs"] / peaks["hbm_gbs"],
                                           "e2e": results[b]["e2e_tokens_per_s"]} for b in batches},
        "e2e": {"value": main_result["e2e_tokens_per_s"], "unit": "tokens/s", "ms_per_step": main_result["e2e_ms"],
                "h2d_bytes_per_step": main_result["h2d"], "d2h_bytes_per_step": main_result["d2h"],
                "settle_steps": E2E_SETTLE_STEPS},
        "gpu_launches": main_result["kernels"] * steps,
        "clocks": clock_record,
        "checked": bool(checks) and all(b in checks for b in batches),
        "check": {f"decode_b{b}": checks[b] for b in checks},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
