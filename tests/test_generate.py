"""Generation through the Python entry point and the command line against the plain implementation."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import TINY, random_tokens, write_tiny_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request, tmp_path_factory):
    folder = str(tmp_path_factory.mktemp(f"gen{request.param}"))
    raw = write_tiny_model(folder, request.param)
    config, weights = plain.read_model_folder(folder)
    return dict(name=request.param, folder=folder, raw=raw, config=config, weights=weights, page=TINY[request.param][1])


def plain_sampled(config, weights, prompt, count, temperature, top_p, seed):
    from kirai_b200.sampling import rng

    tokens, out = list(prompt), []
    for k in range(count):
        logits = plain.forward_logits(config, weights, tokens)[-1]
        token = plain.argmax_first(logits) if temperature == 0.0 else plain.sample_top_p(logits, temperature, top_p, rng.draw(seed, k))
        out.append(token)
        tokens.append(token)
    return out


def margin_ok(config, weights, prompt, generated, temperature):
    """True when greedy choices are not near-ties (a near-tie may flip with rounding)."""
    if temperature != 0.0:
        return True
    logits = plain.forward_logits(config, weights, list(prompt) + list(generated))
    top2 = torch.topk(logits[len(prompt) - 1 : -1], 2, dim=-1).values
    return bool(((top2[:, 0] - top2[:, 1]) > 1e-4).all())


def test_greedy_generation_float32(tiny):
    from kirai_b200 import Engine, SamplingParams

    engine = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_prefill_tokens=16,
                    max_concurrent_requests=3, max_new_tokens=16, max_cache_tokens=256)
    prompts = [random_tokens(n, tiny["raw"]["vocab_size"], 50 + n) for n in (5, 11, 17, 3, 24)]
    outputs = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
    for prompt, output in zip(prompts, outputs):
        expected = plain.greedy_generate(tiny["config"], tiny["weights"], prompt, 8)
        assert margin_ok(tiny["config"], tiny["weights"], prompt, expected, 0.0)
        assert output.token_ids == expected and output.finish_reason == "length"
        assert (output.prompt_tokens, output.completion_tokens) == (len(prompt), 8)
    stats = engine.stats()
    assert stats["cache"]["live_requests"] == 0 and all(g["used"] == 0 for g in stats["cache"]["groups"])


def test_temperature_sampling_with_seed_float32(tiny):
    from kirai_b200 import Engine, SamplingParams

    engine = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_prefill_tokens=16,
                    max_concurrent_requests=4, max_new_tokens=16, max_cache_tokens=256)
    prompts = [random_tokens(n, tiny["raw"]["vocab_size"], 80 + n) for n in (3, 24, 40, 9)]
    params = [SamplingParams(temperature=0.7, top_p=1.0, seed=11, max_new_tokens=12),
              SamplingParams(temperature=0.7, top_p=0.9, seed=12, max_new_tokens=12),
              SamplingParams(temperature=1.3, top_p=0.5, seed=13, max_new_tokens=12),
              SamplingParams(temperature=0.0, max_new_tokens=12)]
    outputs = engine.generate(prompts, params)
    again = engine.generate(prompts, params)
    for prompt, p, output, second in zip(prompts, params, outputs, again):
        expected = plain_sampled(tiny["config"], tiny["weights"], prompt, 12, p.temperature, p.top_p, p.seed or 0)
        assert output.token_ids == expected
        assert second.token_ids == output.token_ids  # the same seed gives the same tokens


def test_greedy_generation_bfloat16_follows_plain(tiny):
    """bfloat16 rounds activations, so a near-tie may resolve differently from the plain implementation, and from
    there on the two generate different texts.  The whole generation is followed all the same: at every step the
    plain logits are computed for the prompt and the tokens that the ENGINE has generated so far, and the engine's
    next token must be the plain maximum or within the bfloat16 bound of it.  Most steps must agree exactly."""
    from kirai_b200 import Engine, SamplingParams

    engine = Engine(tiny["folder"], dtype="bfloat16", page_size=tiny["page"], max_prefill_tokens=16,
                    max_concurrent_requests=2, max_new_tokens=16, max_cache_tokens=256)
    prompts = [random_tokens(n, tiny["raw"]["vocab_size"], 60 + n) for n in (6, 19, 33)]
    outputs = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    agreed = steps = 0
    for prompt, output in zip(prompts, outputs):
        assert len(output.token_ids) == 12
        tokens = list(prompt)
        for token in output.token_ids:
            logits = plain.forward_logits(tiny["config"], tiny["weights"], tokens)[-1]
            best = plain.argmax_first(logits)
            assert float(logits[best] - logits[token]) <= 0.02 * float(logits.abs().max()), (len(tokens), token, best)
            agreed += token == best
            steps += 1
            tokens.append(token)  # the engine's token, whichever it was: the next step is judged on the engine's own text
    assert steps == 36 and agreed >= 30


def test_eviction_and_recompute_give_the_same_tokens(tiny):
    from kirai_b200 import Engine, SamplingParams

    params = SamplingParams(temperature=0.8, top_p=0.95, seed=5, max_new_tokens=14)
    prompts = [random_tokens(17, tiny["raw"]["vocab_size"], 1), random_tokens(18, tiny["raw"]["vocab_size"], 2)]
    roomy = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=16, max_cache_tokens=256)
    expected = [o.token_ids for o in roomy.generate(prompts, params)]
    tight = Engine(tiny["folder"], dtype="float32", page_size=tiny["page"], max_new_tokens=16, max_cache_tokens=48)
    outputs = tight.generate(prompts, params)
    assert [o.token_ids for o in outputs] == expected
    assert tight.stats()["scheduler"]["preemptions"] >= 1 and sum(o.preemptions for o in outputs) >= 1


def test_steps_queued_ahead_give_the_same_tokens_and_drop_what_follows_a_stop(tiny):
    """Decode steps are queued one ahead of the host's knowledge of their input tokens.  With and without that, the
    same requests (different lengths, seeded sampling, one stop token that ends a request early while its next
    step is already queued) must produce the same tokens, and nothing stays reserved."""
    from kirai_b200 import Engine, SamplingParams

    vocab = tiny["raw"]["vocab_size"]
    prompts = [random_tokens(n, vocab, 30 + n) for n in (7, 12, 4)]
    base = dict(dtype="float32", page_size=tiny["page"], max_prefill_tokens=16, max_concurrent_requests=3,
                max_new_tokens=32, max_cache_tokens=512)
    plain_params = [SamplingParams(temperature=0.9, top_p=0.95, seed=21 + i, max_new_tokens=24, ignore_eos=True) for i in range(3)]
    reference = Engine(tiny["folder"], overlap_steps=False, **base).generate(prompts, plain_params)
    # a stop token for the second request: the 6th token that it generates without one
    stop = reference[1].token_ids[5]
    params = list(plain_params)
    params[1] = SamplingParams(temperature=0.9, top_p=0.95, seed=22, max_new_tokens=24, eos_token_id=stop)
    expected = Engine(tiny["folder"], overlap_steps=False, **base).generate(prompts, params)
    assert expected[1].finish_reason == "stop" and len(expected[1].token_ids) <= 6
    engine = Engine(tiny["folder"], overlap_steps=True, **base)
    outputs = engine.generate(prompts, params)
    for got, want in zip(outputs, expected):
        assert got.token_ids == want.token_ids and got.finish_reason == want.finish_reason
    stats = engine.stats()
    assert stats["graph_steps"] > 0
    assert stats["cache"]["live_requests"] == 0 and all(g["used"] == 0 for g in stats["cache"]["groups"])
    # step by step: every call returns the requests that one step finished, and a drained engine holds nothing
    stepping = Engine(tiny["folder"], overlap_steps=True, **base)
    requests = [stepping.add_request(p, q) for p, q in zip(prompts, params)]
    finished = []
    while stepping.scheduler.has_work():
        finished += stepping.step()
    finished += stepping.drain()
    assert sorted(id(r) for r in finished) == sorted(id(r) for r in requests)
    assert [r.output for r in requests] == [o.token_ids for o in expected]


def test_abort_between_steps_leaves_the_others_untouched(tiny):
    """A request is ended while it decodes (a step for it may already be queued) and another while it still waits:
    the rest generate what they generate without them, and nothing stays reserved."""
    from kirai_b200 import Engine, SamplingParams

    vocab = tiny["raw"]["vocab_size"]
    prompts = [random_tokens(n, vocab, 50 + n) for n in (9, 5, 13, 6)]
    base = dict(dtype="float32", page_size=tiny["page"], max_prefill_tokens=16, max_concurrent_requests=3,
                max_new_tokens=32, max_cache_tokens=512)
    params = [SamplingParams(temperature=0.7, top_p=0.9, seed=40 + i, max_new_tokens=20, ignore_eos=True) for i in range(4)]
    expected = Engine(tiny["folder"], **base).generate(prompts, params)
    engine = Engine(tiny["folder"], **base)
    requests = [engine.add_request(p, q) for p, q in zip(prompts, params)]
    finished = []
    while len(requests[1].output) < 7:  # the second request is in the middle of its decoding
        finished += engine.step()
    finished += engine.abort(requests[1])
    finished += engine.abort(requests[3])  # the fourth still waits for a free place among the running
    assert requests[1].finish_reason == "aborted" and 7 <= len(requests[1].output) < 20
    assert requests[3].finish_reason == "aborted" and requests[3].output == []
    assert requests[1].output == expected[1].token_ids[: len(requests[1].output)]
    while engine.scheduler.has_work():
        finished += engine.step()
    finished += engine.drain()
    assert requests[0].output == expected[0].token_ids and requests[2].output == expected[2].token_ids
    assert sorted(id(r) for r in finished) == sorted(id(requests[i]) for i in (0, 2))
    stats = engine.stats()
    assert stats["cache"]["live_requests"] == 0 and all(g["used"] == 0 for g in stats["cache"]["groups"])
    assert engine.abort(requests[0]) == [] and requests[0].finish_reason == "length"  # ending a finished request changes nothing


def test_command_line(tiny):
    command = [sys.executable, os.path.join(ROOT, "bin", "kirai"), "generate", "--snapshot", tiny["folder"],
               "--prompt-ids", "5,17,3,44", "--prompt-ids", "9,8,7", "--max-tokens", "6", "--temperature", "0",
               "--dtype", "float32", "--page-size", str(tiny["page"]), "--max-new-tokens", "16", "--log-level", "trace",
               "--prefill-chunk", "3", "--num-pages", "24"]
    result = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    stats = json.loads(result.stderr.strip().splitlines()[-1].split("[kirai] ", 1)[1])  # the last log line: the engine's counters
    assert stats["cache"]["groups"][0]["pages"] == 24 + 1  # the pool asked for, and the page of the padding rows
    # the prompt of four tokens went in two portions (3 + 1): one step more than its six tokens alone would take
    assert stats["steps"] == 7 and stats["kernel_launches"]["kirai_sample_rows"] >= 1  # replays of captured steps call no entry point
    lines = [json.loads(line) for line in result.stdout.strip().splitlines()]
    assert len(lines) == 2
    for prompt, line in zip(([5, 17, 3, 44], [9, 8, 7]), lines):
        assert line["token_ids"] == plain.greedy_generate(tiny["config"], tiny["weights"], prompt, 6)
        assert line["finish_reason"] == "length" and line["prompt_tokens"] == len(prompt)


def test_command_line_with_text(tiny, tmp_path):
    """With a tokenizer.json in the model folder, --prompt takes text and the output lines carry the generated text."""
    tokenizers = pytest.importorskip("tokenizers")
    import shutil

    folder = str(tmp_path / "with_tokenizer")
    shutil.copytree(tiny["folder"], folder)
    vocab = {f"w{i}": i for i in range(tiny["raw"]["vocab_size"])}
    tokenizer = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="w0"))
    tokenizer.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tokenizer.decoder = tokenizers.decoders.Fuse()
    tokenizer.save(os.path.join(folder, "tokenizer.json"))
    base = [sys.executable, os.path.join(ROOT, "bin", "kirai"), "generate", "--snapshot", folder, "--max-tokens", "5",
            "--temperature", "0", "--dtype", "float32", "--page-size", str(tiny["page"]), "--max-new-tokens", "16", "--log-level", "off"]
    by_text = subprocess.run(base + ["--prompt", "w5 w17 w3 w44"], capture_output=True, text=True, timeout=600)
    by_ids = subprocess.run(base + ["--prompt-ids", "5,17,3,44"], capture_output=True, text=True, timeout=600)
    assert by_text.returncode == 0, by_text.stderr
    assert by_ids.returncode == 0, by_ids.stderr
    text_line, ids_line = json.loads(by_text.stdout.strip().splitlines()[-1]), json.loads(by_ids.stdout.strip().splitlines()[-1])
    assert text_line["token_ids"] == ids_line["token_ids"] == plain.greedy_generate(tiny["config"], tiny["weights"], [5, 17, 3, 44], 5)
    assert text_line["prompt_tokens"] == 4
    assert text_line["text"] == "".join(f"w{t}" for t in text_line["token_ids"]) == ids_line["text"]
    # without a tokenizer in the folder, text is refused with a message that says what is missing
    refused = subprocess.run([a if a != folder else tiny["folder"] for a in base] + ["--prompt", "w5"], capture_output=True, text=True, timeout=600)
    assert refused.returncode != 0 and "tokenizer.json" in refused.stderr
