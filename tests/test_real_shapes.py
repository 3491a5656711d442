"""The engine at the layer sizes of a real model (hidden 4096, 32 query heads over 8 kv heads of
128, intermediate 12288; two layers and a small vocabulary so that the plain implementation stays
fast): logits under several ways of cutting the work, in 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, head_dim=128, vocab_size=1000,
            max_position_embeddings=8192, rms_norm_eps=1e-6, rope_theta=1000000.0)
CONFIGS = {
    # hidden, heads and intermediate of the 8-billion-parameter shape (untied), of the 4-billion one (tied; query
    # width 4096 over a hidden size of 2560) and of the 32-billion one (64 query heads in groups of 8)
    "8b": dict(BASE, hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8, tie_word_embeddings=False),
    "4b": dict(BASE, hidden_size=2560, intermediate_size=9728, num_attention_heads=32, num_key_value_heads=8, tie_word_embeddings=True),
    "32b": dict(BASE, hidden_size=5120, intermediate_size=25600, num_attention_heads=64, num_key_value_heads=8, tie_word_embeddings=False),
}


@pytest.fixture(scope="module", params=["8b", "4b", "32b"])
def model(request, tmp_path_factory):
    CONFIG = CONFIGS[request.param]
    import kirai_b200  # noqa: F401
    from kirai_b200.registry import config_from_dict
    from kirai_b200.weights import write_random_model

    folder = str(tmp_path_factory.mktemp("real"))
    write_random_model(folder, config_from_dict(CONFIG), seed=2, std=0.02, norm_jitter=0.1)
    config, weights = plain.read_model_folder(folder)
    tokens = torch.randint(0, CONFIG["vocab_size"], (150,), generator=torch.Generator().manual_seed(3)).tolist()
    return dict(name=request.param, folder=folder, tokens=tokens, config=config, weights=weights,
                reference=plain.forward_logits(config, weights, tokens).numpy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuts_at_real_layer_sizes(model, dtype):
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner

    runner = ModelRunner.from_folder(model["folder"], dtype=dtype, page_size=16, max_tokens=512, num_slots=4)
    tokens, reference = model["tokens"], model["reference"]
    bound = 1e-4 if dtype == "float32" else 0.02 * float(np.abs(reference).max())

    def run(request_id, cuts):
        request = runner.cache.open(request_id)
        rows, start = [], 0
        for count in cuts:
            rows.append(runner.step([StepEntry(request, tokens[start : start + count], range(count))]).cpu().numpy())
            start += count
        runner.cache.close(request)
        return np.concatenate(rows)

    whole = run("whole", [150])
    assert float(np.abs(whole - reference).max()) <= bound
    portions = run("portions", [70, 17, 2, 33, 1, 1, 1, 25])  # crosses the 64-token GEMM variants and page edges
    assert float(np.abs(portions - reference).max()) <= bound
    # two requests side by side: one decodes while the other brings a prompt portion
    a, b = runner.cache.open("a"), runner.cache.open("b")
    first = runner.step([StepEntry(a, tokens[:100], [99])]).cpu().numpy()
    mixed = runner.step([StepEntry(a, tokens[100:101], [0]), StepEntry(b, tokens[:40], range(40))]).cpu().numpy()
    assert float(np.abs(first[0] - reference[99]).max()) <= bound
    assert float(np.abs(mixed[0] - reference[100]).max()) <= bound
    assert float(np.abs(mixed[1:] - reference[:40]).max()) <= bound
    decode = runner.step([StepEntry(a, tokens[101:102], [0]), StepEntry(b, tokens[40:41], [0])]).cpu().numpy()  # decode-only batch
    assert float(np.abs(decode[0] - reference[101]).max()) <= bound
    assert float(np.abs(decode[1] - reference[40]).max()) <= bound


LONG = 4300  # tokens of the long sequence: contexts beyond 4,096, so that a decode step cuts the keys into several splits


@pytest.fixture(scope="module")
def long_reference(model):
    """One long sequence and its plain logits at the places the tests below look at.  Requests of different lengths
    are prefixes of it: logits at a position do not depend on what follows, so one plain pass serves them all."""
    vocab = model["config"]["vocab_size"]
    tokens = torch.randint(0, vocab, (LONG,), generator=torch.Generator().manual_seed(11)).tolist()
    with torch.no_grad():
        logits = plain.forward_logits(model["config"], model["weights"], tokens).numpy()
    return dict(tokens=tokens, logits=logits)


# lengths of the live requests' caches before the checked step: long and equal (several splits over the context),
# unequal (the kernel that cuts all keys into equal ranges), and more than 16 rows (norms as kernels of their own)
BATCHES = {
    "one": [4200],
    "eight_equal": [4100] * 8,
    "eight_unequal": [4200, 37, 4111, 1500, 64, 2300, 900, 4160],
    "twenty": [4200, 37, 4111, 1500, 64, 2300, 900, 4160, 15, 16, 17, 3000, 4096, 4095, 1, 2048, 333, 4250, 129, 640],
    # a hundred short requests: the products take tiles of 128 tokens through the weight-streaming kernel, in the decode
    # step and in the prompts of 65 to 128 tokens that fill the caches
    "hundred": [(i * 37) % 290 + 1 for i in range(100)],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps_at_long_contexts(model, long_reference, dtype):
    """What a benchmark of decode steps times, checked: the captured decode step, and the step queued behind it that
    takes its tokens from the first on the device, against the step function on the same cache state (logits, both
    steps) and against the plain implementation (first step), at real layer widths, contexts beyond 4,096 tokens,
    batches of 1, 8, 20 and 100, equal and unequal lengths."""
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.graphs import DecodeGraphs, captured_and_eager_logits
    from kirai_b200.engine.runner import ModelRunner

    tokens, reference = long_reference["tokens"], long_reference["logits"]
    scale = float(np.abs(reference).max())
    bound = 1e-4 if dtype == "float32" else 0.02 * scale
    most = max(sum(lengths) for lengths in BATCHES.values()) + 3400  # and the two requests of the mixed step
    runner = ModelRunner.from_folder(model["folder"], dtype=dtype, page_size=16, max_tokens=most + 64 * 104, num_slots=104)
    graphs = DecodeGraphs(runner)
    kernels_seen = set()
    for name, lengths in BATCHES.items():
        requests = [runner.cache.open((name, i)) for i in range(len(lengths))]
        for request, n in zip(requests, lengths):  # fill the caches: prompts in portions of at most 2,048 tokens
            for start in range(0, n, 2048):
                runner.step([StepEntry(request, tokens[start : min(n, start + 2048)], [])])
        result = captured_and_eager_logits(graphs, requests, [tokens[n] for n in lengths])
        kernels_seen.add(result["balanced"])
        captured, eager = result["captured"], result["eager"]
        for step in range(2):
            difference = float((captured[step] - eager[step]).abs().max())
            assert difference <= bound, f"{name}: captured step {step} differs from the step function by {difference}"
        expected = reference[lengths]  # the token at position n is the last of a sequence of n + 1 tokens
        for which, logits in (("captured", captured[0]), ("step function", eager[0])):
            difference = float(np.abs(logits.cpu().numpy() - expected).max())
            assert difference <= bound, f"{name}: {which} differs from the plain implementation by {difference}"
        # the sampled tokens that the queued step took as its input are the greatest logits of the first step
        assert result["sampled"] == captured[0].argmax(dim=-1).tolist()
        if name == "eight_unequal":
            # a mixed step: the same requests decode on (their caches hold the sequence's tokens up to n, then the two
            # sampled ones, so only what a fresh prompt gives can be compared with the plain logits) beside a prompt
            # portion of another request, given FIRST: inside the batch the single tokens stand first and take the
            # decode kernels, and the logits come back in the order asked for
            fresh = runner.cache.open((name, "fresh"))
            again = runner.cache.open((name, "again"))
            runner.step([StepEntry(again, tokens[:3000], [])])
            mixed = runner.step([StepEntry(fresh, tokens[:300], [299, 0]), StepEntry(again, [tokens[3000]], [0])]
                                + [StepEntry(r, [5], []) for r in requests[:3]]).cpu().numpy()
            assert mixed.shape[0] == 3
            for row, place in enumerate([299, 0, 3000]):
                difference = float(np.abs(mixed[row] - reference[place]).max())
                assert difference <= bound, f"mixed step, place {place}: {difference}"
            for request in (fresh, again):
                runner.cache.close(request)
            lengths = [n + 1 if i < 3 else n for i, n in enumerate(lengths)]
        for request, n in zip(requests, lengths):
            assert request.length == n + 2
            runner.cache.close(request)
    if dtype == "bfloat16":
        assert kernels_seen == {False, True}  # both decode attention kernels were captured and checked
    assert all(g["used"] == 0 for g in runner.cache.stats()["groups"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_schedule_on_a_full_pool_at_real_layer_sizes(model, dtype):
    """The mixed schedule of the replay tests (up to four live requests, portions of some beside decoded tokens of
    others) at real layer widths, on a pool exactly as large as the most that is ever held, so that it runs full and
    pages are used again."""
    if model["name"] != "8b":
        pytest.skip("once, at the widths of the 8-billion-parameter shape")
    from test_replay import mixed_schedule, tokens_held_at_most

    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner

    vocab = model["config"]["vocab_size"]
    sizes = [("a", 75), ("b", 40), ("c", 53), ("d", 9), ("e", 61), ("f", 34)]
    sequences = {rid: torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(200 + k)).tolist()
                 for k, (rid, n) in enumerate(sizes)}
    reference = {rid: plain.forward_logits(model["config"], model["weights"], toks).numpy() for rid, toks in sequences.items()}
    steps = mixed_schedule(sequences)
    page = 16
    most = tokens_held_at_most(steps, page)
    runner = ModelRunner.from_folder(model["folder"], dtype=dtype, page_size=page, max_tokens=most, num_slots=4)
    live = {}
    for entries, end in steps:
        batch = []
        for rid, first, count in entries:
            if rid not in live:
                live[rid] = runner.cache.open(rid)
            batch.append(StepEntry(live[rid], sequences[rid][first : first + count], range(count)))
        logits = runner.step(batch).cpu().numpy()
        row = 0
        for rid, first, count in entries:
            expected = reference[rid][first : first + count]
            bound = 1e-4 if dtype == "float32" else 0.02 * float(np.abs(reference[rid]).max())
            difference = float(np.abs(logits[row : row + count] - expected).max())
            assert difference <= bound, f"{rid} at {first}+{count}: {difference}"
            row += count
        for rid in end:
            runner.cache.close(live.pop(rid))
    group = runner.cache.stats()["groups"][0]
    handed_out = sum(-(-n // page) for _, n in sizes)
    assert group["pages"] == most // page == group["high_water"] and group["used"] == 0
    assert group["handed_out"] == handed_out > group["pages"]


def test_steps_with_products_launched_as_one_kernel(model, monkeypatch):
    """The model's steps with ``ops.chain_products`` set (a layer's weight-streaming products as phases of one
    persistent kernel): single decoded tokens of three requests side by side, norms folded into the products, against
    the plain implementation."""
    if model["name"] == "32b":
        pytest.skip("two shapes are enough here")
    from kirai_b200.csrc import ops
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.engine.runner import ModelRunner

    monkeypatch.setattr(ops, "chain_products", True)
    runner = ModelRunner.from_folder(model["folder"], dtype="bfloat16", page_size=16, max_tokens=1024, num_slots=4)
    tokens, reference = model["tokens"], model["reference"]
    bound = 0.02 * float(np.abs(reference).max())
    heads = [100, 37, 64]
    requests = [runner.cache.open(i) for i in range(3)]
    for request, head in zip(requests, heads):
        runner.step([StepEntry(request, tokens[:head], [])])
    before = ops.launch_count
    for k in range(6):
        logits = runner.step([StepEntry(r, [tokens[h + k]], [0]) for r, h in zip(requests, heads)]).cpu().numpy()
        for row, head in enumerate(heads):
            assert float(np.abs(logits[row] - reference[head + k]).max()) <= bound, (k, row)
    # per step and layer one launch for the four products instead of four (2 layers: 6 launches fewer a step)
    chained = (ops.launch_count - before) / 6
    monkeypatch.setattr(ops, "chain_products", False)
    before = ops.launch_count
    runner.step([StepEntry(r, [tokens[h + 6]], [0]) for r, h in zip(requests, heads)])
    assert ops.launch_count - before > chained + 3
