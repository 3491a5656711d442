"""Trace replay against the plain implementation: the same requests whole, with the last
32 tokens decoded one by one, in portions of changing size, and mixed with other requests
on so few pages that they are used again; in 32-bit and in bfloat16."""
import numpy as np
import pytest

import plain_qwen3 as plain
from replay_client import Replay
from tiny_configs import TINY, random_tokens, write_tiny_model

pytestmark = pytest.mark.gpu

# 32-bit: the engine and the plain implementation differ by summation order only.
FP32_TOL = 2e-5
# bfloat16: activations are rounded to 8 significant bits between kernels; the bound is a
# fraction of the largest logit of the sequence.
BF16_REL = 0.02


def tolerance(dtype, reference):
    return FP32_TOL if dtype == "float32" else BF16_REL * float(np.abs(reference).max())


@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(f"tiny{name}"))
    raw = write_tiny_model(folder, name)
    config, weights = plain.read_model_folder(folder)
    sequences = {rid: random_tokens(n, raw["vocab_size"], 100 + k)
                 for k, (rid, n) in enumerate([("a", 75), ("b", 40), ("c", 53), ("d", 9), ("e", 61), ("f", 34)])}
    reference = {rid: plain.forward_logits(config, weights, toks).numpy() for rid, toks in sequences.items()}
    return dict(name=name, folder=folder, raw=raw, page=TINY[name][1], sequences=sequences, reference=reference)


def check(dtype, got, reference, rows, what):
    expected = reference[rows]
    assert got.shape == expected.shape, what
    diff = float(np.abs(got - expected).max())
    assert diff <= tolerance(dtype, reference), f"{what}: max abs diff {diff}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_requests(tiny, dtype, tmp_path):
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=128, page_size=tiny["page"])
    for rid in ("a", "b", "d"):
        toks = tiny["sequences"][rid]
        got = replay.step([(rid, toks, range(len(toks)))], end=[rid])
        check(dtype, got, tiny["reference"][rid], list(range(len(toks))), f"whole {rid}")
    assert replay.close() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_one_by_one(tiny, dtype, tmp_path):
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=128, page_size=tiny["page"])
    for rid in ("a", "c"):
        toks = tiny["sequences"][rid]
        head = len(toks) - 32
        got = replay.step([(rid, toks[:head], [head - 1])])
        check(dtype, got, tiny["reference"][rid], [head - 1], f"{rid} prompt")
        for i in range(head, len(toks)):
            got = replay.step([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
            check(dtype, got, tiny["reference"][rid], [i], f"{rid} decode at {i}")
    assert replay.close() == 0


@pytest.mark.parametrize("forced", ["0", "1"])
def test_decoding_with_either_attention_kernel(tiny, forced, tmp_path, monkeypatch):
    """The decode step picks between two attention kernels by the batch's lengths (equal splits per request, or all
    keys cut into equal ranges); each is forced here, for three requests of unequal length decoding side by side."""
    monkeypatch.setenv("KIRAI_DECODE_BALANCED", forced)
    replay = Replay(tiny["folder"], "bfloat16", str(tmp_path / "out"), max_tokens=256, page_size=tiny["page"])
    rids = ("a", "c", "d")
    heads = {"a": 43, "c": 21, "d": 2}
    for rid in rids:
        got = replay.step([(rid, tiny["sequences"][rid][: heads[rid]], [heads[rid] - 1])])
        check("bfloat16", got, tiny["reference"][rid], [heads[rid] - 1], f"{rid} prompt")
    for k in range(7):
        live = [rid for rid in rids if heads[rid] + k < len(tiny["sequences"][rid])]
        got = replay.step([(rid, [tiny["sequences"][rid][heads[rid] + k]], [0]) for rid in live])
        for row, rid in enumerate(live):
            check("bfloat16", got[row : row + 1], tiny["reference"][rid], [heads[rid] + k], f"{rid} decode {k} (balanced={forced})")
    assert replay.close() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_changing_size(tiny, dtype, tmp_path):
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=128, page_size=tiny["page"])
    toks = tiny["sequences"]["a"]
    sizes = [13, 2, 7, 16, 5, 3, 2, 11, 9, 2, 5]
    assert sum(sizes) == len(toks)
    start = 0
    for size in sizes:
        got = replay.step([("a", toks[start : start + size], range(size))])
        check(dtype, got, tiny["reference"]["a"], list(range(start, start + size)), f"portion at {start}+{size}")
        start += size
    replay.step([], end=["a"])
    assert replay.close() == 0


def mixed_schedule(sequences):
    """Up to four live requests; prompt portions of some beside decoded tokens of others.
    Returns a list of steps: (entries [(id, first, count)], end [ids])."""
    plan = {
        "a": [20, 30] + [1] * 25,            # 75
        "b": [17, 2] + [1] * 21,             # 40
        "c": [5, 9, 24] + [1] * 15,          # 53
        "d": [3, 2, 2, 1, 1],                # 9
        "e": [33, 16] + [1] * 12,            # 61
        "f": [2, 12, 8] + [1] * 12,          # 34
    }
    for rid, cuts in plan.items():
        assert sum(cuts) == len(sequences[rid]), rid
    arrival = ["a", "b", "c", "d", "e", "f"]
    waiting, live, progress, cursor = list(arrival), [], {r: 0 for r in arrival}, {r: 0 for r in arrival}
    steps = []
    tick = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, end = [], []
        for position, rid in enumerate(list(live)):
            if (tick + position) % 5 == 4 and len(live) > 1:
                continue  # a request may sit a step out and go on later
            count = plan[rid][cursor[rid]]
            entries.append((rid, progress[rid], count))
            progress[rid] += count
            cursor[rid] += 1
            if cursor[rid] == len(plan[rid]):
                end.append(rid)
                live.remove(rid)
        steps.append((entries, end))
        tick += 1
    return steps


def tokens_held_at_most(steps, page_size):
    """The most tokens that live requests hold at any time under a schedule, each request's count rounded up to
    whole pages: a request holds its pages from its first step until the step that names it in ``end`` is over."""
    held, most = {}, 0
    for entries, end in steps:
        for rid, first, count in entries:
            held[rid] = -(-(first + count) // page_size) * page_size
        most = max(most, sum(held.values()))
        for rid in end:
            del held[rid]
    return most


def run_mixed(replay, sequences, reference, dtype, steps):
    for entries, end in steps:
        batch = [(rid, sequences[rid][first : first + count], range(count)) for rid, first, count in entries]
        got = replay.step(batch, end=end)
        row = 0
        for rid, first, count in entries:
            check(dtype, got[row : row + count], reference[rid], list(range(first, first + count)),
                  f"mixed {rid} at {first}+{count}")
            row += count
    assert replay.close() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_requests_with_page_reuse(tiny, dtype, tmp_path):
    """Six requests, at most four live, on a pool that is exactly as large as the most that live requests ever
    hold at once (counted in whole pages), so that the pool runs full and every later request gets pages that an
    earlier one gave back.  The cache's own statistics must say so: the high-water mark is the pool size, and more
    pages were handed out than the pool has."""
    sequences, reference = tiny["sequences"], tiny["reference"]
    steps = mixed_schedule(sequences)
    page = tiny["page"]
    most = tokens_held_at_most(steps, page)
    everything = sum(-(-len(tokens) // page) * page for tokens in sequences.values())
    assert most <= 0.8 * everything  # the six requests would not fit together
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=most, page_size=page,
                    extra=("--stats", str(tmp_path / "out" / "stats.json")))
    run_mixed(replay, sequences, reference, dtype, steps)
    stats = replay.stats()
    assert stats["live_requests"] == 0
    full = [g for g in stats["groups"] if g["window"] is None]
    assert full, "every tiny configuration has a layer that keeps all keys"
    for group in full:
        assert group["pages"] == most // page and group["high_water"] == group["pages"] and group["used"] == 0
        assert group["handed_out"] == everything // page > group["pages"]
    for group in stats["groups"]:
        if group["window"] is not None:  # pages behind the window went back while their requests were still live
            assert group["handed_out"] == everything // page and group["high_water"] < group["pages"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(tiny, dtype, tmp_path):
    """The first tokens of a sequence (positions 0, 1, 2 alone), then decoding far past the
    window and over many page edges."""
    config, weights = plain.read_model_folder(tiny["folder"])
    toks = random_tokens(150, tiny["raw"]["vocab_size"], 7)
    reference = plain.forward_logits(config, weights, toks).numpy()
    replay = Replay(tiny["folder"], dtype, str(tmp_path / "out"), max_tokens=192, page_size=tiny["page"])
    for i, token in enumerate(toks):
        got = replay.step([("long", [token], [0])])
        check(dtype, got, reference, [i], f"decode at {i}")
    assert replay.close() == 0


def test_tolerance_would_show_a_window_off_by_one(tiny):
    """The bound used above must be able to show a fault at the window's edge: the plain logits with a
    window one key shorter or longer differ from the true ones by many times the bfloat16 bound."""
    if "sliding_window" not in tiny["raw"]:
        pytest.skip("configuration without a window")
    config, weights = plain.read_model_folder(tiny["folder"])
    tokens = tiny["sequences"]["a"]
    true = tiny["reference"]["a"]
    for wrong in (config["sliding_window"] - 1, config["sliding_window"] + 1):
        other = plain.forward_logits({**config, "sliding_window": wrong}, weights, tokens).numpy()
        start = config["sliding_window"] + 2  # positions where the window has begun to cut
        assert float(np.abs(other[start:] - true[start:]).max()) > 5 * tolerance("bfloat16", true)
