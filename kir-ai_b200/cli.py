"""Command line: ``kirai generate --snapshot <dir> ...`` prints generated token ids.

Flags are parsed in the reference's manner, a hand-rolled ``--flag value`` scan
with the help text as the schema (crates/llm-engine/src/main.rs:55-76,423-475), and keep
its names and defaults where it has them: ``--snapshot``, ``--max-new-tokens``
(256), ``--max-prefill-tokens`` (2048), ``--max-concurrent-requests`` (4),
``--log-level``.  The reference has no ``generate`` subcommand (it serves HTTP);
the request options take the names of its API fields: ``--temperature``,
``--top-p``, ``--max-tokens``.  Prompts are token ids.  Text (``--prompt``, and a
``text`` field in the output) is offered where the model folder holds a
tokenizer.json and the ``tokenizers`` package is installed; the engine itself
knows token ids only.
"""
from __future__ import annotations

import json
import os
import sys
from typing import List, Optional

HELP = """\
Usage: kirai generate [OPTIONS]

Options:
  --snapshot <path>                 Model folder (config.json + model.safetensors)
  --random-weights <seed>           Use random weights made from --snapshot's config.json (or --config) and this seed
  --config <path>                   config.json to use with --random-weights when there is no snapshot folder
  --write-snapshot <path>           With --random-weights: write the model folder there and exit
  --prompt-ids <ids>                Comma-separated token ids; repeat the flag for several prompts
  --prompt-file <path>              JSON file with a list of prompts (lists of token ids)
  --prompt <text>                   A prompt as text; needs tokenizer.json in the model folder and the `tokenizers`
                                    package.  With a tokenizer present the output lines carry the generated text too
  --max-tokens <n>                  Tokens to generate per request [default: --max-new-tokens]
  --temperature <t>                 0 = greedy [default: 1.0, range 0..2]
  --top-p <p>                       Nucleus mass [default: 1.0, range (0,1]]
  --seed <n>                        Seed of the sampler's draws [default: from the system]
  --eos-token-id <id>               Stop when this token is sampled
  --dtype <bfloat16|float32>        [default: bfloat16]
  --max-new-tokens <n>              Maximum generated tokens a request may ask for [default: 256]
  --max-prefill-tokens <n>          Token budget of a step (prompt portions are cut to it) [default: 2048]
  --max-concurrent-requests <n>     Requests running at a time [default: 4]
  --prefill-chunk <n>               Longest portion of one prompt in a step [default: the step's budget]
  --page-size <n>                   Tokens per cache page [default: 16]
  --max-cache-tokens <n>            Size of the cache pool in tokens [default: from the limits above]
  --num-pages <n>                   Size of the cache pool in pages (instead of --max-cache-tokens)
  --log-level <level>               trace|debug|info|warn|error|off [default: info]; trace also marks every layer
                                    call as an NVTX range
  -h, --help                        Print help
"""


def flag_values(args: List[str], flag: str) -> List[str]:
    values = []
    for index, arg in enumerate(args):
        if arg == flag:
            if index + 1 >= len(args):
                raise SystemExit(f"{flag} requires a value")
            values.append(args[index + 1])
        elif arg.startswith(flag + "="):
            values.append(arg[len(flag) + 1 :])
    return values


def flag_value(args: List[str], flag: str) -> Optional[str]:
    values = flag_values(args, flag)
    return values[-1] if values else None


def has_flag(args: List[str], flag: str) -> bool:
    return flag in args


def _int(args, flag, default):
    value = flag_value(args, flag)
    if value is None:
        return default
    try:
        return int(value)
    except ValueError:
        raise SystemExit(f"{flag} expects an integer, got {value!r}")


def _float(args, flag, default):
    value = flag_value(args, flag)
    if value is None:
        return default
    try:
        return float(value)
    except ValueError:
        raise SystemExit(f"{flag} expects a number, got {value!r}")


def _load_tokenizer(snapshot: Optional[str]):
    """The tokenizer of a model folder, if it has a tokenizer.json and the `tokenizers` package is installed; else None.
    Text is a convenience of the command line only: the engine takes and gives token ids."""
    if snapshot is None:
        return None
    path = os.path.join(snapshot, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


def generate_command(args: List[str]) -> int:
    if has_flag(args, "--help") or has_flag(args, "-h"):
        print(HELP)
        return 0
    level = (flag_value(args, "--log-level") or "info").lower()
    if level not in ("trace", "debug", "info", "warn", "error", "off"):
        raise SystemExit("--log-level must be one of trace|debug|info|warn|error|off")

    def log(message):
        if level in ("trace", "debug", "info"):
            print(f"[kirai] {message}", file=sys.stderr, flush=True)

    from .registry import config_from_dict, load_config
    from .sampling.params import SamplingParams

    snapshot = flag_value(args, "--snapshot")
    random_seed = flag_value(args, "--random-weights")
    config = None
    if random_seed is not None:
        config_path = flag_value(args, "--config")
        if config_path:
            with open(config_path) as handle:
                config = config_from_dict(json.load(handle))
        elif snapshot:
            config = load_config(snapshot)
        else:
            raise SystemExit("--random-weights needs --config or --snapshot for the configuration")
        target = flag_value(args, "--write-snapshot")
        if target:
            from .weights import write_random_model

            write_random_model(target, config, int(random_seed))
            log(f"wrote {target}")
            return 0
    elif snapshot is None:
        raise SystemExit("kirai generate needs --snapshot <path> (or --random-weights <seed> with --config)")

    tokenizer = _load_tokenizer(snapshot)
    prompts = []
    for text in flag_values(args, "--prompt-ids"):
        prompts.append([int(t) for t in text.replace(" ", "").split(",") if t])
    for text in flag_values(args, "--prompt"):
        if tokenizer is None:
            raise SystemExit("--prompt needs tokenizer.json in the model folder and the `tokenizers` package; give --prompt-ids")
        prompts.append(list(tokenizer.encode(text).ids))
    prompt_file = flag_value(args, "--prompt-file")
    if prompt_file:
        with open(prompt_file) as handle:
            prompts.extend(json.load(handle))
    if not prompts:
        raise SystemExit("give --prompt-ids 1,2,3 or --prompt-file prompts.json")

    from .engine.engine import Engine

    seed = flag_value(args, "--seed")
    eos = flag_value(args, "--eos-token-id")
    max_tokens = flag_value(args, "--max-tokens")
    params = SamplingParams(
        temperature=_float(args, "--temperature", 1.0), top_p=_float(args, "--top-p", 1.0),
        seed=int(seed) if seed is not None else None,
        max_new_tokens=int(max_tokens) if max_tokens is not None else None,
        eos_token_id=int(eos) if eos is not None else None,
    )
    cache_tokens = _int(args, "--max-cache-tokens", None)
    num_pages = _int(args, "--num-pages", None)
    if num_pages is not None:
        if cache_tokens is not None:
            raise SystemExit("give --max-cache-tokens or --num-pages, not both")
        cache_tokens = num_pages * _int(args, "--page-size", 16)
    engine = Engine(
        snapshot if random_seed is None else None, config=config,
        random_weights_seed=int(random_seed) if random_seed is not None else None,
        dtype=flag_value(args, "--dtype") or "bfloat16",
        max_new_tokens=_int(args, "--max-new-tokens", 256), max_prefill_tokens=_int(args, "--max-prefill-tokens", 2048),
        max_concurrent_requests=_int(args, "--max-concurrent-requests", 4), page_size=_int(args, "--page-size", 16),
        max_cache_tokens=cache_tokens, prefill_chunk=_int(args, "--prefill-chunk", None),
    )
    engine.runner.model.nvtx = level == "trace"
    log(f"loaded {type(engine.runner.config).__name__}; generating for {len(prompts)} prompt(s)")
    for output in engine.generate(prompts, params):
        line = {"token_ids": output.token_ids, "finish_reason": output.finish_reason,
                "prompt_tokens": output.prompt_tokens, "completion_tokens": output.completion_tokens}
        if tokenizer is not None:
            line["text"] = tokenizer.decode(output.token_ids)
        print(json.dumps(line))
    log(json.dumps(engine.stats()))
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    command = argv[0] if argv else "--help"
    if command in ("--help", "-h", "help"):
        print(HELP)
        return 0
    if command == "generate":
        return generate_command(argv[1:])
    raise SystemExit(f"unknown command {command!r}; known: generate")


if __name__ == "__main__":
    sys.exit(main())
