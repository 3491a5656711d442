"""Drives ``bin/trace_run`` as a user would: a child process, steps on its standard
input, ``done <step>`` lines back, logits read from the files it writes."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Replay:
    def __init__(self, model_dir: str, dtype: str, out_dir: str, max_tokens: int, page_size: int, extra=()):
        self.out_dir = out_dir
        os.makedirs(out_dir, exist_ok=True)
        command = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                   "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size), *extra]
        self.process = subprocess.Popen(command, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.step_index = 0

    def step(self, entries, end=()):
        """entries: list of (id, tokens, want).  Returns the logits [wanted, vocab] or None."""
        record = {"step": self.step_index,
                  "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries], "end": list(end)}
        self.process.stdin.write(json.dumps(record) + "\n")
        self.process.stdin.flush()
        line = self.process.stdout.readline()
        if line.strip() != f"done {self.step_index}":
            raise RuntimeError(f"trace_run answered {line!r} to step {self.step_index} (exit code {self.process.poll()})")
        wanted = sum(len(w) for _, _, w in entries)
        result = None
        if wanted:
            flat = np.fromfile(os.path.join(self.out_dir, f"{self.step_index}.f32"), dtype="<f4")
            result = flat.reshape(wanted, -1)
        self.step_index += 1
        return result

    def close(self) -> int:
        self.process.stdin.close()
        code = self.process.wait(timeout=120)
        self.process.stdout.close()
        return code

    def stats(self) -> dict:
        """The cache's statistics as trace_run wrote them at exit (needs ``extra=("--stats", <out_dir>/stats.json)``)."""
        with open(os.path.join(self.out_dir, "stats.json")) as handle:
            return json.load(handle)
