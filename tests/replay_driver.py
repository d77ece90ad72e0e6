"""Drives bin/trace_run as a user does: one JSON step on standard input, wait for ``done <step>``,
read ``<out>/<step>.f32``."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Replay:
    def __init__(self, model_dir, dtype, out_dir, max_tokens, vocab, extra_args=()):
        self.out_dir, self.vocab, self.n = str(out_dir), vocab, 0
        self.pages = {}          # with --show-pages: step -> {request id: [page ids per cache group]}
        os.makedirs(self.out_dir, exist_ok=True)
        self.proc = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
             "--out", self.out_dir, "--max-tokens", str(max_tokens), *extra_args],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)

    def step(self, entries, end=()):
        """entries: [(id, tokens, want)].  Returns the logits [wanted, vocab] or None."""
        step = self.n
        self.n += 1
        msg = {"step": step, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(msg) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.startswith(f"pages {step} "):
            self.pages[step] = json.loads(line.split(" ", 2)[2])
            line = self.proc.stdout.readline()
        if line.strip() != f"done {step}":
            rest = self.proc.stdout.read()
            raise RuntimeError(f"trace_run said {line!r} {rest!r} (exit {self.proc.poll()})")
        if not any(len(w) for _, _, w in entries):
            return None
        a = np.fromfile(os.path.join(self.out_dir, f"{step}.f32"), dtype="<f4")
        return a.reshape(-1, self.vocab)

    def close(self):
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        assert code == 0, f"trace_run exited with {code}"

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if exc[0] is None:
            self.close()
        else:
            self.proc.kill()
