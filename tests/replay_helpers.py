"""Builds traces for bin/trace_run and compares what it writes with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

import plain_gpt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Trace:
    """Collects steps; remembers for every wanted row which (request, position) it is."""

    def __init__(self):
        self.steps = []
        self.fed = {}           # request -> tokens fed so far
        self.wanted = []        # per step: list of (request, position)

    def step(self, entries, end=()):
        """entries: list of (request, tokens, want-indices)."""
        rec, rows = [], []
        for rid, toks, want in entries:
            base = len(self.fed.setdefault(rid, []))
            self.fed[rid] += list(toks)
            rec.append({"id": rid, "tokens": list(map(int, toks)), "want": list(map(int, want))})
            rows += [(rid, base + w) for w in want]
        self.steps.append({"step": len(self.steps), "entries": rec, "end": list(end)})
        self.wanted.append(rows)

    def live_tokens_bound(self):
        """Most tokens held at a time, each request rounded up to 64 (what --max-tokens means)."""
        held, worst = {}, 0
        for st in self.steps:
            for e in st["entries"]:
                held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
            worst = max(worst, sum(-(-n // 64) * 64 for n in held.values()))
            for rid in st["end"]:
                held.pop(rid, None)
        return worst


def run_trace(trace, folder, dtype, out_dir, max_tokens=None, page_size=None, timeout=600, env=None):
    cmd = [sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens or trace.live_tokens_bound())]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout,
                       env=dict(os.environ, **env) if env else None)
    assert r.returncode == 0, f"trace_run failed:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(trace.steps))], r.stdout[-2000:]
    return r


def read_logits(trace, out_dir, vocab):
    """{(request, position): [logits rows written for it]} from the <step>.f32 files."""
    got = {}
    for i, rows in enumerate(trace.wanted):
        path = os.path.join(out_dir, f"{i}.f32")
        if not rows:
            assert not os.path.exists(path)
            continue
        arr = np.fromfile(path, dtype="<f4")
        assert arr.size == len(rows) * vocab, (i, arr.size, len(rows), vocab)
        arr = arr.reshape(len(rows), vocab)
        for (rid, pos), row in zip(rows, arr):
            got.setdefault((rid, pos), []).append(row)
    return got


def plain_logits(folder, sequences, weights_dtype=torch.float64):
    """{name: float64 logits [T, V]} of whole sequences by the plain implementation."""
    cfg, w = plain_gpt.read_model_folder(folder, weights_dtype)
    with torch.no_grad():
        return cfg, {name: plain_gpt.forward(cfg, w, toks).double().numpy() for name, toks in sequences.items()}
