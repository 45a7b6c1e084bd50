"""Trace replay through bin/trace_run against the plain implementation (GPU), in 32-bit and bfloat16:
each request alone and whole; most of it in one step and the last 32 tokens one by one; in portions
of changing size down to two tokens; and mixed, up to four live requests, portions of some beside
decoded tokens of others, with so few pages that they are used again."""
import numpy as np
import pytest
import torch

from replay_helpers import Trace, plain_logits, read_logits, run_trace

pytestmark = pytest.mark.gpu

# abs tolerance on logits: 32-bit path; bfloat16 path as a fraction of the largest plain logit
TOL_F32 = 1e-4
TOL_BF16_REL = 0.02


def sequences_for(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    P, V = cfg["n_positions"], cfg["vocab_size"]
    lens = {"whole": P, "tail": P - 3, "cut": P - 1, "m0": 70, "m1": 45, "m2": P, "m3": 33, "m4": 64, "m5": 2}
    return {k: torch.randint(0, V, (n,), generator=g).tolist() for k, n in lens.items()}


def build_trace(seqs):
    t = Trace()
    # (1) alone and whole
    t.step([("whole", seqs["whole"], range(len(seqs["whole"])))], end=["whole"])
    # (2) most in one step, the last 32 one by one
    s = seqs["tail"]
    n0 = len(s) - 32
    t.step([("tail", s[:n0], range(n0))])
    for i in range(n0, len(s)):
        t.step([("tail", s[i:i + 1], [0])], end=["tail"] if i == len(s) - 1 else [])
    # (3) portions of changing size, down to two tokens, crossing page edges mid-portion
    s = seqs["cut"]
    sizes, pos = [16, 7, 2, 5, 2, 9, 3, 2, 17, 2, 4, 31, 2], 0
    k = 0
    while pos < len(s):
        n = min(sizes[k % len(sizes)], len(s) - pos)
        if len(s) - pos - n == 1:       # never leave a single token: portions have at least two
            n += 1
        t.step([("cut", s[pos:pos + n], range(n))], end=["cut"] if pos + n == len(s) else [])
        pos += n
        k += 1
    # (4) mixed: up to four live; pages are given back and used again
    plan = {"m0": [30, 2, 1, 1, 1, 1, 1, 1, 32], "m1": [2, 20, 1, 1, 1, 1, 19], "m2": [50, 11, 2, 1, 1, 1, 1, 1],
            "m3": [33], "m4": [3, 1, 1, 1, 1, 57], "m5": [2]}
    plan["m2"].append(len(seqs["m2"]) - sum(plan["m2"]))
    for k_, v in plan.items():
        assert sum(v) == len(seqs[k_]), (k_, sum(v), len(seqs[k_]))
    waiting = ["m0", "m1", "m2", "m3", "m4", "m5"]
    live, at, fed = [], {}, {}
    rnd = np.random.RandomState(0)
    while waiting or live:
        while waiting and len(live) < 4:
            r = waiting.pop(0)
            live.append(r); at[r] = 0; fed[r] = 0
        entries, ended = [], []
        for r in list(live):
            if len(live) > 1 and rnd.rand() < 0.25:
                continue                                    # a request may sit a step out
            n = plan[r][at[r]]
            toks = seqs[r][fed[r]:fed[r] + n]
            want = list(range(n)) if n <= 8 else sorted({0, 1, n // 2, n - 2, n - 1})
            entries.append((r, toks, want))
            fed[r] += n; at[r] += 1
            if at[r] == len(plan[r]):
                ended.append(r); live.remove(r)
        if entries:
            t.step(entries, end=ended)
    return t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_modes(tiny, dtype, tmp_path):
    folder, cfg, page = tiny
    seqs = sequences_for(cfg, seed=cfg["n_layer"])
    trace = build_trace(seqs)
    bound = trace.live_tokens_bound()
    assert bound < sum(-(-len(s) // 64) * 64 for s in seqs.values())      # the pool is smaller than all requests together
    out = str(tmp_path / "out")
    run_trace(trace, folder, dtype, out, max_tokens=bound, page_size=page)
    got = read_logits(trace, out, cfg["vocab_size"])
    _, ref = plain_logits(folder, seqs)
    worst, worst_at = 0.0, None
    for (rid, pos), rows in got.items():
        scale = np.abs(ref[rid]).max()
        tol = TOL_F32 if dtype == "float32" else TOL_BF16_REL * scale
        for row in rows:
            d = np.abs(row.astype(np.float64) - ref[rid][pos]).max()
            if d > worst:
                worst, worst_at = d, (rid, pos)
            assert d < tol, f"request {rid} position {pos}: max abs diff {d:.3e} (tolerance {tol:.3e})"
    for rid in ("whole", "tail", "cut"):                                    # every position was asked for
        assert all((rid, p) in got for p in range(len(seqs[rid])))
    print(f"{dtype}: worst max-abs diff {worst:.3e} at {worst_at}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_freed_pages_filled_with_nan(tiny, dtype, tmp_path):
    """The same trace in the debugging mode that overwrites every page a request gives back with NaN before the
    next step: pages change hands many times (the pool is smaller than the requests together), and a kernel that
    read a page its request no longer holds, or a token slot beyond its request's length in a page that was used
    before, would put NaN into some logit.  Every logit is finite and equal to the plain implementation's."""
    import re
    folder, cfg, page = tiny
    seqs = sequences_for(cfg, seed=cfg["n_layer"])
    trace = build_trace(seqs)
    out = str(tmp_path / "out")
    r = run_trace(trace, folder, dtype, out, max_tokens=trace.live_tokens_bound(), page_size=page,
                  env={"CBIS_POISON_FREED_PAGES": "1"})
    m = re.search(r"(\d+) freed pages were filled with NaN", r.stderr)
    assert m and int(m.group(1)) >= 20, r.stderr[-500:]
    got = read_logits(trace, out, cfg["vocab_size"])
    _, ref = plain_logits(folder, seqs)
    for (rid, pos), rows in got.items():
        scale = np.abs(ref[rid]).max()
        tol = TOL_F32 if dtype == "float32" else TOL_BF16_REL * scale
        for row in rows:
            assert np.isfinite(row).all(), f"request {rid} position {pos}: a logit is not finite"
            assert np.abs(row.astype(np.float64) - ref[rid][pos]).max() < tol, (rid, pos)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuts_agree_with_each_other(tiny, dtype, tmp_path):
    """The same request whole, token by token and in portions, within one run: logits at a position
    do not depend on the cut beyond rounding."""
    folder, cfg, page = tiny
    g = torch.Generator().manual_seed(9)
    s = torch.randint(0, cfg["vocab_size"], (cfg["n_positions"] - 5,), generator=g).tolist()
    t = Trace()
    t.step([("a", s, range(len(s)))], end=["a"])
    for i in range(len(s)):
        t.step([("b", s[i:i + 1], [0])], end=["b"] if i == len(s) - 1 else [])
    pos, k, sizes = 0, 0, [5, 2, 13, 2, 3, 8]
    while pos < len(s):
        n = min(sizes[k % len(sizes)], len(s) - pos)
        t.step([("c", s[pos:pos + n], range(n))], end=["c"] if pos + n == len(s) else [])
        pos += n; k += 1
    out = str(tmp_path / "out")
    run_trace(t, folder, dtype, out, page_size=page)
    got = read_logits(t, out, cfg["vocab_size"])
    scale = max(np.abs(r[0]).max() for r in got.values())
    tol = 1e-5 if dtype == "float32" else 4e-3 * scale
    for p in range(len(s)):
        a, b, c = got[("a", p)][0], got[("b", p)][0], got[("c", p)][0]
        assert np.abs(a - b).max() < tol and np.abs(a - c).max() < tol, p


def test_trace_run_refuses_bad_steps(folder_a, tmp_path):
    t = Trace()
    t.step([("a", [1, 2, 3], [0])])
    t.steps[0]["entries"][0]["tokens"][1] = 999                             # outside the vocabulary
    import subprocess, sys, json
    from replay_helpers import TRACE_RUN
    r = subprocess.run([sys.executable, TRACE_RUN, "--model", folder_a, "--dtype", "float32", "--out",
                        str(tmp_path / "o"), "--max-tokens", "64"], input=json.dumps(t.steps[0]) + "\n",
                       capture_output=True, text=True, timeout=300)
    assert r.returncode != 0 and "outside the vocabulary" in r.stderr
    t2 = Trace()
    t2.step([("a", list(range(70)), [0])])                                  # 70 tokens into a pool of 64
    r = subprocess.run([sys.executable, TRACE_RUN, "--model", folder_a, "--dtype", "float32", "--out",
                        str(tmp_path / "o"), "--max-tokens", "64"], input=json.dumps(t2.steps[0]) + "\n",
                       capture_output=True, text=True, timeout=300)
    assert r.returncode != 0 and "no pages left" in r.stderr
