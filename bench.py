#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Cerebras-GPT-1.3B shapes (random weights).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

One "step" is one decode step of the whole batch.  The default run has the layer sizes of
the 1.3B configuration, bfloat16, a batch of 8 requests with 1,024-token prompts decoded
towards the context length 2,048.  It prints ONE JSON line:

* ``value``: decoded tokens per second, timed on the device with CUDA events around K replays
  of the captured decode step (model, argmax and the move to the next position all on the
  device);
* ``e2e``: the same through the Python entry point (``Engine.step``: scheduler, packed inputs
  copied from pinned host memory, sampled tokens read back every step);
* ``prefill``: one 2,048-token prompt in one step, tokens per second and the fraction of the
  bf16 matrix peak its flops reach;
* ``roofline``: bytes a decode step has to read (every weight once and the cache of the live
  requests) over its time, against the measured copy bandwidth;
* ``points``: decode at batch 1 and 64.

Peaks come from MEASURED_PEAKS.json beside this file when it exists.  This engine runs on one
GPU: with --gpus N > 1 it says so and exits with status 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Cerebras-GPT-1.3B layer sizes (GPT2LMHeadModel)
CONFIG_1_3B = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=24, n_embd=2048, n_head=16,
                   n_inner=8192, vocab_size=50257, n_positions=2048, activation_function="gelu",
                   layer_norm_epsilon=1e-5, tie_word_embeddings=True)
# Cerebras-GPT-6.7B and GPT-2 XL layer sizes (further configurations of the benchmark set)
CONFIG_6_7B = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=32, n_embd=4096, n_head=32,
                   n_inner=16384, vocab_size=50257, n_positions=2048, activation_function="gelu",
                   layer_norm_epsilon=1e-5, tie_word_embeddings=True)
CONFIG_XL = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=48, n_embd=1600, n_head=25,
                 n_inner=6400, vocab_size=50257, n_positions=1024, activation_function="gelu_new",
                 layer_norm_epsilon=1e-5, tie_word_embeddings=True)
# the reference's one fixed model (include/config.hpp:5-21) for its own workload (--config batching)
CONFIG_REFERENCE = dict(architectures=["TinyGPT"], n_layer=4, n_embd=256, n_head=8, n_inner=1024, vocab_size=1000,
                        n_positions=2048, activation_function="gelu", layer_norm_epsilon=1e-5, tie_word_embeddings=False)
REFERENCE_BUILD = os.path.join(ROOT, "baseline", "_ref")     # the unmodified reference, built with its own CMakeLists
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="1.3b", choices=["1.3b", "6.7b", "xl", "batching"],
                    help="1.3b: the default measurement; 6.7b: batch-64 decode at context 2,048; "
                         "xl: 64 mixed requests through the scheduler (prompts 32-768, 256 outputs each); "
                         "batching: the reference's own workload at the reference's own sizes (both --impl arms)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1/64, prefill and e2e")
    ap.add_argument("--prefill-only", action="store_true", help="time only the 2,048-token prefill (for profilers)")
    ap.add_argument("--prefill-portion", type=int, default=None, help="with --prefill-only: the prompt in steps of this many tokens")
    args = ap.parse_args()

    if args.config == "batching":
        return reference_workload(args)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference cannot run this configuration: its model sizes are compile-time constants "
                          "(include/config.hpp:5-21: 4 layers, width 256, vocabulary 1000) and it computes in fp32 only; "
                          "built unmodified with its own CMakeLists it runs its own workload here: "
                          "bench.py --config batching --impl reference"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on ONE GPU; --gpus {args.gpus} is not supported (single-GPU tier)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    from cbis_b200.kernels import ops

    torch.cuda.set_device(0)
    if args.config == "xl":
        return mixed_workload(args, cb, torch)
    if args.config == "6.7b":
        args.skip_points = True
        args.batch = args.batch or 64
        args.steps = min(args.steps, 64)
        args.prompt_len = args.prompt_len or (CONFIG_6_7B["n_positions"] - args.warmup - args.steps - 24)
    args.batch = args.batch or 8
    args.prompt_len = args.prompt_len or 1024
    cfgd = dict(CONFIG_6_7B if args.config == "6.7b" else CONFIG_1_3B)
    n_layer_config = cfgd["n_layer"]
    if args.layers:
        cfgd["n_layer"] = args.layers
    P = cfgd["n_positions"]
    K, W, B, PL = args.steps, args.warmup, args.batch, args.prompt_len
    K = max(1, min(K, P - PL - W - 20))
    pk = peaks()
    max_b = B if args.skip_points else max(B, 64)
    if args.prefill_only:
        max_b = 1
    eng = cb.Engine.from_random(cfgd, seed=1234, dtype="bfloat16", page_size=args.page_size,
                                max_tokens=max_b * P, max_num_seqs=max_b, max_batched_tokens=2048,
                                prefill_chunk=2048)
    model, runner, mgr = eng.model, eng.runner, eng.pool.manager
    V = cfgd["vocab_size"]
    gen = torch.Generator().manual_seed(0)

    def prompts(n, length):
        return torch.randint(0, V, (n, length), generator=gen).tolist()

    def prefill_slots(ps):
        """Prefills prompts through the step function (two per step); returns their slots."""
        slots = [eng.open_request(i) for i in range(len(ps))]
        per = max(1, 2048 // len(ps[0]))
        for i in range(0, len(ps), per):
            eng.forward_step([StepEntry(slots[j], 0, ps[j], []) for j in range(i, min(i + per, len(ps)))])
        return slots

    def decode_device(batch, steps, warm, prompt_len=None):
        """tokens/s of `steps` captured decode steps after `warm` untimed ones; also ms/step, launches/step."""
        PL = prompt_len or args.prompt_len
        ps = prompts(batch, PL)
        slots = prefill_slots(ps)
        for s in slots:
            assert mgr.append(s, warm + steps + 2)
        ops.reset_launch_count()
        loop = runner.decode_loop([StepEntry(s, PL, [1], [0]) for s in slots])
        per_step = ops.launch_count() // 2          # the loop ran its step twice: warm-up and capture
        loop.run(warm)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loop.run(steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        for s in slots:
            eng.close_request(s)
        del loop
        return batch * steps / (ms / 1e3), ms / steps, per_step

    def prefill_once(T, portion=None):
        """Median milliseconds of one T-token prompt run as ONE step, or in steps of ``portion`` tokens
        (3 warm-ups, 5 timed)."""
        toks = prompts(1, T)[0]
        portion = portion or T
        times = []
        for it in range(3 + 5):
            slot = eng.open_request(1000 + it)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for at in range(0, T, portion):
                part = toks[at:at + portion]
                eng.forward_step([StepEntry(slot, at, part, [len(part) - 1] if at + portion >= T else [])])
            e1.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(e0.elapsed_time(e1))
            eng.close_request(slot)
        return statistics.median(times)

    if args.prefill_only:
        ms = prefill_once(2048, args.prefill_portion)
        print(json.dumps({"prefill_ms": round(ms, 3), "tokens": 2048, "portion": args.prefill_portion or 2048,
                          "n_layer": cfgd["n_layer"]}))
        return 0

    # ---- main measurement: decode at the default batch, clocks sampled meanwhile -------------
    sampler = ClockSampler()
    sampler.start()
    value, ms_per_step, launches_per_step = decode_device(B, K, W)
    clocks = sampler.stop()
    ctx_mean = PL + 1 + W + K / 2.0
    step_bytes = model.weight_bytes() + B * ctx_mean * eng.pool.bytes_per_token()
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    result = {
        "metric": f"decode tokens/s (Cerebras-GPT-{args.config.upper()} shapes, batch {B}, context {PL}->{P})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "impl": "b200",
        "config": {"model": f"Cerebras-GPT-{args.config.upper()} shapes (GPT2LMHeadModel)", "n_layer": cfgd["n_layer"],
                   "n_layer_config": n_layer_config, "n_embd": cfgd["n_embd"], "n_head": cfgd["n_head"],
                   "n_inner": cfgd["n_inner"], "vocab_size": V, "n_positions": P, "activation": "gelu",
                   "tied_head": True, "global_batch": B, "prompt_len": PL, "seq_len": P,
                   "page_size": args.page_size, "parallelism": "single GPU",
                   "l2": "inputs larger than L2: every step reads all weights and the live cache"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"],
                     "bytes_per_step": int(step_bytes)},
        "clocks": clocks,
        "gpu_launches": int(launches_per_step * K),
    }

    if not args.skip_points:
        # ---- prefill of 2,048 tokens in one step ------------------------------------------------
        T = 2048
        ms = prefill_once(T)
        d, F, L = cfgd["n_embd"], cfgd["n_inner"], cfgd["n_layer"]
        flops = L * (2 * T * (3 * d * d + d * d + 2 * d * F) + 2 * T * T * d) + 2 * d * V
        result["prefill"] = {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3),
                             "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                             "flops": int(flops), "peak_tflops": pk["bf16_tflops"], "of": pk["source"]}
        ms512 = prefill_once(T, 512)     # the same prompt in four steps of 512 tokens, as a scheduler would cut it
        result["prefill"]["in_portions_of_512"] = {"value": round(T / (ms512 / 1e3), 1), "ms": round(ms512, 3)}
        # ---- decode at batch 1 and 64 -----------------------------------------------------------
        pts = {}
        for b in (1, 64):
            v, _, _ = decode_device(b, min(K, 256), W)
            pts[f"decode_b{b}"] = round(v, 1)
        # the default batch at the two ends of the context range: 32 steps from context 1,024 and 32 steps up to the last position
        v, _, _ = decode_device(B, 32, 3, prompt_len=PL)
        pts[f"decode_b{B}_ctx{PL}"] = round(v, 1)
        v, _, _ = decode_device(B, 32, 3, prompt_len=P - 40)
        pts[f"decode_b{B}_ctx{P}"] = round(v, 1)
        result["points"] = pts
        # ---- end to end through the Python entry point -------------------------------------------
        ps = prompts(B, PL)
        n_new = W + K + 16                      # no request ends inside the timed region
        for p in ps:
            eng.add_request(p, cb.SamplingParams(max_new_tokens=n_new))
        while not all_decoding(eng, B):
            eng.step()
        for _ in range(W):
            eng.step()
        torch.cuda.synchronize()
        tokens_before = eng.tokens_run
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        steps_e2e, tokens_e2e = K, eng.tokens_run - tokens_before
        while eng.has_unfinished():
            eng.step()
        result["e2e"] = {"value": round(tokens_e2e / wall, 1), "unit": "tokens/s", "steps": steps_e2e,
                         "ms_per_step": round(wall * 1e3 / steps_e2e, 4),
                         "h2d_bytes_per_step": int(runner.bytes_per_step_h2d()), "d2h_bytes_per_step": 4 * B,
                         "device_ms_per_step": round(e0.elapsed_time(e1) / steps_e2e, 4)}
    print(json.dumps(result))
    return 0


def reference_workload(args) -> int:
    """The reference's own workload (src/bench_batching.cpp:26-33: 240 requests, Poisson arrivals 6 ms apart, prompts of
    4-16 and outputs of 8-32 tokens, 16 slots) at the reference's own model sizes.  --impl reference runs the unmodified
    reference's bench_batching (built with its own CMakeLists into baseline/_ref; its sm_89 PTX is compiled for the GPU
    at load) on its committed weights; the default arm runs this engine (bin/bench_batching) on random weights of the
    same sizes.  The throughput of both is set by the arrival rate; the latencies are what the engines decide."""
    import re
    import tempfile
    line = {"metric": "the reference's continuous-batching workload: tokens/s (prompt + output) and request latency",
            "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "data": "synthetic (uniform random token ids)",
            "config": {"model": "TinyGPT, the reference's sizes", "n_layer": 4, "n_embd": 256, "n_head": 8, "n_inner": 1024,
                       "vocab_size": 1000, "requests": 240, "mean_interarrival_ms": 6.0, "max_live": 16}}
    if args.impl == "reference":
        exe, weights = os.path.join(REFERENCE_BUILD, "build", "bench_batching"), os.path.join(REFERENCE_BUILD, "weights.bin")
        if not (os.path.isfile(exe) and os.path.isfile(weights)):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no build of the reference "
                              "(cmake -S <reference> -B baseline/_ref/build && cmake --build baseline/_ref/build; "
                              "its python/weights.bin copied to baseline/_ref/weights.bin)"}))
            return 0
        r = subprocess.run([exe, weights], capture_output=True, text=True, timeout=600)
        part = r.stdout.split("== static")[0]
        m = re.search(r"wall clock\s*:\s*([\d.]+) ms.*?token throughput\s*:\s*([\d.]+) tok/s.*?p50/p95/p99\s*:\s*([\d.]+) / "
                      r"([\d.]+) / ([\d.]+) ms", part, re.S)
        if r.returncode != 0 or not m:
            print(json.dumps({"impl": "reference", "unavailable": f"the reference's bench_batching ended with {r.returncode}"}))
            return 0
        line.update(impl="reference", dtype="fp32", value=float(m.group(2)), wall_ms=float(m.group(1)),
                    latency_ms={"p50": float(m.group(3)), "p95": float(m.group(4)), "p99": float(m.group(5))})
        print(json.dumps(line))
        return 0
    with tempfile.TemporaryDirectory() as d:
        cfg = os.path.join(d, "config.json")
        with open(cfg, "w") as f:
            json.dump(CONFIG_REFERENCE, f)
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bench_batching"), "--random", cfg, "--json"],
                           capture_output=True, text=True, timeout=900)
    out = [l for l in r.stdout.splitlines() if l.startswith("{")]
    if r.returncode != 0 or not out:
        print(r.stdout[-2000:], r.stderr[-2000:], file=sys.stderr)
        return 1
    mine = json.loads(out[-1])
    line.update(impl="b200", dtype="bf16", value=mine["tokens_per_s"], wall_ms=mine["wall_ms"], latency_ms=mine["latency_ms"])
    print(json.dumps(line))
    return 0


def mixed_workload(args, cb, torch) -> int:
    """GPT-2 XL layer sizes: 64 requests, prompt lengths uniform in 32..768, 256 outputs each, all submitted at
    t = 0 and run by the scheduler (token budget 2,048, prompt portions of 512)."""
    import random
    cfgd = dict(CONFIG_XL)
    if args.layers:
        cfgd["n_layer"] = args.layers
    n_req, n_out = 64, 256
    eng = cb.Engine.from_random(cfgd, seed=1234, dtype="bfloat16", page_size=args.page_size,
                                max_tokens=n_req * cfgd["n_positions"], max_num_seqs=n_req, max_batched_tokens=2048,
                                prefill_chunk=512)
    rng = random.Random(0)
    prompts = [[rng.randrange(cfgd["vocab_size"]) for _ in range(rng.randint(32, 768))] for _ in range(n_req)]
    eng.generate(prompts[:8], cb.SamplingParams(max_new_tokens=4))       # warm-up: kernels
    eng.warm_up()                                                        # the decode graphs of every batch bucket
    torch.cuda.synchronize()
    steps0 = eng.steps
    step_ms, step_tokens = [], []
    ids = [eng.add_request(p, cb.SamplingParams(max_new_tokens=n_out)) for p in prompts]
    done = {}
    t0 = time.perf_counter()
    last = t0
    while eng.has_unfinished():          # what generate() does, with the wall time of every step noted
        for o in eng.step():
            done[o.request_id] = o.tokens
        now = time.perf_counter()        # the step's sampled tokens have been read back: the device has finished it
        step_ms.append((now - last) * 1e3)
        step_tokens.append(eng.last_step_tokens)
        last = now
    wall = last - t0
    outs = [done[i] for i in ids]
    n_prompt, n_gen = sum(map(len, prompts)), sum(map(len, outs))
    edges = [0.5, 1, 2, 3, 4, 6, 8, 12, 16, 24, 32]
    hist, lo = {}, 0.0
    for e in edges + [float("inf")]:
        hist[f"<={e:g}ms" if e != float("inf") else f">{edges[-1]:g}ms"] = sum(1 for t in step_ms if lo < t <= e)
        lo = e
    decode_only = [t for t, n in zip(step_ms, step_tokens) if n <= n_req]
    print(json.dumps({
        "metric": "mixed continuous-batching workload, tokens/s (GPT-2 XL shapes, 64 requests, prompts 32-768, 256 outputs)",
        "value": round((n_prompt + n_gen) / wall, 1), "unit": "tokens/s", "n_gpus": 1, "impl": "b200", "dtype": "bf16",
        "decode_tokens_per_s": round(n_gen / wall, 1), "wall_s": round(wall, 3), "steps": eng.steps - steps0,
        "prompt_tokens": n_prompt, "output_tokens": n_gen, "preemptions": eng.scheduler.preemptions(),
        "graph_replays": eng.runner.graph_replays, "step_shapes_captured": eng.runner.shape_captures,
        "step_ms": {"median": round(statistics.median(step_ms), 3), "p95": round(sorted(step_ms)[int(0.95 * len(step_ms))], 3),
                    "max": round(max(step_ms), 3),
                    "decode_only_median": round(statistics.median(decode_only), 3) if decode_only else None},
        "step_ms_histogram": hist,
        "higher_is_better": True, "data": "synthetic (random weights, uniform random token ids)",
        "config": {"model": "GPT-2 XL shapes (GPT2LMHeadModel)", "n_layer": cfgd["n_layer"], "n_layer_config": 48,
                   "n_embd": 1600, "n_head": 25, "n_inner": 6400, "vocab_size": 50257, "n_positions": 1024,
                   "requests": n_req, "max_batched_tokens": 2048, "prefill_chunk": 512, "page_size": args.page_size}}))
    return 0


def all_decoding(eng, batch):
    """True once every request of the batch has had its prompt run (each step then feeds one token each)."""
    return eng.scheduler.num_running() == batch and eng.last_step_tokens == batch


if __name__ == "__main__":
    sys.exit(main())
