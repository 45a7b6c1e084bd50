"""Generation through the Python entry point and the command line against the plain implementation (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_gpt
import tiny_configs as tc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def prompts_for(cfg, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]


def check_against_plain(folder, prompts, outputs, temperature, seed, first_id, exact):
    """exact: token for token.  Otherwise (bfloat16) every chosen token must be, by the plain
    model's own scores for the engine's sequence, within a small margin of the best one."""
    cfg, w = plain_gpt.read_model_folder(folder, torch.float64)
    for i, (p, out) in enumerate(zip(prompts, outputs)):
        if exact:
            assert out == plain_gpt.generate(cfg, w, p, len(out), temperature, seed, first_id + i), f"request {i}"
            continue
        with torch.no_grad():
            logits = plain_gpt.forward(cfg, w, p + out[:-1]).numpy()
        for j, t in enumerate(out):
            scores = plain_gpt.perturbed_scores(logits[len(p) - 1 + j], temperature, seed, first_id + i, j)
            margin = 0.03 * np.abs(logits).max() / max(temperature, 1.0) if temperature else 0.03 * np.abs(logits).max()
            assert scores[t] >= scores.max() - margin, f"request {i} output {j}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_tiny_a(folder_a, dtype):
    import cbis_b200 as cb
    prompts = prompts_for(tc.TINY_A, [5, 17, 33], 1)
    eng = cb.Engine(folder_a, dtype=dtype, page_size=tc.PAGE_A, num_pages=16, max_num_seqs=3, max_batched_tokens=64)
    outs = eng.generate(prompts, cb.SamplingParams(max_new_tokens=16))
    assert [len(o) for o in outs] == [16, 16, 16]
    check_against_plain(folder_a, prompts, outs, 0.0, 0, 0, exact=dtype == "float32")
    assert eng.pool.manager.free_pages(0) == 16 and eng.pool.manager.check() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_generation_tiny_b_in_portions(folder_b, dtype):
    import cbis_b200 as cb
    prompts = prompts_for(tc.TINY_B, [1, 7, 23, 40, 61], 2)
    eng = cb.Engine(folder_b, dtype=dtype, page_size=tc.PAGE_B, num_pages=64, max_num_seqs=5, max_batched_tokens=40,
                    prefill_chunk=16)
    outs = eng.generate(prompts, cb.SamplingParams(max_new_tokens=16, temperature=0.8, seed=4321))
    assert [len(o) for o in outs] == [16] * 5
    check_against_plain(folder_b, prompts, outs, 0.8, 4321, 0, exact=dtype == "float32")
    # the draws do not depend on the batch: one request alone gives the same tokens
    solo = cb.Engine(folder_b, dtype=dtype, page_size=tc.PAGE_B, num_pages=64, max_num_seqs=1, max_batched_tokens=96)
    rid = solo.add_request(prompts[3], cb.SamplingParams(max_new_tokens=16, temperature=0.8, seed=4321), request_id=3)
    res = {}
    while solo.has_unfinished():
        for o in solo.step():
            res[o.request_id] = o.tokens
    if dtype == "float32":
        assert res[rid] == outs[3]


def test_long_decoding_to_the_last_position(folder_a):
    import cbis_b200 as cb
    P = tc.TINY_A["n_positions"]
    eng = cb.Engine(folder_a, dtype="float32", page_size=16, num_pages=8, max_num_seqs=1, max_batched_tokens=16)
    prompt = [7, 3, 200]
    out = eng.generate([prompt], cb.SamplingParams(max_new_tokens=500))[0]
    assert len(out) == P - len(prompt) + 1                      # every position was fed; the last output has none left
    cfg, w = plain_gpt.read_model_folder(folder_a, torch.float64)
    assert out == plain_gpt.generate(cfg, w, prompt, len(out))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_the_context_classes_of_the_decode_graphs(tmp_path, dtype):
    """Decode-only steps replay a graph captured for a class of context lengths (256, 1024, ... up to the model's
    positions), for which the attention kernels size their split of the keys.  Requests decode across the bounds 256
    and 1024 side by side and a short one goes on alone: every token is the plain implementation's, and all three
    classes were captured."""
    import cbis_b200 as cb
    cfgd = dict(tc.TINY_B, n_positions=1300)
    folder = str(tmp_path / "long_b")
    cb.write_model_folder(folder, cb.config_from_dict(cfgd), seed=5, scheme=cb.InitScheme(*tc.INIT_B))
    eng = cb.Engine(folder, dtype=dtype, page_size=8, max_tokens=2700, max_num_seqs=3, max_batched_tokens=512)
    prompts = prompts_for(cfgd, [250, 1015, 10], seed=9)
    outs = eng.generate(prompts, [cb.SamplingParams(max_new_tokens=n) for n in (16, 16, 40)])   # the short one ends alone
    check_against_plain(folder, prompts, outs, 0.0, 0, 0, exact=dtype == "float32")
    if eng.runner.use_graphs:
        assert {limit for _, limit in eng.runner._graphs} == {256, 1024, 1300}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_warm_up_captures_every_decode_graph_and_changes_no_token(tmp_path, dtype):
    """``Engine.warm_up`` captures the decode step of every batch-size bucket and context class with requests of its
    own and gives everything back; generation afterwards captures nothing more and gives the plain
    implementation's tokens (the same requests as in the test above, whose graphs were captured on the way)."""
    import cbis_b200 as cb
    cfgd = dict(tc.TINY_B, n_positions=1300)
    folder = str(tmp_path / "long_b")
    cb.write_model_folder(folder, cb.config_from_dict(cfgd), seed=5, scheme=cb.InitScheme(*tc.INIT_B))
    eng = cb.Engine(folder, dtype=dtype, page_size=8, max_tokens=2700, max_num_seqs=3, max_batched_tokens=512)
    free = eng.pool.manager.free_pages(0)
    n = eng.warm_up(small_steps=False)
    assert n == len(eng.runner._graphs) == 3 * 3         # buckets 1, 2, 3 (the most requests) x classes 256, 1024, 1300
    assert eng.warm_up(small_steps=False) == 0
    assert eng.pool.manager.free_pages(0) == free and eng.pool.manager.check() == "" and eng.scheduler.idle()
    replays = eng.runner.graph_replays
    prompts = prompts_for(cfgd, [250, 1015, 10], seed=9)
    outs = eng.generate(prompts, [cb.SamplingParams(max_new_tokens=n) for n in (16, 16, 40)])
    check_against_plain(folder, prompts, outs, 0.0, 0, 0, exact=dtype == "float32")
    assert len(eng.runner._graphs) == 9 and eng.runner.graph_replays > replays
    assert eng.pool.manager.free_pages(0) == free and eng.pool.manager.check() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_steps_launched_ahead_give_the_tokens_of_steps_in_turn(folder_b, dtype, temperature):
    """While a decode step runs, the next is planned and launched with the sampled tokens fed on the device
    (CBIS_STEP_AHEAD, on by default).  The same requests with it and without: the same tokens, also when a request
    stops on an end-of-sequence token while its row of the next step is on its way (the rows of the step after no
    longer line up with the sampled tokens), when requests end by length at different steps, and when pages run out
    and a request is preempted."""
    import cbis_b200 as cb
    prompts = prompts_for(tc.TINY_B, [3, 17, 9, 30, 5], 21)
    lens = [12, 25, 7, 18, 30]

    def run(ahead, eos, num_pages=40):
        eng = cb.Engine(folder_b, dtype=dtype, page_size=tc.PAGE_B, num_pages=num_pages, max_num_seqs=4,
                        max_batched_tokens=48, prefill_chunk=16)
        eng.step_ahead = ahead
        params = [cb.SamplingParams(max_new_tokens=n, temperature=temperature, seed=5, eos_token_id=e)
                  for n, e in zip(lens, eos)]
        outs = eng.generate(prompts, params)
        assert eng.pool.manager.check() == "" and eng.pool.manager.free_pages(0) == num_pages and eng._in_flight is None
        return outs, eng

    none = [None] * 5
    base, eng = run(False, none)
    assert eng.steps_ahead == 0
    got, eng = run(True, none)
    assert got == base and eng.steps_ahead > 20
    if dtype == "float32":
        check_against_plain(folder_b, prompts, got, temperature, 5, 0, exact=True)
    # requests 1 and 4 stop early: on the token they produced as their 6th and 11th output
    eos = [None, base[1][5], None, None, base[4][10]]
    want, _ = run(False, eos)
    assert len(want[1]) <= 6 and len(want[4]) <= 11 and want[1][-1] == eos[1] and want[4][-1] == eos[4]
    got, eng = run(True, eos)
    assert got == want and eng.steps_ahead > 5
    # few pages: the newest request is preempted and recomputed; planning ahead stops where pages are short
    want, e0 = run(False, none, num_pages=12)
    got, e1 = run(True, none, num_pages=12)
    assert got == want == base and e0.scheduler.preemptions() > 0 and e1.scheduler.preemptions() > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b"])
def test_small_steps_with_prompt_portions_replay_a_graph(folder_a, folder_b, which, dtype):
    """Small steps that hold prompt portions are captured per size (rows rounded up to a power of two, laid out for
    all request slots, every segment through the kernels of the longer ones): while serving, once a size has come
    a few times and a timed run has shown the device waiting for the host (here: from the third time on); or ahead
    of serving by ``warm_up``, which keeps a graph if its replay is faster than the launches.  Many short requests
    through few slots: the same tokens as without such graphs, and the plain implementation's."""
    import cbis_b200 as cb
    folder, cfg, page = (folder_a, tc.TINY_A, tc.PAGE_A) if which == "a" else (folder_b, tc.TINY_B, tc.PAGE_B)
    g = torch.Generator().manual_seed(77)
    lens = [int(n) for n in torch.randint(1, 15, (40,), generator=g)]
    prompts = prompts_for(cfg, lens, 12)
    news = [int(n) for n in torch.randint(2, 9, (40,), generator=g)]

    def run(on, warm=False):
        eng = cb.Engine(folder, dtype=dtype, page_size=page, num_pages=64, max_num_seqs=4, max_batched_tokens=64,
                        prefill_chunk=16)
        eng.runner.small_step_graphs = on
        eng.runner.small_graph_after = 3
        eng.runner.small_graph_span_factor = 100.0       # the mechanism is under test here, not the measurement
        eng.runner.small_graph_host_factor = 0.0         # (warm_up keeps every graph it captures)
        kept = eng.warm_up() if warm else 0
        outs = eng.generate(prompts, [cb.SamplingParams(max_new_tokens=n) for n in news])
        assert eng.pool.manager.check() == "" and eng.pool.manager.free_pages(0) == 64
        return outs, eng, kept

    base, e0, _ = run(False)
    assert e0.runner.small_captures == 0
    got, e1, _ = run(True)
    assert e1.runner.small_captures >= 1 and e1.runner.small_replays >= 5
    check_against_plain(folder, prompts, got, 0.0, 0, 0, exact=dtype == "float32")
    if dtype == "float32":
        assert got == base
    warmed, e2, kept = run(True, warm=True)
    sizes = {k[0] for k in e2.runner._small_graphs}
    assert sizes == {16, 32, 64} and kept >= len(e2.runner._graphs) + len(sizes)      # 64: the most tokens of a step
    assert e2.runner.small_replays > e1.runner.small_replays
    assert warmed == got


@pytest.mark.parametrize("seed", [0, 1])
def test_everything_at_once_gives_the_plain_tokens(folder_b, seed):
    """Sixty requests of random lengths, some greedy and some with a temperature, some with an end-of-sequence
    token that they do produce, arriving a few at a time while others run, through four slots and so few pages that
    requests are preempted; with steps launched ahead, small steps replaying graphs and freed pages filled with NaN.
    32-bit path: every request's tokens are the plain implementation's (cut at the end-of-sequence token)."""
    import random
    import cbis_b200 as cb
    rng = random.Random(seed)
    cfg, w = plain_gpt.read_model_folder(folder_b, torch.float64)
    eng = cb.Engine(folder_b, dtype="float32", page_size=tc.PAGE_B, num_pages=14, max_num_seqs=4, max_batched_tokens=40,
                    prefill_chunk=12, poison_freed_pages=True)
    eng.runner.small_graph_after = 2
    eng.runner.small_graph_span_factor = 100.0
    work = []
    for i in range(60):
        prompt = [rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(1, 30))]
        n = rng.randint(1, 20)
        temp = rng.choice([0.0, 0.0, 0.7, 1.3])
        want = plain_gpt.generate(cfg, w, prompt, n, temp, 11, i)
        eos = None
        if len(want) > 2 and rng.random() < 0.4:
            eos = want[rng.randrange(1, len(want))]
            want = want[:want.index(eos) + 1]
        work.append((prompt, cb.SamplingParams(max_new_tokens=n, temperature=temp, seed=11, eos_token_id=eos), want))
    got, nxt = {}, 0
    while nxt < len(work) or eng.has_unfinished():
        for _ in range(rng.randint(0, 3)):
            if nxt < len(work):
                assert eng.add_request(work[nxt][0], work[nxt][1]) == nxt
                nxt += 1
        for o in eng.step():
            got[o.request_id] = o.tokens
    assert eng._in_flight is None and eng.pool.manager.check() == "" and eng.pool.manager.free_pages(0) == 14
    for i, (_, _, want) in enumerate(work):
        assert got[i] == want, f"request {i}"
    assert eng.steps_ahead > 3 and eng.scheduler.preemptions() > 0 and eng.runner.small_replays > 0 and eng.pages_poisoned > 0


def test_first_tokens_of_a_sequence(tiny):
    import cbis_b200 as cb
    folder, cfg, page = tiny
    eng = cb.Engine(folder, dtype="float32", page_size=page, num_pages=8, max_num_seqs=2, max_batched_tokens=16)
    pcfg, w = plain_gpt.read_model_folder(folder, torch.float64)
    for toks in ([0], [cfg["vocab_size"] - 1], [3, 3], [5, 0, 9]):
        got = eng.logits(toks).double().cpu().numpy()
        with torch.no_grad():
            ref = plain_gpt.forward(pcfg, w, toks).numpy()
        assert np.abs(got - ref).max() < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_gives_the_same_tokens(folder_b, dtype):
    import cbis_b200 as cb
    prompts = prompts_for(tc.TINY_B, [9, 14, 20, 11], 3)
    params = cb.SamplingParams(max_new_tokens=24, temperature=0.7, seed=99)
    roomy = cb.Engine(folder_b, dtype=dtype, page_size=8, num_pages=40, max_num_seqs=4, max_batched_tokens=32)
    want = roomy.generate(prompts, params)
    tight = cb.Engine(folder_b, dtype=dtype, page_size=8, num_pages=11, max_num_seqs=4, max_batched_tokens=32)
    got = tight.generate(prompts, params)
    assert tight.scheduler.preemptions() >= 1
    if dtype == "float32":
        assert got == want
    else:
        check_against_plain(folder_b, prompts, got, 0.7, 99, 0, exact=False)
    assert tight.pool.manager.free_pages(0) == 11 and tight.pool.manager.check() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_with_freed_pages_poisoned(folder_b, dtype):
    """The debugging mode that fills every page a request gives back with NaN before the next step: under
    preemption (pages change hands in the middle of generation) no NaN reaches any logit, and the tokens are those
    of an engine with room for everything."""
    import cbis_b200 as cb
    prompts = prompts_for(tc.TINY_B, [9, 14, 20, 11], 3)
    params = cb.SamplingParams(max_new_tokens=24, temperature=0.7, seed=99)
    roomy = cb.Engine(folder_b, dtype=dtype, page_size=8, num_pages=40, max_num_seqs=4, max_batched_tokens=32)
    want = roomy.generate(prompts, params)
    tight = cb.Engine(folder_b, dtype=dtype, page_size=8, num_pages=11, max_num_seqs=4, max_batched_tokens=32,
                      poison_freed_pages=True)
    seen_nan = []
    run_step = tight.runner.step
    def watched(plan, borrow=False):
        out = run_step(plan, borrow=borrow)
        seen_nan.append(bool(torch.isnan(out).any()))
        return out
    tight.runner.step = watched
    got = tight.generate(prompts, params)
    assert tight.scheduler.preemptions() >= 1 and tight.pages_poisoned >= 4 and not any(seen_nan)
    if dtype == "float32":
        assert got == want
    else:
        check_against_plain(folder_b, prompts, got, 0.7, 99, 0, exact=False)
    # the mode does what it says: the pages given back at the end hold NaN once the next step has been queued
    tight.generate([prompts[0][:3]], cb.SamplingParams(max_new_tokens=1))
    k = tight.pool.layer_cache[0].k
    assert torch.isnan(k.float()).any() and tight.pool.manager.check() == ""


@pytest.mark.parametrize("which", ["a", "b"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_device_decode_loop_gives_the_tokens_of_generate(folder_a, folder_b, which, dtype):
    """The decode loop that never leaves the device (model, argmax and the move to the next position in one
    graph, pages reserved ahead) against greedy generation through the scheduler and against the plain
    implementation, across several page edges."""
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    folder, cfgd, page = (folder_a, tc.TINY_A, tc.PAGE_A) if which == "a" else (folder_b, tc.TINY_B, tc.PAGE_B)
    n_new = 64 if which == "a" else 48                         # 4 pages of 16, 6 pages of 8
    prompts = prompts_for(cfgd, [5, 17, 11], 21)
    opts = dict(dtype=dtype, page_size=page, num_pages=40, max_num_seqs=4, max_batched_tokens=64)
    want = cb.Engine(folder, **opts).generate(prompts, cb.SamplingParams(max_new_tokens=n_new))
    eng = cb.Engine(folder, **opts)
    if not eng.runner.use_graphs:
        pytest.skip("no graphs")
    slots = [eng.open_request(i) for i in range(len(prompts))]
    first = eng.forward_step([StepEntry(s, 0, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).argmax(-1).tolist()
    for s in slots:
        assert eng.pool.manager.append(s, n_new)               # the pages of all steps, taken beforehand
    loop = eng.runner.decode_loop([StepEntry(s, len(p), [t], [0]) for s, p, t in zip(slots, prompts, first)])
    got = [[t] for t in first]
    for o, t in zip(got, loop.last_tokens()):                  # building the loop ran its first step
        o.append(t)
    for _ in range(n_new - 2):
        loop.run(1)
        for o, t in zip(got, loop.last_tokens()):
            o.append(t)
    assert loop.steps_done == n_new - 1
    if dtype == "float32":
        assert got == want
        cfg, w = plain_gpt.read_model_folder(folder, torch.float64)
        assert got == [plain_gpt.generate(cfg, w, p, n_new) for p in prompts]
    else:
        check_against_plain(folder, prompts, got, 0.0, 0, 0, exact=False)
        assert [o[:4] for o in got] == [o[:4] for o in want]   # later, a near-tie may send the two runs different ways
    for s in slots:
        eng.close_request(s)
    assert eng.pool.manager.check() == ""


def test_a_refused_prompt_leaves_nothing_of_the_call_behind(folder_a):
    import cbis_b200 as cb
    eng = cb.Engine(folder_a, dtype="float32", page_size=16, num_pages=8, max_num_seqs=2, max_batched_tokens=32)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.generate([[1, 2, 3], [4, 5], [6, 9999]], cb.SamplingParams(max_new_tokens=4))
    assert eng.scheduler.idle() and not eng._params
    with pytest.raises(ValueError, match="exceeds the model"):
        eng.generate([[1, 2], [3] * 500], cb.SamplingParams(max_new_tokens=4))
    assert eng.scheduler.idle() and not eng._params
    out = eng.generate([[1, 2, 3]], cb.SamplingParams(max_new_tokens=4))
    assert len(out) == 1 and len(out[0]) == 4 and eng.pool.manager.free_pages(0) == 8


def test_abort_while_a_step_is_on_its_way(folder_a):
    """A request dropped in the middle of decoding, while the step launched ahead holds a row of it: the others
    end with the tokens they would have had anyway, the pages are all back."""
    import cbis_b200 as cb
    prompts = prompts_for(tc.TINY_A, [6, 11, 4], 3)
    eng = cb.Engine(folder_a, dtype="float32", page_size=tc.PAGE_A, num_pages=16, max_num_seqs=3, max_batched_tokens=64)
    want = eng.generate(prompts, cb.SamplingParams(max_new_tokens=12))
    ids = [eng.add_request(p, cb.SamplingParams(max_new_tokens=12)) for p in prompts]
    got = {}
    for _ in range(5):
        for o in eng.step():
            got[o.request_id] = o.tokens
    assert eng._in_flight is not None
    assert eng.abort(ids[1]) and not eng.abort(ids[1])
    while eng.has_unfinished():
        for o in eng.step():
            got[o.request_id] = o.tokens
    assert got == {ids[0]: want[0], ids[2]: want[2]}
    assert eng._in_flight is None and eng.pool.manager.check() == "" and eng.pool.manager.free_pages(0) == 16


def test_eos_stops_a_request(folder_a):
    import cbis_b200 as cb
    eng = cb.Engine(folder_a, dtype="float32", page_size=16, num_pages=8, max_num_seqs=2, max_batched_tokens=32)
    prompt = [1, 2, 3, 4]
    free = eng.generate([prompt], cb.SamplingParams(max_new_tokens=12))[0]
    stop_at = free[5]
    k = free.index(stop_at)
    out = eng.generate([prompt], cb.SamplingParams(max_new_tokens=12, eos_token_id=stop_at))[0]
    assert out == free[:k + 1]
    assert eng.generate([prompt], cb.SamplingParams(max_new_tokens=12, eos_token_id=stop_at, ignore_eos=True))[0] == free


def test_build_model_from_a_configuration_and_a_seed():
    import cbis_b200 as cb
    a = cb.build_model(tc.TINY_B, seed=5, dtype="float32", page_size=8, num_pages=16, max_num_seqs=2)
    b = cb.build_model(cb.config_from_dict(tc.TINY_B), seed=5, dtype="float32", page_size=8, num_pages=16, max_num_seqs=2)
    c = cb.build_model(tc.TINY_B, seed=6, dtype="float32", page_size=8, num_pages=16, max_num_seqs=2)
    toks = [4, 8, 15, 16, 23, 42]
    la, lb, lc = a.logits(toks), b.logits(toks), c.logits(toks)
    assert la.shape == (6, 317) and torch.equal(la, lb) and not torch.equal(la, lc)


def test_command_line(folder_a, tmp_path):
    prompts = prompts_for(tc.TINY_A, [4, 9], 8)
    pf = tmp_path / "prompts.txt"
    pf.write_text("\n".join(",".join(map(str, p)) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), folder_a, "--dtype", "float32",
                        "--prompts-file", str(pf), "--max-new-tokens", "6", "--num-pages", "8", "--json"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    outs = [json.loads(l)["tokens"] for l in r.stdout.splitlines() if l.startswith("{")]
    cfg, w = plain_gpt.read_model_folder(folder_a, torch.float64)
    assert outs == [plain_gpt.generate(cfg, w, p, 6) for p in prompts]


def test_repeated_step_shapes_replay_a_graph_and_give_the_same_logits(tiny):
    """A step shape that keeps coming back (here: portions of 6 tokens of one request, then of another) is captured
    as a CUDA graph and replayed; the logits are those of the launch-by-launch path."""
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    folder, cfgd, page = tiny
    toks = [(7 * i + 3) % cfgd["vocab_size"] for i in range(60)]

    def run(after):
        eng = cb.Engine(folder, dtype="bfloat16", page_size=page, num_pages=64, max_num_seqs=2, max_batched_tokens=64)
        eng.runner.shape_graph_after, eng.runner.shape_graph_min_host_s = after, 0.0
        outs = []
        for req in range(2):
            slot = eng.open_request(req)
            for at in range(0, 60, 6):
                outs.append(eng.forward_step([StepEntry(slot, at, toks[at:at + 6], [0, 5])]).float().cpu())
            eng.close_request(slot)
        return torch.cat(outs), eng.runner.shape_captures, eng.runner.shape_replays

    eager, c0, r0 = run(10 ** 9)
    graphed, c1, r1 = run(3)
    assert (c0, r0) == (0, 0) and c1 == 1 and r1 == 17       # 20 steps of one shape: 2 launch by launch, 1 captured, 17 replayed
    assert torch.equal(eager, graphed)
