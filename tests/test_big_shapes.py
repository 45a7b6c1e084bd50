"""The layer sizes of the benchmark configurations (width 2048, 16 heads of 128, inner 8192, vocabulary
50257; the GPT-2 XL sizes; and the 6.7B sizes, width 4096 and inner 16384) with two layers or one (GPU): here the kernels for head sizes 128 and 64 run inside
the engine - the tiled prefill attention, the split-KV decode attention, the few-rows product, the TMA +
tcgen05 products.  The 32-bit path is compared with the plain implementation once (its weights are drawn
on the CPU so that the plain side can draw them again); every way of cutting a request in bfloat16 must
then give the logits of the 32-bit path; a step shape that keeps coming back is replayed from a CUDA graph
and must give the bits of the launch-by-launch run; and the decode loop that stays on the device gives the
tokens of generation."""
import numpy as np
import pytest
import torch

import plain_gpt

pytestmark = pytest.mark.gpu

BIG = dict(architectures=["GPT2LMHeadModel"], n_layer=2, n_embd=2048, n_head=16, n_inner=8192, vocab_size=50257,
           n_positions=2048, activation_function="gelu", layer_norm_epsilon=1e-5, tie_word_embeddings=True)
# GPT-2 XL layer sizes: 25 heads of 64, a width and an inner size that are no powers of two, tanh GELU
XL = dict(architectures=["GPT2LMHeadModel"], n_layer=2, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257,
          n_positions=1024, activation_function="gelu_new", layer_norm_epsilon=1e-5, tie_word_embeddings=True)


# Cerebras-GPT-6.7B layer sizes, one layer: K = 4096 and 16384, 32 heads of 128
WIDE = dict(architectures=["GPT2LMHeadModel"], n_layer=1, n_embd=4096, n_head=32, n_inner=16384, vocab_size=50257,
            n_positions=2048, activation_function="gelu", layer_norm_epsilon=1e-5, tie_word_embeddings=True)


@pytest.fixture(scope="module", params=["1.3b", "xl", "6.7b"])
def engines(request):
    import cbis_b200 as cb
    cfg = {"1.3b": BIG, "xl": XL, "6.7b": WIDE}[request.param]
    opts = dict(page_size=16, num_pages=80, max_num_seqs=4, max_batched_tokens=1024)
    # both engines hold the same bfloat16 values, drawn by the CPU's generator: the plain side draws them again
    e32 = cb.Engine.from_random(cfg, seed=3, dtype="float32", weight_dtype=torch.bfloat16, draw_on="cpu", **opts)
    e16 = cb.Engine.from_random(cfg, seed=3, dtype="bfloat16", draw_on="cpu", **opts)
    e32.config_dict = e16.config_dict = cfg
    yield e32, e16
    del e32, e16
    torch.cuda.empty_cache()


def run_cut(eng, seqs, plan):
    """plan: list of steps, each a list of (name, n_tokens); logits of every token are collected per request."""
    from cbis_b200.engine import StepEntry
    slots = {k: eng.open_request(i) for i, k in enumerate(seqs)}
    fed = {k: 0 for k in seqs}
    got = {k: [] for k in seqs}
    for step in plan:
        entries = []
        for name, n in step:
            toks = seqs[name][fed[name]:fed[name] + n]
            entries.append(StepEntry(slots[name], fed[name], toks, list(range(len(toks)))))
        lg = eng.forward_step(entries).float().cpu()
        r = 0
        for name, n in step:
            n = min(n, len(seqs[name]) - fed[name])
            got[name].append(lg[r:r + n]); r += n; fed[name] += n
    for s in slots.values():
        eng.close_request(s)
    return {k: torch.cat(v) for k, v in got.items()}


def test_every_cut_matches_the_32_bit_path(engines):
    e32, e16 = engines
    g = torch.Generator().manual_seed(0)
    seqs = {"a": torch.randint(0, 50257, (300,), generator=g).tolist(),
            "b": torch.randint(0, 50257, (97,), generator=g).tolist()}
    whole = [[("a", 300)], [("b", 97)]]
    ref = run_cut(e32, seqs, whole)
    scale = max(r.abs().max().item() for r in ref.values())
    got_whole = run_cut(e16, seqs, whole)
    # most in one step, the last 32 one by one, the two requests side by side while decoding
    tail = [[("a", 268)], [("b", 65)]] + [[("a", 1), ("b", 1)] for _ in range(32)]
    got_tail = run_cut(e16, seqs, tail)
    # portions of changing size, mixed with the other request's single tokens
    mixed = [[("a", 130)], [("a", 2), ("b", 70)], [("a", 61), ("b", 1)], [("a", 7), ("b", 1)], [("a", 100), ("b", 25)]]
    got_mixed = run_cut(e16, seqs, mixed)
    for name in seqs:
        for got, what in ((got_whole, "whole"), (got_tail, "tail"), (got_mixed, "mixed")):
            d = (got[name] - ref[name]).abs().max().item()
            assert d < 0.02 * scale, f"{name} {what}: max abs diff {d:.4f} against the 32-bit path (largest logit {scale:.2f})"
        # the cuts agree with each other more closely than with the 32-bit path
        assert (got_tail[name] - got_whole[name]).abs().max().item() < 0.01 * scale
        assert (got_mixed[name] - got_whole[name]).abs().max().item() < 0.01 * scale
    # the 32-bit path itself does not depend on the cut
    ref_tail = run_cut(e32, {"b": seqs["b"]}, [[("b", 65)]] + [[("b", 1)] for _ in range(32)])
    assert (ref_tail["b"] - ref["b"]).abs().max().item() < 2e-4 * max(1.0, scale)


def test_greedy_tokens_of_both_paths_agree_where_the_margin_allows(engines):
    import cbis_b200 as cb
    e32, e16 = engines
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 50257, (n,), generator=g).tolist() for n in (40, 9, 120)]
    out16 = e16.generate(prompts, cb.SamplingParams(max_new_tokens=12))
    # replay the bfloat16 path's sequences through the 32-bit path: each chosen token is within a small margin of its best
    for p, o in zip(prompts, out16):
        lg = e32.logits(p + o[:-1]).float().cpu()
        for j, t in enumerate(o):
            row = lg[len(p) - 1 + j]
            assert row[t] >= row.max() - 0.03 * lg.abs().max()


def test_32_bit_path_matches_the_plain_implementation_at_these_sizes(engines):
    """The chain embed ... logits at head size 128 / width 2048 and at head size 64 / width 1600 (K no power of
    two), 32-bit path against the plain implementation in float64 on the CPU, whole and with the last tokens one
    by one.  (The reference checks its one fixed size this way: src/correctness_check.cpp:75-88.)"""
    from cbis_b200.weights import InitScheme, random_tensors
    e32, _ = engines
    cfg = e32.config_dict
    w = {k: v.double() for k, v in random_tensors(e32.model.declared(), 3, InitScheme(), torch.bfloat16).items()}
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, 50257, (200,), generator=g).tolist()
    with torch.no_grad():
        ref = plain_gpt.forward(cfg, w, toks)
    del w
    scale = ref.abs().max().item()
    whole = run_cut(e32, {"a": toks}, [[("a", 200)]])["a"].double()
    assert (whole - ref).abs().max().item() < 1e-3 * scale
    tail = run_cut(e32, {"a": toks}, [[("a", 190)]] + [[("a", 1)] for _ in range(10)])["a"].double()
    assert (tail - ref).abs().max().item() < 1e-3 * scale


def test_a_repeated_mixed_step_shape_is_replayed_from_a_graph_with_the_same_bits(engines):
    """A 512-token portion beside two decoding rows, again and again: after a few times the shape is captured
    (TMA + tcgen05 products and attention inside a CUDA graph) and replayed; every replayed step gives the bits
    of the same step run launch by launch."""
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    _, e16 = engines
    g = torch.Generator().manual_seed(11)
    long_ = torch.randint(0, 50257, (512 * 7,), generator=g).tolist()
    d1, d2 = torch.randint(0, 50257, (30,), generator=g).tolist(), torch.randint(0, 50257, (40,), generator=g).tolist()

    def run(graphs):
        r = e16.runner
        keep = (r.shape_graphs, r.shape_graph_after, r.shape_graph_min_host_s)
        r.shape_graphs, r.shape_graph_after, r.shape_graph_min_host_s = graphs, 3, 0.0
        r._shape_seen.clear(); r._shape_graphs.clear()
        c0, p0 = r.shape_captures, r.shape_replays
        outs = []
        try:
            sd1, sd2 = e16.open_request(1), e16.open_request(2)
            e16.forward_step([StepEntry(sd1, 0, d1[:20], []), StepEntry(sd2, 0, d2[:33], [])])
            n1, n2 = 20, 33
            for rep in range(7):
                # two portions fill the 1,024 positions of one of the models and most of the pool: a new request then
                if rep % 2 == 0:
                    if rep:
                        e16.close_request(sl)
                    sl, at = e16.open_request(3), 0
                part = long_[rep * 512:(rep + 1) * 512]
                outs.append(e16.forward_step([StepEntry(sl, at, part, [0, 511]), StepEntry(sd1, n1, d1[n1:n1 + 1], [0]),
                                              StepEntry(sd2, n2, d2[n2:n2 + 1], [0])]).clone())
                at += 512; n1 += 1; n2 += 1
            for s_ in (sl, sd1, sd2):
                e16.close_request(s_)
        finally:
            r.shape_graphs, r.shape_graph_after, r.shape_graph_min_host_s = keep
        return torch.stack(outs), r.shape_captures - c0, r.shape_replays - p0

    eager, c_e, p_e = run(False)
    graphed, c_g, p_g = run(True)
    assert (c_e, p_e) == (0, 0) and c_g == 1 and p_g == 4        # steps 1-2 launch by launch, 3 captured, 4-7 replayed
    assert torch.isfinite(eager).all() and torch.equal(eager, graphed)


def test_device_decode_loop_gives_the_tokens_of_generate_at_these_sizes(engines):
    """The loop that the benchmark times (model, argmax and the move to the next position in one graph) against
    greedy generation through the scheduler, 80 steps, across five page edges."""
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    e32, e16 = engines
    g = torch.Generator().manual_seed(13)
    prompts = [torch.randint(0, 50257, (n,), generator=g).tolist() for n in (60, 9, 33)]
    n_new = 80
    for eng, exact in ((e32, True), (e16, False)):
        want = eng.generate(prompts, cb.SamplingParams(max_new_tokens=n_new))
        slots = [eng.open_request(i) for i in range(3)]
        first = eng.forward_step([StepEntry(s, 0, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).argmax(-1).tolist()
        for s in slots:
            assert eng.pool.manager.append(s, n_new)
        loop = eng.runner.decode_loop([StepEntry(s, len(p), [t], [0]) for s, p, t in zip(slots, prompts, first)])
        got = [[t] for t in first]
        for o, t in zip(got, loop.last_tokens()):
            o.append(t)
        for _ in range(n_new - 2):
            loop.run(1)
            for o, t in zip(got, loop.last_tokens()):
                o.append(t)
        del loop
        for s in slots:
            eng.close_request(s)
        if exact:
            assert got == want
        else:   # bfloat16: both runs choose, by the 32-bit path's scores for their own sequence, within a margin of the best
            assert [o[:4] for o in got] == [o[:4] for o in want]
            for p, o in zip(prompts, got):
                lg = e32.logits(p + o[:-1]).float().cpu()
                for j, t in enumerate(o):
                    row = lg[len(p) - 1 + j]
                    assert row[t] >= row.max() - 0.03 * lg.abs().max()


def test_long_positions_change_the_split_of_the_keys_in_a_captured_step():
    """A model with 32,768 positions: a step captured for replay sizes its split of the keys for the bound of the
    positions, not for the step's own context, so the captured launches differ from the launch-by-launch ones;
    the logits agree to rounding and with the 32-bit path."""
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    cfg = dict(architectures=["GPT2LMHeadModel"], n_layer=2, n_embd=256, n_head=2, n_inner=512, vocab_size=1031,
               n_positions=32768, activation_function="gelu", layer_norm_epsilon=1e-5, tie_word_embeddings=True)
    opts = dict(page_size=16, num_pages=200, max_num_seqs=2, max_batched_tokens=512)
    e32 = cb.Engine.from_random(cfg, seed=5, dtype="float32", weight_dtype=torch.bfloat16, draw_on="cpu", **opts)
    e16 = cb.Engine.from_random(cfg, seed=5, dtype="bfloat16", draw_on="cpu", **opts)
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, 1031, (1200,), generator=g).tolist()

    def run(eng, graphs):
        r = eng.runner
        r.shape_graphs, r.shape_graph_after, r.shape_graph_min_host_s = graphs, 2, 0.0
        r._shape_seen.clear(); r._shape_graphs.clear()
        outs = []
        for rep in range(2):
            slot = eng.open_request(rep)
            for at in range(0, 1200, 300):
                outs.append(eng.forward_step([StepEntry(slot, at, toks[at:at + 300], [0, 150, 299])]).clone())
            # then token by token: decode-only steps, captured for a class of context lengths
            outs.append(torch.cat([eng.forward_step([StepEntry(slot, 1200 + i, [toks[i]], [0])]) for i in range(3)]))
            eng.close_request(slot)
        return torch.cat(outs), r.shape_captures

    ref, _ = run(e32, False)
    eager, c0 = run(e16, False)
    graphed, c1 = run(e16, True)
    scale = ref.abs().max().item()
    assert c0 == 0 and c1 >= 1
    assert (eager - ref).abs().max().item() < 0.02 * scale and (graphed - ref).abs().max().item() < 0.02 * scale
    assert (graphed - eager).abs().max().item() < 0.01 * scale
