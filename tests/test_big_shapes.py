"""The layer sizes of the benchmark configuration (width 2048, 16 heads of 128, inner 8192, vocabulary
50257) with two layers (GPU): here the kernels for head size 128 run inside the engine - the tiled
prefill attention, the split-KV decode attention, the few-rows product, the library product - and every
way of cutting a request must give the logits of the 32-bit path, which stands in for the plain
implementation at sizes where that one is too slow."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BIG = dict(architectures=["GPT2LMHeadModel"], n_layer=2, n_embd=2048, n_head=16, n_inner=8192, vocab_size=50257,
           n_positions=2048, activation_function="gelu", layer_norm_epsilon=1e-5, tie_word_embeddings=True)
# GPT-2 XL layer sizes: 25 heads of 64, a width and an inner size that are no powers of two, tanh GELU
XL = dict(architectures=["GPT2LMHeadModel"], n_layer=2, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257,
          n_positions=1024, activation_function="gelu_new", layer_norm_epsilon=1e-5, tie_word_embeddings=True)


@pytest.fixture(scope="module", params=["1.3b", "xl"])
def engines(request):
    import cbis_b200 as cb
    cfg = BIG if request.param == "1.3b" else XL
    opts = dict(page_size=16, num_pages=80, max_num_seqs=4, max_batched_tokens=1024)
    e32 = cb.Engine.from_random(cfg, seed=3, dtype="float32", weight_dtype=torch.bfloat16, **opts)
    e16 = cb.Engine.from_random(cfg, seed=3, dtype="bfloat16", **opts)
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
