"""The two optional forms of a decode step, the persistent kernel (a run of layers in one launch, CBIS_FUSED_DECODE=1)
and the norm inside the product's kernel (CBIS_LN_LINEAR=1), against the same layers run kernel by kernel and
against the plain implementation (GPU): head sizes 64 and 128, shared key/value heads, a window, widths that are
no power of two, 1 to 16 rows, requests of very different lengths side by side, page edges, padding rows of a
captured step, and generation through the scheduler."""
import numpy as np
import pytest
import torch

import plain_gpt

pytestmark = pytest.mark.gpu

SMALL_64 = dict(architectures=["GPT2LMHeadModel"], n_layer=3, n_embd=128, n_head=2, n_inner=320, vocab_size=301,
                n_positions=320, activation_function="gelu_new", layer_norm_epsilon=1e-5, tie_word_embeddings=True)
SMALL_128 = dict(architectures=["TinyGPT"], n_layer=2, n_embd=384, n_head=3, n_inner=712, vocab_size=517,
                 n_positions=200, activation_function="gelu", layer_norm_epsilon=1e-6, tie_word_embeddings=False)
INIT = (0.08, 0.05, 0.1, 0.1)


def folder_of(tmp_path_factory, cfg, seed):
    import cbis_b200 as cb
    d = str(tmp_path_factory.mktemp("dl"))
    cb.write_model_folder(d, cb.config_from_dict(cfg), seed=seed, scheme=cb.InitScheme(*INIT))
    return d


def decode_logits(eng, seqs, n_prompt, fused, ln_linear=False):
    """Prompts in one step each, then all requests token by token side by side: logits of every decoded position."""
    from cbis_b200.engine import StepEntry
    from cbis_b200.kernels import ops
    keep, keep_ln = ops.USE_FUSED_DECODE, ops.USE_LN_LINEAR
    ops.USE_FUSED_DECODE, ops.USE_LN_LINEAR = fused, ln_linear
    eng.runner._graphs.clear()          # captured decode steps hold the launches of the form they were captured with
    try:
        slots = [eng.open_request(i) for i in range(len(seqs))]
        for s, toks, n in zip(slots, seqs, n_prompt):
            eng.forward_step([StepEntry(s, 0, toks[:n], [])])
        fed = list(n_prompt)
        got = [[] for _ in seqs]
        while any(f < len(t) for f, t in zip(fed, seqs)):
            live = [i for i in range(len(seqs)) if fed[i] < len(seqs[i])]
            lg = eng.forward_step([StepEntry(slots[i], fed[i], [seqs[i][fed[i]]], [0]) for i in live]).float().cpu()
            for r, i in enumerate(live):
                got[i].append(lg[r])
                fed[i] += 1
        for s in slots:
            eng.close_request(s)
        ops.raise_if_kernel_errors()
    finally:
        ops.USE_FUSED_DECODE, ops.USE_LN_LINEAR = keep, keep_ln
    return [torch.stack(g) for g in got]


@pytest.mark.parametrize("which", ["hd64", "hd128"])
def test_decode_steps_with_the_norm_inside_the_product_match_kernel_by_kernel_and_plain(tmp_path_factory, which, monkeypatch):
    """CBIS_LN_LINEAR=1: up to 8 rows normalise inside the kernels of the QKV and the first feed-forward product, and
    the attention's and the feed-forward's outputs are added into the residual stream by their products; 9 rows and
    more, and the prompts' steps, go the usual way in the same requests."""
    import cbis_b200 as cb
    from cbis_b200.kernels import ops
    cfg = SMALL_64 if which == "hd64" else SMALL_128
    folder = folder_of(tmp_path_factory, cfg, 77)
    V = cfg["vocab_size"]
    g = torch.Generator().manual_seed(9)
    lens = [150, 40, 97, 33, 64, 18, 129, 70, 51, 20]
    n_prompt = [120, 1, 64, 31, 48, 2, 100, 63, 17, 3]
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]
    pcfg, w = plain_gpt.read_model_folder(folder, torch.float64)
    calls = []
    real = ops.ln_linear
    monkeypatch.setattr(ops, "ln_linear", lambda *a: (calls.append(a[0].shape[0]), real(*a))[1])
    for n_req in (1, 5, 8, 10):
        eng = cb.Engine(folder, dtype="bfloat16", page_size=16, num_pages=80, max_num_seqs=16, max_batched_tokens=256)
        chain = decode_logits(eng, seqs[:n_req], n_prompt[:n_req], fused=False)
        assert not calls
        inside = decode_logits(eng, seqs[:n_req], n_prompt[:n_req], fused=False, ln_linear=True)
        assert calls and max(calls) <= 8
        del calls[:]
        for i in range(n_req):
            with torch.no_grad():
                ref = plain_gpt.forward(pcfg, w, seqs[i])[n_prompt[i]:].float()
            scale = ref.abs().max().item()
            assert torch.isfinite(inside[i]).all()
            assert (inside[i] - ref).abs().max().item() < 0.02 * scale, (n_req, i)
            assert (inside[i] - chain[i]).abs().max().item() < 0.008 * scale, (n_req, i)
        assert eng.pool.manager.check() == ""


@pytest.mark.parametrize("which", ["hd64", "hd128"])
def test_decode_steps_in_one_kernel_match_kernel_by_kernel_and_plain(tmp_path_factory, which):
    import cbis_b200 as cb
    cfg = SMALL_64 if which == "hd64" else SMALL_128
    folder = folder_of(tmp_path_factory, cfg, 31)
    V = cfg["vocab_size"]
    g = torch.Generator().manual_seed(4)
    lens = [150, 40, 97, 33, 64, 18, 129, 70, 51, 20, 88, 35]               # up to 12 rows: the 16-row form
    n_prompt = [120, 1, 64, 31, 48, 2, 100, 63, 17, 3, 60, 16]
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]
    pcfg, w = plain_gpt.read_model_folder(folder, torch.float64)
    for n_req in (1, 3, 8, 12):
        eng = cb.Engine(folder, dtype="bfloat16", page_size=16, num_pages=80, max_num_seqs=16, max_batched_tokens=256)
        chain = decode_logits(eng, seqs[:n_req], n_prompt[:n_req], fused=False)
        assert "_decode_layer_plans" not in eng.runner.__dict__
        fused = decode_logits(eng, seqs[:n_req], n_prompt[:n_req], fused=True)
        plans = eng.runner.__dict__["_decode_layer_plans"]
        assert len(plans) == 1 and all(p is not False and p.n_layers == cfg["n_layer"] for p in plans.values())
        for i in range(n_req):
            with torch.no_grad():
                ref = plain_gpt.forward(pcfg, w, seqs[i])[n_prompt[i]:].float()
            scale = ref.abs().max().item()
            assert torch.isfinite(fused[i]).all()
            assert (fused[i] - ref).abs().max().item() < 0.02 * scale, (n_req, i)
            assert (fused[i] - chain[i]).abs().max().item() < 0.008 * scale, (n_req, i)
        assert eng.pool.manager.check() == ""


def test_shared_key_value_heads_and_a_window_in_one_kernel():
    """Four query heads on two key/value heads of 64, a window of 40 keys, pages of 32: the persistent kernel against
    the same model kernel by kernel and against a plain restatement."""
    import cbis_b200 as cb
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec
    from cbis_b200.models import Model
    from cbis_b200.weights import InitScheme, random_tensors
    W, V, P, H, KV, HD, F = 200, 211, 160, 4, 2, 64, 264
    norm = PartSpec("layernorm", {"width": W, "eps": 1e-5})
    att = PartSpec("attention", {"width": W, "n_head": H, "n_kv_head": KV, "head_dim": HD, "scale": HD ** -0.5, "window": 40})
    ffn = PartSpec("dense", {"width": W, "inner": F, "activation": "gelu_erf"})
    layers = tuple(LayerSpec(f"h.{i}.", "pre_norm", att, ffn, norm, norm) for i in range(2))
    spec = ModelSpec(W, V, P, "wte.weight", PartSpec("learned", {"width": W, "n_positions": P}), layers, (0, 1), norm,
                     "ln_f.", None)
    tensors = random_tensors(Model(spec).declared(), 3, InitScheme(0.08, 0.05, 0.1, 0.1), torch.bfloat16)
    model = Model(spec).load(tensors, "bfloat16", "cuda")
    eng = cb.Engine(model, dtype="bfloat16", page_size=32, num_pages=24, max_num_seqs=4, max_batched_tokens=160)
    w = {k: v.double() for k, v in tensors.items()}

    def plain(tokens):
        T = len(tokens)
        x = plain_gpt.embed(tokens, w["wte.weight"], w["wpe.weight"])
        i = torch.arange(T)
        mask = (i[None, :] > i[:, None]) | (i[:, None] - i[None, :] >= 40)
        for li in range(2):
            p = f"h.{li}."
            h = plain_gpt.layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], 1e-5)
            qkv = h @ w[p + "attn.c_attn.weight"] + w[p + "attn.c_attn.bias"]
            q, k, v = qkv[:, :H * HD], qkv[:, H * HD:(H + KV) * HD], qkv[:, (H + KV) * HD:]
            outs = []
            for hh in range(H):
                kk, vv = k[:, (hh // 2) * HD:(hh // 2 + 1) * HD], v[:, (hh // 2) * HD:(hh // 2 + 1) * HD]
                sc = (q[:, hh * HD:(hh + 1) * HD] @ kk.T) * HD ** -0.5
                outs.append(torch.softmax(sc.masked_fill(mask, float("-inf")), -1) @ vv)
            x = x + torch.cat(outs, 1) @ w[p + "attn.c_proj.weight"] + w[p + "attn.c_proj.bias"]
            x = x + plain_gpt.mlp(plain_gpt.layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], 1e-5),
                                  w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"], w[p + "mlp.c_proj.weight"],
                                  w[p + "mlp.c_proj.bias"], "gelu")
        return plain_gpt.layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], 1e-5) @ w["wte.weight"].T

    g = torch.Generator().manual_seed(8)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (150, 45, 90)]
    n_prompt = [100, 2, 33]
    chain = decode_logits(eng, seqs, n_prompt, fused=False)
    fused = decode_logits(eng, seqs, n_prompt, fused=True)
    assert any(p is not False for p in eng.runner.__dict__["_decode_layer_plans"].values())
    for i in range(3):
        ref = plain(seqs[i])[n_prompt[i]:].float()
        scale = ref.abs().max().item()
        assert (fused[i] - ref).abs().max().item() < 0.02 * scale
        assert (fused[i] - chain[i]).abs().max().item() < 0.008 * scale


def test_generation_with_the_persistent_kernel_equals_generation_without(tmp_path_factory):
    """Greedy generation through the scheduler (captured decode steps with padding rows, requests that end at
    different times, pages that change hands) with and without the persistent kernel: each chosen token is, by the
    plain implementation's scores, within a bfloat16 margin of the best."""
    import cbis_b200 as cb
    from cbis_b200.kernels import ops
    folder = folder_of(tmp_path_factory, SMALL_64, 77)
    V = SMALL_64["vocab_size"]
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in (5, 70, 33, 9, 120)]
    params = [cb.SamplingParams(max_new_tokens=n) for n in (40, 12, 64, 30, 50)]
    eng = cb.Engine(folder, dtype="bfloat16", page_size=16, num_pages=30, max_num_seqs=5, max_batched_tokens=128,
                    poison_freed_pages=True)
    keep, ops.USE_FUSED_DECODE = ops.USE_FUSED_DECODE, True
    try:
        outs = eng.generate(prompts, params)
    finally:
        ops.USE_FUSED_DECODE = keep
    assert [len(o) for o in outs] == [40, 12, 64, 30, 50]
    assert any(p is not False for p in eng.runner.__dict__.get("_decode_layer_plans", {}).values())
    ops.raise_if_kernel_errors()
    pcfg, w = plain_gpt.read_model_folder(folder, torch.float64)
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            lg = plain_gpt.forward(pcfg, w, p + o[:-1]).numpy()
        for j, t in enumerate(o):
            row = lg[len(p) - 1 + j]
            assert row[t] >= row.max() - 0.03 * np.abs(lg).max(), (len(p), j)
