"""Compares tests/plain_gpt.py with the reference's own model code and stores small outputs.

Run once, on the CPU, from the repository root:

    python tests/golden/make_golden.py /path/to/continuous-batching-inference-server

It imports the reference's ``python/model.py`` (TinyGPT, Block), sets that module's size
globals to the two tiny configurations (the classes read them when they are built,
python/model.py:26-33,57-61), copies random GPT-2-format weights into the module
(``wq.weight = c_attn.weight[:, 0:d].T`` and so on), runs ``model(idx)`` and the plain
implementation on the same tokens, asserts that they agree to 1e-5, and writes for each
configuration ``golden_<name>.npz``: the tokens and the reference module's logits at the
first, a middle and the last position.  tests/test_plain.py rebuilds the same weights from
the seed and checks the plain implementation against these files, so the check holds
without the reference being present.

The tanh GELU of tiny-A is not in the reference (python/model.py:50 is the erf form): for
that configuration the module's ``F`` is replaced by a shim whose ``gelu`` is torch's tanh
approximation; the layer-norm eps is set on each ``nn.LayerNorm``; tying is
``lm_head.weight = tok_emb.weight``.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import plain_gpt  # noqa: E402
import tiny_configs as tc  # noqa: E402


def golden_weights(cfg, init, seed):
    """Random GPT-2-format weights in float32, made with torch only (no engine code)."""
    g = torch.Generator().manual_seed(seed)
    d, F, V, P = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"], cfg["n_positions"]
    ms, bs, gs, bes = init

    def n(shape, std, mean=0.0):
        return torch.full(shape, mean) if std == 0 else torch.randn(shape, generator=g) * std + mean

    w = {"wte.weight": n((V, d), ms), "wpe.weight": n((P, d), ms)}
    for i in range(cfg["n_layer"]):
        p = f"h.{i}."
        w[p + "ln_1.weight"], w[p + "ln_1.bias"] = n((d,), gs, 1.0), n((d,), bes)
        w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"] = n((d, 3 * d), ms), n((3 * d,), bs)
        w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"] = n((d, d), ms), n((d,), bs)
        w[p + "ln_2.weight"], w[p + "ln_2.bias"] = n((d,), gs, 1.0), n((d,), bes)
        w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"] = n((d, F), ms), n((F,), bs)
        w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"] = n((F, d), ms), n((d,), bs)
    w["ln_f.weight"], w["ln_f.bias"] = n((d,), gs, 1.0), n((d,), bes)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = n((V, d), ms)
    return w


def reference_logits(ref_dir, cfg, w, tokens):
    spec = importlib.util.spec_from_file_location("ref_model", os.path.join(ref_dir, "python", "model.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    d = cfg["n_embd"]
    m.VOCAB, m.D_MODEL, m.N_HEADS, m.HEAD_DIM = cfg["vocab_size"], d, cfg["n_head"], d // cfg["n_head"]
    m.N_LAYERS, m.MLP_HIDDEN, m.MAX_SEQ_LEN = cfg["n_layer"], cfg["n_inner"], cfg["n_positions"]
    if cfg["activation_function"] == "gelu_new":
        import torch.nn.functional as F
        m.F = types.SimpleNamespace(softmax=F.softmax, gelu=lambda v: F.gelu(v, approximate="tanh"))
    model = m.TinyGPT().eval()
    with torch.no_grad():
        model.tok_emb.weight.copy_(w["wte.weight"])
        model.pos_emb.weight.copy_(w["wpe.weight"])
        for i, blk in enumerate(model.blocks):
            p = f"h.{i}."
            for ln, name in ((blk.ln1, "ln_1"), (blk.ln2, "ln_2")):
                ln.eps = cfg["layer_norm_epsilon"]
                ln.weight.copy_(w[p + name + ".weight"]); ln.bias.copy_(w[p + name + ".bias"])
            ca, cb_ = w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"]
            for j, lin in enumerate((blk.wq, blk.wk, blk.wv)):
                lin.weight.copy_(ca[:, j * d:(j + 1) * d].T); lin.bias.copy_(cb_[j * d:(j + 1) * d])
            blk.wo.weight.copy_(w[p + "attn.c_proj.weight"].T); blk.wo.bias.copy_(w[p + "attn.c_proj.bias"])
            blk.fc1.weight.copy_(w[p + "mlp.c_fc.weight"].T); blk.fc1.bias.copy_(w[p + "mlp.c_fc.bias"])
            blk.fc2.weight.copy_(w[p + "mlp.c_proj.weight"].T); blk.fc2.bias.copy_(w[p + "mlp.c_proj.bias"])
        model.ln_f.eps = cfg["layer_norm_epsilon"]
        model.ln_f.weight.copy_(w["ln_f.weight"]); model.ln_f.bias.copy_(w["ln_f.bias"])
        model.lm_head.weight.copy_(w["wte.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"])
        return model(torch.tensor([tokens]))[0]


def main():
    ref_dir = sys.argv[1]
    for name, cfg, init in (("tiny_a", tc.TINY_A, tc.INIT_A), ("tiny_b", tc.TINY_B, tc.INIT_B)):
        w = golden_weights(cfg, init, seed=2024)
        g = torch.Generator().manual_seed(777)   # the reference's fixture seed (python/export_weights.py:72)
        T = min(64, cfg["n_positions"])
        tokens = torch.randint(0, cfg["vocab_size"], (T,), generator=g).tolist()
        ref = reference_logits(ref_dir, cfg, w, tokens)
        with torch.no_grad():
            mine = plain_gpt.forward(cfg, w, tokens)
        diff = (ref - mine).abs().max().item()
        print(f"{name}: reference module vs plain implementation, {T} tokens: max abs diff {diff:.3e}")
        assert diff < 1e-5, diff
        rows = [0, T // 2, T - 1]
        np.savez(os.path.join(HERE, f"golden_{name}.npz"), tokens=np.asarray(tokens, dtype=np.int32),
                 rows=np.asarray(rows, dtype=np.int32), logits=ref[rows].numpy().astype(np.float32),
                 max_abs_diff_plain_vs_reference=np.float64(diff))


if __name__ == "__main__":
    main()
