"""Each part alone against the plain implementation's function for it (GPU)."""
import pytest
import torch

import plain_gpt

pytestmark = pytest.mark.gpu

W, H, F, V, P, T = 40, 2, 72, 31, 50, 23     # sizes of neither tiny configuration


def make_runner(dtype):
    from cbis_b200.cache import CachePool
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec
    from cbis_b200.engine import ModelRunner
    from cbis_b200.models import Model
    from cbis_b200.weights import InitScheme, random_tensors
    norm = PartSpec("layernorm", {"width": W, "eps": 1e-3})
    layer = LayerSpec("h.0.", "pre_norm",
                      PartSpec("attention", {"width": W, "n_head": H, "n_kv_head": H, "head_dim": W // H,
                                             "scale": (W // H) ** -0.5, "window": 0}),
                      PartSpec("dense", {"width": W, "inner": F, "activation": "gelu_tanh"}), norm, norm)
    spec = ModelSpec(W, V, P, "wte.weight", PartSpec("learned", {"width": W, "n_positions": P}), (layer,), (0,),
                     norm, "ln_f.", None)
    model = Model(spec)
    tensors = random_tensors(model.declared(), 3, InitScheme(0.2, 0.1, 0.2, 0.1), torch.float32)
    model.load(tensors, dtype, "cuda")
    pool = CachePool(model, page_size=4, num_pages=16, max_requests=2)
    return model, pool, ModelRunner(model, pool, max_batched_tokens=64, max_num_seqs=2), {k: v.double() for k, v in tensors.items()}


def whole_context(pool, runner, tokens):
    from cbis_b200.engine import StepEntry
    s = pool.manager.admit(0)
    assert pool.manager.append(s, len(tokens))
    return runner.build_context([StepEntry(s, 0, tokens, [len(tokens) - 1])])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    from cbis_b200.parts import Delta
    model, pool, runner, w = make_runner(dtype)
    if dtype == torch.bfloat16:                       # the plain side gets the weights as the engine holds them
        w = {k: (v.float().to(torch.bfloat16).double() if v.dim() == 2 else v) for k, v in w.items()}
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, V, (T,), generator=g).tolist()
    ctx = whole_context(pool, runner, tokens)
    layer = model.layers[0]

    def close(a, b, scale_tol=tol):
        return (a.double().cpu() - b).abs().max().item() < scale_tol * max(1.0, b.abs().max().item())

    # position encoding + token rows
    x = model.position.embed(ctx, model.token_table)
    x_ref = plain_gpt.embed(tokens, w["wte.weight"], w["wpe.weight"])
    assert x.dtype == torch.float32 and close(x, x_ref, 1e-6)
    # norm, with a pending delta and its bias folded in
    dv = torch.randn(T, W, generator=g)
    db = torch.randn(W, generator=g)
    x1 = x.clone()
    h = layer.norm_mixer.forward(ctx, x1, Delta(dv.cuda().to(dtype), db.cuda()))
    dv_seen = dv.to(dtype).double()
    xs = x_ref + dv_seen + db.double()
    assert h.dtype == dtype and close(x1, xs, 1e-6)
    assert close(h, plain_gpt.layer_norm(xs, w["h.0.ln_1.weight"], w["h.0.ln_1.bias"], 1e-3))
    # mixer
    hin = (torch.randn(T, W, generator=g)).to(dtype)
    d = layer.mixer.forward(ctx, hin.cuda(), ctx.layer_cache(0), None)
    ref = plain_gpt.attention(hin.double(), w["h.0.attn.c_attn.weight"], w["h.0.attn.c_attn.bias"],
                              w["h.0.attn.c_proj.weight"], w["h.0.attn.c_proj.bias"], H)
    assert d.value.dtype == torch.float32 and close(d.value + d.bias, ref)
    # feed-forward
    d = layer.feed_forward.forward(ctx, hin.cuda())
    ref = plain_gpt.mlp(hin.double(), w["h.0.mlp.c_fc.weight"], w["h.0.mlp.c_fc.bias"],
                        w["h.0.mlp.c_proj.weight"], w["h.0.mlp.c_proj.bias"], "gelu_new")
    assert close(d.value + d.bias, ref)
    # the arrangement: x and the pending output together are the block's result
    x2 = x.clone()
    pend = layer.block.forward(ctx, x2, None, ctx.layer_cache(0), None)
    ref = plain_gpt.block(x_ref, w, 0, H, 1e-3, "gelu_new")
    assert close(x2 + pend.value + pend.bias, ref)
    # final norm on chosen rows
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
    hf = model.final_norm.forward(ctx, x2, pend, rows=rows)
    ref_f = plain_gpt.layer_norm(ref, w["ln_f.weight"], w["ln_f.bias"], 1e-3)[[T - 1, 0]]
    assert hf.shape == (2, W) and close(hf, ref_f)


def test_unknown_part_kinds_are_named():
    from cbis_b200.config import PartSpec
    from cbis_b200.parts import make_mixer, make_norm
    with pytest.raises(KeyError, match="unknown mixer kind 'conv'.*attention"):
        make_mixer(PartSpec("conv", {}))
    with pytest.raises(KeyError, match="unknown norm kind 'rms'"):
        make_norm(PartSpec("rms", {}))
