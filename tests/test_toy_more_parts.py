"""More parts defined outside the framework and run without a change to its files (GPU): a norm whose
tensors have names of their own, an embedding with a multiplier, a head with bias, scale and soft cap, a
model without a final norm; a mixer that caches ONE array per token (no keys and values); a position
encoding that acts inside the mixers; and a mixer with state of its own that takes part in CUDA graphs."""
import math

import pytest
import torch

import plain_gpt

pytestmark = pytest.mark.gpu


def cut_and_compare(eng, toks, plain, sizes, tol=1e-4):
    """Runs ``toks`` through the step function in portions of ``sizes`` and compares every logit with ``plain``."""
    from cbis_b200.engine import StepEntry
    ref = plain(toks)
    slot = eng.open_request(0)
    got, pos, k = [], 0, 0
    while pos < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - pos)
        got.append(eng.forward_step([StepEntry(slot, pos, toks[pos:pos + n], list(range(n)))]).double().cpu())
        pos += n
        k += 1
    eng.close_request(slot)
    got = torch.cat(got)
    assert got.shape == ref.shape
    assert (got - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())


def test_norm_by_another_name_embedding_multiplier_head_with_bias_scale_cap_and_no_final_norm():
    import cbis_b200 as cb
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec
    from cbis_b200.models import Model
    from cbis_b200.parts import Norm, register_norm
    from cbis_b200.weights import InitScheme, TensorDecl, random_tensors

    class ScaleNorm(Norm):
        """y = x / rms(x) * scale: one tensor, called ``scale``, declared as a norm's weight."""
        def __init__(self, width, eps):
            self.width, self.eps = width, eps

        def tensors(self, prefix):
            return [TensorDecl(prefix + "scale", (self.width,), "norm_weight")]

        def load(self, prefix, tensors, dtype, device):
            self.scale = tensors[prefix + "scale"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, x, delta, rows=None, out_dtype=None):
            if delta is not None and rows is None:
                x += delta.value.float() + (delta.bias if delta.bias is not None else 0.0)
                v = x
            else:
                v = x[rows.long()] if rows is not None else x
                if delta is not None:
                    v = v + delta.value.float()[rows.long()] + (delta.bias if delta.bias is not None else 0.0)
            y = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + self.eps) * self.scale
            return y.to(out_dtype or ctx.dtype)

    register_norm("scale_norm_test", ScaleNorm)
    W, V, P, H = 48, 53, 40, 3
    norm = PartSpec("scale_norm_test", {"width": W, "eps": 1e-4})
    att = PartSpec("attention", {"width": W, "n_head": H, "n_kv_head": H, "head_dim": 16, "scale": 0.25, "window": 0})
    ffn = PartSpec("dense", {"width": W, "inner": 80, "activation": "gelu_erf"})
    layers = tuple(LayerSpec(f"blk.{i}.", "pre_norm", att, ffn, norm, norm, norm_prefixes=("rms_a.", "rms_b."))
                   for i in range(2))
    spec = ModelSpec(W, V, P,
                     PartSpec("token_table", {"vocab_size": V, "width": W, "tensor": "emb.table", "multiplier": 3.0}),
                     PartSpec("learned", {"width": W, "n_positions": P, "tensor": "emb.positions"}), layers, (0, 1),
                     PartSpec("none", {"width": W}), "unused.",
                     PartSpec("linear", {"vocab_size": V, "width": W, "tensor": "out.weight", "bias": "out.bias",
                                         "logit_scale": 0.5, "soft_cap": 2.0}))
    model = Model(spec)
    names = {d.name: d.role for d in model.declared()}
    assert names["blk.0.rms_a.scale"] == "norm_weight" and names["out.bias"] == "vector" and "emb.table" in names
    assert not any(n.startswith("unused.") for n in names)            # no final norm, no tensors for one
    tensors = random_tensors(model.declared(), 8, InitScheme(0.2, 0.3, 0.1, 0.1), torch.float32)
    assert abs(tensors["blk.1.rms_b.scale"].mean().item() - 1.0) < 0.1   # drawn around 1 by its role, not its name
    model.load(tensors, "float32", "cuda")
    eng = cb.Engine(model, dtype="float32", page_size=4, num_pages=16, max_num_seqs=2, max_batched_tokens=64)
    w = {k: v.double() for k, v in tensors.items()}

    def plain(tokens):
        x = 3.0 * w["emb.table"][tokens] + w["emb.positions"][:len(tokens)]
        rms = lambda v, s: v * torch.rsqrt((v * v).mean(-1, keepdim=True) + 1e-4) * s
        for i in range(2):
            p = f"blk.{i}."
            x = x + plain_gpt.attention(rms(x, w[p + "rms_a.scale"]), w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"],
                                        w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"], H)
            x = x + plain_gpt.mlp(rms(x, w[p + "rms_b.scale"]), w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"],
                                  w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"], "gelu")
        return 2.0 * torch.tanh(0.5 * (x @ w["out.weight"].T + w["out.bias"]) / 2.0)

    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, V, (37,), generator=g).tolist()
    cut_and_compare(eng, toks, plain, [37])
    cut_and_compare(eng, toks, plain, [5, 2, 1, 1, 9, 1, 2])
    # bfloat16 runs the same parts through the bfloat16 kernels (the identity norm's cast, the head's bias and cap)
    model16 = Model(spec).load(tensors, "bfloat16", "cuda")
    eng16 = cb.Engine(model16, dtype="bfloat16", page_size=4, num_pages=16, max_num_seqs=2, max_batched_tokens=64)
    cut_and_compare(eng16, toks, plain, [11, 1, 1, 3], tol=5e-2)


def test_mixer_that_caches_one_array_per_token():
    """A mixer that keeps one compressed vector per token (one array of one head, 10 wide, not a key and a value)
    in pages of its own group, beside built-in attention with its own group; its output for the token at p is the
    mean of the cached vectors 0..p times a matrix.  Portions, single tokens, page edges, and a slot used again."""
    import cbis_b200 as cb
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec
    from cbis_b200.engine import StepEntry
    from cbis_b200.models import Model
    from cbis_b200.parts import CacheArray, CacheNeed, Delta, Mixer, register_mixer
    from cbis_b200.weights import InitScheme, TensorDecl, random_tensors

    class LatentMean(Mixer):
        capturable = False            # forward() reads the step's sizes and tables on the host

        def __init__(self, width, latent):
            self.width, self.latent = width, latent

        def cache_need(self):
            return CacheNeed((CacheArray("latent", 1, self.latent),))

        def tensors(self, prefix):
            return [TensorDecl(prefix + "down.weight", (self.width, self.latent)),
                    TensorDecl(prefix + "up.weight", (self.latent, self.width))]

        def load(self, prefix, tensors, dtype, device):
            self.down = tensors[prefix + "down.weight"].to(device=device, dtype=torch.float32)
            self.up = tensors[prefix + "up.weight"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, h, cache, state):
            pages = cache.arrays["latent"]                              # [num_pages, 1, page_size, latent]
            assert set(cache.arrays) == {"latent"} and pages.shape[1:] == (1, cache.page_size, self.latent)
            flat = pages.view(-1, self.latent)                          # token slot -> vector (one head)
            view = ctx.groups[cache.group]
            c = h.float() @ self.down
            flat[view.slot_mapping[:ctx.n_rows].long()] = c.to(flat.dtype)     # this step's tokens first
            out = torch.empty((ctx.n_rows, self.width), dtype=torch.float32, device=h.device)
            tables, r = view.block_table.tolist(), 0
            ps = cache.page_size
            for s, (n, length) in enumerate(zip(ctx.host_seg_rows, ctx.host_seg_ctx)):
                slots = torch.tensor([tables[s][p // ps] * ps + p % ps for p in range(length)], device=h.device)
                means = flat[slots].float().cumsum(0) / torch.arange(1, length + 1, device=h.device)[:, None]
                out[r:r + n] = means[length - n:] @ self.up
                r += n
            return Delta(out)

    register_mixer("latent_mean_test", LatentMean)
    W, V, P = 32, 41, 64
    norm = PartSpec("layernorm", {"width": W, "eps": 1e-5})
    att = PartSpec("attention", {"width": W, "n_head": 2, "n_kv_head": 2, "head_dim": 16, "scale": 0.25, "window": 0})
    lat = PartSpec("latent_mean_test", {"width": W, "latent": 10})
    ffn = PartSpec("dense", {"width": W, "inner": 40, "activation": "gelu_tanh"})
    layers = (LayerSpec("h.0.", "pre_norm", lat, ffn, norm, norm), LayerSpec("h.1.", "pre_norm", att, ffn, norm, norm),
              LayerSpec("h.2.", "pre_norm", lat, ffn, norm, norm))
    spec = ModelSpec(W, V, P, "wte.weight", PartSpec("learned", {"width": W, "n_positions": P}), layers, (0, 1, 2),
                     norm, "ln_f.", None)
    model = Model(spec)
    tensors = random_tensors(model.declared(), 2, InitScheme(0.25, 0.1, 0.1, 0.1), torch.float32)
    model.load(tensors, "float32", "cuda")
    eng = cb.Engine(model, dtype="float32", page_size=4, num_pages=20, max_num_seqs=2, max_batched_tokens=64)
    groups = eng.pool.groups
    assert [g.layers for g in groups] == [[0, 2], [1]]                  # the two latent layers share a group
    assert [a.name for a in groups[0].need.arrays] == ["latent"] and groups[0].need.elements_per_token() == 10
    assert eng.pool.bytes_per_token() == (2 * 10 + 2 * 2 * 16) * 4
    w = {k: v.double() for k, v in tensors.items()}

    def plain(tokens):
        x = plain_gpt.embed(tokens, w["wte.weight"], w["wpe.weight"])
        T = len(tokens)
        for i in range(3):
            p = f"h.{i}."
            h = plain_gpt.layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], 1e-5)
            if i == 1:
                x = x + plain_gpt.attention(h, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"],
                                            w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"], 2)
            else:
                c = h @ w[p + "down.weight"]
                x = x + (c.cumsum(0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]) @ w[p + "up.weight"]
            x = x + plain_gpt.mlp(plain_gpt.layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], 1e-5),
                                  w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"], w[p + "mlp.c_proj.weight"],
                                  w[p + "mlp.c_proj.bias"], "gelu_new")
        return plain_gpt.layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], 1e-5) @ w["wte.weight"].T

    g = torch.Generator().manual_seed(4)
    a = torch.randint(0, V, (50,), generator=g).tolist()
    b = torch.randint(0, V, (21,), generator=g).tolist()
    cut_and_compare(eng, a, plain, [50])
    cut_and_compare(eng, a, plain, [7, 2, 1, 1, 13, 3, 1])
    # two requests side by side; b ends, its pages go to a third request
    sa, sb = eng.open_request(0), eng.open_request(1)
    eng.forward_step([StepEntry(sa, 0, a[:30], []), StepEntry(sb, 0, b, [])])
    eng.close_request(sb)
    sc = eng.open_request(2)
    lg = eng.forward_step([StepEntry(sa, 30, a[30:], list(range(20))), StepEntry(sc, 0, b[:9], list(range(9)))]).double().cpu()
    assert (lg[:20] - plain(a)[30:]).abs().max() < 1e-4 and (lg[20:] - plain(b[:9])).abs().max() < 1e-4
    eng.close_request(sa); eng.close_request(sc)
    assert eng.pool.manager.check() == "" and eng.pool.manager.free_pages(0) == 20 and eng.pool.manager.free_pages(1) == 20


class ToyRotary:
    """Rotates the pairs (i, i + hd/2) of every head of q and k by position * base^(-2i/hd)."""

    @staticmethod
    def rotate(x, positions, head_dim, base):
        T = x.shape[0]
        v = x.reshape(T, -1, head_dim)
        half = head_dim // 2
        i = torch.arange(half, device=x.device, dtype=torch.float64)
        ang = positions.to(torch.float64)[:, None] * torch.exp(-math.log(base) * 2 * i / head_dim)[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = v[..., :half].to(torch.float64), v[..., half:].to(torch.float64)
        return torch.cat([a * cos - b * sin, a * sin + b * cos], -1).reshape(T, -1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_encoding_that_acts_inside_the_mixers(dtype):
    """Nothing is added at the input; the built-in attention hands its queries and keys to the model's position
    encoding before the keys are cached.  Whole, in portions and token by token (decode steps replay a graph)."""
    import cbis_b200 as cb
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec
    from cbis_b200.kernels import ops
    from cbis_b200.models import Model
    from cbis_b200.parts import PositionEncoding, register_position
    from cbis_b200.weights import InitScheme, random_tensors

    class RotaryTest(PositionEncoding):
        acts_in_mixer = True

        def __init__(self, width, base):
            self.width, self.base = width, base

        def embed(self, ctx, token_table):
            x = torch.empty((ctx.n_rows, self.width), dtype=torch.float32, device=token_table.device)
            ops.embed_pos_add(ctx.tokens, ctx.positions, token_table, None, x, ctx.error_flag)
            return x

        def apply_in_mixer(self, ctx, q, k, head_dim):
            for t in (q, k):
                if t is not None:
                    t.copy_(ToyRotary.rotate(t, ctx.positions[:t.shape[0]], head_dim, self.base).to(t.dtype))

    register_position("rotary_test", RotaryTest)
    W, V, P, H, HD = 64, 37, 80, 4, 16
    norm = PartSpec("layernorm", {"width": W, "eps": 1e-5})
    att = PartSpec("attention", {"width": W, "n_head": H, "n_kv_head": 2, "head_dim": HD, "scale": 0.25, "window": 0})
    ffn = PartSpec("dense", {"width": W, "inner": 96, "activation": "gelu_erf"})
    layers = tuple(LayerSpec(f"h.{i}.", "pre_norm", att, ffn, norm, norm) for i in range(2))
    spec = ModelSpec(W, V, P, "wte.weight", PartSpec("rotary_test", {"width": W, "base": 100.0}), layers, (0, 1), norm,
                     "ln_f.", None)
    model = Model(spec)
    tensors = random_tensors(model.declared(), 6, InitScheme(0.2, 0.1, 0.1, 0.1), torch.float32)
    if dtype == "bfloat16":
        tensors = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in tensors.items()}
    model.load(tensors, dtype, "cuda")
    eng = cb.Engine(model, dtype=dtype, page_size=8, num_pages=24, max_num_seqs=2, max_batched_tokens=96)
    w = {k: v.double() for k, v in tensors.items()}

    def plain(tokens):
        T = len(tokens)
        x = w["wte.weight"][tokens]
        pos = torch.arange(T)
        for i in range(2):
            p = f"h.{i}."
            h = plain_gpt.layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], 1e-5)
            qkv = h @ w[p + "attn.c_attn.weight"] + w[p + "attn.c_attn.bias"]
            q = ToyRotary.rotate(qkv[:, :W], pos, HD, 100.0).reshape(T, H, HD)
            k = ToyRotary.rotate(qkv[:, W:W + 2 * HD], pos, HD, 100.0).reshape(T, 2, HD)
            v = qkv[:, W + 2 * HD:].reshape(T, 2, HD)
            outs = []
            for hh in range(H):                                        # two query heads share a key/value head
                sc = (q[:, hh] @ k[:, hh // 2].T) * 0.25
                sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
                outs.append(torch.softmax(sc, -1) @ v[:, hh // 2])
            x = x + torch.cat(outs, 1) @ w[p + "attn.c_proj.weight"] + w[p + "attn.c_proj.bias"]
            x = x + plain_gpt.mlp(plain_gpt.layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], 1e-5),
                                  w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"], w[p + "mlp.c_proj.weight"],
                                  w[p + "mlp.c_proj.bias"], "gelu")
        return plain_gpt.layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], 1e-5) @ w["wte.weight"].T

    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, V, (70,), generator=g).tolist()
    tol = 1e-4 if dtype == "float32" else 4e-2
    cut_and_compare(eng, toks, plain, [70], tol)
    cut_and_compare(eng, toks, plain, [33, 2, 1, 1, 1, 1, 17, 1, 1, 1], tol)
    if eng.runner.use_graphs:
        assert eng.runner.graph_replays >= 4                           # the single tokens went through a captured step


def test_mixer_with_state_of_its_own_inside_captured_steps():
    """A mixer that keeps a running sum per request in its state slot, written with device operations only, so
    its steps are captured as CUDA graphs like any other.  The step during which a graph is captured must move
    the state on ONCE: a run that crosses captures of decode buckets and of a repeated step shape gives the
    logits of a run without graphs, and of the plain restatement."""
    import cbis_b200 as cb
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec
    from cbis_b200.engine import StepEntry
    from cbis_b200.models import Model
    from cbis_b200.parts import Delta, Mixer, StateNeed, register_mixer
    from cbis_b200.weights import InitScheme, TensorDecl, random_tensors

    class RunningSum(Mixer):
        """state <- state + h_t; out_t = state @ W.  No host reads: capturable."""

        def __init__(self, width):
            self.width = width

        def state_need(self):
            return StateNeed((self.width,), torch.float32)

        def tensors(self, prefix):
            return [TensorDecl(prefix + "mix.weight", (self.width, self.width))]

        def load(self, prefix, tensors, dtype, device):
            self.w = tensors[prefix + "mix.weight"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, h, cache, state):
            T, S = ctx.n_rows, ctx.n_segments
            hf = h.float()
            seg = ctx.row_seq[:T].long()
            valid = (seg >= 0)[:, None]
            hf = hf * valid                                              # padding rows carry nothing
            seg = seg.clamp(min=0)
            cs0 = torch.cat([torch.zeros_like(hf[:1]), hf.cumsum(0)])    # cs0[i]: sum of the rows before i
            cu = ctx.cu_rows[:S + 1].long()
            rows = torch.arange(T, device=h.device)
            inside = cs0[rows + 1] - cs0[cu[seg]]                        # sum over the segment up to and with this row
            slot = ctx.seg_slot[:S].long()
            out = (state[slot[seg]] + inside) @ self.w
            state.index_add_(0, slot, cs0[cu[1:]] - cs0[cu[:-1]])        # empty (padding) segments add nothing
            return Delta(out * valid)

    register_mixer("running_sum_test", RunningSum)
    W, V, P = 24, 33, 64
    norm = PartSpec("layernorm", {"width": W, "eps": 1e-5})
    mix = PartSpec("running_sum_test", {"width": W})
    att = PartSpec("attention", {"width": W, "n_head": 2, "n_kv_head": 2, "head_dim": 12, "scale": 12 ** -0.5, "window": 0})
    ffn = PartSpec("dense", {"width": W, "inner": 40, "activation": "gelu_erf"})
    layers = (LayerSpec("h.0.", "pre_norm", mix, ffn, norm, norm), LayerSpec("h.1.", "pre_norm", att, ffn, norm, norm))
    spec = ModelSpec(W, V, P, "wte.weight", PartSpec("learned", {"width": W, "n_positions": P}), layers, (0, 1), norm,
                     "ln_f.", None)
    tensors = random_tensors(Model(spec).declared(), 9, InitScheme(0.1, 0.05, 0.1, 0.1), torch.float32)
    w = {k: v.double() for k, v in tensors.items()}

    def plain(tokens):
        x = plain_gpt.embed(tokens, w["wte.weight"], w["wpe.weight"])
        for i in range(2):
            p = f"h.{i}."
            h = plain_gpt.layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], 1e-5)
            if i == 0:
                x = x + h.cumsum(0) @ w[p + "mix.weight"]
            else:
                x = x + plain_gpt.attention(h, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"],
                                            w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"], 2)
            x = x + plain_gpt.mlp(plain_gpt.layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], 1e-5),
                                  w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"], w[p + "mlp.c_proj.weight"],
                                  w[p + "mlp.c_proj.bias"], "gelu")
        return plain_gpt.layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], 1e-5) @ w["wte.weight"].T

    g = torch.Generator().manual_seed(5)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (40, 36, 30)]

    def run(use_graphs):
        model = Model(spec).load(tensors, "float32", "cuda")
        eng = cb.Engine(model, dtype="float32", page_size=4, num_pages=40, max_num_seqs=4, max_batched_tokens=64)
        assert eng.runner.use_graphs                                     # every part is capturable
        eng.runner.use_graphs = use_graphs
        eng.runner.shape_graph_after, eng.runner.shape_graph_min_host_s = 2, 0.0
        slots = [eng.open_request(i) for i in range(3)]
        fed = [0, 0, 0]
        got = [[], [], []]

        def step(parts):                                                 # parts: {request: n tokens}
            entries = [StepEntry(slots[r], fed[r], seqs[r][fed[r]:fed[r] + n], list(range(n))) for r, n in parts.items()]
            lg = eng.forward_step(entries).double().cpu()
            at = 0
            for r, n in parts.items():
                got[r].append(lg[at:at + n]); at += n; fed[r] += n

        for _ in range(4):
            step({0: 6})                                                 # one shape four times: launch by launch, captured, replayed
        for _ in range(3):
            step({0: 1})                                                 # decode bucket 1: captured at its first step
        step({1: 9})
        for _ in range(3):
            step({0: 1, 1: 1})                                           # bucket 2
        step({2: 5})
        for _ in range(4):
            step({0: 1, 1: 1, 2: 1})                                     # bucket 4, one padding row
        return [torch.cat(x) for x in got], eng.runner.graph_replays, eng.runner.shape_captures

    plain_run, n0, c0 = run(False)
    graph_run, n1, c1 = run(True)
    assert n0 == 0 and c0 == 0 and n1 >= 7 and c1 == 1
    for r in range(3):
        ref = plain(seqs[r][:len(graph_run[r])])
        assert (plain_run[r] - ref).abs().max().item() < 1e-4
        assert (graph_run[r] - ref).abs().max().item() < 1e-4, f"request {r}: a captured step moved the state on twice?"
