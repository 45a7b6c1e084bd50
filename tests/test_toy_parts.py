"""Parts defined here, outside the framework, can be registered, built and stepped without any change
to the framework's files (GPU): a mixer with fixed-size state of its own (no pages), mixed in one
model with the built-in attention; a layer that reads another layer's cache and is named twice in the
schedule (it writes nothing, so running it twice is well defined under any cut)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def register_toy():
    import cbis_b200 as cb
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec
    from cbis_b200.parts import Delta, Mixer, StateNeed, register_mixer
    from cbis_b200.weights import TensorDecl

    class DecayingSum(Mixer):
        """state <- decay * state + h_t ; out_t = state @ W.  The state lives in the request's slot."""
        capturable = False        # forward() reads the slots on the host

        def __init__(self, width, decay):
            self.width, self.decay = width, decay
            self.w = None

        def state_need(self):
            return StateNeed((self.width,), torch.float32)

        def tensors(self, prefix):
            return [TensorDecl(prefix + "mix.weight", (self.width, self.width))]

        def load(self, prefix, tensors, dtype, device):
            self.w = tensors[prefix + "mix.weight"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, h, cache, state):
            assert cache is None and state is not None
            out = torch.empty((ctx.n_rows, self.width), dtype=torch.float32, device=h.device)
            slots = ctx.seg_slot.tolist()
            r = 0
            for s, n in enumerate(ctx.host_seg_rows):          # tokens of a request in order; the slot carries the state
                st = state[slots[s]]
                for i in range(n):
                    st.mul_(self.decay).add_(h[r + i].float())
                    out[r + i] = st @ self.w
                r += n
            return Delta(out)

    register_mixer("decaying_sum", DecayingSum)

    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return self.d

        def model_spec(self):
            w, v, p = self.d["width"], self.d["vocab"], self.d["positions"]
            norm = PartSpec("layernorm", {"width": w, "eps": 1e-5})
            att = PartSpec("attention", {"width": w, "n_head": 2, "n_kv_head": 1, "head_dim": w // 2,
                                         "scale": (w // 2) ** -0.5, "window": self.d.get("window", 0)})
            toy = PartSpec("decaying_sum", {"width": w, "decay": self.d["decay"]})
            ffn = PartSpec("dense", {"width": w, "inner": 3 * w, "activation": "gelu_erf"})
            layers = (LayerSpec("h.0.", "pre_norm", att, ffn, norm, norm),
                      LayerSpec("h.1.", "pre_norm", toy, ffn, norm, norm),
                      LayerSpec("h.2.", "pre_norm", att, ffn, norm, norm, cache_source=0))
            return ModelSpec(w, v, p, "wte.weight", PartSpec("learned", {"width": w, "n_positions": p}), layers,
                             (0, 1, 2, 2), norm, "ln_f.", None)

    cb.register_architecture("ToyStateModel", ToyConfig)
    return ToyConfig


def plain_toy_forward(w, cfg, tokens):
    """The same model by the plain functions, whole sequence (float64)."""
    import plain_gpt
    d = cfg["width"]
    x = plain_gpt.embed(tokens, w["wte.weight"], w["wpe.weight"])
    ln = lambda x, p: plain_gpt.layer_norm(x, w[p + "weight"], w[p + "bias"], 1e-5)
    ffn = lambda h, p: plain_gpt.mlp(h, w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"], w[p + "mlp.c_proj.weight"],
                                     w[p + "mlp.c_proj.bias"], "gelu")
    hd = d // 2

    def kv_of(h):
        qkv = h @ w["h.0.attn.c_attn.weight"] + w["h.0.attn.c_attn.bias"]
        return qkv[:, d:d + hd], qkv[:, d + hd:]

    def attend(q, k, v, wo, bo):
        T = q.shape[0]
        outs = []
        for hh in range(2):                                   # two query heads share one key/value head
            sc = (q[:, hh * hd:(hh + 1) * hd] @ k.T) * hd ** -0.5
            win = cfg.get("window", 0)
            i = torch.arange(T)
            mask = (i[None, :] > i[:, None]) | ((i[:, None] - i[None, :] >= win) if win else False)
            outs.append(torch.softmax(sc.masked_fill(mask, float("-inf")), -1) @ v)
        return torch.cat(outs, 1) @ wo + bo

    state = {1: torch.zeros(d, dtype=torch.float64)}
    k0 = v0 = None
    for li in (0, 1, 2, 2):
        p = f"h.{li}."
        h = ln(x, p + "ln_1.")
        if li == 0:
            qkv = h @ w[p + "attn.c_attn.weight"] + w[p + "attn.c_attn.bias"]
            k0, v0 = kv_of(h)
            x = x + attend(qkv[:, :d], k0, v0, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])
        elif li == 2:
            q = h @ w[p + "attn.c_attn.weight"] + w[p + "attn.c_attn.bias"]
            x = x + attend(q, k0, v0, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])
        else:
            out = torch.empty_like(h)
            st = state[1]
            for t in range(h.shape[0]):
                st = cfg["decay"] * st + h[t]
                out[t] = st @ w[p + "mix.weight"]
            state[1] = st
            x = x + out
        x = x + ffn(ln(x, p + "ln_2."), p)
    return ln(x, "ln_f.") @ w["wte.weight"].T


@pytest.mark.parametrize("window", [0, 6])
def test_toy_mixer_with_state_builds_and_steps(window):
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    from cbis_b200.models import Model
    from cbis_b200.weights import InitScheme, random_tensors
    register_toy()
    cfgd = {"architectures": ["ToyStateModel"], "width": 24, "vocab": 40, "positions": 48, "decay": 0.9,
            "window": window}
    config = cb.config_from_dict(cfgd)
    model = Model(config.model_spec())
    tensors = random_tensors(model.declared(), 1, InitScheme(0.15, 0.05, 0.1, 0.1), torch.float32)
    model.load(tensors, "float32", "cuda")
    eng = cb.Engine(model, dtype="float32", page_size=4, num_pages=16 if window == 0 else 10, max_num_seqs=3,
                    max_batched_tokens=64)
    assert set(eng.pool.state) == {1} and eng.pool.state[1].shape == (3, 24)
    assert len(eng.pool.groups) == 1 and eng.pool.groups[0].layers == [0] and eng.pool.groups[0].need.arrays[0].heads == 1
    w = {k: v.double() for k, v in tensors.items()}
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, 40, (40,), generator=g).tolist()
    b = torch.randint(0, 40, (17,), generator=g).tolist()
    ref_a, ref_b = plain_toy_forward(w, cfgd, a), plain_toy_forward(w, cfgd, b)
    # a in portions, b beside it from the third step on, then both token by token
    sa, sb = eng.open_request(0), eng.open_request(1)
    got_a, got_b = [], []
    cuts = [(7, 0), (2, 0), (9, 5), (2, 2), (1, 1), (1, 1), (5, 2), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (8, 1)]
    pa = pb = 0
    for na, nb in cuts:
        entries = []
        if na and pa < len(a):
            na = min(na, len(a) - pa)
            entries.append(StepEntry(sa, pa, a[pa:pa + na], list(range(na))))
        if nb and pb < len(b):
            nb = min(nb, len(b) - pb)
            entries.append(StepEntry(sb, pb, b[pb:pb + nb], list(range(nb))))
        lg = eng.forward_step(entries).double().cpu()
        if na and pa < len(a):
            got_a.append(lg[:na]); lg = lg[na:]; pa += na
        if nb and pb < len(b):
            got_b.append(lg[:nb]); pb += nb
    got_a, got_b = torch.cat(got_a), torch.cat(got_b)
    assert (got_a - ref_a[:len(got_a)]).abs().max() < 1e-4
    assert (got_b - ref_b[:len(got_b)]).abs().max() < 1e-4
    assert len(got_a) == 40 and len(got_b) == 17
    # a new request in b's slot starts from a zero state
    eng.close_request(sb)
    sc = eng.open_request(2)
    assert sc == sb
    lg = eng.forward_step([StepEntry(sc, 0, b, list(range(len(b))))]).double().cpu()
    assert (lg - ref_b).abs().max() < 1e-4
    if window:
        assert eng.pool.manager.block_table(sa, 0)[0] == -1     # pages behind the window went back
    # and it generates through the scheduler
    eng.close_request(sa); eng.close_request(sc)
    out = eng.generate([a[:5], b[:3]], cb.SamplingParams(max_new_tokens=6))
    for prompt, o in zip((a[:5], b[:3]), out):
        seq = list(prompt)
        for t in o:
            assert t == int(plain_toy_forward(w, cfgd, seq)[-1].argmax())
            seq.append(t)


def test_toy_feed_forward_with_routing_and_another_position_encoding():
    """A feed-forward that routes every row to one of three small experts (router logits and choice in
    32-bit) and a position encoding computed from the position instead of looked up, both defined here
    and registered without touching the framework; the built-in attention runs between them."""
    import math

    import cbis_b200 as cb
    import plain_gpt
    from cbis_b200.config import LayerSpec, ModelSpec, PartSpec
    from cbis_b200.engine import StepEntry
    from cbis_b200.kernels import ops
    from cbis_b200.models import Model
    from cbis_b200.parts import Delta, FeedForward, PositionEncoding, register_feed_forward, register_position
    from cbis_b200.weights import InitScheme, TensorDecl, random_tensors

    class RoutedExperts(FeedForward):
        capturable = False          # nonzero() below makes the host wait for the device

        def __init__(self, width, inner, n_experts):
            self.width, self.inner, self.n = width, inner, n_experts

        def tensors(self, prefix):
            out = [TensorDecl(prefix + "router.weight", (self.width, self.n))]
            for e in range(self.n):
                out += [TensorDecl(f"{prefix}experts.{e}.up.weight", (self.width, self.inner)),
                        TensorDecl(f"{prefix}experts.{e}.down.weight", (self.inner, self.width))]
            return out

        def load(self, prefix, tensors, dtype, device):
            f = lambda name: tensors[prefix + name].to(device=device, dtype=torch.float32)
            self.router = f("router.weight")
            self.up = [f(f"experts.{e}.up.weight") for e in range(self.n)]
            self.down = [f(f"experts.{e}.down.weight") for e in range(self.n)]

        def forward(self, ctx, h):
            h = h.float()
            choice = (h @ self.router).argmax(-1)                   # routing decided on the device, per row
            out = torch.zeros_like(h)
            for e in range(self.n):
                rows = (choice == e).nonzero().squeeze(-1)          # a step-local index tensor
                if rows.numel():
                    out.index_add_(0, rows, torch.relu(h[rows] @ self.up[e]) @ self.down[e])
            return Delta(out)

    class SinusoidalPositions(PositionEncoding):
        def __init__(self, width, base):
            self.width, self.base = width, base

        def embed(self, ctx, token_table):
            x = torch.empty((ctx.n_rows, self.width), dtype=torch.float32, device=token_table.device)
            ops.embed_pos_add(ctx.tokens, ctx.positions, token_table, None, x, ctx.error_flag)   # token rows only
            i = torch.arange(self.width // 2, device=x.device, dtype=torch.float32)
            ang = ctx.positions.float()[:, None] * torch.exp(-math.log(self.base) * 2 * i / self.width)[None, :]
            return x + torch.cat([ang.sin(), ang.cos()], 1)

    register_feed_forward("routed_test", RoutedExperts)
    register_position("sinusoidal_test", SinusoidalPositions)
    W, V, P = 32, 29, 40
    norm = PartSpec("layernorm", {"width": W, "eps": 1e-5})
    att = PartSpec("attention", {"width": W, "n_head": 2, "n_kv_head": 2, "head_dim": 16, "scale": 0.25, "window": 0})
    layers = (LayerSpec("h.0.", "pre_norm", att, PartSpec("routed_test", {"width": W, "inner": 20, "n_experts": 3}), norm, norm),
              LayerSpec("h.1.", "pre_norm", att, PartSpec("dense", {"width": W, "inner": 48, "activation": "gelu_tanh"}), norm, norm))
    spec = ModelSpec(W, V, P, "wte.weight", PartSpec("sinusoidal_test", {"width": W, "base": 50.0}), layers, (0, 1),
                     norm, "ln_f.", None)
    model = Model(spec)
    tensors = random_tensors(model.declared(), 4, InitScheme(0.3, 0.1, 0.1, 0.1), torch.float32)
    model.load(tensors, "float32", "cuda")
    eng = cb.Engine(model, dtype="float32", page_size=4, num_pages=24, max_num_seqs=2, max_batched_tokens=64)
    w = {k: v.double() for k, v in tensors.items()}

    def plain(tokens):
        T = len(tokens)
        i = torch.arange(W // 2, dtype=torch.float64)
        ang = torch.arange(T, dtype=torch.float64)[:, None] * torch.exp(-math.log(50.0) * 2 * i / W)[None, :]
        x = w["wte.weight"][tokens] + torch.cat([ang.sin(), ang.cos()], 1)
        for li in (0, 1):
            p = f"h.{li}."
            ln = lambda x, q: plain_gpt.layer_norm(x, w[p + q + "weight"], w[p + q + "bias"], 1e-5)
            x = x + plain_gpt.attention(ln(x, "ln_1."), w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"],
                                        w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"], 2)
            h = ln(x, "ln_2.")
            if li == 0:
                choice = (h @ w[p + "router.weight"]).argmax(-1)
                f = torch.stack([torch.relu(h[t] @ w[f"{p}experts.{int(choice[t])}.up.weight"])
                                 @ w[f"{p}experts.{int(choice[t])}.down.weight"] for t in range(T)])
                assert len(set(choice.tolist())) > 1                # the rows really go to different experts
            else:
                f = plain_gpt.mlp(h, w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"], w[p + "mlp.c_proj.weight"],
                                  w[p + "mlp.c_proj.bias"], "gelu_new")
            x = x + f
        return plain_gpt.layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], 1e-5) @ w["wte.weight"].T

    g = torch.Generator().manual_seed(6)
    toks = torch.randint(0, V, (37,), generator=g).tolist()
    ref = plain(toks)
    slot = eng.open_request(0)
    got, pos = [], 0
    for n in (9, 2, 1, 1, 13, 2, 1, 1, 1, 6):                       # portions and single tokens
        got.append(eng.forward_step([StepEntry(slot, pos, toks[pos:pos + n], list(range(n)))]).double().cpu())
        pos += n
    assert pos == len(toks) and (torch.cat(got) - ref).abs().max() < 1e-4
