"""Each CUDA kernel alone against a plain torch reference, at sizes other than the engine's (GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_gpt

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from cbis_b200.kernels import ops as o
    return o


def dev(t):
    return t.cuda().contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [7, 100, 1032])
def test_embed_pos_add(ops, dtype, d):
    g = torch.Generator().manual_seed(d)
    V, P, T = 53, 19, 37
    wte, wpe = torch.randn(V, d, generator=g).to(dtype), torch.randn(P, d, generator=g).to(dtype)
    tok, pos = torch.randint(0, V, (T,), generator=g).int(), torch.randint(0, P, (T,), generator=g).int()
    out = torch.full((T, d), float("nan"), device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed_pos_add(dev(tok), dev(pos), dev(wte), dev(wpe), out, err)
    ref = wte.float()[tok.long()] + wpe.float()[pos.long()]
    assert torch.equal(out.cpu(), ref) and err.item() == 0
    ops.embed_pos_add(dev(tok), dev(pos), dev(wte), None, out, err)
    assert torch.equal(out.cpu(), wte.float()[tok.long()])
    tok[5] = V
    ops.embed_pos_add(dev(tok), dev(pos), dev(wte), dev(wpe), out, err)
    assert err.item() == 1 and torch.equal(out[5].cpu(), torch.zeros(d))
    err.zero_(); tok[5] = 0; pos[3] = P
    ops.embed_pos_add(dev(tok), dev(pos), dev(wte), dev(wpe), out, err)
    assert err.item() == 2


@pytest.mark.parametrize("d", [5, 96, 1000, 2500, 20000])
@pytest.mark.parametrize("delta_dtype,out_dtype", [(None, torch.float32), (torch.float32, torch.float32),
                                                    (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16)])
def test_add_layernorm(ops, d, delta_dtype, out_dtype):
    g = torch.Generator().manual_seed(d)
    T, eps = 9, 3e-6
    x = torch.randn(T, d, generator=g) * 3 + 1.5
    delta = (torch.randn(T, d, generator=g)).to(delta_dtype) if delta_dtype else None
    bias = torch.randn(d, generator=g) if delta_dtype else None
    gamma, beta = torch.randn(d, generator=g), torch.randn(d, generator=g)
    xs = x.double() + (delta.double() + bias.double() if delta is not None else 0)
    ref = plain_gpt.layer_norm(xs, gamma.double(), beta.double(), eps)
    xd = dev(x)
    out = torch.empty(T, d, dtype=out_dtype, device="cuda")
    ops.add_layernorm(xd, dev(delta) if delta is not None else None, dev(bias) if bias is not None else None,
                      dev(gamma), dev(beta), eps, out)
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    assert (out.double().cpu() - ref).abs().max() < tol * max(1.0, ref.abs().max().item())
    assert (xd.double().cpu() - xs).abs().max() < 1e-6 * 20          # the residual stream moved on, in 32-bit
    # row selection: only the chosen rows, x untouched
    rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32)
    xd2 = dev(x)
    out2 = torch.empty(4, d, dtype=out_dtype, device="cuda")
    ops.add_layernorm(xd2, dev(delta) if delta is not None else None, dev(bias) if bias is not None else None,
                      dev(gamma), dev(beta), eps, out2, dev(rows))
    assert torch.equal(out2.cpu(), out.cpu()[rows.long()]) and torch.equal(xd2.cpu(), x)


def test_add_layernorm_refuses_a_width_it_cannot_stage(ops):
    x = torch.zeros(1, 60000, device="cuda")
    with pytest.raises(ops.KernelError, match="too large"):
        ops.add_layernorm(x, None, None, x[0], x[0], 1e-5, torch.empty_like(x))


def test_layernorm_of_large_offsets_is_centred(ops):
    # E[x^2]-mean^2 (the reference's form, kernels/elementwise.cu:50) loses the variance here; the centred form does not
    d = 512
    x = (torch.randn(3, d) * 0.01 + 300.0)
    ones, zeros = torch.ones(d), torch.zeros(d)
    out = torch.empty(3, d, device="cuda")
    ops.add_layernorm(dev(x), None, None, dev(ones), dev(zeros), 1e-8, out)
    ref = plain_gpt.layer_norm(x.double(), ones.double(), zeros.double(), 1e-8)
    assert (out.double().cpu() - ref).abs().max() < 5e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act,name", [("gelu_erf", "gelu"), ("gelu_tanh", "gelu_new"), (None, None)])
def test_bias_act(ops, dtype, act, name):
    g = torch.Generator().manual_seed(3)
    M, N = 13, 301
    x = (torch.randn(M, N, generator=g) * 2).to(dtype)
    b = torch.randn(N, generator=g)
    xd = dev(x)
    ops.bias_act(xd, dev(b), act)
    v = x.double() + b.double()
    ref = plain_gpt.gelu(v, name) if name else v
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert (xd.double().cpu() - ref).abs().max() < tol * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M", [1, 5, 17, 70, 300])
@pytest.mark.parametrize("N,K", [(33, 5), (100, 64), (513, 300), (64, 1030)])
def test_linear_f32(ops, M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + N)
    x, w, b = torch.randn(M, K, generator=g), torch.randn(K, N, generator=g), torch.randn(N, generator=g)
    ref = x.double() @ w.double() + b.double()
    scale = ref.abs().max().item()
    out = torch.empty(M, N, device="cuda")
    ops.linear_f32(dev(x), dev(w), dev(b), None, out)
    assert (out.double().cpu() - ref).abs().max() < 2e-6 * scale * math.sqrt(K)
    ops.linear_f32(dev(x), dev(w.t()), None, "gelu_erf", out, w_is_nk=True)
    ref2 = plain_gpt.gelu(x.double() @ w.double(), "gelu")
    assert (out.double().cpu() - ref2).abs().max() < 2e-6 * scale * math.sqrt(K)
    # a strided input (columns of a wider matrix) and a strided output
    wide = torch.randn(M, K + 11, generator=g)
    big = torch.zeros(M, N + 5, device="cuda")
    ops.linear_f32(dev(wide)[:, 3:3 + K], dev(w), None, None, big[:, :N])
    assert (big[:, :N].double().cpu() - wide[:, 3:3 + K].double() @ w.double()).abs().max() < 2e-6 * scale * math.sqrt(K)
    assert torch.equal(big[:, N:].cpu(), torch.zeros(M, 5))


@pytest.mark.parametrize("M,N,K", [(512, 256, 1024), (70, 100, 64), (300, 513, 300), (33, 40, 36), (2048, 768, 256), (17, 1000, 8),
                                   (2000, 2500, 68)])
def test_linear_f32_kernels_give_the_same_bits(ops, M, N, K):
    """Every 32-bit product kernel sums along k in the same order: the cp.async kernel (its three tile sizes), the older
    tiled kernels and the few-rows kernel agree bit for bit, so a token's logits do not depend on which step shape
    (and therefore which kernel) computed them."""
    g = torch.Generator().manual_seed(M + N + K)
    x, w, b = dev(torch.randn(M, K, generator=g)), dev(torch.randn(N, K, generator=g)), dev(torch.randn(N, generator=g))
    new, old = torch.full((M, N), float("nan"), device="cuda"), torch.full((M, N), float("nan"), device="cuda")
    ops.linear_f32(x, w, b, "gelu_erf", new, w_is_nk=True)
    ops.linear_f32(x, w, b, "gelu_erf", old, w_is_nk=True, variant=1)
    assert torch.equal(new, old)
    lo = min(5, M - 16)
    few = torch.empty(16, N, device="cuda")
    ops.linear_f32(x[lo:lo + 16], w, b, "gelu_erf", few, w_is_nk=True)    # 16 rows: the few-rows kernel
    assert torch.equal(few, new[lo:lo + 16])
    ref = plain_gpt.gelu(x.double() @ w.double().t() + b.double(), "gelu")
    assert (new.double() - ref).abs().max().item() < 2e-6 * max(1.0, ref.abs().max().item()) * math.sqrt(K)


def test_linear_f32_is_true_32_bit(ops):
    # a product that TF32 (10-bit mantissa) would get wrong by ~1e-3 relative
    g = torch.Generator().manual_seed(1)
    x, w = 1.0 + torch.rand(64, 256, generator=g) * 1e-3, 1.0 + torch.rand(256, 64, generator=g) * 1e-3
    out = torch.empty(64, 64, device="cuda")
    ops.linear_f32(dev(x), dev(w), None, None, out)
    ref = x.double() @ w.double()
    assert ((out.double().cpu() - ref).abs() / ref).max() < 1e-6


def naive_paged_attention(q, k_all, v_all, positions, row_seq, n_head, n_kv_head, hd, scale, window):
    """q [T, H*hd]; k_all/v_all: per segment the full key/value rows [ctx, Hkv*hd] (float64)."""
    out = torch.zeros_like(q)
    for r in range(q.shape[0]):
        s, p = int(row_seq[r]), int(positions[r])
        lo = max(0, p - window + 1) if window else 0
        for h in range(n_head):
            hk = h // (n_head // n_kv_head)
            kk = k_all[s][lo:p + 1, hk * hd:(hk + 1) * hd]
            vv = v_all[s][lo:p + 1, hk * hd:(hk + 1) * hd]
            sc = (kk @ q[r, h * hd:(h + 1) * hd]) * scale
            out[r, h * hd:(h + 1) * hd] = torch.softmax(sc, 0) @ vv
    return out


def paged_case(ops, dtype, n_head, n_kv_head, hd, ps, window, seg_ctx, seg_rows, seed):
    """Random keys/values scattered over random pages by kv_write; queries for the last seg_rows of each segment."""
    g = torch.Generator().manual_seed(seed)
    S = len(seg_ctx)
    max_blocks = max(-(-c // ps) for c in seg_ctx) + 2
    num_pages = sum(-(-c // ps) for c in seg_ctx) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((S, max_blocks), -1, dtype=torch.int32)
    k_all, v_all = [], []
    kc = torch.full((num_pages, n_kv_head, ps, hd), float("nan")).to(dtype).cuda()
    vc = torch.full((num_pages, n_kv_head, ps, hd), float("nan")).to(dtype).cuda()
    dkv = n_kv_head * hd
    for s, c in enumerate(seg_ctx):
        nb = -(-c // ps)
        pages = [perm.pop() for _ in range(nb)]
        bt[s, :nb] = torch.tensor(pages, dtype=torch.int32)
        kv = torch.randn(c, 2 * dkv, generator=g).to(dtype)
        k_all.append(kv[:, :dkv].double()); v_all.append(kv[:, dkv:].double())
        slots = torch.tensor([pages[p // ps] * ps + p % ps for p in range(c)], dtype=torch.int32)
        ops.kv_write(dev(kv), 0, dkv, kc, vc, dev(slots), n_kv_head, hd, ps)
    positions = torch.tensor([p for c, n in zip(seg_ctx, seg_rows) for p in range(c - n, c)], dtype=torch.int32)
    row_seq = torch.tensor([s for s, n in enumerate(seg_rows) for _ in range(n)], dtype=torch.int32)
    q = torch.randn(len(positions), n_head * hd, generator=g).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    ref = naive_paged_attention(q.double(), k_all, v_all, positions, row_seq, n_head, n_kv_head, hd, scale, window)
    return dict(q=q, kc=kc, vc=vc, bt=bt, positions=positions, row_seq=row_seq, ref=ref, scale=scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_head,n_kv_head,hd,ps,window", [
    (3, 3, 24, 8, 0), (2, 2, 32, 16, 0), (6, 2, 80, 4, 0), (5, 5, 128, 16, 0), (2, 1, 256, 32, 0),
    (4, 4, 48, 8, 11), (1, 1, 16, 3, 5)])
def test_kv_write_and_generic_attention(ops, dtype, n_head, n_kv_head, hd, ps, window):
    seg_ctx, seg_rows = [1, 37, 70, 16, 129], [1, 1, 33, 16, 2]
    c = paged_case(ops, dtype, n_head, n_kv_head, hd, ps, window, seg_ctx, seg_rows, seed=hd + ps)
    out = torch.full_like(c["q"], float("nan")).cuda()
    ops.paged_attention_generic(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(c["row_seq"]), dev(c["positions"]),
                                out, n_head, n_kv_head, hd, ps, c["scale"], window)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - c["ref"]).abs().max() < tol * max(1.0, c["ref"].abs().max().item())
    if hd % 4 == 0:   # every row's keys cut into chunks over more warps, merged by the second kernel
        T = len(c["positions"])
        for n_chunks, chunk_keys in [(2, 128), (9, 16), (33, 4)]:
            partial = torch.full((T * n_head * n_chunks * (hd + 4),), float("nan"), device="cuda")
            cut = torch.full_like(c["q"], float("nan")).cuda()
            ops.paged_attention_generic(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(c["row_seq"]), dev(c["positions"]),
                                        cut, n_head, n_kv_head, hd, ps, c["scale"], window, (n_chunks, chunk_keys), partial)
            assert (cut.double().cpu() - c["ref"]).abs().max() < tol * max(1.0, c["ref"].abs().max().item())
        # a padding row (request -1) is left zero by both kernels
        seq = c["row_seq"].clone(); seq[0] = -1
        partial = torch.full((T * n_head * 2 * (hd + 4),), float("nan"), device="cuda")
        ops.paged_attention_generic(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(seq), dev(c["positions"]),
                                    cut, n_head, n_kv_head, hd, ps, c["scale"], window, (2, 128), partial)
        assert cut[0].abs().max().item() == 0 and not torch.isnan(cut.float()).any()
    assert ops.generic_key_chunks(512, 16, 2048, 128) == (1, 0) and ops.generic_key_chunks(1, 8, 32768, 30) == (1, 0)
    n, keys = ops.generic_key_chunks(1, 8, 32768, 32)
    assert n > 1 and (n - 1) * keys < 32768 <= n * keys and keys >= 256


def test_attention_refuses_sizes_it_does_not_take(ops):
    z = torch.zeros(1, 600, device="cuda")
    i = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="head_dim=300"):
        ops.paged_attention_generic(z, z, z, i, i[0], i[0], z, 2, 2, 300, 16, 1.0)
    with pytest.raises(ops.KernelError, match="not a multiple"):
        ops.paged_attention_generic(z, z, z, i, i[0], i[0], z, 3, 2, 32, 16, 1.0)


def test_a_far_key_among_hundreds_is_found(ops):
    # one key, far back and at the edge of a page, matches the query; every other score is small
    hd, ps, ctx = 64, 16, 700
    for far in (0, 15, 16, 463, 464, 699):
        g = torch.Generator().manual_seed(far)
        k = torch.randn(ctx, hd, generator=g) * 0.05
        v = torch.randn(ctx, hd, generator=g)
        q = torch.randn(1, hd, generator=g)
        k[far] = q[0] * 4.0
        pages = torch.randperm(44, generator=g)[:44].int()
        kc = torch.zeros(44, 1, ps, hd, device="cuda"); vc = torch.zeros_like(kc)
        slots = torch.tensor([int(pages[p // ps]) * ps + p % ps for p in range(ctx)], dtype=torch.int32)
        ops.kv_write(dev(torch.cat([k, v], 1)), 0, hd, kc, vc, dev(slots), 1, hd, ps)
        out = torch.empty(1, hd, device="cuda")
        ops.paged_attention_generic(dev(q), kc, vc, dev(pages[None, :]), dev(torch.zeros(1, dtype=torch.int32)),
                                    dev(torch.tensor([ctx - 1], dtype=torch.int32)), out, 1, 1, hd, ps, 1 / 8.0)
        p = torch.softmax((k.double() @ q[0].double()) / 8.0, 0)
        assert p[far] > 0.99
        assert (out.double().cpu()[0] - p @ v.double()).abs().max() < 1e-5


def test_sampling(ops):
    g = torch.Generator().manual_seed(0)
    R, V = 7, 50257
    logits = torch.randn(R, V, generator=g)
    logits[2, 400] = logits[2, 9000] = 50.0                   # a tie: the first wins
    logits[3, 0] = 60.0
    logits[4, V - 1] = 60.0
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), None, None, out)
    exp = logits.argmax(-1)
    exp[2] = 400
    assert out.cpu().tolist() == exp.tolist()
    from cbis_b200.sampling import request_key
    temps = torch.tensor([0.8, 0.0, 1.3, 0.5, 2.0, 0.05, 1.0])
    keys = torch.tensor([request_key(77, r, 5 + r) for r in range(R)], dtype=torch.int64)
    ops.sample(dev(logits), dev(temps), dev(keys), out)
    for r in range(R):
        scores = plain_gpt.perturbed_scores(logits[r].numpy(), float(temps[r]), 77, r, 5 + r)
        assert scores[out[r].item()] >= scores.max() - 1e-4   # 32-bit logs against the plain 64-bit ones
    # a padded row stride
    wide = torch.randn(3, 40, generator=g)
    ops.sample(dev(wide)[:, :33], None, None, out[:3])
    assert out[:3].cpu().tolist() == wide[:, :33].argmax(-1).tolist()


def test_sampling_follows_the_softmax(ops):
    from cbis_b200.sampling import request_key
    logits = torch.tensor([1.0, 0.0, -1.0, 0.5, -30.0])
    n = 6000
    keys = torch.tensor([request_key(1, 2, i) for i in range(n)], dtype=torch.int64)
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits.repeat(n, 1)), dev(torch.full((n,), 0.7)), dev(keys), out)
    counts = np.bincount(out.cpu().numpy(), minlength=5) / n
    p = torch.softmax(logits / 0.7, 0).numpy()
    assert np.abs(counts - p).max() < 0.025
    exp = [plain_gpt.sample(logits.numpy(), 0.7, 1, 2, i) for i in range(200)]
    assert out[:200].cpu().tolist() == exp


@pytest.mark.parametrize("n_head,n_kv_head,hd,ps,window", [
    (3, 3, 24, 8, 0), (2, 2, 32, 16, 0), (6, 2, 80, 4, 0), (5, 5, 128, 16, 0), (2, 1, 256, 32, 0),
    (4, 4, 48, 8, 11), (1, 1, 16, 3, 5), (4, 2, 64, 16, 0), (2, 2, 112, 16, 70)])
@pytest.mark.parametrize("nsplit", [1, 3, 8])
def test_decode_attention_split_kv(ops, n_head, n_kv_head, hd, ps, window, nsplit):
    """One query per request over 1..700 cached keys; the current token's key/value come from the
    projections and are stored by the kernel itself."""
    seg_ctx = [1, 2, 37, 70, 16, 129, 700]
    S = len(seg_ctx)
    c = paged_case(ops, torch.bfloat16, n_head, n_kv_head, hd, ps, window, seg_ctx, [1] * S, seed=hd + ps + nsplit)
    dq, dkv = n_head * hd, n_kv_head * hd
    # qkv rows: q, then the key/value of the current position; wipe those from the cache to see the kernel store them
    qkv = torch.zeros(S + 1, dq + 2 * dkv + 8, dtype=torch.bfloat16, device="cuda")[:, :dq + 2 * dkv]
    slots = torch.full((S + 1,), -1, dtype=torch.int32)
    kc, vc = c["kc"], c["vc"]
    for s, n in enumerate(seg_ctx):
        page, off = int(c["bt"][s, (n - 1) // ps]), (n - 1) % ps
        qkv[s, :dq] = c["q"][s].cuda()
        qkv[s, dq:dq + dkv] = kc[page, :, off, :].reshape(-1)
        qkv[s, dq + dkv:] = vc[page, :, off, :].reshape(-1)
        slots[s] = page * ps + off
        kc[page, :, off, :] = float("nan")
        vc[page, :, off, :] = float("nan")
    row_seq = torch.cat([c["row_seq"], torch.tensor([-1], dtype=torch.int32)])      # a padding row at the end
    positions = torch.cat([c["positions"], torch.tensor([0], dtype=torch.int32)])
    out = torch.full((S + 1, dq), float("nan"), dtype=torch.bfloat16, device="cuda")
    scratch = torch.full((max(1, ops.decode_scratch_floats(S + 1, n_head, hd, nsplit)),), float("nan"), device="cuda")
    counters = torch.zeros((S + 1) * n_head, dtype=torch.int32, device="cuda")
    if hd % 8:
        with pytest.raises(ops.KernelError, match="multiple of 8"):
            ops.paged_decode_bf16(qkv, dq, dq + dkv, kc, vc, dev(c["bt"]), dev(row_seq), dev(positions), dev(slots), out,
                                  scratch, counters, n_head, n_kv_head, hd, ps, c["scale"], window, nsplit)
        return
    bits_before = [t.clone().view(torch.int16) for t in (kc, vc)]
    ops.paged_decode_bf16(qkv, dq, dq + dkv, kc, vc, dev(c["bt"]), dev(row_seq), dev(positions), dev(slots), out,
                          scratch, counters, n_head, n_kv_head, hd, ps, c["scale"], window, nsplit)
    assert (out[:S].double().cpu() - c["ref"]).abs().max() < 1e-2 * max(1.0, c["ref"].abs().max().item())
    assert torch.equal(out[S].cpu(), torch.zeros(dq, dtype=torch.bfloat16))
    # the kernel wrote the S token slots of the current positions and nothing else (the padding row has slot -1)
    written = torch.zeros(kc.shape[0], kc.shape[2], dtype=torch.bool, device="cuda")
    for s, n in enumerate(seg_ctx):
        written[int(c["bt"][s, (n - 1) // ps]), (n - 1) % ps] = True
    for t, before in zip((kc, vc), bits_before):
        changed = (t.view(torch.int16) != before).any(dim=3).any(dim=1)              # [page, offset]
        assert torch.equal(changed, written)
    for s, n in enumerate(seg_ctx):                                                   # the kernel stored k and v
        page, off = int(c["bt"][s, (n - 1) // ps]), (n - 1) % ps
        assert torch.equal(kc[page, :, off, :].reshape(-1), qkv[s, dq:dq + dkv])
        assert torch.equal(vc[page, :, off, :].reshape(-1), qkv[s, dq + dkv:])
    # the same from the cache alone (k_off < 0) gives the same result
    out2 = torch.empty_like(out)
    ops.paged_decode_bf16(qkv, -1, -1, kc, vc, dev(c["bt"]), dev(row_seq), dev(positions), dev(slots), out2, scratch, counters,
                          n_head, n_kv_head, hd, ps, c["scale"], window, nsplit)
    assert torch.equal(out2[:S], out[:S])
    assert int(counters.abs().sum()) == 0                                             # left zero for the next launch


def test_decode_advance_and_slots(ops):
    tokens = dev(torch.tensor([5, 6, 7], dtype=torch.int32)); pos = dev(torch.tensor([3, 7, 0], dtype=torch.int32))
    start, ctxl = pos.clone(), pos.clone() + 1
    ops.decode_advance(tokens, pos, start, ctxl, dev(torch.tensor([9, 8, 1], dtype=torch.int32)), 2)
    assert tokens.tolist() == [9, 8, 7] and pos.tolist() == [4, 8, 0] and ctxl.tolist() == [5, 9, 1]
    bt = dev(torch.tensor([[4, 2, -1], [7, 0, 3]], dtype=torch.int32))
    slots = dev(torch.zeros(3, dtype=torch.int32))
    ops.slots_from_table(pos, dev(torch.tensor([0, 1, -1], dtype=torch.int32)), bt, 4, slots, 3)
    assert slots.tolist() == [2 * 4 + 0, 3 * 4 + 0, -1]


@pytest.mark.parametrize("M", [1, 3, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(40, 64), (2048, 2048), (50257, 96), (6144, 2048), (1000, 8200), (7, 8)])
def test_gemm_small_m(ops, M, N, K):
    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    ref = x.double() @ w.double().t() + b.double()
    scale = max(1.0, ref.abs().max().item())
    out = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_small_m(dev(x), dev(w), dev(b), None, out)
    assert (out.double().cpu() - ref).abs().max() < 1e-5 * scale * math.sqrt(K)      # 32-bit sums of exact products
    out16 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_small_m(dev(x), dev(w), None, "gelu_erf", out16)
    ref2 = plain_gpt.gelu(x.double() @ w.double().t(), "gelu")
    assert (out16.double().cpu() - ref2).abs().max() < 1e-2 * max(1.0, ref2.abs().max().item())
    # rows of a wider matrix as input, columns of a wider matrix as output
    wide = torch.randn(M, K + 16, generator=g).to(torch.bfloat16)
    big = torch.zeros(M, N + 3, device="cuda")
    ops.gemm_small_m(dev(wide)[:, 8:8 + K], dev(w), None, None, big[:, :N])
    ref3 = wide[:, 8:8 + K].double() @ w.double().t()
    assert (big[:, :N].double().cpu() - ref3).abs().max() < 1e-5 * scale * math.sqrt(K)
    assert torch.equal(big[:, N:].cpu(), torch.zeros(M, 3))


@pytest.mark.parametrize("M", [1, 2, 5, 8])
@pytest.mark.parametrize("N,K", [(40, 64), (2048, 2048), (317, 96), (4800, 1600), (1000, 2056), (7, 8), (50, 4104)])
def test_ln_linear_and_accumulating_product(ops, M, N, K):
    """LayerNorm inside the product's kernel (rows in registers up to 2,048 wide, read again beyond that; K that is
    no multiple of the 32-wide K block; one or two column groups to the last block), and the product that adds
    into a 32-bit matrix, each against 64-bit arithmetic."""
    g = torch.Generator().manual_seed(M * 11 + N + K)
    x = torch.randn(M, K, generator=g) * 2.0 + 0.7
    x[:, K // 2] = 40.0                               # one column far from the mean: a centred variance copes
    gamma, beta = 1 + 0.1 * torch.randn(K, generator=g), 0.1 * torch.randn(K, generator=g)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    eps = 3e-5
    xd = x.double()
    hn = (xd - xd.mean(-1, keepdim=True)) / torch.sqrt(xd.var(-1, unbiased=False, keepdim=True) + eps) * gamma.double() + beta.double()
    hb = hn.float().to(torch.bfloat16)                # the kernel rounds the normalised rows to bfloat16 once
    ref = hb.double() @ w.double().t() + b.double()
    scale = max(1.0, ref.abs().max().item())
    out = torch.full((M, N + 2), float("nan"), device="cuda")
    ops.ln_linear(dev(x), dev(gamma), dev(beta), eps, dev(w), dev(b), None, out[:, :N])
    got = out[:, :N].double().cpu()
    # a normalised value that lands on the other side of a bfloat16 rounding boundary moves one product by 2^-8 of it
    assert (got - ref).abs().max() < 2e-3 * scale
    assert (got - (hn @ w.double().t() + b.double())).abs().max() < 2e-2 * scale
    assert torch.isnan(out[:, N:]).all()
    out16 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.ln_linear(dev(x), dev(gamma), dev(beta), eps, dev(w), None, "gelu_tanh", out16)
    ref2 = plain_gpt.gelu(hb.double() @ w.double().t(), "gelu_new")
    assert (out16.double().cpu() - ref2).abs().max() < 1.5e-2 * max(1.0, ref2.abs().max().item())
    # against the norm kernel and the product kernel one after the other: the same roundings, sums in another order
    h2 = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
    ops.add_layernorm(dev(x), None, None, dev(gamma), dev(beta), eps, h2)
    two = torch.empty(M, N, device="cuda")
    ops.gemm_small_m(h2, dev(w), dev(b), None, two)
    assert (two.double().cpu() - got).abs().max() < 2e-3 * scale
    # x += a W^T + b
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    acc = torch.randn(M, N, generator=g)
    want = acc.double() + a.double() @ w.double().t() + b.double()
    accd = dev(acc.clone())
    ops.gemm_small_m(dev(a), dev(w), dev(b), None, accd, accumulate=True)
    assert (accd.double().cpu() - want).abs().max() < 1e-5 * max(1.0, want.abs().max().item()) * math.sqrt(K)


@pytest.mark.parametrize("M,N,K", [(2048, 2048, 2048), (300, 1000, 264), (129, 4800, 72), (513, 24, 4104)])
def test_tcgen05_product_adds_into_a_32_bit_matrix(ops, M, N, K):
    """C += A W^T + bias through the TMA reduction of the pair kernel's epilogue, and the plain 32-bit result through
    its TMA store: rows that are no multiple of the 32-row pieces, a width that is no multiple of the 16-column
    pieces or of the tile, a matrix wider than the result (columns beside it stay as they are)."""
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    acc = torch.randn(M, N + 4, generator=g)
    prod = a.double() @ w.double().t() + b.double()
    tol = 1e-5 * max(1.0, prod.abs().max().item()) * math.sqrt(K)
    big = dev(acc.clone())
    ops.gemm_tcgen05(dev(a), dev(w), dev(b), None, big[:, :N], accumulate=True)
    assert (big[:, :N].double().cpu() - (acc[:, :N].double() + prod)).abs().max() < tol
    assert torch.equal(big[:, N:].cpu(), acc[:, N:])
    ops.gemm_tcgen05(dev(a), dev(w), dev(b), None, big[:, :N], accumulate=True)      # and once more: twice the product
    assert (big[:, :N].double().cpu() - (acc[:, :N].double() + 2 * prod)).abs().max() < 2 * tol
    out = torch.full((M, N + 4), float("nan"), device="cuda")
    ops.gemm_tcgen05(dev(a), dev(w), None, None, out[:, :N])
    assert (out[:, :N].double().cpu() - (prod - b.double())).abs().max() < tol
    assert torch.isnan(out[:, N:]).all()
    assert ops.tcgen05_error_flag("cuda").item() == 0
    with pytest.raises(ops.KernelError):              # up to 128 rows the single-block form runs, which does not add
        ops.gemm_tcgen05(dev(a)[:100], dev(w), dev(b), None, big[:100, :N], accumulate=True)


def test_ln_linear_refuses_what_it_does_not_take(ops):
    w = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    v = torch.ones(64, device="cuda")
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.ln_linear(torch.zeros(9, 64, device="cuda"), v, v, 1e-5, w, None, None, torch.empty(9, 16, device="cuda"))
    w = torch.zeros(16, 60, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.ln_linear(torch.zeros(2, 60, device="cuda"), v[:60], v[:60], 1e-5, w, None, None, torch.empty(2, 16, device="cuda"))
    with pytest.raises(ops.KernelError):
        ops.gemm_small_m(torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda"), torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda"),
                         None, None, torch.empty(2, 16, dtype=torch.bfloat16, device="cuda"), accumulate=True)


def test_gemm_small_m_refuses_what_it_does_not_take(ops):
    x = torch.zeros(65, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.gemm_small_m(x, w, None, None, torch.empty(65, 16, device="cuda"))
    x = torch.zeros(4, 60, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(16, 60, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.gemm_small_m(x, w, None, None, torch.empty(4, 16, device="cuda"))
    # the dispatcher sends such sizes to the library product instead
    out = ops.linear(x, w, None, None, out_dtype=torch.float32)
    assert out.shape == (4, 16)


@pytest.mark.parametrize("M,N,K", [(64, 4800, 1600), (17, 6400, 1600), (40, 317, 96), (300, 1000, 264), (33, 72, 40), (129, 2056, 520)])
def test_linear_between_few_rows_and_many_uses_one_rounding(ops, M, N, K):
    """17 rows and more, below the sizes of the tcgen05 product: bias, and bias with the tanh GELU, applied to the
    32-bit sums and rounded once, whichever way the product goes (the library's epilogue where the bias is exact in
    bfloat16, else 32-bit sums and this package's epilogue kernel); exact-erf GELU always the latter."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.08).to(torch.bfloat16)
    b_exact = torch.randn(N, generator=g).to(torch.bfloat16).float()
    b_32 = b_exact + 1e-4 * torch.randn(N, generator=g)             # not a bfloat16 number: the other way
    for b in (b_exact, b_32):
        lin = x.double() @ w.double().t() + b.double()
        for act, name in ((None, None), ("gelu_tanh", "gelu_new"), ("gelu_erf", "gelu")):
            ref = plain_gpt.gelu(lin, name) if name else lin
            out = ops.linear(dev(x), dev(w), dev(b), act)
            assert out.dtype == torch.bfloat16 and out.shape == (M, N)
            err = (out.double().cpu() - ref).abs()
            # one bfloat16 rounding of the exact value (2^-9 relative) and the 32-bit sum's own error
            assert (err <= ref.abs() * 2 ** -8 + 2e-4 * math.sqrt(K) * 0.08 + 1e-5).all(), (act, err.max().item())
    on = ops.linear(dev(x), dev(w), dev(b_exact), "gelu_tanh")
    keep = ops.USE_LIBRARY_EPILOGUE
    ops.USE_LIBRARY_EPILOGUE = False
    try:
        off = ops.linear(dev(x), dev(w), dev(b_exact), "gelu_tanh")
    finally:
        ops.USE_LIBRARY_EPILOGUE = keep
    # the two ways differ by the order of the 32-bit sums only: at most the last bfloat16 bit here and there
    assert ((on.double() - off.double()).abs() <= off.double().abs() * 2 ** -7 + 1e-5).all()


def test_bias_act_out_rounds_once(ops):
    g = torch.Generator().manual_seed(5)
    src, b = torch.randn(9, 130, generator=g) * 3, torch.randn(130, generator=g)
    dst = torch.empty(9, 130, dtype=torch.bfloat16, device="cuda")
    ops.bias_act_out(dev(src), dev(b), "gelu_tanh", dst)
    ref = plain_gpt.gelu(src.double() + b.double(), "gelu_new")
    # one bfloat16 rounding (2^-8 relative) of a 32-bit GELU (absolute error of tanhf times |x| in the tails)
    close = (dst.double().cpu() - ref).abs() <= (ref.abs() * 2 ** -8 + 4e-6)
    assert close.all()


@pytest.mark.parametrize("n_head,n_kv_head,hd,ps,window", [(2, 2, 128, 16, 0), (4, 2, 64, 16, 0), (3, 1, 128, 64, 0),
                                                           (2, 2, 64, 8, 0), (2, 2, 128, 16, 100), (1, 1, 64, 32, 37),
                                                           (8, 8, 32, 16, 0), (2, 1, 16, 8, 0), (3, 3, 48, 16, 21),
                                                           (2, 2, 80, 16, 0), (2, 1, 96, 32, 0), (1, 1, 112, 16, 0)])
def test_prefill_attention_tensor_cores(ops, n_head, n_kv_head, hd, ps, window):
    """Segments of 1..200 rows at the end of contexts of up to 333 keys: first portions, later portions,
    rows that are not a multiple of the 64-row tile, contexts that end inside a page and inside a key tile."""
    seg_ctx, seg_rows = [200, 333, 64, 70, 1, 130], [200, 77, 64, 3, 1, 65]
    c = paged_case(ops, torch.bfloat16, n_head, n_kv_head, hd, ps, window, seg_ctx, seg_rows, seed=hd + ps + window)
    S = len(seg_ctx)
    cu = torch.tensor([0] + list(np.cumsum(seg_rows)), dtype=torch.int32)
    start = torch.tensor([cx - n for cx, n in zip(seg_ctx, seg_rows)], dtype=torch.int32)
    out = torch.full_like(c["q"], float("nan")).cuda()
    ops.paged_prefill_bf16(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), out, 0, S, max(seg_rows),
                           n_head, n_kv_head, hd, ps, c["scale"], window)
    err = (out.double().cpu() - c["ref"]).abs().max().item()
    assert err < 1.5e-2 * max(1.0, c["ref"].abs().max().item()), err
    # only some of the segments (the first two count as decoded elsewhere): their rows stay untouched
    out2 = torch.full_like(c["q"], float("nan")).cuda()
    ops.paged_prefill_bf16(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), out2, 2, S - 2, max(seg_rows[2:]),
                           n_head, n_kv_head, hd, ps, c["scale"], window)
    r2 = int(cu[2])
    assert torch.isnan(out2[:r2].float()).all() and torch.equal(out2[r2:], out[r2:])
    # the keys cut into chunks over more blocks and merged by the second kernel: the same to rounding
    T = len(c["positions"])
    for n_chunks, chunk_keys, s0 in [(2, 256, 0), (6, 64, 0), (3, 128, 2)]:
        r0 = int(cu[s0])
        partial = torch.full(((T - r0) * n_head * n_chunks * (hd + 4),), float("nan"), device="cuda")
        cut = torch.full_like(c["q"], float("nan")).cuda()
        ops.paged_prefill_bf16(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), cut, s0, S - s0,
                               max(seg_rows[s0:]), n_head, n_kv_head, hd, ps, c["scale"], window, (n_chunks, chunk_keys),
                               partial, dev(c["positions"]), r0, T - r0)
        assert torch.isnan(cut[:r0].float()).all()
        assert (cut[r0:].float() - out[r0:].float()).abs().max().item() < 1.5e-2 * max(1.0, c["ref"].abs().max().item())


@pytest.mark.parametrize("n_head,n_kv_head,hd,ps,window", [(2, 2, 128, 16, 0), (4, 2, 64, 16, 0), (3, 1, 32, 64, 0),
                                                           (8, 8, 32, 16, 0), (2, 1, 16, 3, 0), (3, 3, 48, 16, 21),
                                                           (2, 2, 80, 5, 100), (2, 1, 96, 32, 0), (1, 1, 112, 16, 37)])
def test_prefill_attention_32_bit_tiled(ops, n_head, n_kv_head, hd, ps, window):
    """The 32-bit tiled form (64 rows to a block, keys through shared memory in tiles of 32): the cases of the
    tensor-core form, page sizes that are no power of two, in a cache whose unused slots hold NaN; it agrees with
    the general kernel (one warp per row) to 32-bit rounding."""
    seg_ctx, seg_rows = [200, 333, 64, 70, 1, 130, 600], [200, 77, 64, 3, 1, 65, 257]
    c = paged_case(ops, torch.float32, n_head, n_kv_head, hd, ps, window, seg_ctx, seg_rows, seed=hd + ps + window)
    S = len(seg_ctx)
    cu = torch.tensor([0] + list(np.cumsum(seg_rows)), dtype=torch.int32)
    start = torch.tensor([cx - n for cx, n in zip(seg_ctx, seg_rows)], dtype=torch.int32)
    out = torch.full_like(c["q"], float("nan")).cuda()
    ops.paged_prefill_f32(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), out, 0, S, max(seg_rows),
                          n_head, n_kv_head, hd, ps, c["scale"], window)
    bound = 2e-6 * max(1.0, c["ref"].abs().max().item())
    assert (out.double().cpu() - c["ref"]).abs().max().item() < bound
    general = torch.empty_like(out)
    ops.paged_attention_generic(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(c["row_seq"]), dev(c["positions"]),
                                general, n_head, n_kv_head, hd, ps, c["scale"], window)
    assert (out - general).abs().max().item() < bound
    # the keys cut into chunks (by absolute index) and merged by the second kernel: the same to rounding
    T = len(c["positions"])
    for n_chunks, chunk_keys in [(3, 256), (10, 64), (20, 32)]:
        partial = torch.full((T * n_head * n_chunks * (hd + 4),), float("nan"), device="cuda")
        cut = torch.full_like(c["q"], float("nan")).cuda()
        ops.paged_prefill_f32(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), cut, 0, S, max(seg_rows),
                              n_head, n_kv_head, hd, ps, c["scale"], window, (n_chunks, chunk_keys), partial,
                              dev(c["positions"]), 0, T)
        assert (cut - out).abs().max().item() < bound, (n_chunks, chunk_keys)
    r2 = int(cu[2])
    partial = torch.full(((T - r2) * n_head * 5 * (hd + 4),), float("nan"), device="cuda")
    cut = torch.full_like(c["q"], float("nan")).cuda()
    ops.paged_prefill_f32(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), cut, 2, S - 2, max(seg_rows[2:]),
                          n_head, n_kv_head, hd, ps, c["scale"], window, (5, 128), partial, dev(c["positions"]), r2, T - r2)
    assert torch.isnan(cut[:r2]).all() and (cut[r2:] - out[r2:]).abs().max().item() < bound
    # only the segments from the third on: the rows before stay untouched
    out2 = torch.full_like(c["q"], float("nan")).cuda()
    ops.paged_prefill_f32(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), out2, 2, S - 2, max(seg_rows[2:]),
                          n_head, n_kv_head, hd, ps, c["scale"], window)
    assert torch.isnan(out2[:r2]).all() and torch.equal(out2[r2:], out[r2:])
    with pytest.raises(ops.KernelError, match="head_dim=24"):
        ops.paged_prefill_f32(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), out2, 0, S, max(seg_rows),
                              n_head, n_kv_head, 24, ps, c["scale"], window)


def test_prefill_key_chunks_fill_the_gpu_and_cover_the_context(ops):
    assert ops.prefill_key_chunks(80, 16, 1, 2048) == (1, 0)              # enough blocks without a cut
    assert ops.prefill_key_chunks(16, 16, 1, 2048, 2, 2) == (1, 0)        # the tcgen05 kernel: two blocks a tile, two an SM
    assert ops.prefill_key_chunks(4, 16, 1, 2048, 2, 2, 8192) == (1, 0) and ops.prefill_key_chunks(4, 16, 1, 32768, 2, 2, 8192) == (2, 16384)
    assert ops.prefill_key_chunks(1, 2, 1, 200) == (1, 0)                 # too short to cut
    for tiles, heads, segs, limit in [(8, 8, 1, 32768), (1, 1, 1, 5000), (2, 3, 2, 257), (8, 8, 1, 700)]:
        n, keys = ops.prefill_key_chunks(tiles, heads, segs, limit)
        assert n > 1 and keys % 32 == 0 and keys >= 256 and keys & (keys - 1) == 0
        assert (n - 1) * keys < limit <= n * keys


def test_prefill_attention_finds_a_far_key_and_respects_the_diagonal(ops):
    hd, ps, T = 128, 16, 300
    g = torch.Generator().manual_seed(4)
    k = (torch.randn(T, hd, generator=g) * 0.05).to(torch.bfloat16)
    v = torch.randn(T, hd, generator=g).to(torch.bfloat16)
    q = (torch.randn(T, hd, generator=g) * 0.05).to(torch.bfloat16)
    # row 250 matches key 3 strongly; row 100 would match key 101 (the future) strongly, which it must not see
    q[250] = torch.randn(hd, generator=g).to(torch.bfloat16)
    q[100] = torch.randn(hd, generator=g).to(torch.bfloat16)
    k[3] = q[250]
    k[101] = q[100]
    pages = torch.randperm(19, generator=g).int()
    kc = torch.zeros(19, 1, ps, hd, dtype=torch.bfloat16, device="cuda"); vc = torch.zeros_like(kc)
    slots = torch.tensor([int(pages[p // ps]) * ps + p % ps for p in range(T)], dtype=torch.int32)
    ops.kv_write(dev(torch.cat([k, v], 1)), 0, hd, kc, vc, dev(slots), 1, hd, ps)
    out = torch.empty(T, hd, dtype=torch.bfloat16, device="cuda")
    ops.paged_prefill_bf16(dev(q), kc, vc, dev(pages[None, :]), dev(torch.tensor([0, T], dtype=torch.int32)),
                           dev(torch.tensor([0], dtype=torch.int32)), out, 0, 1, T, 1, 1, hd, ps, hd ** -0.5)
    sc = (q.double() @ k.double().t()) * hd ** -0.5
    sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    p = torch.softmax(sc, -1)
    assert p[250, 3] > 0.9 and p[100, 101] == 0
    assert (out.double().cpu() - p @ v.double()).abs().max() < 2e-2


@pytest.mark.parametrize("M,N,K,ksplit", [(1, 48, 64, 1), (5, 4800, 1600, 0), (8, 8192, 2048, 0), (8, 6144, 2048, 4),
                                          (16, 2048, 8192, 8), (3, 1000, 520, 2), (8, 2048, 2048, 0), (33, 777, 264, 1),
                                          (64, 4096, 1024, 2), (20, 50257, 256, 0)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_few_rows_tcgen05(ops, M, N, K, ksplit, out_dtype):
    """The few-rows product with swapped operands (weights by TMA, tcgen05, K split over a cluster): sizes that are
    no multiple of its tiles, every cluster size, against the product in 64-bit."""
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device="cuda")
    ops.gemm_few_rows(dev(x), dev(w), dev(b), "gelu_erf", out, ksplit)
    ref = plain_gpt.gelu(x.double() @ w.double().t() + b.double(), "gelu")
    tol = 1e-5 * math.sqrt(K) if out_dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - ref).abs().max() < tol * max(1.0, ref.abs().max().item())
    assert ops.tcgen05_error_flag("cuda").item() == 0


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 300, 136), (1000, 512, 2048), (77, 5001, 96), (2048, 768, 320),
                                   (257, 520, 72), (2304, 8200, 128), (300, 40, 64), (129, 17, 8), (4096, 264, 40)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05(ops, M, N, K, out_dtype):
    """The TMA + tcgen05 product with its fused epilogue: sizes that are no multiple of its tiles (128x256x64 on
    one block up to 128 rows, 256x256x64 on pairs of blocks above), one of them with several tiles per block."""
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device="cuda")
    ops.gemm_tcgen05(dev(x), dev(w), dev(b), "gelu_tanh", out)
    ref = plain_gpt.gelu(x.double() @ w.double().t() + b.double(), "gelu_new")
    tol = 1e-5 * math.sqrt(K) if out_dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - ref).abs().max() < tol * max(1.0, ref.abs().max().item())
    assert ops.tcgen05_error_flag("cuda").item() == 0            # no bounded wait ran out


@pytest.mark.parametrize("n_head,n_kv_head,ps,window", [(2, 2, 16, 0), (4, 2, 16, 0), (3, 1, 64, 0), (2, 2, 8, 0),
                                                        (2, 2, 16, 100), (1, 1, 32, 37), (2, 1, 128, 0)])
@pytest.mark.parametrize("hd", [128, 64])
def test_prefill_attention_tcgen05(ops, n_head, n_kv_head, ps, window, hd):
    """The TMA + tcgen05 form (head sizes 128 and 64): the same cases as the mma.sync form, in a cache whose unused
    slots hold NaN (what an earlier owner of a page may have left must not reach another request)."""
    seg_ctx, seg_rows = [200, 333, 64, 70, 1, 130, 600], [200, 77, 64, 3, 1, 65, 257]
    c = paged_case(ops, torch.bfloat16, n_head, n_kv_head, hd, ps, window, seg_ctx, seg_rows, seed=ps + window)
    S = len(seg_ctx)
    cu = torch.tensor([0] + list(np.cumsum(seg_rows)), dtype=torch.int32)
    start = torch.tensor([cx - n for cx, n in zip(seg_ctx, seg_rows)], dtype=torch.int32)
    out = torch.full_like(c["q"], float("nan")).cuda()
    ops.paged_prefill_tc5(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), out, 0, S, max(seg_rows),
                          n_head, n_kv_head, hd, ps, c["scale"], window)
    assert ops.tcgen05_error_flag("cuda").item() == 0
    err = (out.double().cpu() - c["ref"]).abs().max().item()
    assert err < 1.5e-2 * max(1.0, c["ref"].abs().max().item()), err
    # the keys cut into chunks over more clusters and merged by the second kernel: the same to rounding
    T = len(c["positions"])
    for n_chunks, chunk_keys, s0 in [(3, 256, 0), (10, 64, 0), (5, 128, 2)]:
        r0 = int(cu[s0])
        partial = torch.full(((T - r0) * n_head * n_chunks * (hd + 4),), float("nan"), device="cuda")
        cut = torch.full_like(c["q"], float("nan")).cuda()
        ops.paged_prefill_tc5(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), cut, s0, S - s0,
                              max(seg_rows[s0:]), n_head, n_kv_head, hd, ps, c["scale"], window, (n_chunks, chunk_keys),
                              partial, dev(c["positions"]), r0, T - r0)
        assert ops.tcgen05_error_flag("cuda").item() == 0
        assert torch.isnan(cut[:r0].float()).all()
        assert (cut[r0:].float() - out[r0:].float()).abs().max().item() < 1.5e-2 * max(1.0, c["ref"].abs().max().item())
    # agrees with the mma.sync form to rounding
    out2 = torch.empty_like(out)
    ops.paged_prefill_bf16(dev(c["q"]), c["kc"], c["vc"], dev(c["bt"]), dev(cu), dev(start), out2, 0, S, max(seg_rows),
                           n_head, n_kv_head, hd, ps, c["scale"], window)
    assert (out.float() - out2.float()).abs().max().item() < 2e-2 * max(1.0, c["ref"].abs().max().item())


def test_prefill_attention_tcgen05_is_repeatable(ops):
    """Three hundred launches of a case with many short key ranges (where the threads of a block run furthest
    apart): every launch gives the bits of the first, and no bounded wait runs out."""
    hd, ps, n_head = 128, 16, 4
    seg_ctx, seg_rows = [193, 72, 400, 130, 64, 1000], [61, 70, 2, 130, 7, 300]
    c = paged_case(ops, torch.bfloat16, n_head, n_head, hd, ps, 0, seg_ctx, seg_rows, seed=5)
    S = len(seg_ctx)
    cu = dev(torch.tensor([0] + list(np.cumsum(seg_rows)), dtype=torch.int32))
    start = dev(torch.tensor([cx - n for cx, n in zip(seg_ctx, seg_rows)], dtype=torch.int32))
    q, bt = dev(c["q"]), dev(c["bt"])
    first = None
    for _ in range(300):
        out = torch.full_like(c["q"], float("nan")).cuda()
        ops.paged_prefill_tc5(q, c["kc"], c["vc"], bt, cu, start, out, 0, S, max(seg_rows), n_head, n_head, hd, ps,
                              c["scale"], 0)
        if first is None:
            first = out
            assert (out.double().cpu() - c["ref"]).abs().max().item() < 1.5e-2 * max(1.0, c["ref"].abs().max().item())
        else:
            assert torch.equal(out, first)
    assert ops.tcgen05_error_flag("cuda").item() == 0


def test_prefill_attention_tcgen05_two_blocks_per_sm(ops):
    """Its shared memory, registers and tensor memory are sized so that an SM holds two blocks: one block's
    softmax runs while the other's products do."""
    assert ops.paged_prefill_tc5_blocks_per_sm() == 2     # a kilobyte more shared memory, or 147 registers, and it reads 1


def test_a_wait_that_runs_out_is_reported_and_the_kernel_returns(ops):
    """The TMA + tcgen05 product is told to request no operands and to give every wait a short limit: its waits
    for operands wait for a signal that nothing sends, run out, the kernel sets the error flag, frees its tensor
    memory and returns (no copy in flight, no trap).  The host sees the flag as an exception that names the cause
    and clears it; the next launch, of the same kernel with the same tensor memory, gives the right result."""
    g = torch.Generator().manual_seed(3)
    M, N, K = 96, 512, 256
    x = dev(torch.randn(M, K, generator=g).to(torch.bfloat16))
    w = dev((torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16))
    flag = ops.tcgen05_error_flag("cuda")
    assert flag.item() == 0
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05(x, w, None, None, out, spin_limit=64, starve=True)
    torch.cuda.synchronize()                                                        # it came back by itself
    assert flag.item() != 0
    with pytest.raises(ops.KernelError, match="bounded wait"):
        ops.raise_if_kernel_errors("cuda")
    assert flag.item() == 0                                                         # reported once, then cleared
    ops.raise_if_kernel_errors("cuda")
    ops.gemm_tcgen05(x, w, None, None, out)                                         # tensor memory was given back
    ref = x.double() @ w.double().t()
    assert (out.double() - ref).abs().max().item() < 1e-2 * ref.abs().max().item()
    assert flag.item() == 0
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.gemm_tcgen05(dev(torch.zeros(300, K, dtype=torch.bfloat16)), w, None, None,
                         torch.empty(300, N, dtype=torch.bfloat16, device="cuda"), starve=True)


def test_error_flag_set_from_the_host_reaches_every_reporting_path(ops, folder_a):
    """What the engine does when a kernel has reported a wait that ran out, shown by writing the flag from the
    host: the blocking check raises and clears; the polling check raises within two calls; a bare step reports it
    at one of the next calls or when the request is closed; the engine's own step raises."""
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    flag = ops.tcgen05_error_flag("cuda")
    flag.fill_(13)
    with pytest.raises(ops.KernelError, match="code 13"):
        ops.raise_if_kernel_errors("cuda")
    assert flag.item() == 0
    flag.fill_(2)
    with pytest.raises(ops.KernelError, match="code 2"):
        for _ in range(3):
            ops.poll_kernel_errors("cuda")
            torch.cuda.synchronize()
    assert flag.item() == 0
    ops.poll_kernel_errors("cuda"); torch.cuda.synchronize(); ops.poll_kernel_errors("cuda")   # clean again
    eng = cb.Engine(folder_a, dtype="bfloat16", page_size=16, num_pages=8, max_num_seqs=2, max_batched_tokens=32)
    slot = eng.open_request(0)
    eng.forward_step([StepEntry(slot, 0, [1, 2, 3, 4], [3])])
    flag.fill_(11)
    with pytest.raises(ops.KernelError, match="code 11"):
        eng.forward_step([StepEntry(slot, 4, [5, 6], [1])])
        eng.close_request(slot)                                 # at the latest here
    assert flag.item() == 0
    if eng.pool.manager.live(slot):
        eng.close_request(slot)
    flag.fill_(21)
    with pytest.raises(ops.KernelError, match="code 21"):
        eng.generate([[1, 2, 3, 4, 5]], cb.SamplingParams(max_new_tokens=2))       # a step with a prompt portion checks
    assert flag.item() == 0
