"""Times single kernels at given sizes, inside a CUDA graph over distinct buffers (so that every
launch streams from HBM, as in a real step) or launch by launch for profilers.

    python -m cbis_b200.kernels.microbench --op decode_attn --rows 8 --ctx 1536 --layers 24
    python -m cbis_b200.kernels.microbench --op gemm --rows 8 --n 6144 --k 2048
    python -m cbis_b200.kernels.microbench --op gemm_tc --rows 2048 --n 8192 --k 2048
    python -m cbis_b200.kernels.microbench --op gemm_f32 --rows 512 --n 256 --k 1024
    python -m cbis_b200.kernels.microbench --op layernorm --rows 8 --k 2048
    python -m cbis_b200.kernels.microbench --op sample --rows 8 --n 50257
    python -m cbis_b200.kernels.microbench --op prefill_attn --rows 512 --ctx 32768 --heads 8 --head-dim 32 [--dtype float32]
    python -m cbis_b200.kernels.microbench --op decode_layers_phases --rows 8 --ctx 1024 --layers 6

``--no-graph`` launches the kernels directly (a profiler then sees ordinary launches).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def timed(fn, use_graph=True, reps=20):
    """Microseconds per call of fn()."""
    fn()
    torch.cuda.synchronize()
    if use_graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        run = g.replay
    else:
        run = fn
    run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def decode_layers_phases(rows: int, ctx_len: int, layers: int):
    """Microseconds per phase and layer of the persistent decode kernel as its block 0 sees them (1.3B layer sizes)."""
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    from cbis_b200.kernels import ops
    cfg = dict(architectures=["GPT2LMHeadModel"], n_layer=layers, n_embd=2048, n_head=16, n_inner=8192, vocab_size=50257,
               n_positions=2048, activation_function="gelu", layer_norm_epsilon=1e-5, tie_word_embeddings=True)
    eng = cb.Engine.from_random(cfg, seed=1, dtype="bfloat16", page_size=16, max_tokens=rows * 2048, max_num_seqs=rows,
                                max_batched_tokens=2048, prefill_chunk=2048)
    g = torch.Generator().manual_seed(0)
    slots = [eng.open_request(i) for i in range(rows)]
    for s in slots:
        eng.forward_step([StepEntry(s, 0, torch.randint(0, 50257, (ctx_len,), generator=g).tolist(), [])])
    eng.runner.use_graphs, ops.USE_FUSED_DECODE = False, True
    for step in range(4):
        eng.forward_step([StepEntry(s, ctx_len + step, [5], [0]) for s in slots])
    plan = next(iter(eng.runner.__dict__["_decode_layer_plans"].values()))
    plan.trace = torch.zeros(256, dtype=torch.int64, device="cuda")
    eng.forward_step([StepEntry(s, ctx_len + 4, [5], [0]) for s in slots])
    torch.cuda.synchronize()
    t = plan.trace.cpu().tolist()
    names = ["LN1", "QKV", "meet", "attention", "meet", "O", "meet", "LN2", "FC", "meet", "PROJ", "meet"]
    for layer in range(min(layers, 21)):
        row = t[layer * 12:layer * 12 + 13]
        if 0 in row:
            break
        print(f"layer {layer}: " + " ".join(f"{n}={(b - a) / 1e3:.1f}" for n, a, b in zip(names, row, row[1:])) +
              f" | total {(row[12] - row[0]) / 1e3:.1f} us")


def main():
    from cbis_b200.kernels import ops
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["decode_attn", "prefill_attn", "gemm", "gemm_tc", "gemm_f32", "layernorm", "sample",
                                                    "decode_layers_phases"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="prefill_attn: the path")
    ap.add_argument("--chunks", type=int, default=-1, help="prefill_attn: key chunks (-1: the engine's own choice, 1: none)")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--ctx", type=int, default=1536)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0, help="0: the engine's own choice")
    ap.add_argument("--layers", type=int, default=24, help="distinct weight/cache buffers per timed call")
    ap.add_argument("--act", default="gelu_erf", choices=["none", "gelu_erf", "gelu_tanh"], help="gemm_tc: the fused activation")
    ap.add_argument("--accumulate", action="store_true", help="gemm_tc: 32-bit result added into the output (TMA reduction)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--reps", type=int, default=20)
    a = ap.parse_args()
    if a.op == "decode_layers_phases":
        return decode_layers_phases(a.rows, a.ctx, a.layers)
    dev, M, L = "cuda", a.rows, a.layers
    torch.manual_seed(0)
    if a.op == "gemm":
        W = [torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(L)]
        x = torch.randn(M, a.k, device=dev, dtype=torch.bfloat16)
        bias = torch.randn(a.n, device=dev)
        out = torch.empty(M, a.n, device=dev, dtype=torch.bfloat16)

        def fn():
            for l in range(L):
                ops.gemm_small_m(x, W[l], bias, None, out)

        def lib():
            for l in range(L):
                torch.mm(x, W[l].t(), out=out)
        mb = a.n * a.k * 2 / 1e6
        t = timed(fn, not a.no_graph, a.reps) / L
        tl = timed(lib, not a.no_graph, a.reps) / L

        def few():
            for l in range(L):
                ops.gemm_few_rows(x, W[l], bias, None, out, a.splits)
        try:
            tf = timed(few, not a.no_graph, a.reps) / L
        except ops.KernelError:          # a split it does not take at this size
            tf = float("nan")

        print(f"gemm M={M} N={a.n} K={a.k}: {mb:.1f} MB  mma.sync {t:.2f} us ({mb / t:.2f} TB/s)  tcgen05 swapped {tf:.2f} us "
              f"({mb / tf:.2f} TB/s)  library {tl:.2f} us ({mb / tl:.2f} TB/s)  flag {ops.tcgen05_error_flag(dev).item()}")
    elif a.op == "gemm_tc":
        x = torch.randn(M, a.k, device=dev, dtype=torch.bfloat16)
        W = [torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(min(L, 4))]
        bias = torch.randn(a.n, device=dev)
        out = torch.empty(M, a.n, device=dev, dtype=torch.bfloat16)
        if a.accumulate:         # the result added into 32-bit rows (attention output, feed-forward output of a prompt)
            out = torch.zeros(M, a.n, device=dev)
            a.act = "none"

        def fn():
            for w in W:
                ops.gemm_tcgen05(x, w, bias, a.act, out, accumulate=a.accumulate)

        def lib():
            for w in W:
                if a.accumulate:
                    torch.mm(x, w.t(), out_dtype=torch.float32)
                else:
                    torch.mm(x, w.t(), out=out)
        fl = 2.0 * M * a.n * a.k
        t = timed(fn, not a.no_graph, a.reps) / len(W)
        tl = timed(lib, not a.no_graph, a.reps) / len(W)
        print(f"gemm_tc M={M} N={a.n} K={a.k}: tcgen05 with bias+{a.act} {t:.1f} us ({fl / t / 1e6:.0f} TFLOP/s)  "
              f"library, no epilogue {tl:.1f} us ({fl / tl / 1e6:.0f} TFLOP/s)  error flag {ops.tcgen05_error_flag(dev).item()}")
    elif a.op == "gemm_f32":
        x = torch.randn(M, a.k, device=dev)
        W = [torch.randn(a.n, a.k, device=dev) * 0.02 for _ in range(min(L, 4))]
        bias = torch.randn(a.n, device=dev)
        out = torch.empty(M, a.n, device=dev)
        fl = 2.0 * M * a.n * a.k
        for name, variant in (("cp.async kernel", 0), ("older tiled kernels", 1)):
            def fn():
                for w in W:
                    ops.linear_f32(x, w, bias, a.act if a.act != "none" else None, out, w_is_nk=True, variant=variant)
            t = timed(fn, not a.no_graph, a.reps) / len(W)
            print(f"gemm_f32 M={M} N={a.n} K={a.k} {name}: {t:.1f} us ({fl / t / 1e6:.1f} TFLOP/s)")
    elif a.op == "layernorm":
        x = torch.randn(M, a.k, device=dev)
        delta = torch.randn(M, a.k, device=dev)
        gm, bt = torch.ones(a.k, device=dev), torch.zeros(a.k, device=dev)
        out = torch.empty(M, a.k, device=dev, dtype=torch.bfloat16)

        def fn():
            for l in range(L):
                ops.add_layernorm(x, delta, bt, gm, bt, 1e-5, out)
        print(f"add_layernorm rows={M} width={a.k}: {timed(fn, not a.no_graph, a.reps) / L:.2f} us")
    elif a.op == "sample":
        lg = torch.randn(M, a.n, device=dev)
        out = torch.empty(M, dtype=torch.int32, device=dev)

        def fn():
            for l in range(L):
                ops.sample(lg, None, None, out)
        print(f"sample rows={M} vocab={a.n}: {timed(fn, not a.no_graph, a.reps) / L:.2f} us")
    elif a.op == "prefill_attn":
        # the last `rows` tokens of one request of `ctx` tokens (a portion of a prompt behind ctx - rows cached tokens)
        H, hd, ps, ctx = a.heads, a.head_dim, a.page_size, a.ctx
        dt = torch.float32 if a.dtype == "float32" else torch.bfloat16
        L = min(L, 4)
        nblk = -(-ctx // ps)
        kc = torch.randn(L, nblk, H, ps, hd, device=dev, dtype=dt)
        vc = torch.randn_like(kc)
        bt_ = torch.randperm(nblk, device=dev).int().view(1, nblk).contiguous()
        q = torch.randn(M, H * hd, device=dev, dtype=dt)
        out = torch.empty_like(q)
        cu = torch.tensor([0, M], dtype=torch.int32, device=dev)
        start = torch.tensor([ctx - M], dtype=torch.int32, device=dev)
        pos = torch.arange(ctx - M, ctx, dtype=torch.int32, device=dev)
        chunks = ops.prefill_key_chunks(-(-M // 64), H, 1, ctx)
        if a.chunks == 1:
            chunks = (1, 0)
        elif a.chunks > 1:
            keys = 64
            while keys * a.chunks < ctx:
                keys *= 2
            chunks = (-(-ctx // keys), keys)
        partial = torch.empty(max(1, M * H * chunks[0] * (hd + 4)), device=dev)
        fl = 4.0 * H * hd * (M * (ctx - M) + M * (M + 1) / 2)
        forms = []
        if dt == torch.float32:
            forms.append(("32-bit tiled", lambda l: ops.paged_prefill_f32(q, kc[l], vc[l], bt_, cu, start, out, 0, 1, M, H, H, hd, ps,
                                                                         hd ** -0.5, 0, chunks, partial, pos, 0, M)))
        else:
            forms.append(("mma.sync tiled", lambda l: ops.paged_prefill_bf16(q, kc[l], vc[l], bt_, cu, start, out, 0, 1, M, H, H, hd,
                                                                            ps, hd ** -0.5, 0, chunks, partial, pos, 0, M)))
            if hd in (64, 128) and 8 <= ps <= 128:
                ch5 = ops.prefill_key_chunks(-(-M // 128), H, 1, ctx, 2, 2, 8192) if a.chunks < 0 else chunks
                part5 = torch.empty(max(1, M * H * ch5[0] * (hd + 4)), device=dev)
                forms.append((f"tcgen05 (key chunks {ch5[0]} x {ch5[1]})",
                              lambda l: ops.paged_prefill_tc5(q, kc[l], vc[l], bt_, cu, start, out, 0, 1, M, H, H, hd, ps,
                                                              hd ** -0.5, 0, ch5, part5, pos, 0, M)))
        print(f"prefill_attn {a.dtype} rows={M} ctx={ctx} heads={H} head_dim={hd} page={ps}: {fl / 1e9:.2f} GFLOP, "
              f"key chunks {chunks[0]} x {chunks[1]}")
        for name, form in forms:
            def fn():
                for l in range(L):
                    form(l)
            t = timed(fn, not a.no_graph, a.reps) / L
            print(f"   {name}: {t:.1f} us ({fl / t / 1e6:.1f} TFLOP/s)")
        print(f"   error flag {ops.tcgen05_error_flag(dev).item()}")
    else:
        H, hd, ps, ctx = a.heads, a.head_dim, a.page_size, a.ctx
        nblk = -(-ctx // ps)
        npages = M * nblk
        kc = torch.randn(L, npages, H, ps, hd, device=dev, dtype=torch.bfloat16)
        vc = torch.randn_like(kc)
        mb_ = max(nblk, 128)
        bt_ = (torch.arange(M * mb_, dtype=torch.int32, device=dev).view(M, mb_) % nblk
               + (torch.arange(M, dtype=torch.int32, device=dev) * nblk)[:, None]).int().contiguous()
        d = H * hd
        qkv = torch.randn(M, 3 * d, device=dev, dtype=torch.bfloat16)
        rs = torch.arange(M, dtype=torch.int32, device=dev)
        pos = torch.full((M,), ctx - 1, dtype=torch.int32, device=dev)
        sm = (bt_[:, (ctx - 1) // ps] * ps + (ctx - 1) % ps).int().contiguous()
        out = torch.empty(M, d, device=dev, dtype=torch.bfloat16)
        ns = a.splits or ops.decode_splits(M, H, ctx)
        scratch = torch.empty(max(1, ops.decode_scratch_floats(M, H, hd, ns)), device=dev)
        cnt = torch.zeros(M * H, dtype=torch.int32, device=dev)

        def fn():
            for l in range(L):
                ops.paged_decode_bf16(qkv, d, 2 * d, kc[l], vc[l], bt_, rs, pos, sm, out, scratch, cnt, H, H, hd, ps,
                                      hd ** -0.5, 0, ns)
        mb = M * ctx * d * 2 * 2 / 1e6
        t = timed(fn, not a.no_graph, a.reps) / L
        print(f"decode_attn rows={M} ctx={ctx} heads={H} head_dim={hd} splits={ns}: {mb:.1f} MB  {t:.2f} us ({mb / t:.2f} TB/s)")


if __name__ == "__main__":
    main()
