"""Python faces of the CUDA kernels: argument checks, then a ctypes call on the current stream.

Every function works on CUDA tensors only and raises if the kernel library is missing;
nothing here falls back to torch operators.  The dense matrix products of the bfloat16
path go to the library GEMM (cuBLASLt through ``torch``), as the reference's go to
``cublasSgemm`` (kernels/linear.cu:25-27); everything around them is this package's own.
"""
from __future__ import annotations

import ctypes
import weakref
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from .library import kernels, optional_kernels

F32, BF16 = 0, 1
ACT = {None: 0, "none": 0, "gelu_erf": 1, "gelu_tanh": 2}

_STATUS = {-1: "unsupported dtype", -2: "a size that the kernel does not take",
           -3: "misaligned pointer or stride", -4: "size too large for this kernel"}


class KernelError(RuntimeError):
    pass


_launches = 0


def launch_count() -> int:
    """Kernel launches of this package since the last reset (captured launches count once, at capture)."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def _check(status: int, what: str, detail: str = "", launches: int = 1) -> None:
    global _launches
    if status == 0:
        _launches += launches
        return
    if status < 0:
        raise KernelError(f"{what}: {_STATUS.get(status, 'error %d' % status)}{(' (' + detail + ')') if detail else ''}")
    raise KernelError(f"{what}: CUDA error {status} at launch {detail}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is not supported (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream of the current device as a raw handle.  torch.cuda.current_stream() builds a Python
    object through several layers (about 5 us, a third of the host's share of a launch); the two calls below are
    what it ends in."""
    if _raw_stream is not None and _raw_device is not None:
        return c_void_p(_raw_stream(_raw_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def raw_stream_handle():
    """The current stream's raw handle (an int), or None where torch does not offer the fast call."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return None


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only; there is no CPU path")


NORM_MAX_WIDTH = 200 * 1024 // 4 - 33     # the widest row add_layernorm takes (cbis_norm_max_width() says the same)
ATTENTION_MAX_HEAD_DIM = 256             # the general attention kernel's limit; the tiled ones take less and say so


def embed_pos_add(tokens, positions, wte, wpe, out, err, multiplier: float = 1.0):
    """out[r] = wte[tokens[r]] * multiplier + wpe[positions[r]] in 32-bit; err (int32[1]) is set on a bad index."""
    _need_cuda(tokens, positions, wte, wpe, out, err)
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and wte.is_contiguous()
    assert tokens.dtype == torch.int32 and positions.dtype == torch.int32
    st = kernels().cbis_embed_pos_add(_ptr(tokens), _ptr(positions), _ptr(wte), _ptr(wpe), _ptr(out),
                                      c_int(T), c_int(d), c_int(wte.shape[0]),
                                      c_int(wpe.shape[0] if wpe is not None else 0),
                                      c_int(dtype_code(wte.dtype)), c_float(multiplier), _ptr(err), _stream())
    _check(st, "embed_pos_add", f"T={T} d={d}")


def add_layernorm(x, delta, delta_bias, gamma, beta, eps, out, rows=None):
    """x += delta + delta_bias (32-bit, in place unless ``rows``); out = LayerNorm(x) * gamma + beta.

    ``rows`` (int32[R]) selects source rows: out[r] = LN(x[rows[r]] + ...), x is left as it is.
    ``gamma`` None: no normalisation, out = x + delta + delta_bias in ``out``'s dtype."""
    _need_cuda(x, delta, delta_bias, gamma, beta, out, rows)
    d = x.shape[-1]
    R = rows.shape[0] if rows is not None else x.shape[0]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape[-1] == d
    assert gamma is None or gamma.dtype == torch.float32
    assert beta is None or (gamma is not None and beta.dtype == torch.float32)
    assert delta is None or (delta.is_contiguous() and delta.shape == x.shape)
    assert delta_bias is None or delta_bias.dtype == torch.float32
    assert out.shape[0] >= R
    st = kernels().cbis_add_layernorm(_ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype) if delta is not None else 0),
                                      _ptr(delta_bias), _ptr(gamma), _ptr(beta), c_float(eps), _ptr(out),
                                      c_int(dtype_code(out.dtype)), _ptr(rows), c_int(R), c_int(d), _stream())
    _check(st, "add_layernorm", f"rows={R} width={d}")


def add_delta(x, delta, delta_bias):
    """x += delta + delta_bias (the 32-bit residual stream, in place): what a layer left pending, added without a
    norm for a part that normalises inside its own kernel."""
    add_layernorm(x, delta, delta_bias, None, None, 0.0, torch.empty_like(x, dtype=torch.bfloat16))


def bias_act(x, bias, act):
    """x = act(x + bias) in place, arithmetic in 32-bit."""
    _need_cuda(x, bias)
    M, N = x.shape
    assert x.is_contiguous()
    st = kernels().cbis_bias_act(_ptr(x), _ptr(bias), c_int(ACT[act]), c_int(M), c_int(N),
                                 c_int(dtype_code(x.dtype)), _stream())
    _check(st, "bias_act", f"M={M} N={N}")


def scale_soft_cap(x, scale: float, cap: float):
    """x = cap * tanh(x * scale / cap) if cap > 0 else x * scale, in place on 32-bit values."""
    _need_cuda(x)
    M, N = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    st = kernels().cbis_scale_soft_cap(_ptr(x), c_float(scale), c_float(cap), c_int(M), c_int(N), _stream())
    _check(st, "scale_soft_cap", f"M={M} N={N}")


def bias_act_out(src, bias, act, dst):
    """dst = act(src + bias): 32-bit sums in, activations out with one rounding."""
    _need_cuda(src, bias, dst)
    M, N = src.shape
    assert src.dtype == torch.float32 and src.is_contiguous() and dst.is_contiguous() and dst.shape == src.shape
    st = kernels().cbis_bias_act_out(_ptr(src), _ptr(bias), c_int(ACT[act]), _ptr(dst), c_int(M), c_int(N),
                                     c_int(dtype_code(dst.dtype)), _stream())
    _check(st, "bias_act_out", f"M={M} N={N}")


def linear_f32(x, w, bias, act, out, w_is_nk=False, variant=0):
    """out = act(x @ W + bias) on the FP32 units; W is [K,N], or [N,K] with ``w_is_nk``.  ``variant`` 1 keeps the
    cp.async kernel out (all kernels sum along k in the same order and give the same bits)."""
    _need_cuda(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0] if w_is_nk else w.shape[1]
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32
    assert (w.shape[1] if w_is_nk else w.shape[0]) == K and w.is_contiguous()
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] >= M and out.shape[1] == N
    st = kernels().cbis_linear_f32(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), c_int(M), c_int(N), c_int(K),
                                   c_int(1 if w_is_nk else 0), c_int(ACT[act]), c_int(x.stride(0)),
                                   c_int(out.stride(0)), c_int(variant), _stream())
    _check(st, "linear_f32", f"M={M} N={N} K={K}")


SMALL_M = int(__import__("os").environ.get("CBIS_SMALL_M", "16"))      # rows up to which the weight-streaming kernel takes a bfloat16 product (it can take 64; measured at batch 32 and 64 of the 1.3B sizes: the library product is 27-33 % faster per step there)


_next_weight = {}      # data_ptr of a weight -> weak reference to the weight used after it
PREFETCH_AHEAD = int(__import__("os").environ.get("CBIS_PREFETCH_AHEAD", "1"))   # products ahead (measured: 1 is best, 6,305 tok/s at batch 8; 0: 6,014, 2: 6,205, 3: 5,975)
PREFETCH_CAP = 64 << 20   # bytes of a successor's weights brought into L2 ahead of time (L2 holds 126 MB)


def add_weight_order(weights) -> None:
    """Tells the few-rows product in which order a decode step uses its weights (a cycle: after the
    last comes the first of the next step), so that each product can prefetch its successor's weights
    into L2 while it runs.  Only weak references are kept: a freed model's entries die with it."""
    import weakref
    ws = [w for w in weights if w is not None and w.is_cuda and w.dtype == torch.bfloat16]
    ahead = PREFETCH_AHEAD % max(1, len(ws))
    for a, b in zip(ws, ws[ahead:] + ws[:ahead]):
        if a.data_ptr() != b.data_ptr():
            _next_weight[a.data_ptr()] = weakref.ref(b)
    for k in [k for k, r in _next_weight.items() if r() is None]:
        del _next_weight[k]


def _next_of(w_nk):
    """(pointer, bytes) of the weight used after ``w_nk``, for the L2 prefetch the weight-streaming kernels issue."""
    ref = _next_weight.get(w_nk.data_ptr())
    nxt = ref() if ref is not None else None
    return _ptr(nxt), ctypes.c_ulonglong(min(nxt.numel() * 2, PREFETCH_CAP) if nxt is not None else 0)


SMALL_WEIGHT = 1 << 20


def gemm_small_m(x, w_nk, bias, act, out, accumulate=False):
    """out = act(x @ w_nk^T + bias) for up to 64 rows of bfloat16, 32-bit accumulation (weight streaming).
    ``accumulate`` (32-bit ``out`` only): the result is added to what ``out`` holds."""
    _need_cuda(x, w_nk, bias, out)
    M, K = x.shape
    N = w_nk.shape[0]
    assert x.dtype == torch.bfloat16 and w_nk.dtype == torch.bfloat16 and w_nk.is_contiguous() and w_nk.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N)
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm_small_m: a product is added into a 32-bit matrix only")
    nxt, nbytes = _next_of(w_nk)
    st = kernels().cbis_gemm_small_m_bf16(_ptr(x), c_int(x.stride(0)), _ptr(w_nk), _ptr(bias), _ptr(out),
                                          c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(ACT[act]),
                                          c_int(dtype_code(out.dtype)), nxt, nbytes, c_int(1 if accumulate else 0), _stream())
    _check(st, "gemm_small_m", f"M={M} N={N} K={K}")


LN_LINEAR_MAX_ROWS = 8


_ln_max_k = []


def ln_linear_max_k() -> int:
    if not _ln_max_k:
        _ln_max_k.append(int(kernels().cbis_gemm_ln_small_m_max_k()))
    return _ln_max_k[0]


# 1: decode steps of up to 8 rows normalise inside the product's kernel and add the layer's results straight into the
# residual stream (5 kernels a layer instead of 7).  Off by default: measured at the 1.3B sizes it is the slower form,
# 0.941 ms against 0.900 per step at batch 1 and 1.258 against 1.220 at batch 8; with programmatic dependent launch the
# separate norm kernel already runs under the next product's first weight loads.
USE_LN_LINEAR = __import__("os").environ.get("CBIS_LN_LINEAR", "0") == "1"


def ln_linear_takes(ctx, norm, w_nk) -> bool:
    """Whether this step's rows can go through ``ln_linear`` with this norm and weight: a bfloat16 step of up to 8
    rows, a LayerNorm with weight and bias over rows the kernel takes."""
    if not USE_LN_LINEAR or ctx.dtype != torch.bfloat16 or not 0 < ctx.n_rows <= LN_LINEAR_MAX_ROWS:
        return False
    if norm.as_layernorm() is None:
        return False
    if w_nk is None or not w_nk.is_cuda or w_nk.dtype != torch.bfloat16:
        return False
    K = w_nk.shape[1]
    return K == norm.as_layernorm()[0].numel() and K % 8 == 0 and K <= ln_linear_max_k()


def ln_linear(x, gamma, beta, eps, w_nk, bias, act, out):
    """out = act(LayerNorm(x) @ w_nk^T + bias) for up to 8 rows: x the 32-bit rows, statistics in 32-bit, the
    normalised rows rounded to bfloat16 (as the separate norm kernel hands them to the product), w_nk bfloat16."""
    _need_cuda(x, gamma, beta, w_nk, bias, out)
    M, K = x.shape
    N = w_nk.shape[0]
    assert x.dtype == torch.float32 and w_nk.dtype == torch.bfloat16 and w_nk.is_contiguous() and w_nk.shape[1] == K
    assert gamma.dtype == torch.float32 and beta.dtype == torch.float32 and gamma.numel() == K and beta.numel() == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N)
    nxt, nbytes = _next_of(w_nk)
    st = kernels().cbis_gemm_ln_small_m(_ptr(x), c_int(x.stride(0)), _ptr(gamma), _ptr(beta), ctypes.c_float(eps),
                                        _ptr(w_nk), _ptr(bias), _ptr(out), c_int(out.stride(0)), c_int(M), c_int(N),
                                        c_int(K), c_int(ACT[act]), c_int(dtype_code(out.dtype)), nxt, nbytes, _stream())
    _check(st, "ln_linear", f"M={M} N={N} K={K}")


def gemm_few_rows(x, w_nk, bias, act, out, ksplit=0):
    """out = act(x @ w_nk^T + bias) for up to 64 rows of bfloat16 on the tcgen05 tensor cores with the operands
    swapped: the weights stream through shared memory by TMA, K split over the blocks of a cluster
    (``ksplit`` 0: the launcher's choice)."""
    _need_cuda(x, w_nk, bias, out)
    M, K = x.shape
    N = w_nk.shape[0]
    assert x.dtype == torch.bfloat16 and w_nk.dtype == torch.bfloat16 and w_nk.is_contiguous() and w_nk.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N)
    ref = _next_weight.get(w_nk.data_ptr())
    nxt = ref() if ref is not None else None
    st = kernels().cbis_gemm_few_rows_tc5(_ptr(x), c_int(x.stride(0)), _ptr(w_nk), _ptr(bias), _ptr(out),
                                          c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(ACT[act]),
                                          c_int(dtype_code(out.dtype)), c_int(ksplit), _ptr(nxt),
                                          ctypes.c_ulonglong(min(nxt.numel() * 2, PREFETCH_CAP) if nxt is not None else 0),
                                          _ptr(tcgen05_error_flag(x.device)), _stream())
    _check(st, "gemm_few_rows", f"M={M} N={N} K={K} ksplit={ksplit}")


_tc_error = {}
USE_TCGEN05 = __import__("os").environ.get("CBIS_TCGEN05", "1") != "0"
USE_KEY_CHUNKS = __import__("os").environ.get("CBIS_KEY_CHUNKS", "1") != "0"   # 0: attention kernels never cut the keys over more blocks
USE_TILED_F32 = __import__("os").environ.get("CBIS_TILED_F32", "1") != "0"   # 0: the general kernel for 32-bit prompts
USE_FEW_ROWS = USE_TCGEN05 and __import__("os").environ.get("CBIS_FEW_ROWS", "1") != "0"


def raise_if_kernel_errors(device="cuda") -> None:
    """Reads the error flag of the tcgen05 product (a 4-byte copy: call it where the host waits anyway)."""
    key = torch.device(device).index or 0
    flag = _tc_error.get(key)
    if flag is not None:
        code = int(flag.item())
        if code:
            flag.zero_()
            _tc_pending.pop(key, None)      # a copy of the flag asked for earlier would report the same event again
            raise KernelError(f"a bounded wait inside a TMA kernel ran out (code {code}: 1-6 and 21-24 the tcgen05 "
                              f"product, 11-19 the prefill attention, 31-34 the persistent decode kernel); the step's "
                              f"results are invalid")



_tc_pending = {}     # device index -> (pinned copy of the flag, event recorded after the copy)


def poll_kernel_errors(device="cuda") -> None:
    """The same check without making the host wait: looks at the copy of the flag that the call before this one
    asked for (if that copy has been made by now) and asks for a new one behind the work queued so far.  A step
    whose wait ran out is therefore reported one or two calls late, but steps keep overlapping with the host."""
    key = torch.device(device).index or 0
    flag = _tc_error.get(key)
    if flag is None:
        return
    pending = _tc_pending.get(key)
    if pending is not None:
        host, event = pending
        if not event.query():
            return                      # the copy asked for earlier has not run yet: ask again next time
        code = int(host[0])
        if code:
            _tc_pending.pop(key, None)
            flag.zero_()
            raise KernelError(f"a bounded wait inside a TMA kernel ran out (code {code}: 1-6 and 21-24 the tcgen05 "
                              f"product, 11-19 the prefill attention, 31-34 the persistent decode kernel); the results "
                              f"of a recent step are invalid")
    else:
        host, event = torch.zeros(1, dtype=torch.int32).pin_memory(), torch.cuda.Event()
    host.copy_(flag, non_blocking=True)
    event.record()
    _tc_pending[key] = (host, event)


def tcgen05_error_flag(device) -> torch.Tensor:
    """int32[1] on the device that the tcgen05 product sets when one of its bounded waits runs out."""
    key = torch.device(device).index or 0
    if key not in _tc_error:
        _tc_error[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_error[key]


def gemm_tcgen05(x, w_nk, bias, act, out, spin_limit: int = 0, starve: bool = False, accumulate: bool = False):
    """out = act(x @ w_nk^T + bias) on the tcgen05 tensor cores (TMA operands, accumulator in tensor
    memory, bias and activation on the 32-bit sums).  bfloat16, K a multiple of 8.
    ``spin_limit`` (0: the service limit) bounds every wait inside the kernel; ``starve`` (up to 128 rows,
    for the test of the give-up path) makes the kernel request no operands, so that its waits run out:
    it then sets the error flag (``tcgen05_error_flag``), frees its tensor memory and returns.
    ``accumulate`` (32-bit ``out``, more than 128 rows): the result is added into ``out`` (a TMA reduction)."""
    _need_cuda(x, w_nk, bias, out)
    M, K = x.shape
    N = w_nk.shape[0]
    assert x.dtype == torch.bfloat16 and w_nk.dtype == torch.bfloat16 and w_nk.is_contiguous() and w_nk.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N)
    st = kernels().cbis_gemm_tcgen05_bf16_ex(_ptr(x), c_int(x.stride(0)), _ptr(w_nk), _ptr(bias), _ptr(out),
                                             c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(ACT[act]),
                                             c_int(dtype_code(out.dtype)), _ptr(tcgen05_error_flag(x.device)), _stream(),
                                             ctypes.c_uint(spin_limit), c_int(1 if starve else 0), c_int(1 if accumulate else 0))
    _check(st, "gemm_tcgen05", f"M={M} N={N} K={K}" + (" accumulate" if accumulate else ""))


# 1: products whose result is added to the residual stream (attention output, feed-forward output) add it there
# themselves where the TMA + tcgen05 product has tiles enough (prompts): bias and sum in its epilogue, a TMA reduction
# into the 32-bit rows; 0: the library product writes 32-bit sums and the next norm adds them.
USE_LINEAR_ADD = __import__("os").environ.get("CBIS_LINEAR_ADD", "1") != "0"
USE_TCGEN05_PAIR = __import__("os").environ.get("CBIS_TCGEN05_PAIR", "1") != "0"    # the kernel library reads the same variable


def linear_add_takes(x, w_nk, residual) -> bool:
    """Whether ``linear_add`` takes this product: bfloat16 rows enough for the tcgen05 product's tiles, aligned."""
    if not (USE_LINEAR_ADD and USE_TCGEN05 and USE_TCGEN05_PAIR) or residual is None or x.dtype != torch.bfloat16:
        return False
    M, K = x.shape
    N = w_nk.shape[0]
    return (M > 128 and tc_tiles(M, N) and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and residual.dtype == torch.float32 and residual.stride(0) % 4 == 0 and residual.data_ptr() % 16 == 0 and N >= 16)


def linear_add(x, w_nk, bias, residual) -> None:
    """residual += x @ w_nk^T + bias (32-bit residual rows, bfloat16 operands, 32-bit sums)."""
    gemm_tcgen05(x, w_nk, bias, None, residual, accumulate=True)


def linear(x, w_nk, bias, act=None, out_dtype=None):
    """act(x @ W^T + bias) with W stored [N, K] (K contiguous).

    32-bit inputs: this package's FFMA kernel (no reduced-precision matrix mode).  bfloat16
    inputs: up to 16 rows go to the weight-streaming mma.sync kernel; a head over a vocabulary at
    17..64 rows goes to the TMA + tcgen05 kernel with swapped operands; more rows with a bias or an
    activation go to the TMA + tcgen05 kernel; all apply bias and activation to the 32-bit sums and
    round once.  More rows without an epilogue go to the library GEMM."""
    M, K = x.shape
    N = w_nk.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        linear_f32(x, w_nk, bias, act, out, w_is_nk=True)
        return out
    _need_cuda(x, w_nk)
    out_dtype = out_dtype or x.dtype
    aligned = K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
    # up to 16 rows; up to 64 where the weight is small (a million elements: any kernel takes a few microseconds, and the
    # library's call costs the host 15-60 us, this one 6, with the epilogue inside)
    if aligned and (M <= SMALL_M or (M <= 64 and N * K <= SMALL_WEIGHT)):
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        gemm_small_m(x, w_nk, bias, act, out)
        return out
    plain = bias is None and not ACT[act]
    if USE_FEW_ROWS and M <= 64 and aligned and plain and (N % 8 != 0 or N >= 32768):
        # a head over a vocabulary at 17..64 rows: the library product is slow when N is no multiple of 8 (212 us at
        # 64 rows of 50,257 x 2,048), the TMA + tcgen05 kernel with swapped operands streams it at 4.9 TB/s (42 us).
        # (Up to 16 rows, and inside a layer, the mma.sync kernel stays: the tcgen05 one is as fast alone and keeps
        # more bytes in flight on large matrices, 5.8 TB/s on 134 MB against 4.4, but its blocks need 90 KB of
        # shared memory each and cannot start beside the blocks of the kernel before them: in the chain of a
        # decode step that costs more than it wins, 1.75 ms per step against 1.29.)
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        gemm_few_rows(x, w_nk, bias, act, out)
        return out
    if out_dtype != torch.float32 and plain:
        return torch.mm(x, w_nk.t())
    if USE_LIBRARY_EPILOGUE and out_dtype == torch.bfloat16 and bias is not None and ACT[act] in (0, 2) and not (USE_TCGEN05 and tc_tiles(M, N)):
        # 17 rows up to where the tcgen05 product has tiles enough: the library product with the library's own epilogue
        # (bias, or bias and tanh GELU, applied to its 32-bit sums, rounded once) instead of 32-bit sums and a kernel
        # for the epilogue: 9.1 -> 6.6 us (bias) and 9.2 -> 8.0 us (bias, GELU) on 64 x 6400 x 1600.  It wants the
        # bias in bfloat16: taken only where that copy is exact.  The GELU form only with every operand aligned: on
        # other sizes the library adds the bias, rounds, and then applies the activation to the rounded values.
        b16 = _bias_bf16(bias)
        if b16 is not None:
            if ACT[act] == 0:
                return torch.addmm(b16, x, w_nk.t())
            if aligned and N % 8 == 0 and x.is_contiguous():
                return torch._addmm_activation(b16, x, w_nk.t(), use_gelu=True)
    if (USE_TCGEN05 and tc_tiles(M, N) and out_dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        # a product with an epilogue: TMA + tcgen05 with bias and activation applied to the sums in tensor memory
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        gemm_tcgen05(x, w_nk, bias, act, out)
        return out
    acc = torch.mm(x, w_nk.t(), out_dtype=torch.float32)
    if out_dtype == torch.float32:
        if not plain:
            bias_act(acc, bias, act)
        return acc
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    bias_act_out(acc, bias, act, out)     # one rounding, as in the few-rows kernel
    return out


def tc_tiles(M: int, N: int) -> bool:
    """Whether the 128x256 tiles of the TMA + tcgen05 product cover most of the 148 SMs."""
    return -(-M // 128) * -(-N // 256) >= 96


USE_LIBRARY_EPILOGUE = __import__("os").environ.get("CBIS_LIBRARY_EPILOGUE", "1") != "0"
_bias16 = {}     # data_ptr of a 32-bit bias -> (weak reference to it, its bfloat16 copy or None if the copy is not exact)


def _bias_bf16(bias):
    key = bias.data_ptr()
    hit = _bias16.get(key)
    if hit is not None and hit[0]() is bias:
        return hit[1]
    b16 = bias.to(torch.bfloat16)
    if not torch.equal(b16.float(), bias.float()):
        b16 = None
    if len(_bias16) > 4096:
        for k in [k for k, (r, _) in _bias16.items() if r() is None]:
            del _bias16[k]
    _bias16[key] = (weakref.ref(bias), b16)
    return b16


def kv_write(qkv, k_off, v_off, k_cache, v_cache, slot_mapping, n_kv_head, head_dim, page_size):
    """Rows of this step's K and V (columns k_off.. and v_off.. of qkv) go to their token slots."""
    _need_cuda(qkv, k_cache, v_cache, slot_mapping)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    assert slot_mapping.dtype == torch.int32 and slot_mapping.shape[0] >= T
    st = kernels().cbis_kv_write(_ptr(qkv), c_int(qkv.stride(0)), c_int(k_off), c_int(v_off), _ptr(k_cache),
                                 _ptr(v_cache), _ptr(slot_mapping), c_int(T), c_int(n_kv_head), c_int(head_dim),
                                 c_int(page_size), c_int(dtype_code(qkv.dtype)), _stream())
    _check(st, "kv_write", f"T={T} kv_heads={n_kv_head} head_dim={head_dim} page={page_size}")


def generic_key_chunks(rows: int, n_head: int, max_context: int, head_dim: int):
    """(n_chunks, chunk_keys) for the general attention kernel (a warp per row and head): no cut (1, 0) when rows and
    heads alone give 16 warps to each of the 148 SMs, or the head size is no multiple of 4; else chunks of a power
    of two of keys, at least 256, that do."""
    want = -(-16 * 148 // max(1, rows * n_head))
    if want <= 1 or max_context <= 256 or head_dim % 4 or not USE_KEY_CHUNKS:
        return 1, 0
    chunk = 256
    while chunk * want < max_context:
        chunk *= 2
    n = -(-max_context // chunk)
    return (n, chunk) if n > 1 else (1, 0)


def paged_attention_generic(q, k_cache, v_cache, block_table, row_seq, positions, out, n_head, n_kv_head,
                            head_dim, page_size, scale, window=0, chunks=(1, 0), partial=None):
    """Attention of every row over its request's pages: keys max(0,p-window+1)..p for the query at p.
    ``chunks`` = (n, keys) from ``generic_key_chunks`` cuts every row's keys n ways over as many warps (every
    context below n * keys); ``partial`` then holds ``rows * n_head * n * (head_dim + 4)`` floats."""
    _need_cuda(q, k_cache, v_cache, block_table, row_seq, positions, out, partial)
    T = q.shape[0]
    if head_dim > 256:
        raise KernelError(f"attention: head_dim={head_dim} is above the kernel's limit of 256")
    if n_head % n_kv_head:
        raise KernelError(f"attention: n_head={n_head} is not a multiple of n_kv_head={n_kv_head}")
    assert q.stride(1) == 1 and out.stride(1) == 1 and block_table.dtype == torch.int32
    assert block_table.is_contiguous() and row_seq.dtype == torch.int32 and positions.dtype == torch.int32
    n_chunks, chunk_keys = chunks
    if n_chunks > 1:
        assert partial.dtype == torch.float32 and partial.numel() >= T * n_head * n_chunks * (head_dim + 4)
        if out.stride(0) % 4 or out.data_ptr() % 16:
            n_chunks, chunk_keys = 1, 0
    st = kernels().cbis_paged_attention_generic(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(row_seq), _ptr(positions), _ptr(out), c_int(out.stride(0)), c_int(T), c_int(n_head), c_int(n_kv_head),
        c_int(head_dim), c_int(page_size), c_float(scale), c_int(window), c_int(dtype_code(q.dtype)),
        c_int(n_chunks), c_int(chunk_keys), _ptr(partial), _stream())
    _check(st, "paged_attention_generic", f"T={T} heads={n_head}/{n_kv_head} head_dim={head_dim} page={page_size} "
                                          f"chunks={n_chunks}x{chunk_keys}")


def decode_splits(rows: int, n_head: int, max_context: int) -> int:
    """How many ways the decode kernel splits a request's keys.  A block takes (row, head, split) and
    4 blocks fit on each of the 148 SMs: split as far as one round of blocks allows, in pieces of at
    least 32 keys, at most 32 ways; with a round or more of (row, head) pairs there is no split."""
    slots = 4 * 148
    pairs = max(1, rows * n_head)
    return max(1, min(slots // pairs, 32, max(1, max_context // 32)))


def decode_scratch_floats(rows: int, n_head: int, head_dim: int, nsplit: int) -> int:
    """Floats of scratch for the decode kernel's partial results."""
    return rows * n_head * nsplit * (head_dim + 2) if nsplit > 1 else 0


def paged_decode_bf16(qkv, k_off, v_off, k_cache, v_cache, block_table, row_seq, positions, slot_mapping, out,
                      scratch, counters, n_head, n_kv_head, head_dim, page_size, scale, window, nsplit):
    """Decode attention (one query per row) with the keys split ``nsplit`` ways; with ``k_off >= 0`` the
    current token's key/value are taken from ``qkv`` and stored into the cache by the same kernel.
    ``scratch``: ``decode_scratch_floats`` floats; ``counters``: rows*n_head int32, zero before the
    first launch (every launch leaves them zero)."""
    _need_cuda(qkv, k_cache, v_cache, block_table, row_seq, positions, slot_mapping, out, scratch, counters)
    rows = qkv.shape[0]
    if head_dim % 8 or head_dim > 256:
        raise KernelError(f"decode attention: head_dim={head_dim} must be a multiple of 8, at most 256")
    assert qkv.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    if nsplit > 1:
        assert scratch.dtype == torch.float32 and scratch.numel() >= decode_scratch_floats(rows, n_head, head_dim, nsplit)
        assert counters.dtype == torch.int32 and counters.numel() >= rows * n_head
    st = kernels().cbis_paged_decode_bf16(
        _ptr(qkv), c_int(qkv.stride(0)), c_int(k_off), c_int(v_off), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
        c_int(block_table.shape[1]), _ptr(row_seq), _ptr(positions), _ptr(slot_mapping), _ptr(out),
        c_int(out.stride(0)), _ptr(scratch), _ptr(counters), c_int(rows), c_int(n_head), c_int(n_kv_head),
        c_int(head_dim), c_int(page_size), c_float(scale), c_int(window), c_int(nsplit), _stream())
    _check(st, "paged_decode_bf16", f"rows={rows} heads={n_head}/{n_kv_head} head_dim={head_dim} splits={nsplit}")


def paged_prefill_bf16(q, k_cache, v_cache, block_table, cu_rows, seg_start, out, seg0, n_seg, max_seg_rows,
                       n_head, n_kv_head, head_dim, page_size, scale, window=0, chunks=(1, 0), partial=None,
                       positions=None, row0=0, n_rows=0):
    """Attention of the segments seg0..seg0+n_seg-1 (runs of rows given by ``cu_rows``, first positions
    ``seg_start``) over their pages, on the tensor cores.  Head sizes 16, 32, ... 128, page sizes 2^k.
    ``chunks`` = (n, keys) from ``prefill_key_chunks`` cuts the keys n ways over more blocks (every context of the
    step below n * keys); ``partial`` then holds ``n_rows * n_head * n * (head_dim + 4)`` floats, ``positions`` the
    position of every row, ``row0`` and ``n_rows`` name the rows of these segments."""
    _need_cuda(q, k_cache, v_cache, block_table, cu_rows, seg_start, out, partial, positions)
    if head_dim % 16 or not 16 <= head_dim <= 128:
        raise KernelError(f"prefill attention: head_dim={head_dim} is no multiple of 16 up to 128 (the general kernel takes it)")
    if page_size & (page_size - 1):
        raise KernelError(f"prefill attention: page_size={page_size} is not a power of two (the general kernel takes it)")
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and block_table.is_contiguous()
    n_chunks, chunk_keys = chunks
    if n_chunks > 1:
        assert partial.dtype == torch.float32 and partial.numel() >= n_rows * n_head * n_chunks * (head_dim + 4)
        assert positions.dtype == torch.int32 and positions.numel() >= row0 + n_rows
    st = kernels().cbis_paged_prefill_bf16(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(cu_rows), _ptr(seg_start), _ptr(out), c_int(out.stride(0)), c_int(seg0), c_int(n_seg),
        c_int(max_seg_rows), c_int(n_head), c_int(n_kv_head), c_int(head_dim), c_int(page_size), c_float(scale),
        c_int(window), c_int(n_chunks), c_int(chunk_keys), _ptr(partial), _ptr(positions), c_int(row0), c_int(n_rows),
        _stream())
    _check(st, "paged_prefill_bf16", f"segments={n_seg} heads={n_head}/{n_kv_head} head_dim={head_dim} page={page_size} "
                                     f"chunks={n_chunks}x{chunk_keys}")


def prefill_key_chunks(row_tiles: int, n_head: int, n_seg: int, max_context: int, blocks_per_tile: int = 1,
                       blocks_per_sm: int = 8, min_chunk: int = 256):
    """(n_chunks, chunk_keys) for the tiled prefill attention kernels: no cut (1, 0) when (row tile, head, segment)
    alone give ``blocks_per_sm`` blocks to each of the 148 SMs; else chunks of a power of two of keys, at least
    ``min_chunk``, that do.  The tcgen05 kernel has two blocks per row tile and two per SM, and a block of it costs
    some 8 us before its first tile: it is cut only into chunks of 8,192 keys or more (measured at 512 rows, 16 heads
    of 128: 2,048 keys 32 us whole, 42 us in two chunks; 32,768 keys 385 us whole, 230 us in two, 291 us in eight)."""
    base = max(1, row_tiles * n_head * n_seg * blocks_per_tile)
    want = -(-blocks_per_sm * 148 // base)
    if want <= 1 or max_context <= min_chunk or not USE_KEY_CHUNKS:
        return 1, 0
    chunk = min_chunk
    while chunk * want < max_context:
        chunk *= 2
    n = -(-max_context // chunk)
    return (n, chunk) if n > 1 else (1, 0)


def paged_prefill_f32(q, k_cache, v_cache, block_table, cu_rows, seg_start, out, seg0, n_seg, max_seg_rows,
                      n_head, n_kv_head, head_dim, page_size, scale, window=0, chunks=(1, 0), partial=None,
                      positions=None, row0=0, n_rows=0):
    """The same attention as ``paged_prefill_bf16`` in true 32-bit (no tensor cores): a block takes 64 rows of one
    head and brings keys and values through shared memory once.  Head sizes 16, 32, ... 128, any page size;
    ``q`` and ``out`` in full row numbering.  ``chunks`` = (n, keys) from ``prefill_key_chunks`` cuts the keys n
    ways (every context of the step below n * keys); ``partial`` then holds ``n_rows * n_head * n * (head_dim + 4)``
    floats, ``positions`` the position of every row, ``row0`` and ``n_rows`` name the rows of these segments."""
    _need_cuda(q, k_cache, v_cache, block_table, cu_rows, seg_start, out, partial, positions)
    if head_dim % 16 or not 16 <= head_dim <= 128:
        raise KernelError(f"32-bit prefill attention: head_dim={head_dim} is no multiple of 16 up to 128 (the general kernel takes it)")
    assert q.dtype == torch.float32 and k_cache.dtype == torch.float32 and out.dtype == torch.float32
    assert q.stride(1) == 1 and out.stride(1) == 1 and block_table.is_contiguous() and k_cache.is_contiguous()
    n_chunks, chunk_keys = chunks
    if n_chunks > 1:
        assert partial.dtype == torch.float32 and partial.numel() >= n_rows * n_head * n_chunks * (head_dim + 4)
        assert positions.dtype == torch.int32 and positions.numel() >= row0 + n_rows
    st = kernels().cbis_paged_prefill_f32(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(cu_rows), _ptr(seg_start), _ptr(out), c_int(out.stride(0)), c_int(seg0), c_int(n_seg),
        c_int(max_seg_rows), c_int(n_head), c_int(n_kv_head), c_int(head_dim), c_int(page_size), c_float(scale),
        c_int(window), c_int(n_chunks), c_int(chunk_keys), _ptr(partial), _ptr(positions), c_int(row0), c_int(n_rows),
        _stream())
    _check(st, "paged_prefill_f32", f"segments={n_seg} heads={n_head}/{n_kv_head} head_dim={head_dim} page={page_size} "
                                    f"chunks={n_chunks}x{chunk_keys}")


def paged_prefill_tc5(q, k_cache, v_cache, block_table, cu_rows, seg_start, out, seg0, n_seg, max_seg_rows,
                      n_head, n_kv_head, head_dim, page_size, scale, window=0, chunks=(1, 0), partial=None,
                      positions=None, row0=0, n_rows=0):
    """The same attention as ``paged_prefill_bf16`` on the tcgen05 tensor cores (TMA operands, S and the output in
    tensor memory).  Head size 64 or 128, page sizes 8..128 (powers of two); ``q`` and ``out`` in full row numbering.
    ``chunks``, ``partial``, ``positions``, ``row0``, ``n_rows`` as for ``paged_prefill_bf16`` (chunks from
    ``prefill_key_chunks`` with two blocks per 128-row tile, two per SM and chunks of at least 8,192 keys)."""
    _need_cuda(q, k_cache, v_cache, block_table, cu_rows, seg_start, out, partial, positions)
    if head_dim not in (64, 128):
        raise KernelError(f"tcgen05 prefill attention: head_dim={head_dim} is neither 64 nor 128")
    if page_size & (page_size - 1) or not 8 <= page_size <= 128:
        raise KernelError(f"tcgen05 prefill attention: page_size={page_size} is not a power of two in 8..128")
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and block_table.is_contiguous() and k_cache.is_contiguous()
    n_chunks, chunk_keys = chunks
    if n_chunks > 1:
        assert partial.dtype == torch.float32 and partial.numel() >= n_rows * n_head * n_chunks * (head_dim + 4)
        assert positions.dtype == torch.int32 and positions.numel() >= row0 + n_rows
    st = kernels().cbis_paged_prefill_tc5(
        _ptr(q), c_int(q.stride(0)), c_int(q.shape[0]), _ptr(k_cache), _ptr(v_cache), c_int(k_cache.shape[0]),
        _ptr(block_table), c_int(block_table.shape[1]), _ptr(cu_rows), _ptr(seg_start), _ptr(out),
        c_int(out.stride(0)), c_int(seg0), c_int(n_seg), c_int(max_seg_rows), c_int(n_head), c_int(n_kv_head),
        c_int(head_dim), c_int(page_size), c_float(scale), c_int(window), c_int(n_chunks), c_int(chunk_keys),
        _ptr(partial), _ptr(positions), c_int(row0), c_int(n_rows), _ptr(tcgen05_error_flag(q.device)), _stream())
    _check(st, "paged_prefill_tc5", f"segments={n_seg} heads={n_head}/{n_kv_head} page={page_size} chunks={n_chunks}x{chunk_keys}")


def paged_prefill_tc5_blocks_per_sm() -> int:
    """How many blocks of the tcgen05 prefill attention an SM has room for at a time (it is sized for two): from the
    registers, shared memory and tensor memory a block takes as compiled and what the device's SMs have."""
    n = kernels().cbis_paged_prefill_tc5_blocks_per_sm()
    if n < 0:
        raise KernelError(f"paged_prefill_tc5: a device query failed with CUDA error {-n}")
    return n


# 1: decode steps of up to 16 rows run their layers in ONE persistent kernel (csrc/kernels/decode_layers.cu).  Off by
# default: measured at the 1.3B sizes it takes 1.6 ms per step at batch 1 and 2.1 ms at batch 8, the chain of kernels 0.95
# and 1.24 ms (its twelve dependent phases per layer each wait for L2 or for the other blocks while the memory system is
# kept busy by its own weight stream, and eight warps per SM do not hide that).
USE_FUSED_DECODE = __import__("os").environ.get("CBIS_FUSED_DECODE", "0") == "1"
FUSED_DECODE_MAX_ROWS = 16


def decode_layers_blocks(n_min: int) -> int:
    """Blocks the persistent decode kernel runs with: one per SM, fewer when the narrowest product of a layer has
    fewer than 8 columns per block."""
    n = optional_kernels().cbis_decode_layers_blocks(c_int(n_min))
    if n <= 0:
        raise KernelError("decode_layers: the device could not be queried")
    return n


def decode_layers_map(w_nk, blocks: int) -> torch.Tensor:
    """The 128-byte TMA descriptor of a weight matrix ``[N, K]`` for ``blocks`` blocks, as a CPU uint8 tensor."""
    _need_cuda(w_nk)
    assert w_nk.dtype == torch.bfloat16 and w_nk.is_contiguous() and w_nk.dim() == 2
    out = torch.zeros(128, dtype=torch.uint8)
    st = optional_kernels().cbis_decode_layers_map(c_void_p(out.data_ptr()), _ptr(w_nk), c_int(w_nk.shape[0]), c_int(w_nk.shape[1]),
                                          c_int(blocks))
    _check(st, "decode_layers_map", f"N={w_nk.shape[0]} K={w_nk.shape[1]} blocks={blocks}", launches=0)
    return out


def decode_layers_desc_bytes() -> int:
    return int(optional_kernels().cbis_decode_layers_desc_bytes())


def decode_layers_splits(rows: int, n_head: int, max_context: int, blocks: int) -> int:
    """How many ways the persistent decode kernel splits a request's keys: its (row, head, split) items go to the two
    groups of four warps of every block.  An item has a fixed cost (its query, the meeting of its warps, the merge),
    so the items are as long as one round over the groups allows: pieces of 64 keys or more, at most 32 ways."""
    groups, pairs = 2 * blocks, max(1, rows * n_head)
    return max(1, min(32, groups // pairs, max_context // 64))


def decode_layers(maps, layers, n_layers, blocks, M, d, n_head, n_kv_head, head_dim, F, page_size, act, window, scale,
                  nsplit, x, qkv, attn, hidden, block_table, row_seq, positions, slot_mapping, part, counters,
                  grid_counter, trace=None):
    """``n_layers`` pre-norm layers of a decode step of ``M`` <= 16 rows in one persistent kernel (see
    csrc/kernels/decode_layers.cu).  ``grid_counter`` (int32[1]) must be zero; a wait that runs out inside the kernel
    sets the flag that ``raise_if_kernel_errors`` reads.  ``trace`` (int64[256], for measuring): block 0's
    nanosecond timer at every phase boundary, 12 per layer."""
    _need_cuda(maps, layers, x, qkv, attn, hidden, block_table, row_seq, positions, slot_mapping, part, counters, grid_counter)
    assert x.dtype == torch.float32 and x.is_contiguous() and qkv.dtype == torch.bfloat16 and hidden.dtype == torch.bfloat16
    assert block_table.is_contiguous() and block_table.dtype == torch.int32
    st = optional_kernels().cbis_decode_layers(
        _ptr(maps), _ptr(layers), c_int(n_layers), c_int(blocks), c_int(M), c_int(d), c_int(n_head), c_int(n_kv_head),
        c_int(head_dim), c_int(F), c_int(page_size), c_int(ACT[act]), c_int(window), c_float(scale), c_int(nsplit), _ptr(x),
        _ptr(qkv), _ptr(attn), _ptr(hidden), _ptr(block_table), c_int(block_table.shape[1]), _ptr(row_seq), _ptr(positions),
        _ptr(slot_mapping), _ptr(part), _ptr(counters), _ptr(grid_counter), _ptr(tcgen05_error_flag(x.device)), _stream(),
        _ptr(trace))
    _check(st, "decode_layers", f"layers={n_layers} rows={M} width={d} heads={n_head}/{n_kv_head} head_dim={head_dim} inner={F}")


def decode_advance(tokens, positions, seg_start, seg_ctx, sampled, n):
    """tokens <- sampled, positions/seg_start/seg_ctx += 1 for the first n rows (all on the device)."""
    st = kernels().cbis_decode_advance(_ptr(tokens), _ptr(positions), _ptr(seg_start), _ptr(seg_ctx), _ptr(sampled),
                                       c_int(n), _stream())
    _check(st, "decode_advance")


def slots_from_table(positions, row_seq, block_table, page_size, slot_mapping, n):
    """slot_mapping[r] = token slot of positions[r] by the request's block table (-1 for padding rows)."""
    st = kernels().cbis_slots_from_table(_ptr(positions), _ptr(row_seq), _ptr(block_table),
                                         c_int(block_table.shape[1]), c_int(page_size), _ptr(slot_mapping), c_int(n),
                                         _stream())
    _check(st, "slots_from_table")


_sample_scratch = {}
_sample_outgrown = []     # buffers that a later call outgrew: a captured graph may still hold their addresses


def _sample_buffers(device, R: int, chunks: int):
    """Scratch of the sampling kernel, kept per device and grown as needed; counters start at zero
    and every launch leaves them zero."""
    key = device.index     # one scratch per device: launches on different streams must not overlap
    have = _sample_scratch.get(key)
    if have is None or have[0].numel() < R * chunks or have[2].numel() < R:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("sampling scratch would have to grow during graph capture")
        n = max(R * chunks, 64 * 64)
        if have is not None:
            _sample_outgrown.append(have)
        have = (torch.empty(n, dtype=torch.float32, device=device), torch.empty(n, dtype=torch.int32, device=device),
                torch.zeros(max(R, 1024), dtype=torch.int32, device=device))
        _sample_scratch[key] = have
    return have


def sample(logits, temperature, keys, out):
    """out[r] = argmax_i(logits[r,i]) (temperature[r] <= 0 or None) or the Gumbel-max draw keyed by keys[r]."""
    _need_cuda(logits, temperature, keys, out)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert temperature is None or temperature.dtype == torch.float32
    assert keys is None or keys.dtype == torch.int64
    chunks = kernels().cbis_sample_chunks(c_int(V))
    pv, pi, cnt = _sample_buffers(logits.device, R, chunks)
    st = kernels().cbis_sample(_ptr(logits), c_int(logits.stride(0)), _ptr(temperature), _ptr(keys), _ptr(out),
                               c_int(R), c_int(V), _ptr(pv), _ptr(pi), _ptr(cnt), _stream())
    _check(st, "sample", f"R={R} V={V}")
