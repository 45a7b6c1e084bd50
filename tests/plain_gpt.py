"""Plain, slow TinyGPT (GPT-2 style) for tests: whole sequences, no cache, one
function per part, torch CPU ops only.

It shares no code with the engine.  Every function is written from the formulas
of Manas103/continuous-batching-inference-server; the file:line beside each one
is the place in that project where the formula stands.  Weights come in GPT-2
naming and Conv1D layout (``[in, out]``, ``y = x @ W + b``); the reference keeps
``nn.Linear`` ``[out, in]`` weights, so ``W_here = W_ref.T``.

``tests/golden/make_golden.py`` compares this file with the reference's own
``python/model.py`` on two tiny random models and stores small outputs.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# --------------------------------------------------------------------------
# reading a model folder (independent of the engine's reader)
# --------------------------------------------------------------------------

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64, "F64": torch.float64}


def read_model_folder(folder: str, dtype=torch.float64):
    """Returns (config dict, {name: tensor in `dtype`}) of a model folder."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    data = raw[8 + n:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=_ST_DTYPES[meta["dtype"]])
        t = t.reshape(meta["shape"])
        if name.startswith("transformer."):
            name = name[len("transformer."):]
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, out


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed(tokens, wte, wpe, first_position=0):
    """x[r] = wte[tok[r]] + wpe[pos[r]], pos counted from 0.
    python/model.py:65-66; kernels/elementwise.cu:12-16."""
    pos = torch.arange(first_position, first_position + len(tokens))
    return wte[torch.as_tensor(tokens, dtype=torch.long)] + wpe[pos]


def layer_norm(x, gamma, beta, eps):
    """Biased variance over the last dim, y = (x-mean)*rsqrt(var+eps)*gamma+beta.
    kernels/elementwise.cu:21-57 (eps literal there: :51); python/model.py:26,31,60."""
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * gamma + beta


def gelu(v, kind):
    """'gelu': 0.5*v*(1+erf(v/sqrt 2)), kernels/elementwise.cu:59-66 and
    python/model.py:50.  'gelu_new': the tanh form GPT-2 folders name,
    0.5*v*(1+tanh(sqrt(2/pi)*(v+0.044715 v^3)))."""
    if kind == "gelu":
        return 0.5 * v * (1.0 + torch.erf(v / math.sqrt(2.0)))
    if kind == "gelu_new":
        return 0.5 * v * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (v + 0.044715 * v ** 3)))
    raise ValueError(kind)


def attention(h, c_attn_w, c_attn_b, c_proj_w, c_proj_b, n_head):
    """Causal multi-head attention over a whole sequence.
    q|k|v = h @ c_attn + b split at d and 2d (python/model.py:37-39 has three
    separate projections; src/transformer.cpp:71-73); head i owns columns
    i*hd..(i+1)*hd (python/model.py:37; kernels/attention.cu:70,81); scores
    (q.k)/sqrt(hd) (python/model.py:40; kernels/attention.cu:72,84), keys
    0..p for the query at p (python/model.py:41-42; kernels/attention.cu:67-68,78),
    softmax, times v, heads side by side, output projection
    (python/model.py:43-46; kernels/attention.cu:86-97)."""
    T, d = h.shape
    hd = d // n_head
    qkv = h @ c_attn_w + c_attn_b
    q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
    q = q.reshape(T, n_head, hd).transpose(0, 1)
    k = k.reshape(T, n_head, hd).transpose(0, 1)
    v = v.reshape(T, n_head, hd).transpose(0, 1)
    scores = (q @ k.transpose(-2, -1)) / math.sqrt(hd)
    future = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    scores = scores.masked_fill(future, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = (probs @ v).transpose(0, 1).reshape(T, d)
    return out @ c_proj_w + c_proj_b


def mlp(h, c_fc_w, c_fc_b, c_proj_w, c_proj_b, activation):
    """act(h @ W1 + b1) @ W2 + b2.  python/model.py:50; src/transformer.cpp:86-88."""
    return gelu(h @ c_fc_w + c_fc_b, activation) @ c_proj_w + c_proj_b


def block(x, w, i, n_head, eps, activation):
    """x += attn(ln_1(x)); x += mlp(ln_2(x)).
    python/model.py:48-51; src/transformer.cpp:67-90."""
    p = f"h.{i}."
    x = x + attention(layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps),
                      w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"],
                      w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"], n_head)
    x = x + mlp(layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps),
                w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"],
                w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"], activation)
    return x


def lm_head(x, w, cfg):
    """logits = ln_f(x) @ head^T without bias (python/model.py:69-70;
    src/transformer.cpp:92-93); head is wte when tie_word_embeddings."""
    eps = cfg.get("layer_norm_epsilon", 1e-5)
    h = layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], eps)
    head = w["wte.weight"] if cfg.get("tie_word_embeddings", True) else w["lm_head.weight"]
    return h @ head.T


def forward(cfg, w, tokens):
    """Logits [T, V] of one whole sequence.  python/model.py:63-70."""
    eps = cfg.get("layer_norm_epsilon", 1e-5)
    act = cfg.get("activation_function", "gelu_new")
    x = embed(tokens, w["wte.weight"], w["wpe.weight"])
    for i in range(cfg["n_layer"]):
        x = block(x, w, i, cfg["n_head"], eps, act)
    return lm_head(x, w, cfg)


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

_M64 = (1 << 64) - 1


def _splitmix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def gumbel_noise(seed: int, request: int, output_index: int, vocab: int):
    """g_i = -log(-log u_i); u_i from a counter generator keyed by
    (seed, request, output index, i), so a draw does not depend on batching."""
    key = _splitmix64((seed & _M64) ^ _splitmix64(((request & 0xFFFFFFFF) << 32) | (output_index & 0xFFFFFFFF)))
    i = np.arange(vocab, dtype=np.uint64)
    z = (np.uint64(key) + (i + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15))
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    z = z ^ (z >> np.uint64(31))
    u = ((z >> np.uint64(41)).astype(np.float64) + 0.5) * (2.0 ** -23)
    return -np.log(-np.log(u))


def sample(logits_row, temperature=0.0, seed=0, request=0, output_index=0):
    """Greedy: first maximum wins (src/server_demo.cpp:70-74).  temperature>0:
    argmax(logit/temperature + gumbel), a draw from softmax(logit/temperature)."""
    row = np.asarray(logits_row, dtype=np.float64)
    if temperature <= 0.0:
        return int(np.argmax(row))
    return int(np.argmax(row / temperature + gumbel_noise(seed, request, output_index, row.shape[0])))


def perturbed_scores(logits_row, temperature, seed, request, output_index):
    row = np.asarray(logits_row, dtype=np.float64)
    if temperature <= 0.0:
        return row
    return row / temperature + gumbel_noise(seed, request, output_index, row.shape[0])


def generate(cfg, w, prompt, max_new_tokens, temperature=0.0, seed=0, request=0):
    """Recomputes the whole sequence for every new token (no cache).  A request
    with g outputs runs g forward passes; the g-th token is not fed back
    (src/server_demo.cpp:162-185)."""
    toks = list(prompt)
    out = []
    with torch.no_grad():
        for j in range(max_new_tokens):
            if len(toks) > cfg["n_positions"]:
                break
            logits = forward(cfg, w, toks)[-1]
            t = sample(logits.numpy(), temperature, seed, request, j)
            out.append(t)
            toks.append(t)
    return out
