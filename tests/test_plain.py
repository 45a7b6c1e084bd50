"""The plain implementation itself (CPU): against the reference module's stored outputs, and its parts."""
import math
import os

import numpy as np
import torch

import plain_gpt
import tiny_configs as tc
from golden.make_golden import golden_weights

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_matches_the_reference_modules_outputs():
    for name, cfg, init in (("tiny_a", tc.TINY_A, tc.INIT_A), ("tiny_b", tc.TINY_B, tc.INIT_B)):
        g = np.load(os.path.join(GOLDEN, f"golden_{name}.npz"))
        w = golden_weights(cfg, init, seed=2024)
        with torch.no_grad():
            logits = plain_gpt.forward(cfg, w, g["tokens"].tolist())
        assert np.abs(logits[g["rows"].tolist()].numpy() - g["logits"]).max() < 1e-5
        assert float(g["max_abs_diff_plain_vs_reference"]) < 1e-5


def test_parts_against_torch():
    torch.manual_seed(0)
    x = torch.randn(5, 12, dtype=torch.float64)
    g, b = torch.randn(12, dtype=torch.float64), torch.randn(12, dtype=torch.float64)
    assert torch.allclose(plain_gpt.layer_norm(x, g, b, 1e-6), torch.nn.functional.layer_norm(x, (12,), g, b, 1e-6))
    assert torch.allclose(plain_gpt.gelu(x, "gelu"), torch.nn.functional.gelu(x))
    assert torch.allclose(plain_gpt.gelu(x, "gelu_new"), torch.nn.functional.gelu(x, approximate="tanh"))


def test_attention_is_causal_and_scaled():
    torch.manual_seed(1)
    d, H, T = 8, 2, 6
    h = torch.randn(T, d, dtype=torch.float64)
    wa, ba = torch.randn(d, 3 * d, dtype=torch.float64), torch.randn(3 * d, dtype=torch.float64)
    wo, bo = torch.eye(d, dtype=torch.float64), torch.zeros(d, dtype=torch.float64)
    full = plain_gpt.attention(h, wa, ba, wo, bo, H)
    for t in range(1, T + 1):                       # a prefix gives the same rows: nothing looks ahead
        assert torch.allclose(plain_gpt.attention(h[:t], wa, ba, wo, bo, H), full[:t])
    qkv = h @ wa + ba                               # row 1, head 0, by hand
    q, k, v = qkv[1, :4], qkv[:2, d:d + 4], qkv[:2, 2 * d:2 * d + 4]
    p = torch.softmax((k @ q) / math.sqrt(4), 0)
    assert torch.allclose(full[1, :4], p @ v)


def test_sampling_rules():
    row = np.array([0.1, 3.0, 3.0, -1.0])
    assert plain_gpt.sample(row) == 1               # first maximum wins
    a = plain_gpt.gumbel_noise(5, 2, 3, 1000)
    assert np.array_equal(a, plain_gpt.gumbel_noise(5, 2, 3, 1000))
    assert not np.array_equal(a, plain_gpt.gumbel_noise(5, 2, 4, 1000))
    assert not np.array_equal(a[:10], plain_gpt.gumbel_noise(5, 3, 3, 10))
    # draws follow softmax(logits / temperature)
    logits = np.array([1.0, 0.0, -1.0, 0.5])
    n = 4000
    counts = np.bincount([plain_gpt.sample(logits, 0.7, 9, 1, i) for i in range(n)], minlength=4) / n
    p = np.exp(logits / 0.7) / np.exp(logits / 0.7).sum()
    assert np.abs(counts - p).max() < 0.03


def test_generate_feeds_back_all_but_the_last_token():
    cfg, w = tc.TINY_A, golden_weights(tc.TINY_A, tc.INIT_A, 3)
    out = plain_gpt.generate(cfg, w, [1, 2, 3], 4)
    with torch.no_grad():
        assert out[0] == int(plain_gpt.forward(cfg, w, [1, 2, 3])[-1].argmax())
        assert out[3] == int(plain_gpt.forward(cfg, w, [1, 2, 3] + out[:3])[-1].argmax())
