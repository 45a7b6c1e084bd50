"""The host's choice of how attention kernels cut a long context over more blocks (no GPU needed)."""
import random

from cbis_b200.kernels import ops


def test_chunks_cover_every_context_and_are_whole_key_tiles():
    rng = random.Random(3)
    for _ in range(2000):
        tiles, heads, segs = rng.randint(1, 40), rng.randint(1, 40), rng.randint(1, 4)
        limit = rng.randint(1, 200_000)
        per_tile, per_sm, least = rng.choice([(1, 8, 256), (2, 2, 8192), (1, 3, 64)])
        n, keys = ops.prefill_key_chunks(tiles, heads, segs, limit, per_tile, per_sm, least)
        if n == 1:
            assert keys == 0
            continue
        assert keys >= least and keys % 64 == 0 and keys & (keys - 1) == 0
        assert (n - 1) * keys < limit <= n * keys            # every key has a chunk, no chunk is wholly beyond the limit
        blocks = tiles * heads * segs * per_tile
        assert blocks < per_sm * 148                          # cut only when the grid alone does not fill the SMs
        want = -(-per_sm * 148 // blocks)                     # chunks that would fill the SMs
        assert keys == least or (keys // 2) * want < limit    # the smallest power of two that gets by with `want` chunks


def test_general_kernel_chunks():
    rng = random.Random(4)
    for _ in range(2000):
        rows, heads, limit, hd = rng.randint(1, 600), rng.randint(1, 40), rng.randint(1, 200_000), rng.choice([16, 24, 30, 64, 128, 250])
        n, keys = ops.generic_key_chunks(rows, heads, limit, hd)
        if hd % 4 or limit <= 256 or rows * heads >= 16 * 148:
            assert (n, keys) == (1, 0)                        # the merge kernel reads 16 bytes at a time; enough warps anyway
            continue
        if n > 1:
            assert keys >= 256 and keys & (keys - 1) == 0 and (n - 1) * keys < limit <= n * keys


def test_chunks_can_be_switched_off(monkeypatch):
    monkeypatch.setattr(ops, "USE_KEY_CHUNKS", False)
    assert ops.prefill_key_chunks(1, 1, 1, 100_000) == (1, 0)
    assert ops.generic_key_chunks(1, 1, 100_000, 64) == (1, 0)
