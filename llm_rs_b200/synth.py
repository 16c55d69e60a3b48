"""Seeded synthetic Q4_K / Q6_K weights and activations with the value distributions the
benchmark configurations name.  They stand in for real GGUF tensors (the reference's own
benches also measure on random blocks: examples/bench_q4k_gemv.rs:32-46).

Counter-based: value i of tensor `tid` depends only on (seed, tid, i), so any shard of a
tensor can be generated on its own and every rank of a multi-GPU run sees the same bytes.
"""
from __future__ import annotations

import numpy as np

DEFAULT_SEED = 0x5EEDB200
_C1 = np.uint64(0xD1B54A32D192ED03)
_WORDS_PER_BLOCK = 32          # counter stride per block (>= 27 words for 210 bytes)


def splitmix64(x: np.ndarray) -> np.ndarray:
    """Vectorised SplitMix64 output function on uint64 counters."""
    with np.errstate(over="ignore"):
        z = x + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _stream(seed: int, tid: int, start: int, count: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = np.uint64(seed) ^ (np.uint64(tid) * _C1)
        idx = np.arange(start, start + count, dtype=np.uint64)
        return splitmix64(base ^ idx)


def _unit(u: np.ndarray) -> np.ndarray:
    """uint64 -> float64 uniform in [0, 1)."""
    return (u >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))


def _block_bytes(seed: int, tid: int, first_block: int, n_blocks: int, block_bytes: int) -> np.ndarray:
    words = (block_bytes + 7) // 8
    with np.errstate(over="ignore"):
        base = np.uint64(seed) ^ (np.uint64(tid) * _C1)
        blk = np.arange(first_block, first_block + n_blocks, dtype=np.uint64)[:, None] * np.uint64(_WORDS_PER_BLOCK)
        ctr = blk + np.arange(words, dtype=np.uint64)[None, :]
        u = splitmix64(base ^ ctr)
    return u.view(np.uint8).reshape(n_blocks, words * 8)[:, :block_bytes].copy(), u


def q4k_blocks(n_blocks: int, *, seed: int = DEFAULT_SEED, tid: int = 0, first_block: int = 0,
               chunk: int = 1 << 18) -> np.ndarray:
    """[n_blocks, 144] uint8.  d, dmin = f16 of uniform [1e-3, 2e-2]; the other 140 bytes are
    uniform, which makes the 6-bit scales/mins uniform in 0..63 and the nibbles in 0..15."""
    out = np.empty((n_blocks, 144), dtype=np.uint8)
    for a in range(0, n_blocks, chunk):
        n = min(chunk, n_blocks - a)
        b, u = _block_bytes(seed, tid, first_block + a, n, 144)
        # two extra draws per block for d / dmin (counter slots 30 and 31 of the block)
        with np.errstate(over="ignore"):
            base = np.uint64(seed) ^ (np.uint64(tid) * _C1)
            blk = np.arange(first_block + a, first_block + a + n, dtype=np.uint64) * np.uint64(_WORDS_PER_BLOCK)
            ud = _unit(splitmix64(base ^ (blk + np.uint64(30))))
            um = _unit(splitmix64(base ^ (blk + np.uint64(31))))
        b[:, 0:2] = (1e-3 + ud * (2e-2 - 1e-3)).astype(np.float16).view(np.uint8).reshape(n, 2)
        b[:, 2:4] = (1e-3 + um * (2e-2 - 1e-3)).astype(np.float16).view(np.uint8).reshape(n, 2)
        out[a:a + n] = b
    return out


def q6k_blocks(n_blocks: int, *, seed: int = DEFAULT_SEED, tid: int = 0, first_block: int = 0,
               chunk: int = 1 << 18) -> np.ndarray:
    """[n_blocks, 210] uint8.  d = f16 of uniform [1e-3, 1e-2]; 16 int8 sub-scales uniform in
    [-32, 31]; ql/qh uniform bytes, i.e. 6-bit quants uniform in 0..63."""
    out = np.empty((n_blocks, 210), dtype=np.uint8)
    for a in range(0, n_blocks, chunk):
        n = min(chunk, n_blocks - a)
        b, u = _block_bytes(seed, tid, first_block + a, n, 210)
        b[:, 192:208] = ((b[:, 192:208] & 63).astype(np.int16) - 32).astype(np.int8).view(np.uint8)
        with np.errstate(over="ignore"):
            base = np.uint64(seed) ^ (np.uint64(tid) * _C1)
            blk = np.arange(first_block + a, first_block + a + n, dtype=np.uint64) * np.uint64(_WORDS_PER_BLOCK)
            ud = _unit(splitmix64(base ^ (blk + np.uint64(30))))
        b[:, 208:210] = (1e-3 + ud * (1e-2 - 1e-3)).astype(np.float16).view(np.uint8).reshape(n, 2)
        out[a:a + n] = b
    return out


def weight(dtype: int, K: int, N: int, *, seed: int = DEFAULT_SEED, tid: int = 0,
           rows: tuple[int, int] | None = None) -> np.ndarray:
    """Raw GGUF bytes of a [K, N] weight (dtype 12 = Q4_K, 14 = Q6_K), or of its rows a..b:
    N rows of K/256 consecutive blocks."""
    assert K % 256 == 0
    nb = K // 256
    a, b = rows if rows is not None else (0, N)
    gen = q4k_blocks if dtype == 12 else q6k_blocks
    return gen((b - a) * nb, seed=seed, tid=tid, first_block=a * nb).reshape(-1)


def activations(M: int, K: int, *, seed: int = DEFAULT_SEED, tid: int = 1000) -> np.ndarray:
    """float32 [M, K] ~ N(0, 1) by Box-Muller on the counter stream."""
    n = M * K
    pairs = (n + 1) // 2                    # each pair of draws gives two normals
    u1 = 1.0 - _unit(_stream(seed, tid, 0, pairs))     # (0, 1]
    u2 = _unit(_stream(seed, tid, 1 << 40, pairs))
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.concatenate([r * np.cos(2 * np.pi * u2), r * np.sin(2 * np.pi * u2)])[:n]
    return z.astype(np.float32).reshape(M, K)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even; finite inputs."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) >> np.uint32(16)).astype(np.uint16)
