"""ctypes binding of the CPU oracle (test infrastructure; see llmrs_oracle.c).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import this
module.  The CUDA library and the llm_rs_b200 package never do.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "llmrs_oracle.c")
_LIB = os.path.join(_HERE, "libllmrs_oracle.so")

Q4K, Q6K = 12, 14          # GGUF dtype ids (reference: src/tensor/mod.rs:14,16)
F32, F16, Q4_0, Q8_0, BF16 = 0, 1, 2, 8, 30      # the other weight types the dispatcher accepts (src/tensor/mod.rs:3-33)
BLOCK_BYTES = {Q4K: 144, Q6K: 210, F32: 4, F16: 2, BF16: 2, Q4_0: 18, Q8_0: 34}
BLOCK_ELEMS = {Q4K: 256, Q6K: 256, F32: 1, F16: 1, BF16: 1, Q4_0: 32, Q8_0: 32}

# -ffp-contract=off and no -ffast-math: every float operation happens as written.
_FLAGS = ["-O2", "-march=native", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-Wall"]


def build(force: bool = False) -> str:
    """Compile llmrs_oracle.c next to this file.  OpenMP is used when a compiler
    that has it is found (some gcc wrappers ship without libgomp)."""
    if not force and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    errors = []
    for cc in ("/usr/bin/gcc", "gcc", "cc"):
        for omp in (["-fopenmp"], []):
            cmd = [cc, *_FLAGS, *omp, "-o", _LIB, _SRC, "-lm"]
            try:
                r = subprocess.run(cmd, capture_output=True, text=True)
            except FileNotFoundError as e:
                errors.append(str(e))
                continue
            if r.returncode == 0:
                return _LIB
            errors.append(" ".join(cmd) + "\n" + r.stderr[-400:])
    raise RuntimeError("could not build the oracle:\n" + "\n".join(errors))


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        u8p, f32p, u16p = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_uint16)
        L.llmrs_oracle_f16_to_f32.restype = C.c_float
        L.llmrs_oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.llmrs_oracle_f32_to_f16.restype = C.c_uint16
        L.llmrs_oracle_f32_to_f16.argtypes = [C.c_float]
        L.llmrs_oracle_bf16_to_f32.restype = C.c_float
        L.llmrs_oracle_bf16_to_f32.argtypes = [C.c_uint16]
        L.llmrs_oracle_f32_to_bf16.restype = C.c_uint16
        L.llmrs_oracle_f32_to_bf16.argtypes = [C.c_float]
        L.llmrs_oracle_unpack_q4k_scale.restype = None
        L.llmrs_oracle_unpack_q4k_scale.argtypes = [u8p, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        L.llmrs_oracle_q6k_elem.restype = C.c_uint8
        L.llmrs_oracle_q6k_elem.argtypes = [u8p, u8p, C.c_uint]
        L.llmrs_oracle_dequant.restype = C.c_int
        L.llmrs_oracle_dequant.argtypes = [C.c_int, u8p, C.c_size_t, C.c_size_t, f32p, C.c_int]
        L.llmrs_oracle_matmul.restype = C.c_int
        L.llmrs_oracle_matmul.argtypes = [C.c_int, u8p, C.c_size_t, C.c_size_t, f32p, C.c_size_t, f32p,
                                          C.c_size_t, C.c_size_t, C.c_int, C.c_int]
        L.llmrs_oracle_matmul_fast.restype = C.c_int
        L.llmrs_oracle_matmul_fast.argtypes = [C.c_int, u8p, C.c_size_t, C.c_size_t, f32p, C.c_size_t, f32p,
                                               C.c_size_t, C.c_size_t, C.c_int]
        L.llmrs_oracle_ref_case_q4k.restype = C.c_int
        L.llmrs_oracle_ref_case_q4k.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, u8p, u16p]
        L.llmrs_oracle_ref_tolerance_failures.restype = C.c_size_t
        L.llmrs_oracle_ref_tolerance_failures.argtypes = [f32p, f32p, C.c_size_t, C.c_size_t, f32p]
        L.llmrs_oracle_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a: np.ndarray, ty):
    return a.ctypes.data_as(C.POINTER(ty))


def max_threads() -> int:
    return int(lib().llmrs_oracle_max_threads())


def f16_to_f32(h: int) -> float:
    return float(lib().llmrs_oracle_f16_to_f32(h))


def f32_to_f16(f: float) -> int:
    return int(lib().llmrs_oracle_f32_to_f16(np.float32(f)))


def bf16_to_f32(b: int) -> float:
    return float(lib().llmrs_oracle_bf16_to_f32(b))


def f32_to_bf16(f: float) -> int:
    return int(lib().llmrs_oracle_f32_to_bf16(np.float32(f)))


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) -> float32, exact."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def unpack_q4k_scale(scales12: np.ndarray, sb: int) -> tuple[int, int]:
    s = np.ascontiguousarray(scales12, dtype=np.uint8)
    sc, m = C.c_uint32(), C.c_uint32()
    lib().llmrs_oracle_unpack_q4k_scale(_p(s, C.c_uint8), sb, C.byref(sc), C.byref(m))
    return sc.value, m.value


def q6k_elem(ql: np.ndarray, qh: np.ndarray, i: int) -> int:
    ql = np.ascontiguousarray(ql, dtype=np.uint8)
    qh = np.ascontiguousarray(qh, dtype=np.uint8)
    return int(lib().llmrs_oracle_q6k_elem(_p(ql, C.c_uint8), _p(qh, C.c_uint8), i))


def _check_weight(dtype: int, w: np.ndarray, K: int, N: int) -> np.ndarray:
    w = np.ascontiguousarray(w).view(np.uint8).reshape(-1)
    be = BLOCK_ELEMS[dtype]
    assert K % be == 0 and w.size == N * (K // be) * BLOCK_BYTES[dtype], (w.size, K, N)
    return w


def dequant(dtype: int, w: np.ndarray, K: int, N: int, threads: int | None = None) -> np.ndarray:
    """Raw GGUF blocks of an [K, N] weight -> float32 [N, K] (row r = output feature r)."""
    w = _check_weight(dtype, w, K, N)
    out = np.empty((N, K), dtype=np.float32)
    rc = lib().llmrs_oracle_dequant(dtype, _p(w, C.c_uint8), K, N, _p(out, C.c_float), threads or max_threads())
    assert rc == 0, rc
    return out


def embed(dtype: int, w: np.ndarray, K: int, N: int, tokens, *, bf16: bool = False) -> np.ndarray:
    """Embedding lookup (src/backend/mod.rs:25-27; shaders/ops.metal:917-965): float32
    [len(tokens), K], row i = dequantised row tokens[i] of the [K, N] table -- the float32 values
    of the reference's CPU dequantisation (tests/ops.rs:41-59), rounded to bf16 (round to nearest
    even, as half::bf16::from_f32) and widened again when bf16=True."""
    w = _check_weight(dtype, w, K, N)
    row_bytes = (K // BLOCK_ELEMS[dtype]) * BLOCK_BYTES[dtype]
    rows = np.stack([w[int(t) * row_bytes:(int(t) + 1) * row_bytes] for t in tokens]) if len(tokens) else \
        np.empty((0, row_bytes), dtype=np.uint8)
    out = dequant(dtype, np.ascontiguousarray(rows).reshape(-1), K, len(tokens)) if len(tokens) else \
        np.empty((0, K), dtype=np.float32)
    if bf16:
        out = bf16_bits_to_f32(f32_to_bf16_bits(out)).reshape(out.shape)
    return out


def _round_io(v: np.ndarray, bf16: bool) -> np.ndarray:
    v = np.asarray(v, dtype=np.float32)
    return bf16_bits_to_f32(f32_to_bf16_bits(v)).reshape(v.shape) if bf16 else v


def silu(x: np.ndarray, *, bf16: bool = False) -> np.ndarray:
    """shaders/ops.metal:762-771: v / (1 + exp(-v)) in float32 (exp evaluated in double here), then the
    output rounding."""
    v = np.asarray(x, dtype=np.float32).astype(np.float64)
    return _round_io((v / (1.0 + np.exp(-v))).astype(np.float32), bf16)


def mul(a: np.ndarray, b: np.ndarray, *, bf16: bool = False) -> np.ndarray:
    """shaders/ops.metal:785-793: float(a) * float(b), one rounding."""
    return _round_io(np.asarray(a, np.float32) * np.asarray(b, np.float32), bf16)


def add(a: np.ndarray, b: np.ndarray, *, bf16: bool = False) -> np.ndarray:
    """shaders/ops.metal:775-783."""
    return _round_io(np.asarray(a, np.float32) + np.asarray(b, np.float32), bf16)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float, *, bf16: bool = False) -> np.ndarray:
    """shaders/ops.metal:970-1003 per row of x [rows, dim]: inv = rsqrt(sum(v^2) / dim + eps);
    out = (v * inv) * weight.  The sum of squares is taken in double (the shader's own order of
    float additions depends on its thread count); inv and the products are float32."""
    v = np.asarray(x, dtype=np.float32)
    ss = (v.astype(np.float64) ** 2).sum(axis=-1, keepdims=True)
    inv = (1.0 / np.sqrt(ss / v.shape[-1] + np.float64(np.float32(eps)))).astype(np.float32)
    return _round_io((v * inv) * np.asarray(weight, np.float32), bf16)


def argmax(x: np.ndarray) -> int:
    """shaders/ops.metal:803-835 for distinct maxima; the smallest index among equal maxima."""
    return int(np.argmax(np.asarray(x, dtype=np.float32)))


def rope(x: np.ndarray, positions, head_dim: int, theta: float, *, split_half: bool = False,
         bf16: bool = False) -> np.ndarray:
    """shaders/ops.metal:1011-1042 on x [seq_len, row_stride] (rows of heads of head_dim): pair i of a
    head is (2i, 2i+1), or (i, i + head_dim/2) when split_half; angle = position * theta^(-2i/head_dim);
    (x0, x1) -> (x0 cos - x1 sin, x0 sin + x1 cos).  Frequency and angle are float32 values as in the
    shader (the angle's rounding, position * 2^-24 radians, is part of the reference's result); cosine,
    sine and the rotation are taken in double."""
    v = np.asarray(x, dtype=np.float32).astype(np.float64)
    seq, stride = v.shape
    half = head_dim // 2
    i = np.arange(half, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(theta), np.float32(2.0) * i / np.float32(head_dim))).astype(np.float32)
    out = v.copy()
    for s in range(seq):
        ang = (np.float32(int(positions[s])) * freq).astype(np.float32).astype(np.float64)
        c, sn = np.cos(ang), np.sin(ang)
        for h in range(stride // head_dim):
            base = h * head_dim
            ia = base + (np.arange(half) if split_half else 2 * np.arange(half))
            ib = ia + half if split_half else ia + 1
            x0, x1 = v[s, ia], v[s, ib]
            out[s, ia] = x0 * c - x1 * sn
            out[s, ib] = x0 * sn + x1 * c
    return _round_io(out.astype(np.float32), bf16)


def scatter_kv(pool: np.ndarray, src: np.ndarray, slot_mapping, kv_dim: int, num_tokens: int) -> np.ndarray:
    """shaders/ops.metal:841-853: pool[slot_mapping[t] * kv_dim + d] = src[t * kv_dim + d]."""
    out = np.array(pool, copy=True).reshape(-1, kv_dim)
    s = np.asarray(src).reshape(-1)[:num_tokens * kv_dim].reshape(num_tokens, kv_dim)
    for t in range(num_tokens):
        out[int(slot_mapping[t])] = s[t]
    return out.reshape(np.asarray(pool).shape)


def gather(src: np.ndarray, indices, num_indices: int) -> np.ndarray:
    """shaders/ops.metal:859-873 on src [seq_len, dim]: row c of the result = row indices[c]."""
    return np.asarray(src)[[int(i) for i in indices[:num_indices]]]


def attention(q: np.ndarray, k_pool: np.ndarray, v_pool: np.ndarray, block_table, query_starts, seq_lens,
              n_heads: int, n_kv_heads: int, head_dim: int, block_size: int, max_blocks_per_seq: int,
              *, bf16: bool = False) -> np.ndarray:
    """shaders/ops.metal:636-758: q [total_query_tokens, n_heads * head_dim]; pools [slots, n_kv_heads *
    head_dim] with slot = page * block_size + offset; request r owns query tokens query_starts[r] ..
    query_starts[r+1], has seq_lens[r] positions, page p = block_table[r * max_blocks_per_seq + p];
    query token i of c sees positions 0 .. seq_len - c + i; softmax(q.k / sqrt(head_dim)) v per head,
    head h reading kv head h / (n_heads / n_kv_heads).  In double."""
    qf = np.asarray(q, dtype=np.float32).astype(np.float64)
    kf = np.asarray(k_pool, dtype=np.float32).astype(np.float64).reshape(-1, n_kv_heads * head_dim)
    vf = np.asarray(v_pool, dtype=np.float32).astype(np.float64).reshape(-1, n_kv_heads * head_dim)
    out = np.zeros_like(qf)
    group = n_heads // n_kv_heads
    for r in range(len(seq_lens)):
        q0, q1 = int(query_starts[r]), int(query_starts[r + 1])
        count = q1 - q0
        for li in range(count):
            n_pos = int(seq_lens[r]) - count + li + 1
            slots = [int(block_table[r * max_blocks_per_seq + t // block_size]) * block_size + t % block_size
                     for t in range(n_pos)]
            for h in range(n_heads):
                kv = (h // group) * head_dim
                qq = qf[q0 + li, h * head_dim:(h + 1) * head_dim]
                sc = kf[slots, kv:kv + head_dim] @ qq / np.sqrt(np.float64(head_dim))
                p = np.exp(sc - sc.max())
                out[q0 + li, h * head_dim:(h + 1) * head_dim] = (p / p.sum()) @ vf[slots, kv:kv + head_dim]
    return _round_io(out.astype(np.float32), bf16)


def matmul(dtype: int, w: np.ndarray, K: int, N: int, x: np.ndarray, *, acc: str = "f64",
           rows: tuple[int, int] | None = None, threads: int | None = None, fast: bool = False) -> np.ndarray:
    """Out[M, N] = X[M, K] . W[N, K]^T.  acc="f32": the reference's sequential float
    accumulate; acc="f64": products and sums in double (used as truth for relative-L2).
    rows=(a, b) computes only output features a..b (the rest of `out` stays 0)."""
    w = _check_weight(dtype, w, K, N)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, K)
    M = x.shape[0]
    out = np.zeros((M, N), dtype=np.float32)
    a, b = rows if rows is not None else (0, N)
    t = threads or max_threads()
    if fast:
        rc = lib().llmrs_oracle_matmul_fast(dtype, _p(w, C.c_uint8), K, N, _p(x, C.c_float), M,
                                            _p(out, C.c_float), a, b, t)
    else:
        rc = lib().llmrs_oracle_matmul(dtype, _p(w, C.c_uint8), K, N, _p(x, C.c_float), M,
                                       _p(out, C.c_float), a, b, 1 if acc == "f64" else 0, t)
    assert rc == 0, rc
    return out


def ref_case_q4k(in_f: int, out_f: int, seq_len: int) -> tuple[np.ndarray, np.ndarray]:
    """The inputs check_matmul_q4k(in_f, out_f, seq_len) of the reference's test draws:
    (Q4_K weight bytes, bf16 activation bit patterns)."""
    w = np.empty(out_f * (in_f // 256) * 144, dtype=np.uint8)
    x = np.empty(in_f * seq_len, dtype=np.uint16)
    rc = lib().llmrs_oracle_ref_case_q4k(in_f, out_f, seq_len, _p(w, C.c_uint8), _p(x, C.c_uint16))
    assert rc == 0, rc
    return w, x


def ref_tolerance_failures(expected: np.ndarray, got: np.ndarray, in_f: int) -> tuple[int, float]:
    """Number of elements failing the reference test's criterion, and its max relative error."""
    e = np.ascontiguousarray(expected, dtype=np.float32).reshape(-1)
    g = np.ascontiguousarray(got, dtype=np.float32).reshape(-1)
    assert e.size == g.size
    mr = C.c_float()
    bad = lib().llmrs_oracle_ref_tolerance_failures(_p(e, C.c_float), _p(g, C.c_float), e.size, in_f, C.byref(mr))
    return int(bad), float(mr.value)


def rel_l2(got: np.ndarray, truth: np.ndarray) -> float:
    g = np.asarray(got, dtype=np.float64).reshape(-1)
    t = np.asarray(truth, dtype=np.float64).reshape(-1)
    return float(np.linalg.norm(g - t) / max(np.linalg.norm(t), 1e-300))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
