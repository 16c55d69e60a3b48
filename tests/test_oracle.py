"""The CPU oracle against everything that pins it: IEEE conversions, hand-derived
known-answer blocks, an independent pure-Python restatement of the reference's CPU code,
the gguf-py golden fixtures, and the reference test's own generator and seven cases."""
import os

import numpy as np
import pytest

from oracle import oracle as O


# ---------- conversions (crate `half` semantics) ----------

def test_f16_to_f32_exhaustive():
    hs = np.arange(65536, dtype=np.uint16)
    ref = hs.view(np.float16).astype(np.float32)
    got = np.array([O.f16_to_f32(int(h)) for h in hs], dtype=np.float32)
    ok = ~np.isnan(ref)
    assert np.array_equal(got.view(np.uint32)[ok], ref.view(np.uint32)[ok])
    assert np.isnan(got[~ok]).all()


def test_f32_to_f16_round_to_nearest_even():
    rng = np.random.default_rng(1)
    xs = (rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 6, 20000)).astype(np.float32)
    # every f16 value, and the midpoints between neighbours (ties)
    h = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float32)
    mids = ((h[:-1].astype(np.float64) + h[1:].astype(np.float64)) / 2).astype(np.float32)
    xs = np.concatenate([xs, h, -h, mids, -mids, np.float32([65519.9, 65520.0, 1e9, 2.0 ** -25, 2.0 ** -24])])
    with np.errstate(over="ignore"):
        ref = xs.astype(np.float16).view(np.uint16)
    got = np.array([O.f32_to_f16(float(v)) for v in xs], dtype=np.uint16)
    assert np.array_equal(got, ref)


def test_bf16_conversions():
    import torch
    rng = np.random.default_rng(2)
    xs = (rng.standard_normal(20000) * 10.0 ** rng.integers(-20, 20, 20000)).astype(np.float32)
    ties = (np.arange(1, 2000, dtype=np.uint32) << 16 | 0x8000).view(np.float32)
    xs = np.concatenate([xs, ties])
    ref = torch.from_numpy(xs).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got = np.array([O.f32_to_bf16(float(v)) for v in xs], dtype=np.uint16)
    assert np.array_equal(got, ref)
    assert np.array_equal(O.f32_to_bf16_bits(xs), ref)
    back = np.array([O.bf16_to_f32(int(b)) for b in ref[:1000]], dtype=np.float32)
    assert np.array_equal(back, O.bf16_bits_to_f32(ref[:1000]))


# ---------- independent pure-Python restatement (small cases only) ----------

def py_unpack_q4k_scale(scales, sb):
    """tests/ops.rs:29-39, written out with Python ints."""
    if sb < 4:
        return scales[sb] & 63, scales[sb + 4] & 63
    sc = (scales[sb + 4] & 0x0F) | ((scales[sb - 4] >> 6) << 4)
    m = (scales[sb + 4] >> 4) | ((scales[sb] >> 6) << 4)
    return sc, m


def py_dequant_q4k_block(blk):
    d = np.frombuffer(bytes(blk[0:2]), dtype=np.float16)[0].astype(np.float32)
    dmin = np.frombuffer(bytes(blk[2:4]), dtype=np.float16)[0].astype(np.float32)
    scales = [int(v) for v in blk[4:16]]
    qs = [int(v) for v in blk[16:144]]
    out = np.zeros(256, dtype=np.float32)
    for sb in range(8):
        sc, m = py_unpack_q4k_scale(scales, sb)
        for j in range(32):
            packed = qs[(sb // 2) * 32 + j]
            q = (packed >> 4) if sb % 2 else (packed & 0x0F)
            out[sb * 32 + j] = np.float32(np.float32(d * np.float32(sc)) * np.float32(q)) - np.float32(dmin * np.float32(m))
    return out


def py_dequant_q6k_block(blk):
    """shaders/ops.metal:28-42 and :322-334 with Python ints."""
    ql = [int(v) for v in blk[0:128]]
    qh = [int(v) for v in blk[128:192]]
    sc = np.frombuffer(bytes(blk[192:208]), dtype=np.int8)
    d = np.frombuffer(bytes(blk[208:210]), dtype=np.float16)[0].astype(np.float32)
    out = np.zeros(256, dtype=np.float32)
    for i in range(256):
        h, j = divmod(i, 128)
        lo = (ql[h * 64 + j] & 0x0F) if j < 64 else (ql[h * 64 + j - 64] >> 4)
        if j < 32:
            hi = qh[h * 32 + j] & 3
        elif j < 64:
            hi = (qh[h * 32 + j - 32] >> 2) & 3
        elif j < 96:
            hi = (qh[h * 32 + j - 64] >> 4) & 3
        else:
            hi = (qh[h * 32 + j - 96] >> 6) & 3
        q = lo | (hi << 4)
        out[i] = np.float32(d * np.float32(sc[i // 16])) * np.float32(q - 32)
    return out


def test_unpack_q4k_scale_all_sub_blocks():
    rng = np.random.default_rng(3)
    for _ in range(200):
        s = rng.integers(0, 256, 12, dtype=np.uint8)
        for sb in range(8):
            assert O.unpack_q4k_scale(s, sb) == py_unpack_q4k_scale([int(v) for v in s], sb)
    # the packing is a bijection onto 16 six-bit fields: all-ones gives 63 everywhere
    assert all(O.unpack_q4k_scale(np.full(12, 255, np.uint8), sb) == (63, 63) for sb in range(8))


def test_q6k_elem_matches_restatement():
    rng = np.random.default_rng(4)
    blk = rng.integers(0, 256, 210, dtype=np.uint8)
    blk[208:210] = np.array([1.0], dtype=np.float16).view(np.uint8)
    blk[192:208] = 1
    deq = py_dequant_q6k_block(blk)
    for i in range(256):
        assert O.q6k_elem(blk[0:128], blk[128:192], i) - 32 == int(deq[i])


def test_dequant_matches_python_restatement():
    rng = np.random.default_rng(5)
    b4 = rng.integers(0, 256, (6, 144), dtype=np.uint8)
    b4[:, 0:2] = rng.uniform(0.001, 0.05, 6).astype(np.float16).view(np.uint8).reshape(6, 2)
    b4[:, 2:4] = rng.uniform(0.001, 0.05, 6).astype(np.float16).view(np.uint8).reshape(6, 2)
    got = O.dequant(O.Q4K, b4.reshape(-1), 512, 3)
    ref = np.stack([py_dequant_q4k_block(b) for b in b4]).reshape(3, 512)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    b6 = rng.integers(0, 256, (6, 210), dtype=np.uint8)
    b6[:, 208:210] = rng.uniform(0.001, 0.01, 6).astype(np.float16).view(np.uint8).reshape(6, 2)
    got = O.dequant(O.Q6K, b6.reshape(-1), 512, 3)
    ref = np.stack([py_dequant_q6k_block(b) for b in b6]).reshape(3, 512)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


# ---------- hand-derived known answers ----------

def test_q4k_known_answer_block():
    """d = 0.5, dmin = 0.25; sub-block sb has scale sb+1 and min 2*sb; nibble value = j % 16 for
    even sub-blocks and 15 - j % 16 for odd ones.  Weight = 0.5*(sb+1)*q - 0.25*2*sb."""
    blk = np.zeros(144, dtype=np.uint8)
    blk[0:2] = np.array([0.5], dtype=np.float16).view(np.uint8)
    blk[2:4] = np.array([0.25], dtype=np.float16).view(np.uint8)
    sc = [sb + 1 for sb in range(8)]
    mn = [2 * sb for sb in range(8)]
    s = [0] * 12
    for sb in range(4):                       # packing inverse of tests/ops.rs:29-39
        s[sb] = sc[sb] | ((sc[sb + 4] >> 4) << 6)
        s[sb + 4] = mn[sb] | ((mn[sb + 4] >> 4) << 6)
        s[sb + 8] = (sc[sb + 4] & 0xF) | ((mn[sb + 4] & 0xF) << 4)
    blk[4:16] = s
    for pair in range(4):
        for j in range(32):
            blk[16 + pair * 32 + j] = (j % 16) | ((15 - j % 16) << 4)
    got = O.dequant(O.Q4K, blk, 256, 1)[0]
    for sb in range(8):
        for j in range(32):
            q = (15 - j % 16) if sb % 2 else (j % 16)
            assert got[sb * 32 + j] == 0.5 * (sb + 1) * q - 0.25 * 2 * sb


def test_q6k_known_answer_block():
    """d = 0.25, scale of group g16 = g16 - 8; quant of element i = i % 64 -> weight 0.25*(g16-8)*(i%64-32)."""
    blk = np.zeros(210, dtype=np.uint8)
    for i in range(256):
        q = i % 64
        h, j = divmod(i, 128)
        if j < 64:
            blk[h * 64 + j] |= q & 0xF
        else:
            blk[h * 64 + j - 64] |= (q & 0xF) << 4
        blk[128 + h * 32 + j % 32] |= (q >> 4) << (2 * (j // 32))
    blk[192:208] = (np.arange(16) - 8).astype(np.int8).view(np.uint8)
    blk[208:210] = np.array([0.25], dtype=np.float16).view(np.uint8)
    got = O.dequant(O.Q6K, blk, 256, 1)[0]
    for i in range(256):
        assert got[i] == 0.25 * (i // 16 - 8) * (i % 64 - 32)


# ---------- golden fixtures from gguf-py ----------

GOLDEN_CASES = [(k, K, N, M) for k in ("q4k", "q6k") for (K, N, M) in [(256, 8, 1), (512, 5, 3), (1024, 33, 4), (2048, 16, 7)]]


@pytest.mark.parametrize("kind,K,N,M", GOLDEN_CASES)
def test_oracle_vs_golden(golden, kind, K, N, M):
    tag = f"{kind}_{K}_{N}_{M}"
    dt = O.Q4K if kind == "q4k" else O.Q6K
    blocks, want_w, x, want_y = (golden[tag + s] for s in ("_blocks", "_dequant", "_x", "_y"))
    got_w = O.dequant(dt, blocks, K, N)
    assert np.array_equal(got_w.view(np.uint32), want_w.view(np.uint32)), "dequantised weights must be bit-exact"
    assert O.rel_l2(O.matmul(dt, blocks, K, N, x, acc="f64"), want_y) < 1e-7
    assert O.rel_l2(O.matmul(dt, blocks, K, N, x, acc="f32", threads=1), want_y) < 1e-5
    assert O.rel_l2(O.matmul(dt, blocks, K, N, x, fast=True), want_y) < 1e-5


# ---------- the reference test's generator and cases (tests/ops.rs:14-25, 66-96, 166-185) ----------

def py_xor_stream(seed, n):
    mask = (1 << 64) - 1
    s = ((seed * 0x9E3779B97F4A7C15) & mask) | 1
    out = []
    for _ in range(n):
        s ^= (s << 13) & mask
        s ^= s >> 7
        s ^= (s << 17) & mask
        out.append(s)
    return out


def test_reference_generator_prefix():
    in_f, out_f, seq = 256, 8, 4
    w, x = O.ref_case_q4k(in_f, out_f, seq)
    n_blocks = in_f * out_f // 256
    stream = py_xor_stream(0xC0FFEE ^ (in_f * out_f * seq), n_blocks * 142 + in_f * seq)
    it = iter(stream)
    wb = w.reshape(n_blocks, 144)
    for b in range(n_blocks):
        d = np.float32(0.02) + np.float32(np.float32(next(it) & 0xFF) / np.float32(255.0)) * np.float32(0.03)
        dm = np.float32(0.01) + np.float32(np.float32(next(it) & 0xFF) / np.float32(255.0)) * np.float32(0.02)
        assert wb[b, 0:2].copy().view(np.float16)[0] == np.float16(d)
        assert wb[b, 2:4].copy().view(np.float16)[0] == np.float16(dm)
        assert [int(v) for v in wb[b, 4:]] == [next(it) & 0xFF for _ in range(140)]
    for i in range(in_f * seq):
        f = np.float32(np.float32(next(it) >> 40) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
        assert x[i] == O.f32_to_bf16(float(f))


REF_CASES = [(256, 8, 1), (512, 16, 1), (1024, 64, 1), (4096, 4096, 1), (256, 8, 4), (1024, 64, 7), (4096, 1024, 16)]


@pytest.mark.parametrize("in_f,out_f,seq", REF_CASES)
def test_reference_cases_self_consistent(in_f, out_f, seq):
    """The oracle's f32-sequential result (the reference's `expected`) and its f64 truth agree far
    inside the reference's own tolerance, and the all-cores variant matches too."""
    w, xb = O.ref_case_q4k(in_f, out_f, seq)
    x = O.bf16_bits_to_f32(xb).reshape(seq, in_f)
    e32 = O.matmul(O.Q4K, w, in_f, out_f, x, acc="f32")
    e64 = O.matmul(O.Q4K, w, in_f, out_f, x, acc="f64")
    fast = O.matmul(O.Q4K, w, in_f, out_f, x, fast=True)
    assert O.ref_tolerance_failures(e32, e64, in_f)[0] == 0
    assert O.rel_l2(e32, e64) < 1e-5 and O.rel_l2(fast, e64) < 1e-5
    # sampled rows only: the rest of the output stays zero
    part = O.matmul(O.Q4K, w, in_f, out_f, x, acc="f64", rows=(1, min(out_f, 3)))
    assert np.array_equal(part[:, 1:3], e64[:, 1:3]) and not part[:, 3:].any() and not part[:, :1].any()


def test_matmul_f32_is_sequential_sum():
    """acc='f32' reproduces a strictly left-to-right float32 accumulation (tests/ops.rs:127-136)."""
    w, xb = O.ref_case_q4k(256, 8, 1)
    x = O.bf16_bits_to_f32(xb).reshape(1, 256)
    W = O.dequant(O.Q4K, w, 256, 8)
    got = O.matmul(O.Q4K, w, 256, 8, x, acc="f32", threads=1)
    for r in range(8):
        acc = np.float32(0.0)
        for i in range(256):
            acc = np.float32(acc + np.float32(W[r, i] * x[0, i]))
        assert got[0, r] == acc


def test_embed_is_row_lookup_of_dequant():
    """embed = rows of the dequantised table, in token order (src/backend/mod.rs:25-27)."""
    from llm_rs_b200 import synth
    for dt in (O.Q4K, O.Q6K):
        K, N = 512, 40
        w = synth.weight(dt, K, N, tid=91)
        full = O.dequant(dt, w, K, N)
        toks = [7, 0, 39, 7, 13]
        got = O.embed(dt, w, K, N, toks)
        assert got.shape == (5, K) and np.array_equal(got.view(np.uint32), full[toks].view(np.uint32))
        gb = O.embed(dt, w, K, N, toks, bf16=True)
        assert np.array_equal(O.f32_to_bf16_bits(gb), O.f32_to_bf16_bits(full[toks]))     # idempotent rounding
        assert O.embed(dt, w, K, N, []).shape == (0, K)


def test_small_ops_known_values():
    """silu, mul, add, rms_norm, argmax against values worked out by hand."""
    assert np.allclose(O.silu(np.array([0.0, 1.0, -1.0], np.float32)), [0.0, 0.7310586, -0.26894143], atol=1e-7)
    assert np.array_equal(O.mul(np.array([1.5, -2.0], np.float32), np.array([2.0, 0.25], np.float32)), [3.0, -0.5])
    assert np.array_equal(O.add(np.array([1.5, -2.0], np.float32), np.array([2.0, 0.25], np.float32)), [3.5, -1.75])
    x = np.array([[3.0, 4.0, 0.0, 0.0]], np.float32)                  # mean square 6.25
    got = O.rms_norm(x, np.array([1.0, 2.0, 1.0, 1.0], np.float32), 0.0)
    assert np.allclose(got, [[1.2, 3.2, 0.0, 0.0]], rtol=1e-6)
    assert O.argmax(np.array([1.0, 5.0, 5.0, -2.0], np.float32)) == 1
    # bf16 output is a single round-to-nearest-even of the float32 result
    assert O.add(np.array([1.0], np.float32), np.array([2.0 ** -9], np.float32), bf16=True)[0] == 1.0


def test_rope_scatter_gather_attention_known_values():
    # rope: position 0 leaves x alone; a quarter turn of pair 0 (angle = position * 1) maps (1, 0) to (cos, sin)
    x = np.array([[1.0, 0.0, 2.0, 3.0]], np.float32)
    assert np.array_equal(O.rope(x, [0], 4, 10000.0), x)
    got = O.rope(x, [1], 4, 10000.0)
    assert np.allclose(got[0, :2], [np.cos(1.0), np.sin(1.0)], atol=1e-7)
    a = 1.0 / 10000.0 ** 0.5                                            # pair 1: theta^(-2/4)
    assert np.allclose(got[0, 2:], [2 * np.cos(a) - 3 * np.sin(a), 2 * np.sin(a) + 3 * np.cos(a)], atol=1e-6)
    sp = O.rope(x, [1], 4, 10000.0, split_half=True)                    # pairs (0, 2) and (1, 3)
    assert np.allclose(sp[0, [0, 2]], [np.cos(1.0) - 2 * np.sin(1.0), np.sin(1.0) + 2 * np.cos(1.0)], atol=1e-6)
    # scatter / gather
    pool = np.zeros((4, 2), np.float32)
    out = O.scatter_kv(pool, np.array([[1, 2], [3, 4]], np.float32), [3, 0], 2, 2)
    assert np.array_equal(out, [[3, 4], [0, 0], [0, 0], [1, 2]])
    assert np.array_equal(O.gather(out, [3, 3, 0], 3), [[1, 2], [1, 2], [3, 4]])
    # attention: one head, two positions with equal keys -> the mean of the values; causal for the first query token
    k = np.zeros((4, 32), np.float32); v = np.zeros((4, 32), np.float32)
    v[2], v[3] = 1.0, 3.0                                               # page 1 (block_size 2) holds positions 0, 1
    q = np.ones((2, 32), np.float32)
    o = O.attention(q, k, v, [1], [0, 2], [2], 1, 1, 32, 2, 1)
    assert np.allclose(o[0], 1.0) and np.allclose(o[1], 2.0)


# ---------- the other weight types (F16, BF16, Q8_0, Q4_0): gguf-py fixtures ----------

@pytest.fixture(scope="module")
def golden_other():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "other_dtypes_golden.npz"))


@pytest.mark.parametrize("K,N,M", [(64, 5, 1), (256, 8, 3), (1024, 17, 4)])
def test_oracle_other_dtypes_vs_golden(golden_other, K, N, M):
    g, tag = golden_other, f"{K}_{N}_{M}"
    x = g[f"x_{tag}"]
    for name, dt in (("q8_0", O.Q8_0), ("q4_0", O.Q4_0)):
        blocks = g[f"{name}_{tag}_blocks"]
        assert np.array_equal(O.dequant(dt, blocks, K, N).view(np.uint32), g[f"{name}_{tag}_dequant"].view(np.uint32)), name
        assert O.rel_l2(O.matmul(dt, blocks, K, N, x, acc="f64"), g[f"{name}_{tag}_y"]) < 1e-6
    # the reference reads Q4_0 in its own element order, not ggml's: the two differ by a fixed permutation
    ggml = g[f"q4_0_{tag}_dequant_ggml_order"].reshape(-1, 32)
    ours = O.dequant(O.Q4_0, g[f"q4_0_{tag}_blocks"], K, N).reshape(-1, 32)
    assert np.array_equal(ours[:, 0::2], ggml[:, :16]) and np.array_equal(ours[:, 1::2], ggml[:, 16:])
    for name, dt in (("f16", O.F16), ("bf16", O.BF16)):
        bits = g[f"{name}_{tag}_bits"]
        assert np.array_equal(O.dequant(dt, bits, K, N).view(np.uint32), g[f"{name}_{tag}_dequant"].view(np.uint32)), name
