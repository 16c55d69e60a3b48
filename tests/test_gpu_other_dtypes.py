"""The weight types beside Q4_K / Q6_K that the reference's matmul and embed accept (src/backend/metal/mod.rs:
503-518, 542-562, 634-686, 852-859): dense F32 / F16 / BF16 and Q8_0 / Q4_0, on a B200 through the C ABI
against the CPU oracle.  Dequantised values bit-exact; matmul relative L2 <= 1e-4 on the streaming kernel
(float32 accumulation; up to 8 tokens, and every token count for the block formats), <= 2e-3 on the tensor
cores (dense weights from 9 tokens on: 16-bit or tf32 operands, float32 accumulation)."""
import os

import numpy as np
import pytest

from llm_rs_b200 import BackendError, DType, TensorView, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DENSE = (O.F32, O.F16, O.BF16)
ALL = DENSE + (O.Q8_0, O.Q4_0)


def make_weight(dt, K, N, seed):
    """Raw file bytes of a [K, N] weight of type dt, values of the size real weights have."""
    rng = np.random.default_rng(seed)
    if dt in DENSE:
        w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
        return w if dt == O.F32 else w.astype(np.float16) if dt == O.F16 else O.f32_to_bf16_bits(w).reshape(N, K)
    nblk = N * K // 32
    qb = 32 if dt == O.Q8_0 else 16
    b = np.zeros((nblk, 2 + qb), dtype=np.uint8)
    b[:, 0:2] = rng.uniform(1e-3, 5e-2, nblk).astype(np.float16).view(np.uint8).reshape(nblk, 2)
    b[:, 2:] = rng.integers(0, 256, size=(nblk, qb), dtype=np.uint8)
    return b.reshape(-1)


def upload(be, dt, w, K, N):
    return be.upload_tensor(TensorView("w", DType(dt), [K, N], w))


def run(be, wbuf, x, K, N, M, in_bf16=False, out_bf16=False):
    shape = [K] if M == 1 else [K, M]
    xb = be.upload_tensor(TensorView("x", DType.BF16, shape, synth.bf16_bits(x))) if in_bf16 else \
        be.upload_tensor(TensorView("x", DType.F32, shape, np.ascontiguousarray(x, np.float32)))
    out = be.alloc([N] if M == 1 else [N, M], DType.BF16 if out_bf16 else DType.F32)
    be.matmul(out, wbuf, xb)
    be.sync()
    return be.read_to_vec_f32(out).reshape(M, N)


def tol(dt, M):
    return 2e-3 if (M > 8 and dt in DENSE) else 1e-4


@pytest.mark.parametrize("dt", ALL)
@pytest.mark.parametrize("K,N", [(32, 1), (64, 7), (1024, 33), (4096, 64)])
def test_dequant_bit_exact(backend, dt, K, N):
    w = make_weight(dt, K, N, seed=dt * 100 + K)
    got = backend.dequantize(upload(backend, dt, w, K, N))
    assert np.array_equal(got.view(np.uint32), O.dequant(dt, w, K, N).view(np.uint32))


def test_golden_fixtures(backend):
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "other_dtypes_golden.npz"))
    for K, N, M in ((64, 5, 1), (256, 8, 3), (1024, 17, 4)):
        tag = f"{K}_{N}_{M}"
        x = g[f"x_{tag}"]
        for name, dt in (("q8_0", O.Q8_0), ("q4_0", O.Q4_0)):
            wbuf = upload(backend, dt, g[f"{name}_{tag}_blocks"], K, N)
            assert np.array_equal(backend.dequantize(wbuf).view(np.uint32), g[f"{name}_{tag}_dequant"].view(np.uint32)), name
            assert O.rel_l2(run(backend, wbuf, x, K, N, M), g[f"{name}_{tag}_y"]) <= 1e-4, name
        for name, dt in (("f16", O.F16), ("bf16", O.BF16)):
            wbuf = upload(backend, dt, g[f"{name}_{tag}_bits"], K, N)
            assert np.array_equal(backend.dequantize(wbuf).view(np.uint32), g[f"{name}_{tag}_dequant"].view(np.uint32)), name


@pytest.mark.parametrize("dt", ALL)
@pytest.mark.parametrize("K,N,M", [(64, 1, 1), (256, 9, 1), (4096, 4096, 1), (1024, 300, 2), (2048, 77, 3), (4096, 129, 5),
                                   (1024, 64, 8), (1024, 200, 9), (4096, 513, 16), (2048, 96, 40), (1024, 384, 130),
                                   (4096, 1024, 300), (14336, 40, 17)])
def test_matmul_parity(backend, dt, K, N, M):
    w = make_weight(dt, K, N, seed=7 * K + N)
    x = synth.activations(M, K, tid=5000 + M)
    got = run(backend, upload(backend, dt, w, K, N), x, K, N, M)
    err = O.rel_l2(got, O.matmul(dt, w, K, N, x, acc="f64"))
    assert err <= tol(dt, M), err


@pytest.mark.parametrize("dt", ALL)
@pytest.mark.parametrize("M", [1, 4, 33])
@pytest.mark.parametrize("in_bf16,out_bf16", [(True, False), (False, True), (True, True)])
def test_matmul_bf16_io(backend, dt, M, in_bf16, out_bf16):
    """bf16 activations in and out, as every call of the reference makes them (src/arch/llama.rs:61-66)."""
    K, N = 1024, 136
    w = make_weight(dt, K, N, seed=31 + dt)
    x = synth.activations(M, K, tid=5100 + M)
    xr = O.bf16_bits_to_f32(synth.bf16_bits(x)).reshape(M, K) if in_bf16 else x
    got = run(backend, upload(backend, dt, w, K, N), x, K, N, M, in_bf16, out_bf16)
    err = O.rel_l2(got, O.matmul(dt, w, K, N, xr, acc="f64"))
    assert err <= tol(dt, M) + (2.0 ** -8 if out_bf16 else 0.0), err


@pytest.mark.parametrize("dt", DENSE)
@pytest.mark.parametrize("seq", [1, 32, 256])
def test_reference_bench_shape(backend, dt, seq):
    """The shape of the reference's dense bench (examples/bench_gemm.rs:73-77: 4096 x 4096, bf16 in and out)."""
    K = N = 4096
    w = make_weight(dt, K, N, seed=41)
    x = synth.activations(seq, K, tid=5200 + seq)
    xr = O.bf16_bits_to_f32(synth.bf16_bits(x)).reshape(seq, K)
    got = run(backend, upload(backend, dt, w, K, N), x, K, N, seq, True, True)
    truth = O.matmul(dt, w, K, N, xr, acc="f64", rows=(0, 512))
    assert O.rel_l2(got[:, :512], truth[:, :512]) <= tol(dt, seq) + 2.0 ** -8


@pytest.mark.parametrize("dt", DENSE)
@pytest.mark.parametrize("out_bf16", [False, True])
def test_embed_dense_tables(backend, dt, out_bf16):
    K, vocab = 640, 50
    w = make_weight(dt, K, vocab, seed=51)
    table = upload(backend, dt, w, K, vocab)
    toks = [49, 0, 7, 7, 13]
    out = backend.alloc([K, len(toks)], DType.BF16 if out_bf16 else DType.F32)
    backend.embed(out, table, toks)
    backend.sync()
    want = O.embed(dt, w, K, vocab, toks, bf16=out_bf16)
    assert np.array_equal(backend.read_to_vec_f32(out).reshape(len(toks), K).view(np.uint32), want.view(np.uint32))


def test_errors(backend):
    with pytest.raises(BackendError) as e:                  # Q8_0 rows are whole blocks of 32
        backend.upload_tensor(TensorView("w", DType.Q8_0, [48, 2], np.zeros(3 * 34, np.uint8)))
    assert e.value.code == -2
    w = upload(backend, O.F16, make_weight(O.F16, 36, 4, seed=1), 36, 4)      # K = 36: not a multiple of 8
    x = backend.alloc([36], DType.F32)
    out = backend.alloc([4], DType.F32)
    with pytest.raises(BackendError) as e:
        backend.matmul(out, w, x)
    assert e.value.code == -2 and "multiple of 8" in str(e.value)
    with pytest.raises(BackendError) as e:                  # embed takes no block-format table, like the reference
        backend.embed(backend.alloc([64, 1], DType.F32), upload(backend, O.Q8_0, make_weight(O.Q8_0, 64, 4, seed=2), 64, 4), [1])
    assert e.value.code == -3
