"""Parity at the full sizes the benchmark times, for the token counts and shapes whose kernel choice
(decode kernel, two-term or one-term tensor-core kernel, split of the last wave) depends on the shape:
the output projection at 32 and 64 tokens, the feed-forward GEMMs at 128 and 512 tokens, and the
K = 8192 and K = 28672 matrices of a 70B-shaped model.  A seeded sample of output rows, all tokens,
against the float64 oracle (the pattern of the reference's check_matmul, tests/ops.rs:91-157), plus
linearity over the whole output.  Tolerances: 1e-4 up to 64 tokens, 2e-3 above (relative L2)."""
import numpy as np
import pytest

from llm_rs_b200 import DType, TensorView, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _upload_w(be, dt, w, K, N):
    return be.upload_tensor(TensorView("w", DType(dt), [K, N], w))


def _run(be, wbuf, x, K, N, M):
    xb = be.upload_tensor(TensorView("x", DType.F32, [K] if M == 1 else [K, M], np.ascontiguousarray(x, np.float32)))
    out = be.alloc([N] if M == 1 else [N, M], DType.F32)
    be.matmul(out, wbuf, xb)
    be.sync()
    return be.read_to_vec_f32(out).reshape(M, N)


def _tol(M):
    return 1e-4 if M <= 64 else 2e-3


def _check_sampled(got, dt, w, K, N, x, M, seed, n_runs, run=128):
    """`n_runs` runs of `run` consecutive rows (first and last run always) against the oracle."""
    rng = np.random.default_rng(seed)
    starts = sorted({0, N - run} | {int(v) // 8 * 8 for v in rng.integers(0, N - run, max(0, n_runs - 2))})
    for a in starts:
        truth = O.matmul(dt, w, K, N, x, acc="f64", rows=(a, a + run), fast=M > 64 and a not in (0, N - run))
        err = O.rel_l2(got[:, a:a + run], truth[:, a:a + run])
        assert err <= _tol(M), (a, err)


@pytest.fixture(scope="module")
def output_projection(backend):
    K, N = 4096, 128256
    w = synth.weight(O.Q6K, K, N, tid=2)
    return K, N, w, _upload_w(backend, O.Q6K, w, K, N)


@pytest.mark.parametrize("M", [2, 4, 32, 64])
def test_config2_output_projection_more_tokens(backend, output_projection, M):
    K, N, w, wbuf = output_projection
    x1 = synth.activations(M, K, tid=3)
    x2 = synth.activations(M, K, tid=4)
    y1 = _run(backend, wbuf, x1, K, N, M)
    y2 = _run(backend, wbuf, x2, K, N, M)
    y3 = _run(backend, wbuf, np.float32(0.5) * x1 + x2, K, N, M)
    assert O.rel_l2(y3, 0.5 * y1.astype(np.float64) + y2) <= 2 * _tol(M)
    _check_sampled(y1, O.Q6K, w, K, N, x1, M, seed=70 + M, n_runs=8, run=512)      # 4096 rows x all tokens


@pytest.mark.parametrize("M", [128, 512])
def test_config3_feed_forward_gemms_fewer_tokens(backend, M):
    """Q4_K 4096 -> 14336 and Q6_K 14336 -> 4096 at 128 and 512 tokens (the 2048-token case is tested
    with the other prefill tests)."""
    for dt, K, N, tid in ((O.Q4K, 4096, 14336, 61), (O.Q6K, 14336, 4096, 62)):
        w = synth.weight(dt, K, N, tid=tid)
        wbuf = _upload_w(backend, dt, w, K, N)
        x = synth.activations(M, K, tid=63 + M)
        y = _run(backend, wbuf, x, K, N, M)
        _check_sampled(y, dt, w, K, N, x, M, seed=80 + M, n_runs=32)               # 4096 rows x all tokens
        # power-of-two token scaling: the same tensor-core products, so twice the result up to the order
        # in which the K pieces of a split tile are added (which CTA arrives last differs run to run)
        y2 = _run(backend, wbuf, np.float32(2.0) * x, K, N, M)
        assert O.rel_l2(y2, 2.0 * y.astype(np.float64)) <= 1e-6


@pytest.mark.parametrize("dt,K,N", [(O.Q4K, 8192, 1024), (O.Q4K, 8192, 8192), (O.Q6K, 28672, 8192), (O.Q4K, 8192, 28672)])
@pytest.mark.parametrize("M", [1, 4, 16, 64, 512])
def test_config5_70b_shapes(backend, dt, K, N, M):
    if K == 28672 and M == 512:
        n_runs = 4                                               # the oracle's share of the time, not the GPU's
    else:
        n_runs = 8
    w = synth.weight(dt, K, N, tid=5 * K + N)
    wbuf = _upload_w(backend, dt, w, K, N)
    x = synth.activations(M, K, tid=90 + M)
    y = _run(backend, wbuf, x, K, N, M)
    assert np.isfinite(y).all()
    _check_sampled(y, dt, w, K, N, x, M, seed=K + M, n_runs=n_runs)
