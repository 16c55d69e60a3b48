"""The allocation-free matmul entry point (llmrs_cuda_matmul_static_scratch).

Some hosts cannot allocate device memory once they are serving: they gave the whole GPU to their
own pool, or they cannot afford the device-wide synchronisation of cudaMalloc/cudaFree.  For them
the tensor-core GEMM keeps its scratch in an 8 MiB array inside the library.  This file is named so
that pytest collects it last: a run that stops at the first failure has then already run every
other test.  It passes alone in a fresh process and after the rest of the suite.
"""
import numpy as np
import pytest

from llm_rs_b200 import BackendError, DType, TensorView, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

GEMM_TOL = 2e-3      # the tolerance the tensor-core path is held to in test_gpu_parity.py


@pytest.mark.parametrize("dt,K,N,M", [(O.Q4K, 4096, 512, 128), (O.Q6K, 2048, 300, 70)])
def test_static_scratch_matches_matmul_twice(backend, dt, K, N, M):
    """Two calls in a row through the C ABI, different activations each time: the shared array
    keeps the first call's contents and the second call must not see them."""
    w = synth.weight(dt, K, N, tid=71)
    wbuf = backend.upload_tensor(TensorView("w", DType(dt), [K, N], w))
    out_ref = backend.alloc([N, M], DType.F32)
    out_new = backend.alloc([N, M], DType.F32)
    for call in range(2):
        x = synth.activations(M, K, tid=80 + call) * np.float32(1.0 + 3.0 * call)
        xbuf = backend.upload_tensor(TensorView("x", DType.F32, [K, M], x))
        backend.matmul(out_ref, wbuf, xbuf)                      # existing entry point (allocating scratch)
        backend.sync()
        want = backend.read_to_vec_f32(out_ref).reshape(M, N)
        backend.matmul_static_scratch(out_new, wbuf, xbuf)       # the entry point under test
        backend.sync()
        got = backend.read_to_vec_f32(out_new).reshape(M, N)
        assert O.rel_l2(got, want) <= GEMM_TOL, f"call {call}"
        assert O.rel_l2(got, O.matmul(dt, w, K, N, x, acc="f64")) <= GEMM_TOL, f"call {call} vs oracle"


def test_static_scratch_small_m_and_bf16(backend):
    """Any M goes through the tensor-core kernel here, also a single token, also bf16 in/out."""
    K, N = 1024, 200
    w = synth.weight(O.Q4K, K, N, tid=72)
    wbuf = backend.upload_tensor(TensorView("w", DType.Q4K, [K, N], w))
    for M in (1, 5):
        x = synth.activations(M, K, tid=90 + M)
        xe = O.bf16_bits_to_f32(synth.bf16_bits(x)).reshape(M, K)
        xbuf = backend.upload_tensor(TensorView("x", DType.BF16, [K] if M == 1 else [K, M], synth.bf16_bits(x)))
        out = backend.alloc([N] if M == 1 else [N, M], DType.BF16)
        backend.matmul_static_scratch(out, wbuf, xbuf)
        backend.sync()
        got = backend.read_to_vec_f32(out).reshape(M, N)
        assert O.rel_l2(got, O.matmul(O.Q4K, w, K, N, xe, acc="f64")) <= GEMM_TOL + 2.0 ** -8


def test_static_scratch_rejects_oversize(backend):
    """Beyond the 8 MiB array the call fails with a message that names both sizes; nothing ran."""
    K, N, M = 4096, 8, 1100          # 2*K*M = 9 011 200 bytes > 8 388 608
    w = synth.weight(O.Q4K, K, N, tid=73)
    wbuf = backend.upload_tensor(TensorView("w", DType.Q4K, [K, N], w))
    xbuf = backend.alloc([K, M], DType.F32)
    out = backend.alloc([N, M], DType.F32)
    with pytest.raises(BackendError) as e:
        backend.matmul_static_scratch(out, wbuf, xbuf)
    assert e.value.code == -2 and "8388608" in str(e.value) and "scratch" in str(e.value)
    # the regular entry point still serves the same shape
    backend.matmul(out, wbuf, xbuf)
    backend.sync()
