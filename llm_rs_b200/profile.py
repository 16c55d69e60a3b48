"""A few launches of one matmul shape on cuda:0: the small process an `ncu` capture wraps.

    python -m llm_rs_b200.profile DTYPE K N M [ITERS]        (DTYPE 12 = Q4_K, 14 = Q6_K)

Prints the device time per launch (events of the context, not under a profiler when run plainly).
The summaries under profiles/ name the exact command they were made with.
"""
from __future__ import annotations

import sys


def profile_case(dtype: int, K: int, N: int, M: int, iters: int = 3) -> None:
    from . import CudaBackend, DType, TensorView, synth
    be = CudaBackend(0)
    w = be.upload_tensor(TensorView("w", DType(dtype), [K, N], synth.weight(dtype, K, N, tid=1)))
    x = be.upload_tensor(TensorView("x", DType.F32, [K] if M == 1 else [K, M], synth.activations(M, K)))
    out = be.alloc([N] if M == 1 else [N, M], DType.F32)
    be.matmul(out, w, x)                      # one call outside the measurement: scratch, attributes
    be.sync()
    be.reset_gpu_secs()
    for _ in range(iters):
        be.matmul(out, w, x)
    be.sync()
    print(f"dtype={dtype} K={K} N={N} M={M}: {be.gpu_secs_total() / iters * 1e6:.2f} us per launch")
    be.close()


if __name__ == "__main__":
    a = [int(v) for v in sys.argv[1:]]
    if len(a) not in (4, 5):
        sys.exit(__doc__)
    profile_case(*a)
