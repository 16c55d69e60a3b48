"""Generates tests/golden/other_dtypes_golden.npz: vectors for the weight types beside Q4_K / Q6_K that
the reference's matmul accepts (F16, BF16, Q8_0, Q4_0; src/backend/metal/mod.rs:503-518).

Source independent of this repository: gguf-py's numpy dequantisers.  Q8_0 is taken as gguf-py gives
it.  Q4_0 needs care: the reference's kernel (shaders/ops.metal:161-190) reads element e of a block from
byte e/2 (low nibble for even e, high nibble for odd e), whereas ggml's Q4_0, which gguf-py implements,
puts the low nibbles of the 16 bytes into elements 0..15 and the high nibbles into elements 16..31.  The
fixture stores gguf-py's values and the reference-order values obtained from them by that permutation
(ref[2 i] = ggml[i], ref[2 i + 1] = ggml[16 + i]); the oracle and the CUDA path follow the reference.

Run once where gguf-py is importable:  python tests/golden/make_golden_other.py
"""
import os

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import quants

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    rng = np.random.default_rng(20240608)
    out = {}
    for K, N, M in ((64, 5, 1), (256, 8, 3), (1024, 17, 4)):
        x = rng.standard_normal((M, K)).astype(np.float32)
        nblk = N * K // 32
        scale = rng.uniform(1e-3, 5e-2, nblk).astype(np.float16)
        scale[0] = np.float16(-0.01)                                   # a negative scale
        scale[1:2].view(np.uint16)[:] = 0x0001                         # the smallest subnormal
        # Q8_0
        b8 = np.zeros((nblk, 34), dtype=np.uint8)
        b8[:, 0:2] = scale.view(np.uint8).reshape(nblk, 2)
        b8[:, 2:] = rng.integers(0, 256, size=(nblk, 32), dtype=np.uint8)
        w8 = quants.dequantize(b8, T.Q8_0).astype(np.float32).reshape(N, K)
        # Q4_0
        b4 = np.zeros((nblk, 18), dtype=np.uint8)
        b4[:, 0:2] = scale.view(np.uint8).reshape(nblk, 2)
        b4[:, 2:] = rng.integers(0, 256, size=(nblk, 16), dtype=np.uint8)
        g4 = quants.dequantize(b4, T.Q4_0).astype(np.float32).reshape(nblk, 32)
        r4 = np.empty_like(g4)
        r4[:, 0::2] = g4[:, :16]
        r4[:, 1::2] = g4[:, 16:]
        tag = f"{K}_{N}_{M}"
        out[f"x_{tag}"] = x
        out[f"q8_0_{tag}_blocks"] = b8.reshape(-1)
        out[f"q8_0_{tag}_dequant"] = w8
        out[f"q8_0_{tag}_y"] = x.astype(np.float64) @ w8.astype(np.float64).T
        out[f"q4_0_{tag}_blocks"] = b4.reshape(-1)
        out[f"q4_0_{tag}_dequant_ggml_order"] = g4.reshape(N, K)
        out[f"q4_0_{tag}_dequant"] = r4.reshape(N, K)
        out[f"q4_0_{tag}_y"] = x.astype(np.float64) @ r4.reshape(N, K).astype(np.float64).T
        # dense
        wf = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
        out[f"f16_{tag}_bits"] = wf.astype(np.float16).view(np.uint16)
        out[f"f16_{tag}_dequant"] = wf.astype(np.float16).astype(np.float32)
        bf = ((wf.view(np.uint32) + (((wf.view(np.uint32) >> 16) & 1) + 0x7FFF)) >> 16).astype(np.uint16)
        out[f"bf16_{tag}_bits"] = bf
        out[f"bf16_{tag}_dequant"] = (bf.astype(np.uint32) << 16).view(np.float32)
    np.savez_compressed(os.path.join(HERE, "other_dtypes_golden.npz"), **out)
    print("wrote other_dtypes_golden.npz", len(out), "arrays")


if __name__ == "__main__":
    main()
