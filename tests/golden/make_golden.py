"""Generates tests/golden/kquant_golden.npz.

The reference (Rust + Metal) cannot run in this build environment and keeps no vectors on
disk, so the fixtures come from two sources that are independent of this repository's code:

  * gguf-py (`gguf.quants.dequantize`, the GGUF project's own numpy dequantisers for the
    Q4_K / Q6_K block formats the reference reads: src/tensor/mod.rs:71,73);
  * a float64 numpy matmul of those dequantised weights with the stored activations.

Run once where gguf-py is importable:  python tests/golden/make_golden.py
The .npz is committed; tests only read it.
"""
import os

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import quants

HERE = os.path.dirname(os.path.abspath(__file__))


def blocks(rng, n, kind):
    if kind == "q4k":
        b = rng.integers(0, 256, size=(n, 144), dtype=np.uint8)
        b[:, 0:2] = rng.uniform(1e-3, 2e-2, n).astype(np.float16).view(np.uint8).reshape(n, 2)
        b[:, 2:4] = rng.uniform(1e-3, 2e-2, n).astype(np.float16).view(np.uint8).reshape(n, 2)
    else:
        b = rng.integers(0, 256, size=(n, 210), dtype=np.uint8)
        b[:, 208:210] = rng.uniform(1e-3, 1e-2, n).astype(np.float16).view(np.uint8).reshape(n, 2)
    return b


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    cases = [("q4k", 256, 8, 1), ("q4k", 512, 5, 3), ("q4k", 1024, 33, 4), ("q4k", 2048, 16, 7),
             ("q6k", 256, 8, 1), ("q6k", 512, 5, 3), ("q6k", 1024, 33, 4), ("q6k", 2048, 16, 7)]
    for kind, K, N, M in cases:
        b = blocks(rng, N * K // 256, kind)
        # a few extreme blocks: all-zero quants, all-max quants, subnormal / negative d
        b[0, 16 if kind == "q4k" else 0:144 if kind == "q4k" else 192] = 0
        b[1, 16 if kind == "q4k" else 0:144 if kind == "q4k" else 192] = 255
        if kind == "q4k":
            b[2, 0:2] = np.array([0x0001], dtype=np.uint16).view(np.uint8)       # smallest subnormal d
            b[3, 2:4] = np.array([-0.015], dtype=np.float16).view(np.uint8)      # negative dmin
        else:
            b[2, 208:210] = np.array([0x0001], dtype=np.uint16).view(np.uint8)
            b[3, 208:210] = np.array([-0.004], dtype=np.float16).view(np.uint8)
        w = quants.dequantize(b, T.Q4_K if kind == "q4k" else T.Q6_K).astype(np.float32).reshape(N, K)
        x = rng.standard_normal((M, K)).astype(np.float32)
        y = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float64)
        tag = f"{kind}_{K}_{N}_{M}"
        out[tag + "_blocks"] = b.reshape(-1)
        out[tag + "_dequant"] = w
        out[tag + "_x"] = x
        out[tag + "_y"] = y
    np.savez_compressed(os.path.join(HERE, "kquant_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "kquant_golden.npz"), len(out), "arrays")


if __name__ == "__main__":
    main()
