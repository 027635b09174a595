"""Regenerates the golden fixtures in this directory:  python tests/golden/make_golden.py

The reference snapshot holds no vectors for this path, so these are build-owned:
seeded canonical inputs (makepad_b200.synth) with the CPU oracle's outputs.
They pin the oracle against accidental change and give the GPU tests a
committed answer that does not depend on the oracle being rebuilt.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from makepad_b200 import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402

Q4_CASES = [(48, 96, 3, 11), (33, 32, 1, 12), (64, 160, 5, 13), (100, 448, 16, 14)]   # N, K, M, seed
FP4_CASES = [(128, 128, 128, 21), (128, 256, 384, 22)]                                # M, N, K, seed


def main():
    orc.build()
    out = {}
    for i, (N, K, M, seed) in enumerate(Q4_CASES):
        codes, scales = synth.q4_weight(N, K, seed)
        x = synth.activations(M, K, seed)
        out[f"q4_{i}_codes"], out[f"q4_{i}_scales"], out[f"q4_{i}_x"] = codes, scales, x
        out[f"q4_{i}_deq"] = orc.q4_dequantize(codes, scales)
        out[f"q4_{i}_y64"] = orc.q4_matmul_f64(codes, scales, x, threads=1)
    np.savez_compressed(os.path.join(HERE, "q4_small.npz"), **out)
    out = {}
    for i, (M, N, K, seed) in enumerate(FP4_CASES):
        a, sfa = synth.nvfp4_tensor(M, K, seed, 0)
        b, sfb = synth.nvfp4_tensor(N, K, seed, 1)
        c32, c16 = orc.nvfp4_gemm(a, sfa, 1.0, b, sfb, 1.0, threads=1)
        out[f"fp4_{i}_a"], out[f"fp4_{i}_sfa"], out[f"fp4_{i}_b"], out[f"fp4_{i}_sfb"] = a, sfa, b, sfb
        out[f"fp4_{i}_c32"], out[f"fp4_{i}_c16"] = c32, c16
        out[f"fp4_{i}_deq_b"] = orc.nvfp4_dequantize(b, sfb, 1.0)
    np.savez_compressed(os.path.join(HERE, "nvfp4_small.npz"), **out)


if __name__ == "__main__":
    main()
