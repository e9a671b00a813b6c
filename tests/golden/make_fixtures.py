"""Writes tests/golden/gemv_cases.npz: small seeded GEMV cases with the oracle's answers.

The reference is Rust and cannot be run here, so these fixtures are produced by the C oracle
(oracle/candle_q_oracle.c), which tests/test_oracle_golden.py pins to the reference's own known-answer
values.  They let the GPU parity tests run against committed numbers as well as against the live oracle.

    python tests/golden/make_fixtures.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402

CASES = [  # (name, oracle type, k, n, batch)
    ("q4_0", O.Q4_0, 512, 24, 3), ("q8_0", O.Q8_0, 512, 24, 3),
    ("q4_k", O.Q4K, 1024, 20, 4), ("q6_k", O.Q6K, 1024, 20, 4),
    ("q4_k_b8", O.Q4K, 768, 33, 8), ("q6_k_b1", O.Q6K, 2048, 17, 1),
]


def main():
    out = {}
    for i, (name, dt, k, n, b) in enumerate(CASES):
        rng = np.random.default_rng(1000 + i)
        wf = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        x = rng.standard_normal((b, k)).astype(np.float32)
        wq = O.quantize(dt, wf)
        q8 = O.cuda_quantize_q8_1(x)
        out[f"{name}.meta"] = np.array([dt, k, n, b], dtype=np.int64)
        out[f"{name}.w"] = wq
        out[f"{name}.x"] = x
        out[f"{name}.q8_1"] = q8
        out[f"{name}.y_cuda"] = O.cuda_mmvq(dt, wq, q8, k, n)
        out[f"{name}.y_cpu"] = O.matmul(dt, x, wq, n, mode=O.SIMD_ORDER)
        out[f"{name}.act_cpu"] = O.quantize(O.vec_dot_type(dt), x)
    np.savez_compressed(os.path.join(HERE, "gemv_cases.npz"), **out)
    print("wrote", os.path.join(HERE, "gemv_cases.npz"))


if __name__ == "__main__":
    main()
