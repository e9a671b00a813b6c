"""Writes tests/golden/baseline_sha256.json: SHA-256 of the benchmark's own inputs as regenerated from their seeds.

    python tests/golden/make_baseline_sha256.py

For every (block format, K, N) of the GEMV sweep and of the Q4_0 single-matmul case: the quantized weight bytes
(f32 N(0, 0.02), seed 0, through the oracle's restatement of the reference quantizer) and the seed-1 activations;
for the Q4_0 case also the oracle's output.  The GPU parity tests regenerate the same inputs on the GPU box and check
the digests first, so a change of generator, numpy or quantizer cannot pass unnoticed.
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from helpers import baseline_acts, baseline_weights, sha256_hex  # noqa: E402
from oracle import oracle as O  # noqa: E402

SHAPES = [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096), (4096, 128256)]      # (K, N)
TYPES = {"q4_k": O.Q4K, "q6_k": O.Q6K, "q8_0": O.Q8_0}


def main():
    out = {"weights": {}, "acts": {}, "config1": {}}
    for tname, t in TYPES.items():
        for k, n in SHAPES:
            out["weights"][f"{tname}:{k}:{n}"] = sha256_hex(baseline_weights(O, t, k, n))
            print(tname, k, n, flush=True)
    for k in (4096, 14336):
        out["acts"][str(k)] = sha256_hex(baseline_acts(k, 8))
    w = baseline_weights(O, O.Q4_0, 4096, 4096)
    x = baseline_acts(4096, 1)
    out["weights"]["q4_0:4096:4096"] = sha256_hex(w)
    out["config1"]["output_scalar"] = sha256_hex(O.matmul(O.Q4_0, x, w, 4096, mode=O.SCALAR))
    out["config1"]["output_simd_order"] = sha256_hex(O.matmul(O.Q4_0, x, w, 4096, mode=O.SIMD_ORDER))
    json.dump(out, open(os.path.join(HERE, "baseline_sha256.json"), "w"), indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
