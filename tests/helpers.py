"""Helpers shared by the parity tests."""
import numpy as np

# reference GGML ids <-> names used in symbol names
TYPES = {"q4_0": 2, "q4_1": 3, "q5_0": 6, "q5_1": 7, "q8_0": 8, "q2_k": 10, "q3_k": 11, "q4_k": 12, "q5_k": 13, "q6_k": 14}
BLOCK = {2: 32, 3: 32, 6: 32, 7: 32, 8: 32, 10: 256, 11: 256, 12: 256, 13: 256, 14: 256}
TSIZE = {2: 18, 3: 20, 6: 22, 7: 24, 8: 34, 10: 84, 11: 110, 12: 144, 13: 176, 14: 210}


def pad(p, q):
    return (p + q - 1) // q * q


def make_case(oracle, wtype, k, n, b, seed=0, w_std=0.02):
    """Seeded synthetic inputs of the benchmark's kind: W ~ N(0, w_std) quantized with the reference's
    quantizer (restated in the oracle), x ~ N(0, 1)."""
    rng = np.random.default_rng(seed)
    wf = (rng.standard_normal((n, k)) * w_std).astype(np.float32)
    x = rng.standard_normal((b, k)).astype(np.float32)
    wq = oracle.quantize(wtype, wf)
    return wf, x, wq


def rel_err(a, ref):
    """max |a - ref| / max |ref|: the error measure of the parity tests (tolerance 1e-3 per the spec)."""
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30))
