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


# ---- the benchmark's own inputs (its stated configurations), regenerated from seeds ------------------------------------------------
# Weights: f32 N(0, 0.02) from seed 0, quantized by the reference's quantizer (restated in the oracle); activations: f32
# N(0, 1) from seed 1.  numpy's PCG64 + ziggurat float32 stream; rows are drawn in order, so generating in row chunks
# gives the same values as one call.  tests/golden/baseline_sha256.json pins the resulting bytes.
def baseline_weights(oracle, wtype, k, n, chunk_rows=8192):
    rng = np.random.Generator(np.random.PCG64(0))
    parts = []
    for r0 in range(0, n, chunk_rows):
        rows = min(chunk_rows, n - r0)
        wf = rng.standard_normal((rows, k), dtype=np.float32)
        wf *= np.float32(0.02)
        parts.append(oracle.quantize(wtype, wf))
    return np.concatenate(parts, axis=0) if len(parts) > 1 else parts[0]


def baseline_acts(k, rows):
    """The first `rows` rows of the seed-1 activation stream of width k (so batch 2 is the first two rows of batch 8)."""
    rng = np.random.Generator(np.random.PCG64(1))
    return rng.standard_normal((rows, k), dtype=np.float32)


def sha256_hex(a) -> str:
    import hashlib
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8).tobytes()).hexdigest()
