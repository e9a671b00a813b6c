"""Parity at the benchmark's own sizes and seeds, through the C ABI and the public objects.

The other GPU parity files use small matrices; the launch planner then picks other kernel instantiations (rows per
staged batch, grid) than it does for the shapes the benchmark times.  Here every matrix has its full size - the
128256-row vocabulary head included - so the kernels that are timed are the kernels that are checked, and every output
row is compared with the oracle (the CPU restatement is fast enough for that).

Inputs are regenerated from their seeds (helpers.baseline_weights / baseline_acts: weights f32 N(0, 0.02) seed 0 through
the reference quantizer, activations N(0, 1) seed 1) and checked against the committed SHA-256 digests first.

Bars: Q8_1 activation blocks and per-block integer dot products bit-exact; f32 outputs within 1e-3
(max |a - ref| / max |ref|) of the oracle with the CUDA path's Q8_1 arithmetic, and - in CPU-exact mode - of the
reference's CPU vec_dot (candle-core/src/quantized/k_quants.rs:2375-2492), which is the gate the task states.
Reference tests these follow: candle-core/tests/quantized_tests.rs:92-150, 224-259.
"""
import ctypes
import json
import os

import numpy as np
import pytest
import torch

from candle_b200 import capi
from candle_b200.quantized import GgmlDType, QMatMul, QTensor, set_activation_mode
from helpers import TYPES, baseline_acts, baseline_weights, pad, rel_err, sha256_hex
from test_gpu_gemv import ref_call_sequence

pytestmark = pytest.mark.gpu
TOL = 1e-3
SHA = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "baseline_sha256.json")))
SHAPES = [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096), (4096, 128256)]      # (K, N) of the GEMV sweep
SWEEP_TYPES = ["q4_k", "q6_k", "q8_0"]
BATCHES = [1, 2, 4, 8]


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _plan(lib, wt, act, k, n, b):
    out = (ctypes.c_int * 4)()
    assert lib.cq_mmvq_plan(wt, act, k, n, b, out) == 0
    return tuple(out)       # (kernel, rows per batch, grid, threads)


def _cpu_act(wt):
    return capi.ACT_Q8_K if wt in (10, 11, 12, 13, 14) else capi.ACT_Q8_0


def _sample_rows(n, rows_per_batch, grid):
    """Rows whose position inside the launch differs: first / last row of the first batches, of the batches at the
    wrap-around of the persistent grid, of the last batches and the (possibly ragged) tail, plus 64 seeded random rows."""
    rb = max(1, rows_per_batch)
    cand = []
    for batch in (0, 1, grid - 1, grid, grid + 1, 2 * grid - 1, 2 * grid, (n - 1) // rb - 1, (n - 1) // rb):
        if batch >= 0:
            cand += [batch * rb, batch * rb + rb - 1]
    cand += [n - 1, n - 2]
    cand += list(np.random.default_rng(n).integers(0, n, size=64))
    return np.array(sorted({int(r) for r in cand if 0 <= r < n}), dtype=np.int64)


def test_config1_q4_0_single_matmul(lib, oracle, cuda_dev):
    """Benchmark configuration 1 exactly: Q4_0 weight 4096 x 4096 (seed 0), activation [1, 4096] (seed 1), f32 output [1, 4096]
    against the reference's CPU vec_dot; plus the CUDA path's Q8_1 gate on the same inputs."""
    k = n = 4096
    wq = baseline_weights(oracle, oracle.Q4_0, k, n)
    x = baseline_acts(k, 1)
    assert sha256_hex(wq) == SHA["weights"]["q4_0:4096:4096"]
    assert sha256_hex(baseline_acts(k, 8)) == SHA["acts"]["4096"]
    ref_scalar = oracle.matmul(oracle.Q4_0, x, wq, n, mode=oracle.SCALAR)
    ref_simd = oracle.matmul(oracle.Q4_0, x, wq, n, mode=oracle.SIMD_ORDER)
    assert sha256_hex(ref_scalar) == SHA["config1"]["output_scalar"]
    assert sha256_hex(ref_simd) == SHA["config1"]["output_simd_order"]
    mm = QMatMul.from_qtensor(QTensor.from_data(wq, GgmlDType.Q4_0, (n, k), cuda_dev))
    xd = torch.from_numpy(x).to(cuda_dev)
    set_activation_mode(True)
    try:
        y = mm.forward(xd).cpu().numpy()
    finally:
        set_activation_mode(False)
    assert y.shape == (1, n)
    for ref in (ref_scalar, ref_simd):
        assert rel_err(y, ref) <= TOL
    assert rel_err(y, ref_simd) <= 1e-5
    # the CUDA path of the reference (Q8_1 activations): blocks bit-exact, outputs within the same bar
    q8, out = ref_call_sequence(lib, "q4_0", "f32", torch.from_numpy(wq).to(cuda_dev), xd, k, n)
    q8_ref = oracle.cuda_quantize_q8_1(x, pad(k, 512))
    assert np.array_equal(q8.cpu().numpy(), q8_ref)
    assert rel_err(out.cpu().numpy(), oracle.cuda_mmvq(oracle.Q4_0, wq, q8_ref, k, n)) <= 1e-5
    # both arithmetics describe the same product: they agree to the quantization error of the activations
    assert rel_err(out.cpu().numpy(), ref_simd) <= 5e-2


@pytest.mark.parametrize("k,n", SHAPES)
@pytest.mark.parametrize("tname", SWEEP_TYPES)
def test_config2_gemv_sweep_full_size(lib, oracle, cuda_dev, tname, k, n):
    """Benchmark configuration 2: every (format, shape) of the sweep at its full N, batches 1, 2, 4 and 8; all rows compared."""
    wt = TYPES[tname]
    wq = baseline_weights(oracle, wt, k, n)
    assert sha256_hex(wq) == SHA["weights"][f"{tname}:{k}:{n}"]
    x8 = baseline_acts(k, 8)
    assert sha256_hex(x8) == SHA["acts"][str(k)]
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    mm = QMatMul.from_qtensor(QTensor.from_device_blocks(w_dev, GgmlDType(wt), (n, k)))
    q8_ref8 = oracle.cuda_quantize_q8_1(x8, pad(k, 512))
    base_rows = {}
    for b in BATCHES:
        x = x8[:b]
        x_dev = torch.from_numpy(x).to(cuda_dev)
        # --- the reference's CUDA call sequence (Q8_1 activations) ---
        q8, out = ref_call_sequence(lib, tname, "f32", w_dev, x_dev, k, n)
        assert np.array_equal(q8.cpu().numpy(), q8_ref8[:b]), "Q8_1 blocks differ from the reference quantizer"
        got = out.cpu().numpy()
        ref = oracle.cuda_mmvq(wt, wq, q8_ref8[:b], k, n)
        assert rel_err(got, ref) <= TOL
        assert rel_err(got, ref) <= 1e-5           # only the order of f32 additions differs
        # batch invariance (quantized_tests.rs:224-259): row j has the same bits in every batch that holds it
        for j in range(b):
            if j in base_rows:
                assert np.array_equal(got[j], base_rows[j]), f"row {j} changed between batch sizes"
            else:
                base_rows[j] = got[j].copy()
        # --- CPU-exact mode through the public object: the gate against the reference's CPU vec_dot ---
        set_activation_mode(True)
        try:
            y = mm.forward(x_dev).cpu().numpy()
        finally:
            set_activation_mode(False)
        ref_cpu = oracle.matmul(wt, x, wq, n)
        assert rel_err(y, ref_cpu) <= TOL
        assert rel_err(y, ref_cpu) <= 1e-5
    # --- per-block integer dot products, bit-exact, on rows spread over the launch of the timed plan ---
    plan = _plan(lib, wt, capi.ACT_Q8_1, k, n, 1)
    rows = _sample_rows(n, plan[1], plan[2])
    w_s = np.ascontiguousarray(wq[rows])
    ws_dev = torch.from_numpy(w_s).to(cuda_dev)
    nblk = k // capi.BLOCK_ELEMS[wt]
    x1 = torch.from_numpy(x8[:1]).to(cuda_dev)
    for act in (capi.ACT_Q8_1, _cpu_act(wt)):
        y = torch.zeros((pad(k, 512) // 32 * 36,), dtype=torch.uint8, device=cuda_dev)
        lib.cq_quantize_act(x1.data_ptr(), capi.F32, y.data_ptr(), k, pad(k, 512), 1, act, _stream())
        dots = torch.zeros((len(rows), nblk), dtype=torch.int32, device=cuda_dev)
        dmin = torch.zeros_like(dots)
        lib.cq_block_dots(wt, act, ws_dev.data_ptr(), y.data_ptr(), dots.data_ptr(), dmin.data_ptr(), k, len(rows), _stream())
        capi.check("block dots")
        if act == capi.ACT_Q8_1:
            rd, rm = oracle.cuda_block_dots(wt, w_s, q8_ref8[0], k, len(rows))
        else:
            rd, rm = oracle.cpu_block_dots(wt, w_s, oracle.quantize(oracle.vec_dot_type(wt), x8[:1]), k, len(rows))
        assert np.array_equal(dots.cpu().numpy(), rd)
        if wt == 12:
            assert np.array_equal(dmin.cpu().numpy(), rm)
    assert lib.cq_device_timeout_flag() == 0


def test_timed_plans_are_the_checked_plans(lib, cuda_dev):
    """The sweep above runs the benchmark's 60 (format, shape, batch) cases at full size, so each launches the plan the
    benchmark times.  This records those plans (read-only query) and requires that the cases really differ in kernel
    shape: more than one rows-per-batch value and both small and machine-filling grids occur."""
    plans = {}
    for tname in SWEEP_TYPES:
        for k, n in SHAPES:
            for b in BATCHES:
                for act in (capi.ACT_Q8_1, _cpu_act(TYPES[tname])):
                    plans[(tname, k, n, b, act)] = _plan(lib, TYPES[tname], act, k, n, b)
    kinds = {(p[0], p[1]) for p in plans.values()}
    print("distinct (kernel, rows per batch):", sorted(kinds))
    assert len({p[1] for p in plans.values()}) >= 2
    assert len({p[2] for p in plans.values()}) >= 2


@pytest.mark.parametrize("k,n", [(4096, 14336), (14336, 4096)])
def test_config3_prefill_full_size(lib, oracle, cuda_dev, k, n):
    """Benchmark configuration 3: Q4_K weights of 4096 -> 14336 and 14336 -> 4096 (seed 0), activations [M, K] (seed 1) for
    M = 128, 512, 2048 and 8192 in f32 and bf16, through QMatMul.forward.  The GPU computes the whole output; the oracle
    (reference CPU matmul: the prompt kernel uses its Q8_K arithmetic) checks every weight row for sampled tokens:
    first / last token of several 128-token tiles, the last token, and seeded random ones."""
    wt = TYPES["q4_k"]
    wq = baseline_weights(oracle, wt, k, n)
    assert sha256_hex(wq) == SHA["weights"][f"q4_k:{k}:{n}"]
    mm = QMatMul.from_qtensor(QTensor.from_data(wq, GgmlDType.Q4K, (n, k), cuda_dev))
    xall = baseline_acts(k, 8192)
    for m in (128, 512, 2048, 8192):
        x = xall[:m]
        toks = {0, 1, 127, m - 128, m - 1, m // 2, m // 2 - 1} | {int(t) for t in np.random.default_rng(m).integers(0, m, size=17)}
        toks = np.array(sorted(t for t in toks if 0 <= t < m), dtype=np.int64)
        x_dev = torch.from_numpy(x).to(cuda_dev)
        y = mm.forward(x_dev)
        assert y.shape == (m, n) and not bool(torch.isnan(y).any())
        ref = oracle.matmul(wt, x[toks], wq, n)
        got = y[torch.from_numpy(toks).to(cuda_dev)].cpu().numpy()
        assert rel_err(got, ref) <= TOL, (m, "f32")
        assert rel_err(got, ref) <= 1e-5
        # the same token gives the same row at every M (tile position and tile count do not enter the arithmetic)
        if m > 128:
            assert torch.equal(y[:128], first128)
        else:
            first128 = y[:128].clone()
        del y
        xb = x_dev.to(torch.bfloat16)
        yb = mm.forward(xb)
        assert yb.dtype == torch.bfloat16 and yb.shape == (m, n)
        ref_b = oracle.matmul(wt, xb[torch.from_numpy(toks).to(cuda_dev)].float().cpu().numpy(), wq, n)
        ref_b = torch.from_numpy(ref_b).to(torch.bfloat16).float().numpy()
        got_b = yb[torch.from_numpy(toks).to(cuda_dev)].float().cpu().numpy()
        # the f32 result is rounded once to bf16 (8-bit mantissa): one unit in the last place of the largest output
        assert rel_err(got_b, ref_b) <= 2 ** -8 * 1.01, (m, "bf16")
        del yb, xb, x_dev
    assert lib.cq_prefill_timeout_flag() == 0
