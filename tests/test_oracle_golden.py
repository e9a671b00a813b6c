"""Pins the CPU oracle to the known-answer values held by the reference's own tests.

Every expected number below is a constant of candle's test-suite (file:line given per test); none is
produced by this repository.
"""
import numpy as np
import pytest

Q4_0_EXPECT_CPU = [85120.0, 214562.0, 345455.0, 474748.0, 213475.0, 604465.0, 1000686.0, 1388317.0,
                   341876.0, 994283.0, 1655709.0, 2301518.0]
Q4_0_EXPECT_CUDA = [84866.0, 214045.0, 344676.0, 473707.0, 213425.0, 604313.0, 1000431.0, 1387960.0,
                    342030.0, 994630.0, 1656248.0, 2302250.0]
Q4_0_NEG_EXPECT_CPU = [243524.0, -19596.0, -285051.0, -549815.0, 23777.0, 21651.0, 19398.0, 18367.0,
                       -196472.0, 63012.0, 324585.0, 587902.0]
Q4_0_NEG_EXPECT_CUDA = [243740.0, -19762.0, -285476.0, -550498.0, 23774.0, 21645.0, 19395.0, 18364.0,
                        -196045.0, 63030.0, 324120.0, 587079.0]


def _ramp_case(neg):
    m, k, n = 3, 64, 4
    if neg:
        lhs = (np.arange(m * k, dtype=np.float32) - np.float32(m * k) / np.float32(2.0)).reshape(m, k)
        rhs = (np.arange(k * n, dtype=np.float32) - np.float32(k * n) / np.float32(3.0)).astype(np.float32).reshape(n, k)
    else:
        lhs = np.arange(m * k, dtype=np.float32).reshape(m, k)
        rhs = np.arange(k * n, dtype=np.float32).reshape(n, k)
    return lhs, rhs, (m, k, n)


@pytest.mark.parametrize("neg", [False, True])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_q4_0_matmul_cpu_expected(oracle, neg, mode):
    """candle-core/tests/quantized_tests.rs:92-106 and :152-170 (k_quants::matmul on ramps)."""
    lhs, rhs, (m, k, n) = _ramp_case(neg)
    w = oracle.quantize(oracle.Q4_0, rhs)
    out = oracle.matmul(oracle.Q4_0, lhs, w, n, mode=mode)
    assert np.round(out).ravel().tolist() == (Q4_0_NEG_EXPECT_CPU if neg else Q4_0_EXPECT_CPU)


@pytest.mark.parametrize("neg", [False, True])
def test_q4_0_matmul_cuda_expected(oracle, neg):
    """candle-core/tests/quantized_tests.rs:131-138 and :196-203: what candle's CUDA MMVQ path returns."""
    lhs, rhs, (m, k, n) = _ramp_case(neg)
    w = oracle.quantize(oracle.Q4_0, rhs)
    q = oracle.cuda_quantize_q8_1(lhs)
    out = oracle.cuda_mmvq(oracle.Q4_0, w, q, k, n)
    assert np.round(out).ravel().tolist() == (Q4_0_NEG_EXPECT_CUDA if neg else Q4_0_EXPECT_CUDA)


def test_cuda_mmv_q8_1_exact_value(oracle):
    """candle-core/src/quantized/cuda.rs:1028-1052: Q4_0, k = 256, x = w = 0..255 gives exactly 5561664.5."""
    x = np.arange(256, dtype=np.float32).reshape(1, 256)
    w = oracle.quantize(oracle.Q4_0, x)
    q = oracle.cuda_quantize_q8_1(x)
    assert float(oracle.cuda_mmvq(oracle.Q4_0, w, q, 256, 1)[0, 0]) == 5561664.5


def test_q4_0_roundtrip_vector(oracle):
    """candle-core/tests/quantized_tests.rs:345-377."""
    src = np.arange(128, dtype=np.float32)
    d = oracle.dequantize(oracle.Q4_0, oracle.quantize(oracle.Q4_0, src), 128)[0]
    expect = [-0.0, -0.0, 3.875, 3.875, 3.875, 3.875, 7.75, 7.75, 7.75, 7.75, 11.625, 11.625, 11.625,
              11.625, 15.5, 15.5, 15.5, 15.5, 19.375, 19.375, 19.375, 19.375, 23.25, 23.25, 23.25,
              23.25, 27.125, 27.125, 27.125, 27.125, 31.0, 31.0, 31.5, 31.5, 31.5, 31.5, 39.375,
              39.375, 39.375, 39.375, 39.375, 39.375, 39.375, 39.375, 47.25, 47.25, 47.25, 47.25,
              47.25, 47.25, 47.25, 47.25, 55.125, 55.125, 55.125, 55.125, 55.125, 55.125, 55.125,
              55.125, 63.0, 63.0, 63.0, 63.0, 59.375, 59.375, 71.25, 71.25, 71.25, 71.25, 71.25,
              71.25, 71.25, 71.25, 71.25, 71.25, 71.25, 71.25, 83.125, 83.125, 83.125, 83.125,
              83.125, 83.125, 83.125, 83.125, 83.125, 83.125, 83.125, 83.125, 95.0, 95.0, 95.0, 95.0,
              95.0, 95.0, 95.25, 95.25, 95.25, 95.25, 95.25, 95.25, 95.25, 95.25, 111.125, 111.125,
              111.125, 111.125, 111.125, 111.125, 111.125, 111.125, 111.125, 111.125, 111.125,
              111.125, 111.125, 111.125, 111.125, 111.125, 127.0, 127.0, 127.0, 127.0, 127.0, 127.0,
              127.0, 127.0]
    assert d.tolist() == expect


def _round3(v):
    """round_vector of the reference's tests: three decimals (candle-core/tests/quantized_tests.rs:1034-1040)."""
    t = np.asarray(v, dtype=np.float32) * np.float32(1000.0)
    r = np.copysign(np.floor(np.abs(t) + np.float32(0.5)), t).astype(np.float32)      # f32::round: halves away from zero
    return [float(x) for x in r / np.float32(1000.0)]


Q4_1_EXPECT = [
    0.0, 0.0, 2.066, 2.066, 4.133, 4.133, 6.199, 6.199, 8.266, 8.266, 10.332, 10.332,
    12.398, 12.398, 14.465, 14.465, 16.531, 16.531, 18.598, 18.598, 20.664, 20.664, 22.73,
    22.73, 24.797, 24.797, 26.863, 26.863, 28.93, 28.93, 30.996, 30.996, 32.0, 32.0,
    34.066, 34.066, 36.133, 36.133, 38.199, 38.199, 40.266, 40.266, 42.332, 42.332, 44.398,
    44.398, 46.465, 46.465, 48.531, 48.531, 50.598, 50.598, 52.664, 52.664, 54.73, 54.73,
    56.797, 56.797, 58.863, 58.863, 60.93, 60.93, 62.996, 62.996, 64.0, 64.0, 66.066,
    66.066, 68.133, 68.133, 70.199, 70.199, 72.266, 72.266, 74.332, 74.332, 76.398, 76.398,
    78.465, 78.465, 80.531, 80.531, 82.598, 82.598, 84.664, 84.664, 86.73, 86.73, 88.797,
    88.797, 90.863, 90.863, 92.93, 92.93, 94.996, 94.996, 96.0, 96.0, 98.066, 98.066,
    100.133, 100.133, 102.199, 102.199, 104.266, 104.266, 106.332, 106.332, 108.398,
    108.398, 110.465, 110.465, 112.531, 112.531, 114.598, 114.598, 116.664, 116.664,
    118.73, 118.73, 120.797, 120.797, 122.863, 122.863, 124.93, 124.93, 126.996, 126.996]
Q5_0_EXPECT = [
    -0.0, 1.938, 1.938, 3.875, 3.875, 5.813, 5.813, 7.75, 7.75, 9.688, 9.688, 11.625,
    11.625, 13.563, 13.563, 15.5, 15.5, 17.438, 17.438, 19.375, 19.375, 21.313, 21.313,
    23.25, 23.25, 25.188, 25.188, 27.125, 27.125, 29.063, 29.063, 31.0, 31.5, 31.5, 35.438,
    35.438, 35.438, 35.438, 39.375, 39.375, 39.375, 39.375, 43.313, 43.313, 43.313, 43.313,
    47.25, 47.25, 47.25, 47.25, 51.188, 51.188, 51.188, 51.188, 55.125, 55.125, 55.125,
    55.125, 59.063, 59.063, 59.063, 59.063, 63.0, 63.0, 65.313, 65.313, 65.313, 65.313,
    65.313, 71.25, 71.25, 71.25, 71.25, 71.25, 71.25, 77.188, 77.188, 77.188, 77.188,
    77.188, 77.188, 83.125, 83.125, 83.125, 83.125, 83.125, 83.125, 89.063, 89.063, 89.063,
    89.063, 89.063, 89.063, 95.0, 95.0, 95.0, 95.25, 95.25, 95.25, 95.25, 103.188, 103.188,
    103.188, 103.188, 103.188, 103.188, 103.188, 103.188, 111.125, 111.125, 111.125,
    111.125, 111.125, 111.125, 111.125, 111.125, 119.063, 119.063, 119.063, 119.063,
    119.063, 119.063, 119.063, 119.063, 127.0, 127.0, 127.0, 127.0]


@pytest.mark.parametrize("name,expect", [("Q4_1", Q4_1_EXPECT), ("Q5_0", Q5_0_EXPECT), ("Q5_1", [float(v) for v in range(128)])])
def test_q4_1_q5_0_q5_1_roundtrip_vectors(oracle, name, expect):
    """candle-core/tests/quantized_tests.rs:379-411 (Q4_1), :412-444 (Q5_0), :446-474 (Q5_1): 0..127 quantized and back."""
    dt = getattr(oracle, name)
    src = np.arange(128, dtype=np.float32)
    d = oracle.dequantize(dt, oracle.quantize(dt, src), 128)[0]
    assert _round3(d) == [float(np.float32(e)) for e in expect]


def _test_vector2(bound, size):
    v = np.arange(size, dtype=np.float32)
    return ((v - np.float32(size) / np.float32(2.0)) * np.float32(bound) / (np.float32(size) / np.float32(2.0))).astype(np.float32)


@pytest.mark.parametrize("name,probe,tol,tol_big", [
    ("Q2K", [-0.499, -0.366, -0.249, 0.0, 0.295, 0.492], 0.1, 6.0),    # quantized_tests.rs:752-797
    ("Q3K", [-0.493, -0.37, -0.243, -0.0, 0.292, 0.492], 0.03, 3.5),   # quantized_tests.rs:799-844
    ("Q4K", [-0.5, -0.373, -0.25, 0.0, 0.288, 0.498], 0.017, 4.5),     # quantized_tests.rs:846-891
    ("Q5K", [-0.5, -0.373, -0.25, 0.0, 0.279, 0.499], 0.009, 2.5),     # quantized_tests.rs:893-938
    ("Q6K", [-0.497, -0.372, -0.25, -0.0, 0.284, 0.5], 0.008, 2.0),    # quantized_tests.rs:940-985
    ("Q8K", [-0.5, -0.374, -0.25, -0.0, 0.283, 0.499], 0.008, 0.6),    # quantized_tests.rs:987-1032
])
def test_k_quant_roundtrip_probes(oracle, name, probe, tol, tol_big):
    dt = getattr(oracle, name)
    src = _test_vector2(0.5, 1024)
    assert [float(src[i]) for i in (0, 128, 256, 512, 800, 1023)] == [float(np.float32(v)) for v in (-0.5, -0.375, -0.25, 0.0, 0.28125, 0.49902344)]
    d = oracle.dequantize(dt, oracle.quantize(dt, src), 1024)[0]
    assert np.abs(d - src).max() < tol
    r = np.round(np.float32(1000.0) * d) / np.float32(1000.0)
    assert [float(r[i]) for i in (0, 128, 256, 512, 800, 1023)] == [float(np.float32(p)) for p in probe]
    big = _test_vector2(128.0, 1024)
    dbig = oracle.dequantize(dt, oracle.quantize(dt, big), 1024)[0]
    assert np.abs(dbig - big).max() < tol_big


GGML_ERR = {"Q4_0": 0.001143, "Q4_1": 0.008, "Q5_0": 0.001353, "Q5_1": 0.00149, "Q8_0": 0.000092, "Q2K": 0.004086, "Q3K": 0.017, "Q4K": 0.002425, "Q5K": 0.000740, "Q6K": 0.000952}   # quantized_tests.rs:1101-1122


@pytest.mark.parametrize("name", ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2K", "Q3K", "Q4K", "Q5K", "Q6K"])
@pytest.mark.parametrize("variant", [0, 1])
def test_ggml_matmul_error(oracle, name, variant):
    """candle-core/tests/quantized_tests.rs:1126-1191: opt == unopt within 1e-6 * len, matmul == vec_dot,
    error against the exact dot below llama.cpp's figure for the type."""
    dt = getattr(oracle, name)
    n = 4096
    i = np.arange(n, dtype=np.float32)
    if variant == 0:
        a = (np.float32(0.1) + np.float32(2.0) * np.cos(i + np.float32(0.0))).astype(np.float32)
        b = (np.float32(0.1) + np.float32(2.0) * np.cos(i + np.float32(1.0))).astype(np.float32)
        err_m = 1.0
    else:
        a = (i / np.float32(n)).astype(np.float32)
        b = a.copy()
        err_m = 2.0
    wq = oracle.quantize(dt, a)
    aq = oracle.quantize(oracle.vec_dot_type(dt), b)
    unopt = oracle.vec_dot(dt, wq, aq, n, oracle.SCALAR)
    opt = oracle.vec_dot(dt, wq, aq, n, oracle.SIMD_ORDER)
    hw = oracle.vec_dot(dt, wq, aq, n, oracle.SIMD_HW)
    assert abs(opt - unopt) / n <= 1e-6
    assert opt == hw, "portable restatement of the AVX2 order must give the AVX2 bits"
    mm = float(oracle.matmul(dt, b.reshape(1, n), wq, 1, mode=oracle.SIMD_ORDER)[0, 0])
    assert abs(mm - opt) / n <= 1e-6
    exact = float(np.sum(a.astype(np.float32) * b.astype(np.float32), dtype=np.float32))
    for r in (opt, mm):
        err = abs(r - exact) / n
        assert err <= 0.02 and err - 1e-5 <= GGML_ERR[name] * err_m


@pytest.mark.parametrize("name,limit", [("Q4_0", 0.002), ("Q4_1", 0.002), ("Q5_0", 0.002), ("Q5_1", 0.002), ("Q8_0", 0.002), ("Q2K", 0.0075), ("Q3K", 0.0040), ("Q4K", 0.002), ("Q5K", 0.002), ("Q6K", 0.002)])
def test_quantization_rmse(oracle, name, limit):
    """ggml_quantization_error_test, candle-core/tests/quantized_tests.rs:531-552 (limits :14-17)."""
    dt = getattr(oracle, name)
    src = (np.float32(0.1) + np.float32(2.0) * np.cos(np.arange(4096, dtype=np.float32))).astype(np.float32)
    d = oracle.dequantize(dt, oracle.quantize(dt, src), 4096)[0]
    assert float(np.sqrt(((src - d) ** 2).sum()) / 4096) <= limit


def test_batch_invariance(oracle):
    """qmm_batch, candle-core/tests/quantized_tests.rs:224-259: a row gives the same bits inside any batch."""
    rng = np.random.default_rng(5)
    k, n = 256, 6
    w = oracle.quantize(oracle.Q4K, rng.random((n, k), dtype=np.float32) - np.float32(0.5))
    x = rng.random((2, k), dtype=np.float32) - np.float32(0.5)
    mm = oracle.matmul(oracle.Q4K, x, w, n)
    mm3 = oracle.matmul(oracle.Q4K, np.concatenate([x, x, x]), w, n)
    assert (mm3[2:4] == mm).all() and (mm3[4:] == mm).all()


def test_degenerate_blocks_do_not_trap(oracle):
    """All-zero super-blocks: Q6K makes iscale = -128/0 (k_quants.rs:2122-2127); casts saturate, nothing traps."""
    z = np.zeros(512, dtype=np.float32)
    for dt in (oracle.Q4_0, oracle.Q4_1, oracle.Q5_0, oracle.Q5_1, oracle.Q8_0, oracle.Q2K, oracle.Q3K, oracle.Q4K, oracle.Q5K, oracle.Q6K, oracle.Q8K):
        d = oracle.dequantize(dt, oracle.quantize(dt, z), 512)[0]
        assert np.all(d == 0)


def test_prompt_pair_arithmetic_follows_the_tensor_core_variants(oracle):
    """What running the reference's own tiled kernel on a B200 showed (tests/test_gpu_reference_kernels.py): from Turing on
    it computes Q4_0 on signed codes q - 8 and ignores the stored activation sum - so over the DS4 scratch it agrees with
    the CPU `vec_dot` on Q8_0 blocks to rounding, and NOT with the GEMV formula d4 * (sumi * d8 - 8 * s8), which carries the
    quantization error of the activation sum (~1e-2).  Q4_K / Q5_K round d * sc and dmin * m to f16: within 2e-3 of the
    unrounded GEMV arithmetic, not equal to it."""
    rng = np.random.default_rng(21)
    k, n, m = 2048, 48, 6
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    rel = lambda a, b: float(np.abs(a - b).max() / np.abs(b).max())
    wq = oracle.quantize(oracle.Q4_0, w)
    pair = oracle.cuda_mmq(oracle.Q4_0, wq, oracle.cuda_quantize_mmq_q8_1(x, "DS4"), k, n)
    assert rel(pair, oracle.matmul(oracle.Q4_0, x, wq, n)) <= 1e-5
    gemv = oracle.cuda_mmvq(oracle.Q4_0, wq, oracle.cuda_quantize_q8_1(x, 2048), k, n)
    assert 1e-3 < rel(pair, gemv) < 5e-2
    for dt in (oracle.Q4K, oracle.Q5K):
        wq = oracle.quantize(dt, w)
        pair = oracle.cuda_mmq(dt, wq, oracle.cuda_quantize_mmq_q8_1(x, "DS4"), k, n)
        gemv = oracle.cuda_mmvq(dt, wq, oracle.cuda_quantize_q8_1(x, 2048), k, n)
        # the f16 products AND the different sum term (stored f16 sum of the floats here, d8 * sum(q8) in the GEMV) separate them
        assert 1e-5 < rel(pair, gemv) < 2e-2
