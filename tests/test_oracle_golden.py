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


def _test_vector2(bound, size):
    v = np.arange(size, dtype=np.float32)
    return ((v - np.float32(size) / np.float32(2.0)) * np.float32(bound) / (np.float32(size) / np.float32(2.0))).astype(np.float32)


@pytest.mark.parametrize("name,probe,tol,tol_big", [
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


GGML_ERR = {"Q4_0": 0.001143, "Q8_0": 0.000092, "Q4K": 0.002425, "Q5K": 0.000740, "Q6K": 0.000952}   # quantized_tests.rs:1101-1122


@pytest.mark.parametrize("name", ["Q4_0", "Q8_0", "Q4K", "Q5K", "Q6K"])
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


@pytest.mark.parametrize("name,limit", [("Q4_0", 0.002), ("Q8_0", 0.002), ("Q4K", 0.002), ("Q5K", 0.002), ("Q6K", 0.002)])
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
    for dt in (oracle.Q4_0, oracle.Q8_0, oracle.Q4K, oracle.Q5K, oracle.Q6K, oracle.Q8K):
        d = oracle.dequantize(dt, oracle.quantize(dt, z), 512)[0]
        assert np.all(d == 0)
