"""Weight-side quantization (`QTensor::quantize` / `quantize_onto`, candle-core/src/quantized/mod.rs:543-562, 645-671).

The library's host quantizer (the ten GGUF block formats) must write the bytes candle's CPU `from_float` writes: it is compared
with the oracle's restatement of those routines byte for byte, and with the known answers of candle's own tests.
"""
import numpy as np
import pytest
import torch

from candle_b200 import capi
from candle_b200.quantized import GgmlDType, QTensor, quantize_blocks

FORMATS = ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2K", "Q3K", "Q4K", "Q5K", "Q6K"]


def _inputs(k):
    rng = np.random.default_rng(20240611)
    n = 6 * k
    ramp = np.arange(n, dtype=np.float32)
    spikes = rng.standard_normal(n).astype(np.float32)
    spikes[::37] *= 50.0
    yield "normal", rng.standard_normal(n).astype(np.float32)
    yield "ramp", ramp
    yield "centred ramp", ((ramp - np.float32(n) / 2) * np.float32(0.5) / (np.float32(n) / 2)).astype(np.float32)
    yield "cosine", (np.float32(0.1) + np.float32(2.0) * np.cos(ramp)).astype(np.float32)
    yield "zeros", np.zeros(n, dtype=np.float32)
    yield "constant", np.full(n, 0.75, dtype=np.float32)
    yield "negative constant", np.full(n, -3.0, dtype=np.float32)
    yield "one value per block", np.where(np.arange(n) % 32 == 5, np.float32(-1.25), np.float32(0)).astype(np.float32)
    yield "outliers", spikes
    yield "tiny", (rng.standard_normal(n) * 1e-30).astype(np.float32)
    yield "large", (rng.standard_normal(n) * 1e4).astype(np.float32)
    yield "uniform positive", rng.random(n, dtype=np.float32)
    yield "signed zeros", np.where(np.arange(n) % 2 == 0, np.float32(0.0), np.float32(-0.0)).astype(np.float32)


@pytest.mark.parametrize("name", FORMATS)
def test_blocks_equal_the_reference_cpu_quantizer(lib, oracle, name):
    dt, odt = GgmlDType[name], getattr(oracle, name)
    for label, x in _inputs(dt.block_size()):
        mine = np.frombuffer(quantize_blocks(x, dt), dtype=np.uint8)
        ref = oracle.quantize(odt, x).reshape(-1)
        assert mine.size == ref.size == x.size // dt.block_size() * dt.type_size()
        assert np.array_equal(mine, ref), (name, label, int(np.flatnonzero(mine != ref)[0]))


@pytest.mark.parametrize("name", FORMATS)
def test_rows_are_quantized_independently(lib, oracle, name):
    """A [rows, k] tensor gives the rows' blocks one after another (mod.rs:543-562 quantizes the flattened storage)."""
    dt = GgmlDType[name]
    k = 2 * dt.block_size()
    x = np.random.default_rng(7).standard_normal((5, 3, k)).astype(np.float32)
    whole = quantize_blocks(x, dt)
    rows = b"".join(quantize_blocks(r, dt) for r in x.reshape(-1, k))
    assert whole == rows
    assert whole == quantize_blocks(torch.from_numpy(x), dt)


def test_q4_0_known_answer(lib, oracle):
    """candle-core/tests/quantized_tests.rs:345-377: 0..127 through Q4_0 and back (first and last block of the vector)."""
    src = np.arange(128, dtype=np.float32)
    blocks = np.frombuffer(quantize_blocks(src, GgmlDType.Q4_0), dtype=np.uint8)
    d = oracle.dequantize(oracle.Q4_0, blocks.reshape(1, -1), 128)[0]
    assert d[:10].tolist() == [-0.0, -0.0, 3.875, 3.875, 3.875, 3.875, 7.75, 7.75, 7.75, 7.75]
    assert d[30:36].tolist() == [31.0, 31.0, 31.5, 31.5, 31.5, 31.5]
    assert d[-8:].tolist() == [127.0] * 8


@pytest.mark.parametrize("name,probe,tol", [("Q2K", [-0.499, -0.366, -0.249, 0.0, 0.295, 0.492], 0.1),      # quantized_tests.rs:752-797
                                            ("Q3K", [-0.493, -0.37, -0.243, -0.0, 0.292, 0.492], 0.03),     # quantized_tests.rs:799-844
                                            ("Q4K", [-0.5, -0.373, -0.25, 0.0, 0.288, 0.498], 0.017),       # quantized_tests.rs:846-891
                                            ("Q5K", [-0.5, -0.373, -0.25, 0.0, 0.279, 0.499], 0.009),       # quantized_tests.rs:893-938
                                            ("Q6K", [-0.497, -0.372, -0.25, -0.0, 0.284, 0.5], 0.008)])     # quantized_tests.rs:940-985
def test_k_quant_known_answers(lib, oracle, name, probe, tol):
    v = np.arange(1024, dtype=np.float32)
    src = ((v - np.float32(512.0)) * np.float32(0.5) / np.float32(512.0)).astype(np.float32)
    blocks = np.frombuffer(quantize_blocks(src, GgmlDType[name]), dtype=np.uint8)
    d = oracle.dequantize(getattr(oracle, name), blocks.reshape(1, -1), 1024)[0]
    assert np.abs(d - src).max() < tol
    r = np.round(np.float32(1000.0) * d) / np.float32(1000.0)
    assert [float(r[i]) for i in (0, 128, 256, 512, 800, 1023)] == [float(np.float32(p)) for p in probe]


@pytest.mark.parametrize("name,limit", [("Q4_0", 0.002), ("Q4_1", 0.002), ("Q5_0", 0.002), ("Q5_1", 0.002), ("Q8_0", 0.002),
                                        ("Q2K", 0.0075), ("Q3K", 0.0040), ("Q4K", 0.002), ("Q5K", 0.002), ("Q6K", 0.002)])
def test_quantization_rmse(lib, oracle, name, limit):
    """ggml_quantization_error_test, candle-core/tests/quantized_tests.rs:531-552 (limits :14-17)."""
    src = (np.float32(0.1) + np.float32(2.0) * np.cos(np.arange(4096, dtype=np.float32))).astype(np.float32)
    blocks = np.frombuffer(quantize_blocks(src, GgmlDType[name]), dtype=np.uint8)
    d = oracle.dequantize(getattr(oracle, name), blocks.reshape(1, -1), 4096)[0]
    assert float(np.sqrt(((src - d) ** 2).sum()) / 4096) <= limit


def test_errors(lib):
    with pytest.raises(capi.CandleQError, match=r"tensor size \(\[4, 100\]\) is not divisible by block size 32"):
        quantize_blocks(np.zeros((4, 100), dtype=np.float32), GgmlDType.Q8_0)
    with pytest.raises(capi.CandleQError, match=r"tensor size \(\[2, 128\]\) is not divisible by block size 256"):
        quantize_blocks(np.zeros((2, 128), dtype=np.float32), GgmlDType.Q4K)
    with pytest.raises(capi.CandleQError, match="weight-side quantization to Q8K is not built"):
        quantize_blocks(np.zeros((2, 256), dtype=np.float32), GgmlDType.Q8K)
    with pytest.raises(capi.CandleQError, match="expects a `src` to be on the cpu"):
        QTensor.quantize_onto(torch.zeros(2, 256, device="meta"), GgmlDType.Q4K)
    with pytest.raises(capi.CandleQError, match="CUDA devices only"):
        QTensor.quantize(torch.zeros(2, 256), GgmlDType.Q4K)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_quantize_onto_fails_loudly_without_a_gpu(lib):
    """The blocks are made on the host, but the tensor lives on a CUDA device: without one the call is an error."""
    with pytest.raises(capi.CandleQError):
        QTensor.quantize_onto(torch.zeros(2, 256), GgmlDType.Q4K)


@pytest.mark.gpu
@pytest.mark.parametrize("name", FORMATS)
def test_quantize_onto_uploads_the_blocks(lib, name):
    dt = GgmlDType[name]
    x = torch.from_numpy(np.random.default_rng(11).standard_normal((24, 512)).astype(np.float32))
    host = quantize_blocks(x, dt)
    t = QTensor.quantize_onto(x, dt, "cuda:0")
    assert t.shape == (24, 512) and t.dtype is dt and t.data() == host
    t2 = QTensor.quantize(x.to("cuda:0"), dt)
    assert t2.device.type == "cuda" and t2.data() == host


# ---- importance-weighted quantization (`quantize_imatrix`, mod.rs:564-642; `from_float_imatrix`, k_quants.rs) --------------
K_FORMATS = ["Q2K", "Q3K", "Q4K", "Q5K", "Q6K"]


def _imatrix_cases():
    rng = np.random.default_rng(99)
    k = 512
    spikes = rng.standard_normal((3, k)).astype(np.float32)
    spikes[:, ::29] *= 40.0
    imp = (rng.random(k) * 4 + 0.01).astype(np.float32)
    yield "normal", rng.standard_normal((3, k)).astype(np.float32), imp
    yield "outliers", spikes, imp
    yield "uniform importance", rng.standard_normal((2, k)).astype(np.float32), np.ones(k, dtype=np.float32)
    yield "positive values", rng.random((2, k), dtype=np.float32), imp
    yield "zeros", np.zeros((1, k), dtype=np.float32), imp
    yield "constant", np.full((1, k), -1.5, dtype=np.float32), imp
    yield "sparse importance", rng.standard_normal((2, k)).astype(np.float32), np.where(np.arange(k) % 7 == 0, imp, np.float32(0)).astype(np.float32)
    yield "one block per row", rng.standard_normal((4, 256)).astype(np.float32), imp[:256]


@pytest.mark.parametrize("name", K_FORMATS)
def test_imatrix_blocks_equal_the_scalar_restatement(lib, name):
    """The compiled quantizer against oracle/imatrix.py (scalar float32 Python written from the same reference source): byte
    for byte.  The importance row of a block is its position inside the matrix row (rows of two blocks wrap)."""
    from oracle import imatrix as scalar
    for label, x, imp in _imatrix_cases():
        mine = quantize_blocks(x, GgmlDType[name], imatrix=imp)
        assert mine == scalar.quantize_imatrix(name, x, imp), (name, label)


@pytest.mark.parametrize("name", K_FORMATS)
def test_imatrix_lowers_the_error_as_in_the_reference_tests(lib, oracle, name):
    """imatrix_quantize_q6k / q5k / q4k / q3k / q2k, candle-core/tests/quantized_tests.rs:555-750: importance values gathered
    from ten random activation batches; the importance-weighted blocks de-quantize closer to the source (mean absolute
    error) than the plain ones.  Seeded synthetic tensors of the reference's shapes stand in for its unseeded ones."""
    rng = np.random.default_rng(0)
    values, rows, ncall = np.zeros(768, dtype=np.float32), 0, 0
    for _ in range(10):
        res = rng.standard_normal((256, 512)).astype(np.float32) @ rng.standard_normal((512, 768)).astype(np.float32)
        values += (res * res).sum(0)
        rows, ncall = rows + res.shape[0], ncall + 1
    imatrix = (values / np.float32(rows) * np.float32(ncall)).astype(np.float32)
    xs = rng.standard_normal((1024, 768)).astype(np.float32)
    dt, odt = GgmlDType[name], getattr(oracle, name)
    plain = np.frombuffer(quantize_blocks(xs, dt), dtype=np.uint8).reshape(1024, -1)
    weighted = np.frombuffer(quantize_blocks(xs, dt, imatrix=imatrix), dtype=np.uint8).reshape(1024, -1)
    err1 = np.abs(oracle.dequantize(odt, plain, 768) - xs).mean()
    err2 = np.abs(oracle.dequantize(odt, weighted, 768) - xs).mean()
    assert err2 < err1, (err2, err1)


def test_imatrix_errors(lib):
    x = np.zeros((2, 512), dtype=np.float32)
    with pytest.raises(capi.CandleQError, match="imatrix weights must have the same length 256 as the last dim of src 512"):
        quantize_blocks(x, GgmlDType.Q4K, imatrix=np.ones(256, dtype=np.float32))
    with pytest.raises(capi.CandleQError, match="`from_float_imatrix` is unimplemented for Q8_0"):
        quantize_blocks(x, GgmlDType.Q8_0, imatrix=np.ones(512, dtype=np.float32))
    with pytest.raises(capi.CandleQError, match="expects a `src` to be on the cpu"):
        QTensor.quantize_imatrix_onto(torch.zeros(2, 256, device="meta"), np.ones(256, dtype=np.float32), GgmlDType.Q4K)
    with pytest.raises(capi.CandleQError, match="CUDA devices only"):
        QTensor.quantize_imatrix(torch.zeros(2, 256), np.ones(256, dtype=np.float32), GgmlDType.Q4K)


def test_load_imatrix(tmp_path):
    """imatrix_file.rs:10-85: entries (name, ncall, values); values are divided by ncall unless it is zero."""
    import struct
    from candle_b200.imatrix_file import load_imatrix

    def entry(name, ncall, vals):
        raw = name.encode()
        return struct.pack("<i", len(raw)) + raw + struct.pack("<ii", ncall, len(vals)) + np.asarray(vals, dtype="<f4").tobytes()

    p = tmp_path / "m.imatrix"
    p.write_bytes(struct.pack("<i", 2) + entry("blk.0.attn_q.weight", 4, [2.0, 8.0, 1.0]) + entry("output.weight", 0, [3.0, 5.0]))
    got = load_imatrix(p)
    assert set(got) == {"blk.0.attn_q.weight", "output.weight"}
    assert got["blk.0.attn_q.weight"].tolist() == [0.5, 2.0, 0.25] and got["output.weight"].tolist() == [3.0, 5.0]
    assert got["output.weight"].dtype == np.float32
    with pytest.raises(capi.CandleQError, match="Failed to open"):
        load_imatrix(tmp_path / "missing.imatrix")
    (tmp_path / "empty.imatrix").write_bytes(struct.pack("<i", 0))
    with pytest.raises(capi.CandleQError, match="No data in file"):
        load_imatrix(tmp_path / "empty.imatrix")
    (tmp_path / "bad.imatrix").write_bytes(struct.pack("<i", 1) + struct.pack("<i", 1) + b"a" + struct.pack("<ii", 1, 0))
    with pytest.raises(capi.CandleQError, match="Invalid nval for entry 1: 0"):
        load_imatrix(tmp_path / "bad.imatrix")
    (tmp_path / "short.imatrix").write_bytes(struct.pack("<i", 1) + struct.pack("<i", 9) + b"abc")
    with pytest.raises(capi.CandleQError, match="Failed to read name for entry 1"):
        load_imatrix(tmp_path / "short.imatrix")
