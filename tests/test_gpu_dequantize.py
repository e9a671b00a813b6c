"""De-quantize and embedding lookup on the GPU against the oracle's restatement of the CPU `to_float`
(candle-core/src/quantized/k_quants.rs:219-239, 640-656, 1667-1694, 2247-2278): bit-exact f32, round-to-nearest f16 / bf16."""
import numpy as np
import pytest
import torch

from candle_b200 import capi
from candle_b200.capi import CandleQError
from candle_b200.quantized import GgmlDType, QMatMul, QTensor
from helpers import TYPES

pytestmark = pytest.mark.gpu


def _tensor(oracle, wt, n, k, seed):
    rng = np.random.default_rng(seed)
    wf = (rng.standard_normal((n, k)) * rng.uniform(0.01, 2.0, (n, 1))).astype(np.float32)
    wf[0, :min(k, 256)] = 0.0          # an all-zero block
    return oracle.quantize(wt, wf)


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("n,k", [(1, 256), (5, 768), (33, 4096), (2, 14336)])
def test_dequantize_is_bit_exact(oracle, cuda_dev, tname, n, k):
    wt = TYPES[tname]
    wq = _tensor(oracle, wt, n, k, seed=n + k)
    qt = QTensor.from_data(wq.reshape(-1), GgmlDType(wt), (n, k), cuda_dev)
    ref = oracle.dequantize(wt, wq, k)
    got = qt.dequantize()
    assert got.shape == (n, k) and np.array_equal(got.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    assert torch.equal(qt.dequantize(torch.float16), torch.from_numpy(ref).to(cuda_dev).to(torch.float16))
    assert torch.equal(qt.dequantize(torch.bfloat16), torch.from_numpy(ref).to(cuda_dev).to(torch.bfloat16))


@pytest.mark.parametrize("tname", ["q4_k", "q6_k", "q8_0", "q4_0"])
def test_block_formats_with_k_not_a_multiple_of_256(oracle, cuda_dev, tname):
    wt = TYPES[tname]
    if wt in (10, 11, 12, 13, 14):
        pytest.skip("K-quants need K % 256 == 0")
    wq = _tensor(oracle, wt, 3, 288, seed=1)
    qt = QTensor.from_data(wq.reshape(-1), GgmlDType(wt), (3, 288), cuda_dev)
    assert np.array_equal(qt.dequantize().cpu().numpy(), oracle.dequantize(wt, wq, 288))


@pytest.mark.parametrize("tname", list(TYPES))
def test_embedding_gathers_dequantized_rows(oracle, cuda_dev, tname):
    wt = TYPES[tname]
    n, k = 40, 1024
    wq = _tensor(oracle, wt, n, k, seed=7)
    qt = QTensor.from_data(wq.reshape(-1), GgmlDType(wt), (n, k), cuda_dev)
    ids = torch.tensor([[3, 39, 0], [3, 17, 21]], device=cuda_dev)
    out = qt.embedding(ids)
    ref = oracle.dequantize(wt, wq, k)
    assert out.shape == (2, 3, k) and np.array_equal(out.cpu().numpy(), ref[ids.cpu().numpy()])
    with pytest.raises(CandleQError, match="embedding id 40 is out of range for 40 rows"):
        qt.embedding(torch.tensor([1, 40], device=cuda_dev))
    # the C entry point on its own: an id past the end gives zeros and raises the flag
    bad = torch.tensor([2, 1000], dtype=torch.int32, device=cuda_dev)
    o = torch.full((2, k), 7.0, device=cuda_dev)
    L = capi.lib()
    L.cq_get_rows(wt, qt.device_ptr(), bad.data_ptr(), o.data_ptr(), capi.F32, 2, n, k, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.array_equal(o[0].cpu().numpy(), ref[2]) and float(o[1].abs().max()) == 0.0
    assert L.cq_get_rows_bad_id() == 1 and L.cq_get_rows_bad_id() == 0
    L.cq_clear_status()


def test_qmatmul_variants_for_unquantized_tensors_and_dequantize_switches(oracle, cuda_dev, monkeypatch):
    """``QMatMul::from_arc`` (candle-core/src/quantized/mod.rs:837-852): GGUF tensors stored as F32 / F16 / BF16 become the
    dense `Tensor` variant; CANDLE_DEQUANTIZE_ALL turns every tensor into it, CANDLE_DEQUANTIZE_ALL_F16 into `TensorF16`;
    forward of the dense variants is x . W^T over the de-quantized values (:1020-1043)."""
    rng = np.random.default_rng(5)
    n, k = 48, 256
    wf = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((3, 5, k)).astype(np.float32)
    xd = torch.from_numpy(x).to(cuda_dev)
    monkeypatch.delenv("CANDLE_DEQUANTIZE_ALL", raising=False)
    monkeypatch.delenv("CANDLE_DEQUANTIZE_ALL_F16", raising=False)
    for dt, host in ((GgmlDType.F32, wf), (GgmlDType.F16, wf.astype(np.float16)),
                     (GgmlDType.BF16, oracle.f32_to_bf16_bits(wf))):
        qt = QTensor.from_data(host, dt, (n, k), cuda_dev)
        vals = wf if dt == GgmlDType.F32 else host.astype(np.float32) if dt == GgmlDType.F16 else oracle.bf16_bits_to_f32(host)
        assert np.array_equal(qt.dequantize().cpu().numpy(), vals.reshape(n, k))
        mm = QMatMul.from_qtensor(qt)
        assert mm.kind == "Tensor" and mm.dense.dtype == torch.float32
        y = mm.forward(xd).cpu().numpy()
        assert y.shape == (3, 5, n)
        ref = x.reshape(-1, k).astype(np.float64) @ vals.reshape(n, k).astype(np.float64).T
        assert np.abs(y.reshape(-1, n) - ref).max() / np.abs(ref).max() <= 1e-3      # tf32 may be in use for dense f32 products
    # a quantized tensor under the two switches
    wq = oracle.quantize(oracle.Q4K, wf)
    deq = oracle.dequantize(oracle.Q4K, wq, k)
    qt = QTensor.from_data(wq, GgmlDType.Q4K, (n, k), cuda_dev)
    assert QMatMul.from_qtensor(qt).kind == "QTensor"
    for zero_like in ("", "0"):
        monkeypatch.setenv("CANDLE_DEQUANTIZE_ALL", zero_like)
        assert QMatMul.from_qtensor(qt).kind == "QTensor"
    monkeypatch.setenv("CANDLE_DEQUANTIZE_ALL", "1")
    mm = QMatMul.from_qtensor(qt)
    assert mm.kind == "Tensor" and np.array_equal(mm.dense.cpu().numpy(), deq)
    ref = x.reshape(-1, k).astype(np.float64) @ deq.astype(np.float64).T
    assert np.abs(mm.forward(xd).cpu().numpy().reshape(-1, n) - ref).max() / np.abs(ref).max() <= 1e-3
    monkeypatch.delenv("CANDLE_DEQUANTIZE_ALL")
    monkeypatch.setenv("CANDLE_DEQUANTIZE_ALL_F16", "yes")
    mm = QMatMul.from_qtensor(qt)
    assert mm.kind == "TensorF16" and mm.dense.dtype == torch.float16
    y16 = mm.forward(xd)
    assert y16.dtype == torch.float32
    assert np.abs(y16.cpu().numpy().reshape(-1, n) - ref).max() / np.abs(ref).max() <= 2e-2     # f16 weights, inputs and product
    assert torch.equal(mm.dequantize_f16(), mm.dense)
