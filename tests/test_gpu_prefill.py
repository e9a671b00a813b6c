"""GPU parity of the prefill path: activation tiles + int8 tcgen05 GEMM for Q4_K, through the C ABI.

The kernel's arithmetic is candle's CPU one (BlockQ8K activations), so the oracle is k_quants::matmul:
activation int8 values and scales bit-exact, outputs within 1e-3 (max |a - ref| / max |ref|).
"""
import numpy as np
import pytest
import torch

from candle_b200 import capi
from candle_b200.quantized import GgmlDType, QMatMul, QTensor
from candle_b200.synth import random_blocks
from helpers import make_case, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3
Q4K = 12


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _prefill(lib, w_dev, x_dev, k, n, out_dtype=torch.float32, wtype=Q4K):
    tokens = x_dev.shape[0]
    elem = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}
    scratch = torch.full((lib.cq_prefill_scratch_bytes(tokens, k),), 0x5A, dtype=torch.uint8, device=x_dev.device)
    out = torch.full((tokens * n + 32,), float("nan"), dtype=out_dtype, device=x_dev.device)
    lib.cq_prefill_quantize(x_dev.data_ptr(), elem[x_dev.dtype], scratch.data_ptr(), k, tokens, _stream())
    lib.cq_prefill_gemm(wtype, w_dev.data_ptr(), scratch.data_ptr(), out.data_ptr(), elem[out_dtype], k, n, tokens, n, _stream())
    capi.check("prefill")
    torch.cuda.synchronize()
    assert lib.cq_prefill_timeout_flag() == 0
    assert bool(torch.isnan(out[tokens * n:].float()).all()), "output written past its end"
    assert not bool(torch.isnan(out[:tokens * n].float()).any()), "an output element was left unwritten"
    return scratch, out[:tokens * n].view(tokens, n)


def _tiles_to_q8k(scratch, tokens, k):
    """Undo the tensor-core tiling of the scratch: returns (int8 [tokens, k], f32 scales [tokens, k/256],
    int32 sums of the sixteen 16-element runs [tokens, k/16] rebuilt from their 64 * hi + lo split)."""
    s = scratch.cpu().numpy()
    nsb = k // 256
    q = np.zeros((tokens, k), dtype=np.int8)
    d = np.zeros((tokens, nsb), dtype=np.float32)
    bs = np.zeros((tokens, nsb, 16), dtype=np.int32)
    for tt in range((tokens + 127) // 128):
        nt = min(128, tokens - tt * 128)
        rows = (nt + 7) // 8 * 8
        for sb in range(nsb):
            off = tt * 128 * 292 * nsb + sb * rows * 292
            blob = s[off:off + rows * 292]
            slabs = blob[:rows * 288].reshape(18, rows, 16)          # [k/16 | lo | hi][token][16]
            q[tt * 128:tt * 128 + nt, sb * 256:(sb + 1) * 256] = slabs[:16].transpose(1, 0, 2).reshape(rows, 256)[:nt].view(np.int8)
            lo, hi = slabs[16][:nt].astype(np.int32), slabs[17][:nt].view(np.int8).astype(np.int32)
            assert lo.max(initial=0) <= 63
            bs[tt * 128:tt * 128 + nt, sb] = 64 * hi + lo
            d[tt * 128:tt * 128 + nt, sb] = blob[rows * 288:rows * 292].view(np.float32)[:nt]
    return q, d, bs


@pytest.mark.parametrize("tokens,k,n", [(128, 256, 64), (17, 512, 64), (100, 1024, 100), (300, 2048, 200),
                                        (129, 768, 33), (64, 4096, 256), (512, 4096, 384), (1000, 14336, 96)])
def test_prefill_matches_cpu_vec_dot(lib, oracle, cuda_dev, tokens, k, n):
    _, x, wq = make_case(oracle, Q4K, k, n, tokens, seed=tokens + k + n)
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    x_dev = torch.from_numpy(x).to(cuda_dev)
    scratch, out = _prefill(lib, w_dev, x_dev, k, n)
    # activation blocks: identical int8 values and scales to BlockQ8K::from_float
    q, d, bs = _tiles_to_q8k(scratch, tokens, k)
    ref_blocks = oracle.quantize(oracle.Q8K, x).reshape(tokens, k // 256, 292)
    assert np.array_equal(q.reshape(tokens, k // 256, 256), ref_blocks[:, :, 4:260].view(np.int8))
    assert np.array_equal(d, ref_blocks[:, :, 0:4].copy().view(np.float32).reshape(tokens, k // 256))
    assert np.array_equal(bs, ref_blocks[:, :, 260:292].copy().view(np.int16).astype(np.int32).reshape(tokens, k // 256, 16))
    ref = oracle.matmul(Q4K, x, wq, n)
    assert rel_err(out.cpu().numpy(), ref) <= TOL
    assert rel_err(out.cpu().numpy(), ref) <= 1e-5     # only the order of f32 additions differs


@pytest.mark.parametrize("tokens,k,n", [(128, 256, 64), (17, 512, 65), (300, 2048, 200), (130, 4096, 96), (520, 14336, 70)])
def test_prefill_q6k_matches_cpu_vec_dot(lib, oracle, cuda_dev, tokens, k, n):
    Q6K = 14
    _, x, wq = make_case(oracle, Q6K, k, n, tokens, seed=tokens + k + n)
    # include negative, zero and extreme sub-block scales
    blk = wq.reshape(-1, 210)
    blk[0, 192:208] = np.array([-128, 127, 0, -1, 1, -64, 64, 5, -5, 100, -100, 33, -33, 2, -2, 0], dtype=np.int8).view(np.uint8)
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    x_dev = torch.from_numpy(x).to(cuda_dev)
    _, out = _prefill(lib, w_dev, x_dev, k, n, wtype=Q6K)
    ref = oracle.matmul(Q6K, x, wq, n)
    assert rel_err(out.cpu().numpy(), ref) <= TOL
    assert rel_err(out.cpu().numpy(), ref) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prefill_half_types(lib, oracle, cuda_dev, dtype):
    tokens, k, n = 200, 1024, 130
    _, x, wq = make_case(oracle, Q4K, k, n, tokens, seed=5)
    xt = torch.from_numpy(x).to(cuda_dev).to(dtype)
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    _, out = _prefill(lib, w_dev, xt, k, n, out_dtype=dtype)
    ref = torch.from_numpy(oracle.matmul(Q4K, xt.float().cpu().numpy(), wq, n)).to(dtype).float().numpy()
    assert rel_err(out.float().cpu().numpy(), ref) <= (2 ** -8 if dtype == torch.bfloat16 else 2 ** -11) * 1.01


def test_prefill_agrees_with_decode_kernel_at_full_size(lib, cuda_dev):
    """The benchmark's prefill shape (4096 -> 14336, 2048 tokens), synthetic blocks: every sampled token must give
    what the decode GEMV gives for it with the same Q8_K activations (two independent kernels, same integers)."""
    k, n, tokens = 4096, 14336, 2048
    w = random_blocks(GgmlDType.Q4K, n, k, seed=3, device=cuda_dev)
    x = torch.randn((tokens, k), device=cuda_dev, generator=torch.Generator(device=cuda_dev).manual_seed(4))
    _, out = _prefill(lib, w, x, k, n)
    rows = torch.tensor([0, 1, 127, 128, 1000, 2047], device=cuda_dev)
    xs = x[rows].contiguous()
    kp = capi.pad(k, 512)
    y = torch.zeros((len(rows), kp // 32 * 36), dtype=torch.uint8, device=cuda_dev)
    lib.cq_quantize_act(xs.data_ptr(), capi.F32, y.data_ptr(), k, kp, len(rows), capi.ACT_Q8_K, _stream())
    dec = torch.empty((len(rows), n), device=cuda_dev)
    lib.cq_mmvq(Q4K, capi.ACT_Q8_K, capi.F32, w.data_ptr(), y.data_ptr(), dec.data_ptr(), k, n, kp // 32, n, len(rows), _stream())
    capi.check("decode reference")
    assert rel_err(out[rows].cpu().numpy(), dec.cpu().numpy()) <= 1e-5
    # duplicated tokens give identical rows (no dependence on the position inside a tile)
    x2 = torch.cat([x[:300], x[:300]])
    _, out2 = _prefill(lib, w, x2, k, n)
    assert torch.equal(out2[:300], out2[300:])


def test_qmatmul_routes_many_rows_to_prefill(oracle, cuda_dev):
    k, n, tokens = 1024, 96, 77
    _, x, wq = make_case(oracle, Q4K, k, n, tokens, seed=8)
    mm = QMatMul.from_qtensor(QTensor.from_data(wq, GgmlDType.Q4K, (n, k), cuda_dev))
    y = mm.forward(torch.from_numpy(x).to(cuda_dev).view(7, 11, k))
    assert y.shape == (7, 11, n)
    assert rel_err(y.view(tokens, n).cpu().numpy(), oracle.matmul(Q4K, x, wq, n)) <= TOL


# ---- the 32-element block formats (Q4_0, Q8_0): every block is its own MMA step, scaled in the epilogue ----

def _prefill32(lib, wtype, w_dev, x_dev, k, n, out_dtype=torch.float32):
    tokens = x_dev.shape[0]
    elem = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}
    scratch = torch.full((lib.cq_prefill32_scratch_bytes(tokens, k),), 0x5A, dtype=torch.uint8, device=x_dev.device)
    out = torch.full((tokens * n + 32,), float("nan"), dtype=out_dtype, device=x_dev.device)
    lib.cq_prefill32_quantize(x_dev.data_ptr(), elem[x_dev.dtype], scratch.data_ptr(), k, tokens, _stream())
    lib.cq_prefill32_gemm(wtype, w_dev.data_ptr(), scratch.data_ptr(), out.data_ptr(), elem[out_dtype], k, n, tokens, n, _stream())
    capi.check("prefill32")
    torch.cuda.synchronize()
    assert lib.cq_prefill32_timeout_flag() == 0
    assert bool(torch.isnan(out[tokens * n:].float()).all()), "output written past its end"
    assert not bool(torch.isnan(out[:tokens * n].float()).any()), "an output element was left unwritten"
    return scratch, out[:tokens * n].view(tokens, n)


def _tiles_to_q8_0(scratch, tokens, k):
    """Undo the tensor-core tiling: int8 [tokens, k] and the f32 scales [tokens, k/32] (f16 values, widened)."""
    s = scratch.cpu().numpy()
    nch = k // 256
    q = np.zeros((tokens, k), dtype=np.int8)
    d = np.zeros((tokens, k // 32), dtype=np.float32)
    for tt in range((tokens + 127) // 128):
        nt = min(128, tokens - tt * 128)
        rows = (nt + 7) // 8 * 8
        for c in range(nch):
            off = tt * 128 * 288 * nch + c * rows * 288
            blob = s[off:off + rows * 288]
            slabs = blob[:rows * 256].reshape(16, rows, 16)
            q[tt * 128:tt * 128 + nt, c * 256:(c + 1) * 256] = slabs.transpose(1, 0, 2).reshape(rows, 256)[:nt].view(np.int8)
            d[tt * 128:tt * 128 + nt, c * 8:(c + 1) * 8] = blob[rows * 256:].view(np.float32).reshape(8, rows)[:, :nt].T
    return q, d


@pytest.mark.parametrize("tname", ["q8_0", "q4_0"])
@pytest.mark.parametrize("tokens,k,n", [(128, 256, 64), (17, 512, 65), (100, 1024, 100), (300, 2048, 200), (129, 768, 33),
                                        (520, 14336, 70), (1000, 4096, 130), (64, 4096, 256)])
def test_block_format_prefill_matches_cpu_vec_dot(lib, oracle, cuda_dev, tname, tokens, k, n):
    """Q4_0 / Q8_0 prompt kernel: BlockQ8_0 activations bit-exact (values and f16 scales), outputs within 1e-3 of the
    reference's CPU matmul (measured: only the order of f32 additions differs); ragged token and row tiles, 1 to 56 stages."""
    from helpers import TYPES
    wt = TYPES[tname]
    _, x, wq = make_case(oracle, wt, k, n, tokens, seed=tokens + k + n)
    x[0, :32] = 0.0                     # an all-zero block: d = 0, q = 0
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    x_dev = torch.from_numpy(x).to(cuda_dev)
    scratch, out = _prefill32(lib, wt, w_dev, x_dev, k, n)
    q, d = _tiles_to_q8_0(scratch, tokens, k)
    ref_blocks = oracle.quantize(oracle.Q8_0, x).reshape(tokens, k // 32, 34)
    assert np.array_equal(q.reshape(tokens, k // 32, 32), ref_blocks[:, :, 2:].view(np.int8))
    assert np.array_equal(d, ref_blocks[:, :, :2].copy().view(np.float16).astype(np.float32).reshape(tokens, k // 32))
    ref = oracle.matmul(wt, x, wq, n)
    assert rel_err(out.cpu().numpy(), ref) <= TOL
    assert rel_err(out.cpu().numpy(), ref) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_block_format_prefill_half_types(lib, oracle, cuda_dev, dtype):
    from helpers import TYPES
    tokens, k, n = 200, 1024, 130
    for tname in ("q8_0", "q4_0"):
        wt = TYPES[tname]
        _, x, wq = make_case(oracle, wt, k, n, tokens, seed=6)
        xt = torch.from_numpy(x).to(cuda_dev).to(dtype)
        _, out = _prefill32(lib, wt, torch.from_numpy(wq).to(cuda_dev), xt, k, n, out_dtype=dtype)
        ref = torch.from_numpy(oracle.matmul(wt, xt.float().cpu().numpy(), wq, n)).to(dtype).float().numpy()
        assert rel_err(out.float().cpu().numpy(), ref) <= (2 ** -8 if dtype == torch.bfloat16 else 2 ** -11) * 1.01


def test_qmatmul_routes_block_formats_to_their_prefill_kernel(oracle, cuda_dev):
    """More than 16 rows of a Q8_0 / Q4_0 matrix take the tensor-core kernel (CPU arithmetic in every mode) when K is a
    multiple of 256, and the GEMV passes otherwise; duplicated rows give identical outputs; the benchmark's shape class."""
    from helpers import TYPES
    for tname, dt in (("q8_0", GgmlDType.Q8_0), ("q4_0", GgmlDType.Q4_0)):
        wt = TYPES[tname]
        k, n, tokens = 4096, 520, 300
        _, x, wq = make_case(oracle, wt, k, n, tokens, seed=9)
        mm = QMatMul.from_qtensor(QTensor.from_data(wq, dt, (n, k), cuda_dev))
        xd = torch.from_numpy(x).to(cuda_dev)
        y = mm.forward(xd)
        assert rel_err(y.cpu().numpy(), oracle.matmul(wt, x, wq, n)) <= 1e-5
        y2 = mm.forward(torch.cat([xd[:150], xd[:150]]))
        assert torch.equal(y2[:150], y2[150:]) and torch.equal(y2[:150], y[:150])
        # K = 288 is not a whole number of stages: GEMV passes (Q8_1 arithmetic) serve it
        k2 = 288
        _, x2, wq2 = make_case(oracle, wt, k2, 40, 20, seed=10)
        mm2 = QMatMul.from_qtensor(QTensor.from_data(wq2, dt, (40, k2), cuda_dev))
        y3 = mm2.forward(torch.from_numpy(x2).to(cuda_dev))
        ref3 = oracle.cuda_mmvq(wt, wq2, oracle.cuda_quantize_q8_1(x2[:8]), k2, 40)
        assert rel_err(y3[:8].cpu().numpy(), ref3) <= 1e-5
