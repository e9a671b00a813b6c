"""GPU parity of the prompt-phase FFI pair (`launch_mmq_quantize_q8_1_*`, `launch_mmq_gguf_<type>`), driven with the
call sequence of candle-core/src/quantized/fast_mmq.rs:318-385.

Bars: the `block_q8_1_mmq` scratch is bit-exact against the oracle's restatement of the reference quantizer; f32
outputs are within 1e-5 of the oracle's matmul over that scratch (the scratch fixes every rounding but the order of the
f32 additions, which the reference leaves to its tile loops).
"""
import numpy as np
import pytest
import torch

from candle_b200 import capi
from helpers import TYPES, make_case, pad, rel_err

pytestmark = pytest.mark.gpu
LAYOUT = {"q4_0": "DS4", "q4_1": "DS4", "q5_0": "D4", "q5_1": "DS4", "q8_0": "D4", "q2_k": "D2S6", "q3_k": "D4", "q4_k": "DS4", "q5_k": "DS4", "q6_k": "D4"}     # fast_mmq.rs:58-72
GROUP = 144


def _stream():
    return torch.cuda.current_stream().cuda_stream


def quantize_call(lib, layout, x_dev, k, k_padded, ids=None, src_stride=None):
    tokens = x_dev.shape[0] if ids is None else ids.numel()
    groups = k_padded // 128
    scratch = torch.zeros(((groups * tokens + 128) * GROUP,), dtype=torch.uint8, device=x_dev.device)     # fast_mmq.rs:339-345
    scratch[groups * tokens * GROUP:] = 0xCD
    getattr(lib, f"launch_mmq_quantize_q8_1_{layout}")(
        x_dev.data_ptr(), None if ids is None else ids.data_ptr(), scratch.data_ptr(), 0, k, src_stride or k, 0, 0, k_padded,
        tokens, 1, 1, _stream())
    capi.check("mmq quantize")
    torch.cuda.synchronize()
    assert bool((scratch[groups * tokens * GROUP:] == 0xCD).all()), "scratch written past its end"
    return scratch


@pytest.mark.parametrize("layout", ["D4", "DS4", "D2S6"])
@pytest.mark.parametrize("k,tokens", [(128, 1), (300, 5), (4096, 9), (1024, 130)])
def test_mmq_quantizer_is_bit_exact(lib, oracle, cuda_dev, layout, k, tokens):
    rng = np.random.default_rng(k + tokens)
    k4 = pad(k, 4)      # rows are read as float4: candle only calls this with K a multiple of the block size
    x = (rng.standard_normal((tokens, k4)) * rng.uniform(0.01, 30.0, (tokens, 1))).astype(np.float32)
    x[:, k:] = 0
    if tokens > 2:
        x[1, :] = 0.0                 # an all-zero row: d = 0, q = 0 (0 * inf converts to 0)
        x[2, : min(k, 64)] = 0.0      # a zero 32-block inside a live row
    k_padded = pad(pad(k, 512), 128)
    scratch = quantize_call(lib, layout, torch.from_numpy(x).to(cuda_dev), k, k_padded, src_stride=k4)
    got = scratch[: (k_padded // 128) * tokens * GROUP].cpu().numpy().reshape(k_padded // 128, tokens, GROUP)
    ref = oracle.cuda_quantize_mmq_q8_1(np.ascontiguousarray(x[:, :k]), layout, k_padded)
    assert np.array_equal(got, ref)


def test_mmq_quantizer_row_gather(lib, oracle, cuda_dev):
    """`ids` picks source rows (the reference's MoE use of the same kernel)."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 256)).astype(np.float32)
    ids = np.array([4, 0, 0, 5], dtype=np.int32)
    scratch = quantize_call(lib, "DS4", torch.from_numpy(x).to(cuda_dev), 256, 512, ids=torch.from_numpy(ids).to(cuda_dev))
    got = scratch[: 4 * 4 * GROUP].cpu().numpy().reshape(4, 4, GROUP)
    assert np.array_equal(got, oracle.cuda_quantize_mmq_q8_1(x[ids], "DS4", 512))


@pytest.mark.parametrize("tname", list(LAYOUT))
@pytest.mark.parametrize("k,n,tokens", [(256, 3, 1), (512, 70, 9), (4096, 130, 16), (1024, 48, 37), (14336, 24, 11)])
def test_mmq_matmul_matches_oracle(lib, oracle, cuda_dev, tname, k, n, tokens):
    wt = TYPES[tname]
    _, x, wq = make_case(oracle, wt, k, n, tokens, seed=k + n + tokens)
    k_padded = pad(pad(k, 512), 128)
    x_dev, w_dev = torch.from_numpy(x).to(cuda_dev), torch.from_numpy(wq).to(cuda_dev)
    scratch = quantize_call(lib, LAYOUT[tname], x_dev, k, k_padded)
    out = torch.full((tokens * n + 16,), float("nan"), dtype=torch.float32, device=cuda_dev)
    fixup = torch.empty(1024, dtype=torch.float32, device=cuda_dev)
    blk = 256 if tname.endswith("_k") else 32
    getattr(lib, f"launch_mmq_gguf_{tname}")(fixup.data_ptr(), w_dev.data_ptr(), scratch.data_ptr(), out.data_ptr(), k, n, tokens,
                                            k // blk, n, 1000, 148, 232448, 32, _stream())
    capi.check("mmq matmul")
    torch.cuda.synchronize()
    assert lib.cq_mmq_timeout_flag() == 0
    assert bool(torch.isnan(out[tokens * n:]).all()), "output written past its end"
    got = out[: tokens * n].view(tokens, n).cpu().numpy()
    assert not np.isnan(got).any(), "an output element was left unwritten"
    y_ref = oracle.cuda_quantize_mmq_q8_1(x, LAYOUT[tname], k_padded)
    ref = oracle.cuda_mmq(wt, wq, y_ref, k, n)
    assert rel_err(got, ref) <= 1e-5
    # and the Q8_1 arithmetic stays as close to the CPU path as candle's own CUDA kernels do (about 1e-2)
    cpu = oracle.matmul(wt, x, wq, n)
    assert rel_err(got, cpu) <= 3e-2


def test_mmq_argument_checks(lib, cuda_dev):
    lib.cq_clear_status()
    lib.launch_mmq_quantize_q8_1_D4(None, None, None, 0, 256, 256, 0, 0, 512, 1, 1, 1, None)
    assert lib.cq_last_status() == 1
    lib.cq_clear_status()
    buf = torch.zeros(4096, dtype=torch.uint8, device=cuda_dev)
    lib.launch_mmq_quantize_q8_1_D4(buf.data_ptr(), None, buf.data_ptr(), 0, 256, 256, 0, 0, 300, 1, 1, 1, None)   # ne0 % 128
    assert lib.cq_last_status() == 1
    lib.cq_clear_status()
    lib.launch_mmq_gguf_q4_k(None, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), 250, 4, 1, 1, 4, 1000, 148, 0, 32, None)
    assert lib.cq_last_status() == 1
    lib.cq_clear_status()
