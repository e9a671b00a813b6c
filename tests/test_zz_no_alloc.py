"""The allocation-free decode entry point, cq_qmatmul_decode_static.

Some hosts cannot give this library a workspace: they have reserved all device memory for their own use, or
only the tensors of one call cross their plugin boundary.  For them the library carries a fixed Q8_1 scratch in
its own image.  This test calls that entry point through the C ABI twice in a row, with different inputs and
shapes, and requires the same bits as the regular two-launch path, which takes a caller-provided scratch.
The second call runs over whatever the first one left in the shared array.

Collected last on purpose (file name), so a failure here cannot hide the other tests.
"""
import numpy as np
import pytest
import torch

from candle_b200 import capi
from helpers import TYPES, make_case, pad

pytestmark = pytest.mark.gpu


def _regular_path(lib, tname, w_dev, x_dev, k, n):
    b = x_dev.shape[0]
    kp = pad(k, 512)
    s = torch.cuda.current_stream().cuda_stream
    scratch = torch.empty((b * (kp // 32) * 36,), dtype=torch.uint8, device=x_dev.device)
    out = torch.empty((b, n), dtype=torch.float32, device=x_dev.device)
    lib.launch_mmvq_gguf_quantize_q8_1_f32(x_dev.data_ptr(), scratch.data_ptr(), k, kp, b, s)
    getattr(lib, f"launch_mmvq_gguf_{tname}_f32_plain")(w_dev.data_ptr(), scratch.data_ptr(), out.data_ptr(), k, n,
                                                         kp // 32, n, b, s)
    capi.check("regular path")
    return out


def test_static_scratch_entry_point_matches_regular_path(lib, oracle, cuda_dev):
    lib.cq_clear_status()
    s = torch.cuda.current_stream().cuda_stream
    # two calls in a row: the second one is smaller, so stale bytes of the first stay behind it in the array
    for tname, k, n, b, seed in (("q4_k", 4096, 320, 8, 1), ("q6_k", 1024, 96, 3, 2), ("q4_k", 4096, 320, 8, 3)):
        wt = TYPES[tname]
        _, x, wq = make_case(oracle, wt, k, n, b, seed=seed)
        w_dev = torch.from_numpy(wq).to(cuda_dev)
        x_dev = torch.from_numpy(x).to(cuda_dev)
        want = _regular_path(lib, tname, w_dev, x_dev, k, n)
        got = torch.full((b, n), float("nan"), device=cuda_dev)
        lib.cq_qmatmul_decode_static(wt, w_dev.data_ptr(), x_dev.data_ptr(), capi.F32, got.data_ptr(), k, n, b, s)
        capi.check("static-scratch entry point")
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        ref = oracle.cuda_mmvq(wt, wq, oracle.cuda_quantize_q8_1(x, pad(k, 512)), k, n)
        assert np.abs(got.cpu().numpy() - ref).max() / np.abs(ref).max() <= 1e-3


def test_static_scratch_rejects_oversize(lib, cuda_dev):
    lib.cq_clear_status()
    dummy = torch.zeros(64, device=cuda_dev)
    s = torch.cuda.current_stream().cuda_stream
    # 8 rows of 65536 elements need twice the built-in scratch; nothing may be launched
    lib.cq_qmatmul_decode_static(14, dummy.data_ptr(), dummy.data_ptr(), capi.F32, dummy.data_ptr(), 65536, 4, 8, s)
    assert lib.cq_last_status() == 2 and b"exceeds the built-in scratch" in lib.cq_last_message()
    lib.cq_clear_status()
    lib.cq_qmatmul_decode_static(12, dummy.data_ptr(), dummy.data_ptr(), capi.F32, dummy.data_ptr(), 4096, 4, 9, s)
    assert lib.cq_last_status() == 2
    lib.cq_clear_status()
    torch.cuda.synchronize()
