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


ELEMS = {"f32": (capi.F32, torch.float32), "f16": (capi.F16, torch.float16), "bf16": (capi.BF16, torch.bfloat16)}


def _regular_path(lib, tname, w_dev, x_dev, k, n, elem="f32"):
    b = x_dev.shape[0]
    kp = pad(k, 512)
    s = torch.cuda.current_stream().cuda_stream
    scratch = torch.empty((b * (kp // 32) * 36,), dtype=torch.uint8, device=x_dev.device)
    out = torch.empty((b, n), dtype=x_dev.dtype, device=x_dev.device)
    getattr(lib, f"launch_mmvq_gguf_quantize_q8_1_{elem}")(x_dev.data_ptr(), scratch.data_ptr(), k, kp, b, s)
    getattr(lib, f"launch_mmvq_gguf_{tname}_{elem}_plain")(w_dev.data_ptr(), scratch.data_ptr(), out.data_ptr(), k, n,
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


@pytest.mark.parametrize("elem", ["f16", "bf16"])
def test_static_scratch_half_types_and_no_allocation(lib, oracle, cuda_dev, elem):
    """Activations and outputs in f16 / bf16 (the output type follows x_elem), two calls in a row; and the promise in the
    name: free device memory is the same before and after the calls (the scratch is part of the library image)."""
    code, tdt = ELEMS[elem]
    lib.cq_clear_status()
    s = torch.cuda.current_stream().cuda_stream
    cases = []
    for tname, k, n, b, seed in (("q6_k", 2048, 200, 5, 4), ("q8_0", 1024, 64, 2, 5)):
        wt = TYPES[tname]
        _, x, wq = make_case(oracle, wt, k, n, b, seed=seed)
        w_dev = torch.from_numpy(wq).to(cuda_dev)
        x_dev = torch.from_numpy(x).to(cuda_dev).to(tdt)
        want = _regular_path(lib, tname, w_dev, x_dev, k, n, elem)
        got = torch.full((b, n), float("nan"), dtype=tdt, device=cuda_dev)
        cases.append((wt, w_dev, x_dev, want, got, k, n, b))
    # first call on the device (address look-up) is behind us after this warm-up; then measure
    wt, w_dev, x_dev, want, got, k, n, b = cases[0]
    lib.cq_qmatmul_decode_static(wt, w_dev.data_ptr(), x_dev.data_ptr(), code, got.data_ptr(), k, n, b, s)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(cuda_dev)[0]
    for wt, w_dev, x_dev, want, got, k, n, b in cases:
        lib.cq_qmatmul_decode_static(wt, w_dev.data_ptr(), x_dev.data_ptr(), code, got.data_ptr(), k, n, b, s)
    capi.check("static-scratch entry point, half types")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(cuda_dev)[0] == free_before, "the entry point changed the amount of free device memory"
    for wt, w_dev, x_dev, want, got, k, n, b in cases:
        assert torch.equal(got, want)


def test_static_scratch_rejects_unknown_element_type(lib, oracle, cuda_dev):
    """An element type outside f32 / f16 / bf16 is refused before any launch: dst keeps its contents, so the GEMV cannot
    have run over another call's activations."""
    lib.cq_clear_status()
    s = torch.cuda.current_stream().cuda_stream
    wt, k, n, b = TYPES["q4_k"], 1024, 32, 2
    _, x, wq = make_case(oracle, wt, k, n, b, seed=9)
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    x_dev = torch.from_numpy(x).to(cuda_dev)
    dst = torch.full((b, n), 7.0, device=cuda_dev)
    lib.cq_qmatmul_decode_static(wt, w_dev.data_ptr(), x_dev.data_ptr(), 5, dst.data_ptr(), k, n, b, s)
    torch.cuda.synchronize()
    assert lib.cq_last_status() == 1 and b"x_elem" in lib.cq_last_message()
    lib.cq_clear_status()
    assert bool((dst == 7.0).all())


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
