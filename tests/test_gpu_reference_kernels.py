"""This library's kernels, and the CPU oracle, against the REFERENCE'S OWN CUDA kernels run on the same GPU.

oracle/build_ref.py compiles candle-kernels/src/mmvq_gguf.cu and the mmq_gguf sources unmodified for sm_100a into
oracle/_ref/ (test infrastructure; the product never loads them).  Both libraries export the launcher symbols of
candle-kernels/src/ffi.rs, so one call sequence drives either.  Skipped when the reference build is not present."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from candle_b200 import capi
from helpers import pad, rel_err
from test_gpu_gemv import TYPES, make_case, ref_call_sequence

pytestmark = pytest.mark.gpu
REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")
vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64


@pytest.fixture(scope="module")
def ref_mmvq():
    path = os.path.join(REF_DIR, "libcandle_ref_mmvq.so")
    if not os.path.isfile(path):
        pytest.skip("the reference's MMVQ kernels were not built (oracle/build_ref.py)")
    L = C.CDLL(path)
    for e in ("f32", "f16", "bf16"):
        getattr(L, f"launch_mmvq_gguf_quantize_q8_1_{e}").argtypes = [vp, vp, i32, i32, i32, vp]
        getattr(L, f"launch_mmvq_gguf_quantize_q8_1_{e}").restype = None
        for t in TYPES:
            f = getattr(L, f"launch_mmvq_gguf_{t}_{e}_plain")
            f.argtypes, f.restype = [vp, vp, vp, i32, i32, i32, i32, i32, vp], None
    return L


@pytest.fixture(scope="module")
def ref_mmq():
    path = os.path.join(REF_DIR, "libcandle_ref_mmq.so")
    if not os.path.isfile(path):
        pytest.skip("the reference's MMQ kernels were not built (oracle/build_ref.py)")
    L = C.CDLL(path)
    for layout in ("D4", "DS4", "D2S6"):
        f = getattr(L, f"launch_mmq_quantize_q8_1_{layout}")
        f.argtypes, f.restype = [vp, vp, vp, i32, i64, i64, i64, i64, i64, i64, i64, i64, vp], None
    for t in TYPES:
        f = getattr(L, f"launch_mmq_gguf_{t}")
        f.argtypes, f.restype = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i32, i32, i64, i32, vp], None
    return L


@pytest.mark.parametrize("elem", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("k,rows", [(256, 1), (4096, 8), (768, 5), (14336, 3), (1056, 2)])
def test_q8_1_quantizer_gives_the_reference_kernels_bytes(lib, ref_mmvq, oracle, cuda_dev, elem, k, rows):
    """Activation quantization, bit for bit: this library == the reference kernel == the oracle (f32)."""
    dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[elem]
    x = (torch.randn(rows, k, device=cuda_dev, generator=torch.Generator(device=cuda_dev).manual_seed(k + rows)) * 3).to(dt)
    kp = pad(k, 512)
    st = torch.cuda.current_stream().cuda_stream
    mine = torch.zeros(rows * kp // 32 * 36, dtype=torch.uint8, device=cuda_dev)
    theirs = torch.zeros_like(mine)
    getattr(lib, f"launch_mmvq_gguf_quantize_q8_1_{elem}")(x.data_ptr(), mine.data_ptr(), k, kp, rows, st)
    getattr(ref_mmvq, f"launch_mmvq_gguf_quantize_q8_1_{elem}")(x.data_ptr(), theirs.data_ptr(), k, kp, rows, st)
    capi.check("quantize")
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)
    if elem == "f32":
        assert np.array_equal(theirs.cpu().numpy().reshape(rows, -1), oracle.cuda_quantize_q8_1(x.cpu().numpy(), kp))


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("k,n,b", [(256, 3, 2), (4096, 257, 1), (2048, 96, 4), (14336, 48, 8), (4096, 64, 7), (1024, 33, 5)])
def test_gemv_against_the_reference_kernel(lib, ref_mmvq, oracle, cuda_dev, tname, k, n, b):
    """The `_plain` GEMV of all ten formats: this library and the oracle's restatement of the reference's thread map
    against the reference kernel itself on the same inputs (Q8_1 bytes equal; f32 sums differ by their order only)."""
    wt = TYPES[tname]
    _, x, wq = make_case(oracle, wt, k, n, b, seed=k + n + b)
    w_dev, x_dev = torch.from_numpy(wq).to(cuda_dev), torch.from_numpy(x).to(cuda_dev)
    q_mine, y_mine = ref_call_sequence(lib, tname, "f32", w_dev, x_dev, k, n)
    q_ref, y_ref = ref_call_sequence(ref_mmvq, tname, "f32", w_dev, x_dev, k, n)
    assert torch.equal(q_mine, q_ref)
    y_ref = y_ref.cpu().numpy()
    assert rel_err(y_mine.cpu().numpy(), y_ref) <= 1e-5
    y_oracle = oracle.cuda_mmvq(wt, wq, q_ref.cpu().numpy(), k, n)
    assert rel_err(y_oracle, y_ref) <= 1e-5


@pytest.mark.parametrize("tname,elem", [("q4_k", "f16"), ("q6_k", "bf16"), ("q8_0", "f16"), ("q4_0", "bf16")])
def test_gemv_16_bit_results_against_the_reference_kernel(lib, ref_mmvq, oracle, cuda_dev, tname, elem):
    dt = {"f16": torch.float16, "bf16": torch.bfloat16}[elem]
    k, n, b = 4096, 130, 3
    _, x, wq = make_case(oracle, TYPES[tname], k, n, b, seed=5)
    w_dev, x_dev = torch.from_numpy(wq).to(cuda_dev), torch.from_numpy(x).to(cuda_dev).to(dt)
    _, y_mine = ref_call_sequence(lib, tname, elem, w_dev, x_dev, k, n)
    _, y_ref = ref_call_sequence(ref_mmvq, tname, elem, w_dev, x_dev, k, n)
    ulp = 2.0 ** -10 if elem == "f16" else 2.0 ** -7
    a, r = y_mine.float().cpu().numpy(), y_ref.float().cpu().numpy()
    assert np.all(np.abs(a - r) <= ulp * np.maximum(np.abs(r), np.abs(r).max() * 1e-3))     # the same value up to one rounding step


@pytest.mark.parametrize("tname", ["q4_k", "q6_k", "q8_0"])
@pytest.mark.parametrize("b", [1, 8])
def test_vocabulary_head_against_the_reference_kernel(lib, ref_mmvq, cuda_dev, tname, b):
    """4096 -> 128256 at full size on synthetic blocks: every output of this library's GEMV (dp4a at one row, the warp-tile
    tensor-core kernel at eight) against the reference kernel's."""
    from candle_b200.quantized import GgmlDType
    from candle_b200.synth import random_blocks
    k, n = 4096, 128256
    dtype = {"q4_k": GgmlDType.Q4K, "q6_k": GgmlDType.Q6K, "q8_0": GgmlDType.Q8_0}[tname]
    w_dev = random_blocks(dtype, n, k, seed=3, device=cuda_dev)
    x_dev = torch.randn(b, k, device=cuda_dev, generator=torch.Generator(device=cuda_dev).manual_seed(1))
    _, y_mine = ref_call_sequence(lib, tname, "f32", w_dev, x_dev, k, n)
    _, y_ref = ref_call_sequence(ref_mmvq, tname, "f32", w_dev, x_dev, k, n)
    assert rel_err(y_mine.cpu().numpy(), y_ref.cpu().numpy()) <= 1e-5


def _mmq_call(L, tname, layout, w_dev, x_dev, k, n, m):
    """The prompt-phase call pair of candle-core/src/quantized/fast_mmq.rs:318-385 with its workspace sizes."""
    st = torch.cuda.current_stream().cuda_stream
    kp = pad(pad(k, 512), 128)
    scratch = torch.zeros(((kp // 128) * m + 128) * 144, dtype=torch.uint8, device=x_dev.device)
    fixup = torch.zeros(256 * 128 * 128, dtype=torch.float32, device=x_dev.device)
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device=x_dev.device)
    qk = 256 if tname.endswith("_k") else 32
    getattr(L, f"launch_mmq_quantize_q8_1_{layout}")(x_dev.data_ptr(), None, scratch.data_ptr(), 0, k, k, 0, 0, kp, m, 1, 1, st)
    getattr(L, f"launch_mmq_gguf_{tname}")(fixup.data_ptr(), w_dev.data_ptr(), scratch.data_ptr(), y.data_ptr(), k, n, m, k // qk, n,
                                            1000, 148, 232448, 32, st)
    torch.cuda.synchronize()
    return scratch[:(kp // 128) * m * 144], y


MMQ_LAYOUT = {"q4_0": "DS4", "q4_1": "DS4", "q5_0": "D4", "q5_1": "DS4", "q8_0": "D4", "q2_k": "D2S6", "q3_k": "D4", "q4_k": "DS4",
              "q5_k": "DS4", "q6_k": "D4"}       # candle-kernels/src/mmq_gguf/mmq_gguf.cuh:55-90


@pytest.mark.parametrize("tname,layout", list(MMQ_LAYOUT.items()))
@pytest.mark.parametrize("k,n,m", [(512, 70, 9), (2048, 192, 130), (4096, 384, 64)])
def test_prompt_call_pair_against_the_reference_kernel(lib, ref_mmq, oracle, cuda_dev, tname, layout, k, n, m):
    """`launch_mmq_quantize_q8_1_*` + `launch_mmq_gguf_*`: the reference's tiled int8 GEMM (stream-k, fix-up pass) against
    this library's implementation of the same two entry points: scratch bytes equal, outputs equal up to the f32 order."""
    _, x, wq = make_case(oracle, TYPES[tname], k, n, m, seed=k + n + m)
    w_dev, x_dev = torch.from_numpy(wq).to(cuda_dev), torch.from_numpy(x).to(cuda_dev)
    s_ref, y_ref = _mmq_call(ref_mmq, tname, layout, w_dev, x_dev, k, n, m)
    s_mine, y_mine = _mmq_call(lib, tname, layout, w_dev, x_dev, k, n, m)
    capi.check("mmq pair")
    assert torch.equal(s_mine, s_ref)
    assert not bool(torch.isnan(y_ref).any()) and not bool(torch.isnan(y_mine).any())
    assert rel_err(y_mine.cpu().numpy(), y_ref.cpu().numpy()) <= 1e-5
    y_oracle = oracle.cuda_mmq(TYPES[tname], wq, s_ref.cpu().numpy().reshape(-1, m, 144), k, n)
    assert rel_err(y_oracle, y_ref.cpu().numpy()) <= 1e-5


@pytest.fixture(scope="module")
def ref_moe():
    path = os.path.join(REF_DIR, "libcandle_ref_moe.so")
    if not os.path.isfile(path):
        pytest.skip("the reference's MoE kernels were not built (oracle/build_ref.py)")
    L = C.CDLL(path)
    L.moe_gemm_gguf.argtypes, L.moe_gemm_gguf.restype = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp], None
    L.moe_gemm_gguf_prefill.argtypes, L.moe_gemm_gguf_prefill.restype = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp], None
    return L


MOE_CODE = {"q8_0": 0, "q4_k": 1, "q2_k": 2, "q3_k": 3, "q5_k": 4, "q6_k": 5}       # candle-kernels/src/moe/moe_gguf.cu:162


def _moe_case(oracle, tname, tokens, e, topk, n, k, seed):
    rng = np.random.default_rng(seed)
    wf = (rng.standard_normal((e, n, k)) * 0.02).astype(np.float32)
    wq = np.stack([oracle.quantize(TYPES[tname], wf[i]) for i in range(e)])
    ids = np.stack([rng.choice(e, size=topk, replace=False) for _ in range(tokens)]).astype(np.int32)
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable").astype(np.int32)         # pair indices sorted by expert
    return wq, order, flat[order].astype(np.int32), rng


@pytest.mark.parametrize("tname", list(MOE_CODE))
@pytest.mark.parametrize("tokens,e,topk,n,k", [(1, 16, 4, 96, 512), (5, 32, 8, 768, 2048), (7, 8, 2, 130, 1024)])
def test_moe_gemv_against_the_reference_kernel(lib, ref_moe, oracle, cuda_dev, tname, tokens, e, topk, n, k):
    """`moe_gemm_gguf`, the expert-indexed GEMV over sorted (token, expert) pairs - the entry point no reference test
    covers - against the reference kernel itself: the gate / up form (input row = pair / topk, no routing weight) and the
    down form (one input row per pair, scaled by the routing weight, a pair with expert id -1 left untouched)."""
    wq, order, expert_of, rng = _moe_case(oracle, tname, tokens, e, topk, n, k, seed=tokens + e + k)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_dev)
    w_dev, sp, st = dev(wq.reshape(-1)), dev(order), torch.cuda.current_stream().cuda_stream
    pairs = tokens * topk
    x = dev(rng.standard_normal((tokens, k)).astype(np.float32))
    ex = dev(expert_of)
    outs = []
    for L in (ref_moe, lib):
        out = torch.full((pairs, n), 7.0, device=cuda_dev)
        L.moe_gemm_gguf(x.data_ptr(), w_dev.data_ptr(), sp.data_ptr(), ex.data_ptr(), None, out.data_ptr(), e, topk, pairs, n, k,
                        MOE_CODE[tname], st)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy())
    capi.check("moe gate")
    assert rel_err(outs[1], outs[0]) <= 1e-5
    x2 = dev(rng.standard_normal((pairs, k)).astype(np.float32))
    tw = dev(rng.random((pairs,), dtype=np.float32))
    skip = expert_of.copy()
    skip[0] = -1
    ex2 = dev(skip)
    outs = []
    for L in (ref_moe, lib):
        out = torch.full((pairs, n), 7.0, device=cuda_dev)
        L.moe_gemm_gguf(x2.data_ptr(), w_dev.data_ptr(), sp.data_ptr(), ex2.data_ptr(), tw.data_ptr(), out.data_ptr(), e, topk, pairs, n, k,
                        MOE_CODE[tname], st)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy())
    capi.check("moe down")
    assert np.all(outs[0][order[0]] == 7.0) and np.all(outs[1][order[0]] == 7.0)
    assert rel_err(outs[1], outs[0]) <= 1e-5


@pytest.mark.parametrize("tname", ["q4_k", "q6_k", "q8_0"])
def test_moe_prompt_gemm_against_the_reference_kernel(lib, ref_moe, oracle, cuda_dev, tname):
    """`moe_gemm_gguf_prefill`: the reference de-quantizes to f16 and multiplies with wmma, this library keeps integer
    arithmetic - the values agree to f16 accuracy, the row / expert / routing-weight mapping exactly."""
    tokens, e, topk, n, k = 40, 8, 2, 192, 1024
    wq, order, expert_of, rng = _moe_case(oracle, tname, tokens, e, topk, n, k, seed=11)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_dev)
    w_dev, sp, ex, st = dev(wq.reshape(-1)), dev(order), dev(expert_of), torch.cuda.current_stream().cuda_stream
    pairs = tokens * topk
    x = dev(rng.standard_normal((tokens, k)).astype(np.float32)).to(torch.float16)
    x2 = dev(rng.standard_normal((pairs, k)).astype(np.float32)).to(torch.float16)
    tw = dev(rng.random((pairs,), dtype=np.float32))
    for inp, weights in ((x, None), (x2, tw)):
        outs = []
        for L in (ref_moe, lib):
            out = torch.zeros((pairs, n), device=cuda_dev)
            L.moe_gemm_gguf_prefill(inp.data_ptr(), w_dev.data_ptr(), sp.data_ptr(), ex.data_ptr(), None if weights is None else weights.data_ptr(),
                                    out.data_ptr(), e, topk, pairs, n, k, 0, MOE_CODE[tname], st)
            torch.cuda.synchronize()
            outs.append(out.cpu().numpy())
        capi.check("moe prefill")
        assert rel_err(outs[1], outs[0]) <= 2e-2
