"""GPU parity of the decode path (activation quantize + GEMV), called through the C ABI.

Bars (from the task's parity contract):
  * activation blocks: bit-exact against the oracle's restatement of the reference quantizers;
  * per-block integer dot products: bit-exact;
  * final f32 outputs: max |a - ref| / max |ref| <= 1e-3 (only f32 summation order may differ).
"""
import os

import numpy as np
import pytest
import torch

from candle_b200 import capi
from candle_b200.quantized import GgmlDType, QMatMul, QTensor, set_activation_mode
from helpers import TYPES, make_case, pad, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gemv_cases.npz")
TORCH_ELEM = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def ref_call_sequence(lib, tname, elem, w_dev, x_dev, k, n):
    """The two launches candle's host makes for up to 8 rows (candle-core/src/quantized/fast_mmvq.rs:198-247):
    quantize into a scratch of b * k_padded/32 * 36 bytes, then the `_plain` GEMV into an uninitialised output."""
    b = x_dev.shape[0]
    k_padded = pad(k, 512)
    scratch = torch.full((b * (k_padded // 32) * 36 + 64,), 0xCD, dtype=torch.uint8, device=x_dev.device)
    out = torch.full((b * n + 16,), float("nan"), dtype=x_dev.dtype, device=x_dev.device)   # canary tail
    getattr(lib, f"launch_mmvq_gguf_quantize_q8_1_{elem}")(x_dev.data_ptr(), scratch.data_ptr(), k, k_padded, b, _stream())
    getattr(lib, f"launch_mmvq_gguf_{tname}_{elem}_plain")(
        w_dev.data_ptr(), scratch.data_ptr(), out.data_ptr(), k, n, k_padded // 32, n, b, _stream())
    capi.check("reference call sequence")
    torch.cuda.synchronize()
    assert bool((scratch[b * (k_padded // 32) * 36:] == 0xCD).all()), "scratch written past its end"
    assert bool(torch.isnan(out[b * n:].float()).all()), "output written past its end"
    assert not bool(torch.isnan(out[:b * n].float()).any()), "an output element was left unwritten"
    return scratch[:b * (k_padded // 32) * 36].view(b, -1), out[:b * n].view(b, n)


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("k,n,b", [(256, 1, 1), (256, 3, 2), (512, 130, 3), (4096, 257, 1), (2048, 96, 4),
                                   (768, 40, 5), (14336, 48, 8), (4096, 64, 7), (1024, 33, 6)])
def test_gemv_matches_cuda_semantics(lib, oracle, cuda_dev, tname, k, n, b):
    wt = TYPES[tname]
    _, x, wq = make_case(oracle, wt, k, n, b, seed=k + n + b)
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    x_dev = torch.from_numpy(x).to(cuda_dev)
    q8, out = ref_call_sequence(lib, tname, "f32", w_dev, x_dev, k, n)
    q8_ref = oracle.cuda_quantize_q8_1(x, pad(k, 512))
    assert np.array_equal(q8.cpu().numpy(), q8_ref), "Q8_1 blocks differ from the reference quantizer"
    ref = oracle.cuda_mmvq(wt, wq, q8_ref, k, n)
    assert rel_err(out.cpu().numpy(), ref) <= TOL
    # expected to be far inside the bar: only the order of f32 additions differs
    assert rel_err(out.cpu().numpy(), ref) <= 1e-5


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("k,n", [(512, 37), (4096, 130)])
def test_block_integer_dots_exact(lib, oracle, cuda_dev, tname, k, n):
    wt = TYPES[tname]
    _, x, wq = make_case(oracle, wt, k, n, 1, seed=7)
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    x_dev = torch.from_numpy(x).to(cuda_dev)
    nblk = k // capi.BLOCK_ELEMS[wt]
    for act, oracle_dots, act_blocks in (
        (capi.ACT_Q8_1, oracle.cuda_block_dots, None),
        (capi.ACT_Q8_K if nblk * 256 == k and wt in (10, 11, 12, 13, 14) else capi.ACT_Q8_0, oracle.cpu_block_dots, "cpu"),
    ):
        y = torch.zeros((pad(k, 512) // 32 * 36,), dtype=torch.uint8, device=cuda_dev)
        lib.cq_quantize_act(x_dev.data_ptr(), capi.F32, y.data_ptr(), k, pad(k, 512), 1, act, _stream())
        dots = torch.zeros((n, nblk), dtype=torch.int32, device=cuda_dev)
        dmin = torch.zeros_like(dots)
        lib.cq_block_dots(wt, act, w_dev.data_ptr(), y.data_ptr(), dots.data_ptr(), dmin.data_ptr(), k, n, _stream())
        capi.check("block dots")
        if act_blocks is None:
            rd, rm = oracle_dots(wt, wq, oracle.cuda_quantize_q8_1(x, pad(k, 512))[0], k, n)
        else:
            rd, rm = oracle_dots(wt, wq, oracle.quantize(oracle.vec_dot_type(wt), x), k, n)
        assert np.array_equal(dots.cpu().numpy(), rd)
        if wt in (10, 12, 13):
            assert np.array_equal(dmin.cpu().numpy(), rm)


def _unpack_cpu_exact(containers, wt, k):
    """Repack the library's 36-byte containers into the reference's CPU block layout for a byte compare."""
    c = containers.reshape(-1, 36)
    if wt in (3, 7):        # BlockQ8_1 of the CPU path: f16 d, f16 s, 32 int8 -- the container itself
        return c.reshape(-1)
    if wt in (2, 6, 8):     # BlockQ8_0: f16 d + 32 int8 (34 bytes)
        return np.concatenate([c[:, 0:2], c[:, 4:36]], axis=1).reshape(-1)
    nsb = k // 256          # BlockQ8K: f32 d + 256 int8 + 16 int16 bsums (292 bytes)
    c = c[:nsb * 8].reshape(nsb, 8, 36)
    d = c[:, 0, 0:4]
    qs = c[:, :, 4:].reshape(nsb, 256)
    bsums = qs.view(np.int8).astype(np.int32).reshape(nsb, 16, 16).sum(-1).astype(np.int16)
    return np.concatenate([d, qs, bsums.view(np.uint8).reshape(nsb, 32)], axis=1).reshape(-1)


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("k,n,b", [(512, 24, 3), (4096, 96, 1), (14336, 40, 8), (768, 64, 2)])
def test_cpu_exact_mode_matches_cpu_vec_dot(lib, oracle, cuda_dev, tname, k, n, b):
    """With CPU-exact activations the outputs meet the 1e-3 bar against the reference's CPU vec_dot."""
    wt = TYPES[tname]
    if k % capi.BLOCK_ELEMS[wt]:
        pytest.skip("K not a multiple of the block size")
    _, x, wq = make_case(oracle, wt, k, n, b, seed=3 * k + n)
    act = capi.ACT_Q8_K if wt in (10, 11, 12, 13, 14) else capi.ACT_Q8_0
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    x_dev = torch.from_numpy(x).to(cuda_dev)
    kp = pad(k, 512)
    y = torch.zeros((b, kp // 32 * 36), dtype=torch.uint8, device=cuda_dev)
    lib.cq_quantize_act(x_dev.data_ptr(), capi.F32, y.data_ptr(), k, kp, b, act, _stream())
    out = torch.full((b, n), float("nan"), device=cuda_dev)
    lib.cq_mmvq(wt, act, capi.F32, w_dev.data_ptr(), y.data_ptr(), out.data_ptr(), k, n, kp // 32, n, b, _stream())
    capi.check("cpu-exact gemv")
    act_ref = oracle.quantize(oracle.vec_dot_type(wt), x)
    got = np.stack([_unpack_cpu_exact(y[j].cpu().numpy(), wt, k) for j in range(b)])
    assert np.array_equal(got[:, :act_ref.shape[1]], act_ref), "activation blocks differ from the CPU quantizer"
    for mode in (oracle.SCALAR, oracle.SIMD_ORDER):
        ref = oracle.matmul(wt, x, wq, n, mode=mode)
        assert rel_err(out.cpu().numpy(), ref) <= TOL
    assert rel_err(out.cpu().numpy(), oracle.matmul(wt, x, wq, n)) <= 1e-5


@pytest.mark.parametrize("elem", ["f16", "bf16"])
@pytest.mark.parametrize("tname", ["q4_k", "q6_k", "q8_0", "q4_0"])
def test_half_inputs_and_outputs(lib, oracle, cuda_dev, tname, elem):
    """The f16 / bf16 launchers: same blocks as quantizing the up-cast values; output rounded once to the type."""
    wt = TYPES[tname]
    k, n, b = 2048, 70, 3
    _, x, wq = make_case(oracle, wt, k, n, b, seed=11)
    xt = torch.from_numpy(x).to(cuda_dev).to(TORCH_ELEM[elem])
    x_up = xt.float().cpu().numpy()
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    q8, out = ref_call_sequence(lib, tname, elem, w_dev, xt, k, n)
    q8_ref = oracle.cuda_quantize_q8_1(x_up, pad(k, 512))
    assert np.array_equal(q8.cpu().numpy(), q8_ref)
    ref = torch.from_numpy(oracle.cuda_mmvq(wt, wq, q8_ref, k, n)).to(TORCH_ELEM[elem]).float().numpy()
    # one rounding to a 8- or 11-bit mantissa on top of the f32 result
    assert rel_err(out.float().cpu().numpy(), ref) <= (2 ** -8 if elem == "bf16" else 2 ** -11) * 1.01


def test_unaligned_and_ragged_quantize(lib, oracle, cuda_dev):
    """K not a multiple of the vector width or of 32, pointer off 16-byte alignment, zero rows, padding zeroed."""
    for k, rows, off in ((100, 3, 0), (33, 2, 1), (4096, 1, 3), (256, 5, 0)):
        rng = np.random.default_rng(k)
        x = rng.standard_normal((rows, k)).astype(np.float32)
        if rows > 1:
            x[1] = 0.0          # amax == 0 -> q = 0, d = 0
        buf = torch.zeros(rows * k + 8, device=cuda_dev)
        xd = buf[off:off + rows * k].view(rows, k)
        xd.copy_(torch.from_numpy(x))
        kp = pad(k, 512)
        y = torch.full((rows, kp // 32 * 36), 0xEE, dtype=torch.uint8, device=cuda_dev)
        lib.launch_mmvq_gguf_quantize_q8_1_f32(xd.data_ptr(), y.data_ptr(), k, kp, rows, _stream())
        capi.check("quantize")
        assert np.array_equal(y.cpu().numpy(), oracle.cuda_quantize_q8_1(x, kp))


def test_batch_invariance_and_sharding_invariance(lib, oracle, cuda_dev):
    """qmm_batch (candle-core/tests/quantized_tests.rs:224-259): a row must give the same bits inside any batch;
    and, for tensor parallelism, a weight row must give the same bits whether the matrix is whole or cut by rows."""
    for tname in ("q4_k", "q6_k", "q8_0"):
        wt = TYPES[tname]
        k, n = 4096, 512
        _, x, wq = make_case(oracle, wt, k, n, 2, seed=99)
        w_dev = torch.from_numpy(wq).to(cuda_dev)
        base = ref_call_sequence(lib, tname, "f32", w_dev, torch.from_numpy(x).to(cuda_dev), k, n)[1].clone()
        for reps in (2, 3, 4):
            xs = torch.from_numpy(np.concatenate([x] * reps)).to(cuda_dev)
            out = ref_call_sequence(lib, tname, "f32", w_dev, xs, k, n)[1]
            for r in range(reps):
                assert torch.equal(out[2 * r:2 * r + 2], base)
        for shards in (2, 4, 8):
            rows = n // shards
            parts = [ref_call_sequence(lib, tname, "f32", w_dev[s * rows:(s + 1) * rows].contiguous(),
                                       torch.from_numpy(x).to(cuda_dev), k, rows)[1] for s in range(shards)]
            assert torch.equal(torch.cat(parts, dim=1), base)


@pytest.mark.parametrize("tname", ["q4_k", "q6_k", "q8_0"])
@pytest.mark.parametrize("k,n", [(256, 5), (768, 33), (1024, 16), (2048, 100), (4096, 257), (14336, 48), (3072, 40)])
def test_tensor_core_gemv_gives_the_bits_of_the_dp4a_gemv(lib, oracle, cuda_dev, tname, k, n):
    """The mma.sync kernel (2..8 rows) against the dp4a kernel, forced in turn for every batch size: equal bits, with
    partial groups (K below or not a multiple of 2048 / 1024), ragged last tiles and every column count."""
    wt = TYPES[tname]
    _, x, wq = make_case(oracle, wt, k, n, 8, seed=k + n)
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    try:
        for b in range(1, 9):
            xb = torch.from_numpy(x[:b]).to(cuda_dev)
            lib.cq_set_mma_min_batch(9)
            ref = ref_call_sequence(lib, tname, "f32", w_dev, xb, k, n)[1].clone()
            lib.cq_set_mma_min_batch(1)
            lib.cq_set_mma_kernel(1)        # the CTA-shared tensor-core kernel
            got = ref_call_sequence(lib, tname, "f32", w_dev, xb, k, n)[1]
            assert torch.equal(got, ref), f"batch {b}"
            lib.cq_set_mma_kernel(0)
    finally:
        lib.cq_set_mma_min_batch(0)
        lib.cq_set_mma_kernel(0)
    assert lib.cq_device_timeout_flag() == 0


@pytest.mark.parametrize("tname", ["q4_k", "q6_k", "q8_0"])
@pytest.mark.parametrize("k,n", [(2048, 5), (2048, 16), (4096, 257), (14336, 48), (6144, 1000), (4096, 4800), (1024, 40), (4096, 40000),
                                 (14336, 4096), (8192, 700)])
@pytest.mark.parametrize("cluster", [0, 2])
def test_warp_tile_tensor_core_gemv_gives_the_bits_of_the_dp4a_gemv(lib, oracle, cuda_dev, tname, k, n, cluster):
    """The warp-private tensor-core kernel, forced for every batch size 1..8, against the dp4a kernel: equal bits and the
    oracle's bar; single and ragged last tiles, more tiles than warps of one CTA (4800 rows: 300 tiles over many CTAs),
    one to seven groups of 32 chunks; both forms of the kernel - a warp owning whole tiles (40000 rows) and the groups of a
    tile spread over the warps of a CTA with the ordered sum through shared memory (all others with two or more groups) or,
    with `cluster` = 2, over the CTAs of a thread-block cluster with the sums sent through distributed shared memory (plan
    kind 4; clusters of 2 to 7 CTAs, one and several rounds of tiles, ragged last round).  Shapes whose K is not a whole
    number of groups fall back (plan query says so)."""
    import ctypes
    wt = TYPES[tname]
    whole_groups = k % (1024 if tname == "q8_0" else 2048) == 0
    _, x, wq = make_case(oracle, wt, k, n, 8, seed=k + n)
    w_dev = torch.from_numpy(wq).to(cuda_dev)
    groups = k // (1024 if tname == "q8_0" else 2048)
    kinds = set()
    try:
        lib.cq_set_cluster_split(cluster)
        for b in range(1, 9):
            xb = torch.from_numpy(x[:b]).to(cuda_dev)
            lib.cq_set_mma_min_batch(9)
            ref = ref_call_sequence(lib, tname, "f32", w_dev, xb, k, n)[1].clone()
            lib.cq_set_mma_min_batch(1)
            lib.cq_set_mma_kernel(2)
            plan = (ctypes.c_int * 4)()
            assert lib.cq_mmvq_plan(wt, capi.ACT_Q8_1, k, n, b, plan) == 0
            assert (plan[0] in (2, 3, 4)) == whole_groups
            kinds.add(plan[0])
            got = ref_call_sequence(lib, tname, "f32", w_dev, xb, k, n)[1]
            assert torch.equal(got, ref), f"batch {b}"
            lib.cq_set_mma_kernel(0)
            if b in (1, 8):
                want = oracle.cuda_mmvq(wt, wq, oracle.cuda_quantize_q8_1(x[:b], pad(k, 512)), k, n)
                assert rel_err(got.cpu().numpy(), want) <= 1e-5
    finally:
        lib.cq_set_mma_min_batch(0)
        lib.cq_set_mma_kernel(0)
        lib.cq_set_cluster_split(1)
    if whole_groups and groups >= 2 and n < 16 * 148 * 16:
        assert kinds == ({4} if cluster == 2 else {3})
    assert lib.cq_device_timeout_flag() == 0


@pytest.mark.parametrize("k,na,nb", [(256, 3, 2), (4096, 5120, 1024), (1024, 70, 33), (14336, 40, 24)])
def test_paired_launch_gives_the_bits_of_two_launches(oracle, cuda_dev, k, na, nb):
    """QMatMul.forward_q8_1_pair: a Q4_K and a Q6_K matrix over the same Q8_1 row in one launch, and the fall-back to two
    launches for more rows."""
    _, x, wa = make_case(oracle, TYPES["q4_k"], k, na, 3, seed=k)
    _, _, wb = make_case(oracle, TYPES["q6_k"], k, nb, 3, seed=k + 1)
    ma = QMatMul.from_qtensor(QTensor.from_data(wa.reshape(-1), GgmlDType.Q4K, (na, k), cuda_dev))
    mb = QMatMul.from_qtensor(QTensor.from_data(wb.reshape(-1), GgmlDType.Q6K, (nb, k), cuda_dev))
    for rows in (1, 3):
        q8 = torch.from_numpy(oracle.cuda_quantize_q8_1(x[:rows], pad(k, 512))).to(cuda_dev)
        ya, yb = ma.forward_q8_1_pair(mb, q8)
        assert torch.equal(ya, ma.forward_q8_1(q8)) and torch.equal(yb, mb.forward_q8_1(q8))
        assert torch.equal(ya, ma.forward(torch.from_numpy(x[:rows]).to(cuda_dev)))


def test_golden_fixtures(lib, cuda_dev):
    """Committed oracle outputs (tests/golden/make_fixtures.py)."""
    g = np.load(GOLD)
    for name in sorted({key.split(".")[0] for key in g.files}):
        wt, k, n, b = [int(v) for v in g[f"{name}.meta"]]
        tname = {v: key for key, v in TYPES.items()}[wt]
        w_dev = torch.from_numpy(g[f"{name}.w"]).to(cuda_dev)
        x_dev = torch.from_numpy(g[f"{name}.x"]).to(cuda_dev)
        q8, out = ref_call_sequence(lib, tname, "f32", w_dev, x_dev, k, n)
        assert np.array_equal(q8.cpu().numpy(), g[f"{name}.q8_1"])
        assert rel_err(out.cpu().numpy(), g[f"{name}.y_cuda"]) <= TOL
        set_activation_mode(True)
        try:
            qt = QTensor.from_data(g[f"{name}.w"], GgmlDType(wt), (n, k), cuda_dev)
            y = QMatMul.from_qtensor(qt).forward(x_dev)
        finally:
            set_activation_mode(False)
        assert rel_err(y.cpu().numpy(), g[f"{name}.y_cpu"]) <= TOL


def test_qmatmul_forward_api(oracle, cuda_dev):
    """The host objects: upload with tail padding, data() round trip, rank-3 input, error behaviour."""
    wt, k, n = 12, 1024, 48
    _, x, wq = make_case(oracle, wt, k, n, 6, seed=21)
    qt = QTensor.from_data(wq, GgmlDType.Q4K, (n, k), cuda_dev)
    assert qt.data() == wq.tobytes() and qt.shape == (n, k) and qt.storage_size_in_bytes() == wq.size
    mm = QMatMul.from_qtensor(qt)
    x3 = torch.from_numpy(x).to(cuda_dev).view(2, 3, k)
    y = mm.forward(x3)
    assert y.shape == (2, 3, n) and y.dtype == torch.float32
    ref = oracle.cuda_mmvq(wt, wq, oracle.cuda_quantize_q8_1(x, pad(k, 512)), k, n)
    assert rel_err(y.view(6, n).cpu().numpy(), ref) <= TOL
    with pytest.raises(capi.CandleQError, match="mismatch on matmul dim"):
        mm.forward(torch.zeros(2, k + 256, device=cuda_dev))
    with pytest.raises(capi.CandleQError, match="not contiguous"):
        mm.forward(torch.zeros(k, 2, device=cuda_dev).t())
    with pytest.raises(capi.CandleQError, match="byte size does not match"):
        QTensor.from_data(wq, GgmlDType.Q4K, (n + 1, k), cuda_dev)
    # 9..16 rows walk the decode kernel in slices and must agree with it row by row
    xb = torch.from_numpy(np.concatenate([x, x])).to(cuda_dev)
    yb = mm.forward(xb)
    assert rel_err(yb[:6].cpu().numpy(), ref) <= TOL and rel_err(yb[6:].cpu().numpy(), ref) <= TOL
    # more rows go to the tensor-core prefill kernel, whose arithmetic is the CPU path's (Q8_K activations)
    xc = np.concatenate([x] * 5)
    yc = mm.forward(torch.from_numpy(xc).to(cuda_dev))
    assert rel_err(yc.cpu().numpy(), oracle.matmul(wt, xc, wq, n)) <= TOL


def test_forward_over_host_buffers_matches_device_forward(oracle, cuda_dev):
    """QMatMul.forward_host: upload, multiply and copy back inside the library, the copy-back on its own stream.  Ten calls in
    a row (the staging ring has four slots, so slots are reused while earlier copy-backs may still run), different row
    counts, element types and two matrices; after host_flush + synchronize every output has the bits of the device forward."""
    k = 2048
    mats = []
    for tname, n in (("q4_k", 300), ("q8_0", 130)):
        _, _, wq = make_case(oracle, TYPES[tname], k, n, 1, seed=n)
        mats.append(QMatMul.from_qtensor(QTensor.from_data(wq, GgmlDType(TYPES[tname]), (n, k), cuda_dev)))
    rng = np.random.default_rng(3)
    calls = []
    for i in range(10):
        mm = mats[i % 2]
        rows = (1, 8, 3, 40, 2)[i % 5]
        dt = (torch.float32, torch.bfloat16, torch.float16)[i % 3]
        x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).to(dt).pin_memory()
        y = torch.full((rows, mm.qtensor.shape[0]), float("nan"), dtype=dt).pin_memory()
        calls.append((mm, x, y))
    for mm, x, y in calls:
        mm.forward_host(x, y)
    mats[0].host_flush()
    torch.cuda.synchronize()
    for mm, x, y in calls:
        want = mm.forward(x.to(cuda_dev)).cpu()
        assert torch.equal(y, want)
    with pytest.raises(capi.CandleQError, match="output shape"):
        mats[0].forward_host(calls[0][1], torch.empty((2, 2)).pin_memory())
