"""GPU parity of the expert-indexed paths.  The reference has no test for them ("parity unpinned"): the oracle is
the per-expert composition of the pinned pieces (Q8_1 quantize + the reference's MMVQ arithmetic per pair)."""
import numpy as np
import pytest
import torch

from candle_b200 import capi
from candle_b200.moe import moe_gemm_gguf
from candle_b200.quantized import GgmlDType, QTensor, set_activation_mode
from helpers import pad, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3
TYPES = {"q2_k": 10, "q3_k": 11, "q4_k": 12, "q5_k": 13, "q6_k": 14, "q8_0": 8}


def _experts(oracle, wt, e, n, k, seed):
    rng = np.random.default_rng(seed)
    wf = (rng.standard_normal((e, n, k)) * 0.02).astype(np.float32)
    return np.stack([oracle.quantize(wt, wf[i]) for i in range(e)])     # [e, n, row_bytes]


def _route(tokens, e, topk, seed):
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.choice(e, size=topk, replace=False) for _ in range(tokens)]).astype(np.int32)   # [tokens, topk]
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable").astype(np.int32)     # sorted_token_ids: pair indices by expert
    return ids, order, flat[order].astype(np.int32)


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("tokens,e,topk,n,k", [(1, 16, 4, 96, 512), (5, 32, 8, 768, 2048), (3, 8, 2, 2048, 768)])
def test_moe_gemm_gguf_sorted(oracle, cuda_dev, tname, tokens, e, topk, n, k):
    wt = TYPES[tname]
    if k % capi.BLOCK_ELEMS[wt]:
        pytest.skip("K not a multiple of the block size")
    wq = _experts(oracle, wt, e, n, k, seed=tokens + e)
    ids, sorted_pairs, expert_of = _route(tokens, e, topk, seed=3)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((tokens, k)).astype(np.float32)
    tw = rng.random((tokens * topk,), dtype=np.float32)
    qt = QTensor.from_data(wq.reshape(-1), GgmlDType(wt), (e, n, k), cuda_dev)
    dev = lambda a: torch.from_numpy(a).to(cuda_dev)
    # gate/up style: input row = pair / topk, no routing weight
    out = moe_gemm_gguf(dev(x), qt, None, dev(sorted_pairs), dev(expert_of), topk).cpu().numpy()
    q8 = oracle.cuda_quantize_q8_1(x, pad(k, 512))
    ref = np.zeros((tokens * topk, n), dtype=np.float32)
    for pair in range(tokens * topk):
        ex = ids.reshape(-1)[pair]
        ref[pair] = oracle.cuda_mmvq(wt, wq[ex], q8[pair // topk:pair // topk + 1], k, n)[0]
    assert rel_err(out, ref) <= TOL
    # down style: one input row per pair, scaled by the routing weight; expert id -1 skips the pair
    x2 = rng.standard_normal((tokens * topk, k)).astype(np.float32)
    expert_skip = expert_of.copy()
    expert_skip[0] = -1
    out2 = torch.full((tokens * topk, n), 7.0, device=cuda_dev)
    L = capi.lib()
    x2d, sp, es, twd = dev(x2), dev(sorted_pairs), dev(expert_skip), dev(tw)
    L.moe_gemm_gguf(x2d.data_ptr(), qt.device_ptr(), sp.data_ptr(), es.data_ptr(), twd.data_ptr(), out2.data_ptr(), e, topk,
                    tokens * topk, n, k, {10: 2, 11: 3, 12: 1, 13: 4, 14: 5, 8: 0}[wt], torch.cuda.current_stream().cuda_stream)
    capi.check("moe down")
    out2 = out2.cpu().numpy()
    q8b = oracle.cuda_quantize_q8_1(x2, pad(k, 512))
    for j, pair in enumerate(sorted_pairs):
        if j == 0:
            assert np.all(out2[pair] == 7.0)        # skipped pair: untouched
            continue
        ex = expert_of[j]
        r = oracle.cuda_mmvq(wt, wq[ex], q8b[pair:pair + 1], k, n)[0] * tw[pair]
        assert rel_err(out2[pair], r) <= TOL
    assert L.cq_moe_timeout_flag() == 0


@pytest.mark.parametrize("tname", list(TYPES))
@pytest.mark.parametrize("x_dim1_is_one", [True, False])
def test_indexed_moe_forward(oracle, cuda_dev, tname, x_dim1_is_one):
    wt = TYPES[tname]
    e, n, k, batch, topk = 12, 130, 1024, 4, 3
    wq = _experts(oracle, wt, e, n, k, seed=1)
    ids, _, _ = _route(batch, e, topk, seed=5)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((batch, 1 if x_dim1_is_one else topk, k)).astype(np.float32)
    qt = QTensor.from_data(wq.reshape(-1), GgmlDType(wt), (e, n, k), cuda_dev)
    out = qt.indexed_moe_forward(torch.from_numpy(x).to(cuda_dev), torch.from_numpy(ids).to(cuda_dev)).cpu().numpy()
    assert out.shape == (batch, topk, n)
    for b in range(batch):
        for s in range(topk):
            xin = x[b, 0 if x_dim1_is_one else s][None]
            r = oracle.cuda_mmvq(wt, wq[ids[b, s]], oracle.cuda_quantize_q8_1(xin, pad(k, 512)), k, n)[0]
            assert rel_err(out[b, s], r) <= TOL
    # from Q8_1 containers made beforehand (what a fused producer hands over): the same bits, no quantize launch
    xd = torch.from_numpy(x).to(cuda_dev)
    rows_in = xd.shape[0] * xd.shape[1]
    q8 = torch.zeros((rows_in, pad(k, 512) // 32 * 36), dtype=torch.uint8, device=cuda_dev)
    capi.lib().launch_mmvq_gguf_quantize_q8_1_f32(xd.data_ptr(), q8.data_ptr(), k, pad(k, 512), rows_in,
                                                  torch.cuda.current_stream().cuda_stream)
    out_q = qt.indexed_moe_forward_q8_1(q8, xd.shape[1], torch.from_numpy(ids).to(cuda_dev))
    assert np.array_equal(out_q.cpu().numpy(), out)
    # CPU-exact activations: matches the CPU vec_dot per expert
    set_activation_mode(True)
    try:
        out2 = qt.indexed_moe_forward(torch.from_numpy(x).to(cuda_dev), torch.from_numpy(ids).to(cuda_dev)).cpu().numpy()
    finally:
        set_activation_mode(False)
    for b in range(batch):
        for s in range(topk):
            xin = x[b, 0 if x_dim1_is_one else s][None]
            assert rel_err(out2[b, s], oracle.matmul(wt, xin, wq[ids[b, s]], n)[0]) <= TOL


def test_q8_0_experts_use_the_true_expert_stride(oracle, cuda_dev):
    """A stated deviation from the reference.  Its indexed kernel computes the byte distance between experts as
    n * k / 256 * sizeof(block) for every format (candle-kernels/src/quantized.cu:4703), which for Q8_0 - 34-byte blocks
    of 32 values - is an eighth of the true distance, so every expert but the first reads the wrong rows.  This library
    strides by n * row_bytes: expert e's output is the product with expert e's own weights, and it is NOT what the
    reference's address arithmetic would have produced."""
    wt = TYPES["q8_0"]
    e, n, k, batch, topk = 6, 64, 512, 2, 2
    wq = _experts(oracle, wt, e, n, k, seed=9)                                      # [e, n, row_bytes]
    ids = np.array([[1, 4], [5, 2]], dtype=np.int32)
    x = np.random.default_rng(4).standard_normal((batch, 1, k)).astype(np.float32)
    qt = QTensor.from_data(wq.reshape(-1), GgmlDType(wt), (e, n, k), cuda_dev)
    out = qt.indexed_moe_forward(torch.from_numpy(x).to(cuda_dev), torch.from_numpy(ids).to(cuda_dev)).cpu().numpy()
    flat = wq.reshape(-1)
    row_bytes = k // 32 * 34
    for b in range(batch):
        for s_ in range(topk):
            ex = int(ids[b, s_])
            q8 = oracle.cuda_quantize_q8_1(x[b], pad(k, 512))
            right = oracle.cuda_mmvq(wt, wq[ex], q8, k, n)[0]
            assert rel_err(out[b, s_], right) <= TOL
            wrong_start = ex * (n * k // 256 * 34)                                  # the reference's stride
            wrong_w = flat[wrong_start:wrong_start + n * row_bytes].reshape(n, row_bytes)
            wrong = oracle.cuda_mmvq(wt, wrong_w, q8, k, n)[0]
            assert rel_err(out[b, s_], wrong) > 0.1


def test_moe_prefill_entry_point_small_and_large(oracle, cuda_dev):
    """moe_gemm_gguf_prefill: under 64 pairs it is the decode entry point on the up-cast values (same bits); from 64 pairs on
    the grouped tensor-core kernel, whose arithmetic is the CPU path's (Q8_K activations)."""
    wt, e, n, k, topk = 12, 16, 256, 1024, 4
    wq = _experts(oracle, wt, e, n, k, seed=4)
    qt = QTensor.from_data(wq.reshape(-1), GgmlDType(wt), (e, n, k), cuda_dev)
    for tokens in (10, 40):
        ids, sorted_pairs, expert_of = _route(tokens, e, topk, seed=6)
        x = torch.randn((tokens, k), device=cuda_dev).to(torch.float16)
        sp, eo = torch.from_numpy(sorted_pairs).to(cuda_dev), torch.from_numpy(expert_of).to(cuda_dev)
        a = moe_gemm_gguf(x, qt, None, sp, eo, topk, is_prefill=True)
        if tokens * topk < 64:          # (and at least four pairs per expert: 160 >= 4 * 16 in the larger case)
            assert torch.equal(a, moe_gemm_gguf(x.float(), qt, None, sp, eo, topk, is_prefill=False))
        else:
            xf = x.float().cpu().numpy()
            ref = np.stack([oracle.matmul(wt, xf[p // topk][None, :], wq[ids.reshape(-1)[p]], n)[0] for p in range(tokens * topk)])
            assert rel_err(a.cpu().numpy(), ref) <= 1e-5


@pytest.mark.parametrize("is_prefill", [False, True])
def test_fused_moe_block_matches_per_expert_matmuls(oracle, cuda_dev, is_prefill):
    """FusedMoeGGUF::forward (candle-transformers/src/fused_moe.rs:222-301) against the same block written with one
    dense QMatMul per (token, expert): routing, SwiGLU, routing weights, sum over the token's experts.  Then the
    experts are split over two emulated ranks: pair outputs add up to the same bits."""
    from candle_b200.fused_moe import FusedMoeGGUF, route
    from candle_b200.quantized import QMatMul
    e, topk, hidden, inter, tokens = 8, 2, 512, 256, 6
    wt = 12
    g_w = _experts(oracle, wt, e, inter, hidden, seed=1)
    u_w = _experts(oracle, wt, e, inter, hidden, seed=2)
    d_w = _experts(oracle, wt, e, hidden, inter, seed=3)
    mk = lambda w, n, k, lo=0, hi=e: QTensor.from_data(w[lo:hi].reshape(-1), GgmlDType(wt), (hi - lo, n, k), cuda_dev)
    torch.manual_seed(0)
    router = torch.randn(e, hidden, device=cuda_dev) * 0.1
    xs = torch.randn(2, tokens // 2, hidden, device=cuda_dev)
    moe = FusedMoeGGUF(router, mk(g_w, inter, hidden), mk(u_w, inter, hidden), mk(d_w, hidden, inter), topk, True)
    ys = moe.forward(xs, is_prefill)
    assert ys.shape == xs.shape and ys.dtype == xs.dtype
    # the same block, one dense matmul per pair
    x = xs.reshape(-1, hidden)
    tw, ids = route(torch.nn.functional.linear(x, router), topk, True)
    dense = lambda w, n, k, ex: QMatMul.from_qtensor(QTensor.from_data(w[ex].reshape(-1), GgmlDType(wt), (n, k), cuda_dev))
    cast = (lambda t: t.to(torch.bfloat16).to(torch.float32)) if is_prefill else (lambda t: t)
    ref = torch.zeros_like(x)
    for t in range(tokens):
        acc = []
        for s in range(topk):
            ex = int(ids[t, s])
            xin = cast(x[t:t + 1])
            h = dense(u_w, inter, hidden, ex).forward(xin) * torch.nn.functional.silu(dense(g_w, inter, hidden, ex).forward(xin))
            acc.append(dense(d_w, hidden, inter, ex).forward(cast(h)) * tw[t, s])
        ref[t] = torch.stack(acc).sum(dim=0)[0]
    assert rel_err(ys.reshape(-1, hidden).cpu().numpy(), ref.cpu().numpy()) <= 1e-5
    # two emulated expert-parallel ranks: each owns four experts, pair outputs are added
    parts = []
    for r in range(2):
        m = FusedMoeGGUF(router, mk(g_w, inter, hidden, 4 * r, 4 * r + 4), mk(u_w, inter, hidden, 4 * r, 4 * r + 4),
                         mk(d_w, hidden, inter, 4 * r, 4 * r + 4), topk, True, expert_offset=4 * r)
        m.world = 1                      # no process group here: collect the per-rank pair sums by hand
        parts.append(m)
    # run each rank's pairs with zero-initialised outputs and add them, as the all-reduce would
    from candle_b200.fused_moe import sort_pairs
    from candle_b200.moe import moe_gemm_gguf
    experts, pairs = sort_pairs(ids)
    total = None
    for r, m in enumerate(parts):
        loc = experts - 4 * r
        xin = x.to(torch.bfloat16) if is_prefill else x
        g = moe_gemm_gguf(xin, m.gate_experts, None, pairs, loc, topk, is_prefill, zero_init=True)
        u = moe_gemm_gguf(xin, m.up_experts, None, pairs, loc, topk, is_prefill, zero_init=True)
        h = u * torch.nn.functional.silu(g)
        h = h.to(torch.bfloat16) if is_prefill else h
        y = moe_gemm_gguf(h, m.down_experts, tw, pairs, loc, topk, is_prefill, zero_init=True)
        total = y if total is None else total + y
    ep = total.reshape(tokens, topk, hidden).sum(dim=1)
    assert torch.equal(ep, ys.reshape(-1, hidden))


def test_route_kernel_matches_the_tensor_formula(cuda_dev):
    """cq_moe_route_f32 against softmax -> top-k -> renormalise written with tensor ops (fused_moe.rs:233-247)."""
    from candle_b200.fused_moe import route
    L = capi.lib()
    torch.manual_seed(5)
    for tokens, experts, k, norm in ((1, 128, 8, True), (7, 16, 4, False), (33, 60, 6, True), (2, 1024, 32, True)):
        logits = torch.randn(tokens, experts, device=cuda_dev) * 2
        logits[0, 3] = logits[0, 1]                       # a tie: the lower index must come first
        ids = torch.empty((tokens, k), dtype=torch.int32, device=cuda_dev)
        w = torch.empty((tokens, k), dtype=torch.float32, device=cuda_dev)
        L.cq_moe_route_f32(logits.data_ptr(), ids.data_ptr(), w.data_ptr(), tokens, experts, k, 1 if norm else 0,
                           torch.cuda.current_stream().cuda_stream)
        capi.check("route")
        ref_w, ref_ids = route(logits, k, norm)
        assert torch.equal(ids.long(), ref_ids)
        assert torch.allclose(w, ref_w, rtol=1e-5, atol=1e-7)


def test_one_launch_router_and_slot_sum(cuda_dev):
    """cq_moe_router_f32: its logits against the f32 matrix product (summation order differs), its ids and weights bit for
    bit against cq_moe_route_f32 run on those logits, the arrival counters back at zero, twice in a row.
    cq_moe_weighted_sum_f32: the slot-order sum, bit for bit against the same operations written with tensor ops."""
    L = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(11)
    counters = torch.zeros(64, dtype=torch.int32, device=cuda_dev)
    for tokens, experts, d, k, norm in ((1, 128, 2048, 8, True), (8, 128, 2048, 8, True), (5, 60, 516, 6, False), (64, 16, 512, 4, True),
                                        (3, 1024, 64, 32, True)):
        h = torch.randn(tokens, d, device=cuda_dev)
        router = torch.randn(experts, d, device=cuda_dev) * 0.05
        for _ in range(2):
            logits = torch.full((tokens, experts), float("nan"), device=cuda_dev)
            ids = torch.full((tokens, k), -1, dtype=torch.int32, device=cuda_dev)
            w = torch.full((tokens, k), float("nan"), device=cuda_dev)
            L.cq_moe_router_f32(h.data_ptr(), router.data_ptr(), logits.data_ptr(), ids.data_ptr(), w.data_ptr(), counters.data_ptr(),
                                tokens, experts, d, k, 1 if norm else 0, st)
            capi.check("router")
            want = (h.double() @ router.double().t()).float()
            assert torch.allclose(logits, want, rtol=1e-4, atol=1e-5)
            ids2 = torch.empty_like(ids)
            w2 = torch.empty_like(w)
            L.cq_moe_route_f32(logits.data_ptr(), ids2.data_ptr(), w2.data_ptr(), tokens, experts, k, 1 if norm else 0, st)
            capi.check("route")
            assert torch.equal(ids, ids2) and torch.equal(w, w2)
            assert int(counters.abs().sum()) == 0
        y = torch.randn(tokens, k, d, device=cuda_dev)
        out = torch.empty(tokens, d, device=cuda_dev)
        L.cq_moe_weighted_sum_f32(y.data_ptr(), w.data_ptr(), out.data_ptr(), tokens, k, d, st)
        capi.check("weighted sum")
        acc = torch.zeros(tokens, d, device=cuda_dev)
        for s_ in range(k):
            acc = acc + y[:, s_] * w[:, s_:s_ + 1]
        assert torch.equal(out, acc)


def test_qknorm_neox_rope_kernel(cuda_dev):
    """Per-head RMSNorm + non-interleaved RoPE + KV store against the tensor formulas
    (candle-transformers/src/models/quantized_qwen3.rs:136-183)."""
    L = capi.lib()
    torch.manual_seed(6)
    B, T, Hq, Hkv, D, Tmax, pos0, eps = 2, 3, 4, 2, 128, 16, 4, 1e-6
    stride = (Hq + 2 * Hkv) * D
    qkv = torch.randn(B * T, stride, device=cuda_dev)
    qkv0 = qkv.clone()
    qw, kw = torch.rand(D, device=cuda_dev) + 0.5, torch.rand(D, device=cuda_dev) + 0.5
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device=cuda_dev, dtype=torch.float32) / D))
    ang = torch.arange(32, device=cuda_dev, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    kc, vc = torch.zeros(B, Hkv, Tmax, D, device=cuda_dev), torch.zeros(B, Hkv, Tmax, D, device=cuda_dev)
    pos = torch.tensor([pos0], dtype=torch.int32, device=cuda_dev)
    base = qkv.data_ptr()
    L.cq_qknorm_rope_store_kv_f32(base, base + 4 * Hq * D, base + 4 * (Hq + Hkv) * D, qw.data_ptr(), kw.data_ptr(), cos.data_ptr(),
                                  sin.data_ptr(), pos.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, T, Hq, Hkv, D, Tmax, stride, stride,
                                  stride, eps, 1, torch.cuda.current_stream().cuda_stream)
    capi.check("qknorm rope")

    def ref(x, w):          # x [B, T, H, D] double
        x = x.double()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.double()
        c = cos[pos0:pos0 + T][None, :, None, :].double()
        s = sin[pos0:pos0 + T][None, :, None, :].double()
        x1, x2 = x[..., :D // 2], x[..., D // 2:]
        return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1).float()

    q_ref = ref(qkv0[:, :Hq * D].reshape(B, T, Hq, D), qw)
    k_ref = ref(qkv0[:, Hq * D:(Hq + Hkv) * D].reshape(B, T, Hkv, D), kw)
    assert torch.allclose(qkv[:, :Hq * D].reshape(B, T, Hq, D), q_ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(kc[:, :, pos0:pos0 + T], k_ref.permute(0, 2, 1, 3), rtol=1e-5, atol=1e-5)
    assert torch.equal(vc[:, :, pos0:pos0 + T], qkv0[:, (Hq + Hkv) * D:].reshape(B, T, Hkv, D).permute(0, 2, 1, 3))
    assert torch.equal(qkv[:, Hq * D:], qkv0[:, Hq * D:])            # k and v in the projection output stay as they were


def test_moe_decoder_graph_equals_eager(cuda_dev):
    from candle_b200.moe_decoder import MoeDecoderConfig, MoeShapedDecoder
    cfg = MoeDecoderConfig.tiny()
    prompt = torch.randint(0, cfg.vocab, (2, 20), device=cuda_dev, generator=torch.Generator(device=cuda_dev).manual_seed(2))
    m = MoeShapedDecoder(cfg, cuda_dev, batch=2, seed=1)
    eager = m.generate(prompt, 10)
    assert m.capture_decode_step()
    assert torch.equal(m.generate(prompt, 10), eager)
    assert eager.shape == (2, 10) and int(eager.min()) >= 0 and int(eager.max()) < cfg.vocab
    assert not torch.equal(m.generate((prompt + 1) % cfg.vocab, 10), eager)


def test_moe_decode_tokens_do_not_depend_on_fused_quantization(cuda_dev):
    """Decode steps with the norm and the attention storing Q8_1 containers directly (no quantize launch before wqkv and
    wo) against the same steps with f32 results and stand-alone quantization."""
    from candle_b200.moe_decoder import MoeDecoderConfig, MoeShapedDecoder
    cfg = MoeDecoderConfig.tiny()
    prompt = torch.randint(0, cfg.vocab, (2, 20), device=cuda_dev, generator=torch.Generator(device=cuda_dev).manual_seed(5))
    m = MoeShapedDecoder(cfg, cuda_dev, batch=2, seed=2)
    base = m.generate(prompt, 10)
    m.fuse_quantize = False
    assert torch.equal(m.generate(prompt, 10), base)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_tokens_match_single_gpu(tmp_path):
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "ep.txt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(root, "tests", "tp_check.py"), "--moe", "--out", str(out)]
    r = subprocess.run(cmd, cwd=root, env=dict(os.environ, NCCL_NVLS_ENABLE="0"), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert out.read_text().strip() == "identical"


@pytest.mark.parametrize("tname", ["q4_k", "q6_k"])
@pytest.mark.parametrize("with_weights", [False, True])
@pytest.mark.parametrize("e,n,k", [(5, 192, 512), (16, 512, 256), (16, 512, 512), (6, 2048, 768)])
def test_grouped_tensor_core_gemm_matches_cpu_arithmetic(oracle, cuda_dev, tname, with_weights, e, n, k):
    """cq_moe_prefill_gemm: pairs sorted by expert, experts with more than one tile, with an empty expert, and with ids of
    another rank's experts (skipped).  Oracle: the reference CPU matmul (Q8_K activations) of each pair's expert."""
    from candle_b200.moe import moe_prefill_gemm
    wt = TYPES[tname]
    topk = 2       # (16, 512, 256): one super-block per row, many experts with few pairs each - the tiny decoder's shape
    wq = _experts(oracle, wt, e, n, k, seed=11)
    rng = np.random.default_rng(12)
    tokens = 170
    # expert 0 gets 300 pairs (three tiles), expert 2 none, the others a few; two pairs belong to "another rank" (-1, 7)
    flat = np.concatenate([np.zeros(300, np.int32), np.full(17, 1, np.int32), np.full(20, 3, np.int32), np.full(1, 4, np.int32),
                           np.array([-1, e + 2], np.int32)])
    if e > 5:       # spread a part of expert 0's pairs over the further experts (expert 2 stays empty)
        flat[200:300] = rng.integers(5, e, size=100).astype(np.int32)
    assert flat.size == tokens * topk
    rng.shuffle(flat)
    order = np.argsort(flat, kind="stable").astype(np.int32)        # sorted_token_ids
    experts_sorted = flat[order]
    dev = lambda a: torch.from_numpy(a).to(cuda_dev)
    qt = QTensor.from_data(wq.reshape(-1), GgmlDType(wt), (e, n, k), cuda_dev)
    if with_weights:            # down-projection style: one input row per pair, scaled
        x = rng.standard_normal((tokens * topk, k)).astype(np.float32)
        tw = rng.random(tokens * topk, dtype=np.float32)
        out = moe_prefill_gemm(dev(x), qt, dev(tw), dev(order), dev(experts_sorted), topk, zero_init=True).cpu().numpy()
    else:                       # gate / up style: input row = pair // topk
        x = rng.standard_normal((tokens, k)).astype(np.float32)
        tw = None
        out = moe_prefill_gemm(dev(x), qt, None, dev(order), dev(experts_sorted), topk, zero_init=True).cpu().numpy()
    assert capi.lib().cq_prefill_timeout_flag() == 0
    ref = np.zeros_like(out)
    for pair in range(tokens * topk):
        ex = flat[pair]
        if ex < 0 or ex >= e:
            continue
        row = x[pair] if with_weights else x[pair // topk]
        ref[pair] = oracle.matmul(wt, row[None, :], wq[ex], n)[0] * (tw[pair] if with_weights else 1.0)
    assert rel_err(out, ref) <= 1e-5
    skipped = np.where((flat < 0) | (flat >= e))[0]
    assert np.all(out[skipped] == 0.0)
    # bf16 input through the reference's FFI name takes the same kernel
    if not with_weights:
        xb = dev(x).to(torch.bfloat16)
        out_b = moe_gemm_gguf(xb, qt, None, dev(order), dev(experts_sorted), topk, is_prefill=True, zero_init=True).cpu().numpy()
        ref_b = np.zeros_like(out_b)
        xr = xb.to(torch.float32).cpu().numpy()
        for pair in range(tokens * topk):
            ex = flat[pair]
            if 0 <= ex < e:
                ref_b[pair] = oracle.matmul(wt, xr[pair // topk][None, :], wq[ex], n)[0]
        assert rel_err(out_b, ref_b) <= 1e-5
