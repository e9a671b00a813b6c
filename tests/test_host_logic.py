"""Host-side logic that needs no GPU: type registry, shape checks, error behaviour."""
import numpy as np
import pytest
import torch

from candle_b200 import capi
from candle_b200.quantized import GgmlDType, QMatMul, QTensor


def test_type_registry_matches_reference():
    """candle-core/src/quantized/mod.rs:300-342 (ids), :387-421 (sizes)."""
    ids = {"F32": 0, "F16": 1, "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q8_1": 9, "Q2K": 10,
           "Q3K": 11, "Q4K": 12, "Q5K": 13, "Q6K": 14, "Q8K": 15, "BF16": 30}
    for name, u in ids.items():
        assert GgmlDType.from_u32(u) is GgmlDType[name]
    with pytest.raises(capi.CandleQError, match="unknown dtype for tensor 4"):
        GgmlDType.from_u32(4)
    sizes = {"Q4_0": (18, 32), "Q8_0": (34, 32), "Q8_1": (36, 32), "Q4K": (144, 256), "Q6K": (210, 256),
             "Q8K": (292, 256), "Q2K": (84, 256), "Q3K": (110, 256), "Q5K": (176, 256), "Q4_1": (20, 32),
             "Q5_0": (22, 32), "Q5_1": (24, 32), "F32": (4, 1), "F16": (2, 1), "BF16": (2, 1)}
    for name, (ts, bs) in sizes.items():
        assert GgmlDType[name].type_size() == ts and GgmlDType[name].block_size() == bs


def test_oracle_and_library_agree_on_sizes(oracle):
    for name, code in (("Q4_0", capi.Q4_0), ("Q8_0", capi.Q8_0), ("Q4K", capi.Q4_K), ("Q6K", capi.Q6_K)):
        dt = getattr(oracle, name)
        assert oracle.TYPE_SIZE[dt] == capi.TYPE_SIZE[code] == GgmlDType(code).type_size()
        assert oracle.BLOCK_SIZE[dt] == capi.BLOCK_ELEMS[code] == GgmlDType(code).block_size()


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_fails_loudly_without_a_gpu(lib):
    """No CPU fallback: uploading weights or running a matmul without a CUDA device is an error."""
    blocks = np.zeros(4 * 144, dtype=np.uint8)
    with pytest.raises(capi.CandleQError):
        QTensor.from_data(blocks, GgmlDType.Q4K, (4, 256))
    with pytest.raises(capi.CandleQError, match="no CPU path"):
        QMatMul.__new__(QMatMul).forward(torch.zeros(1, 256))


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(capi.CandleQError, match="no CPU or PyTorch fallback"):
        capi.lib()


def test_moe_routing_matches_numpy_restatement():
    """fused_moe.rs:233-260: softmax, top-k (descending), renormalisation, pairs sorted by expert."""
    import numpy as np
    import torch
    from candle_b200.fused_moe import route, sort_pairs
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((7, 16)).astype(np.float32)
    w, ids = route(torch.from_numpy(logits), 4, True)
    e = np.exp(logits - logits.max(-1, keepdims=True))
    p = e / e.sum(-1, keepdims=True)
    ref_ids = np.argsort(-p, axis=-1, kind="stable")[:, :4]
    ref_w = np.take_along_axis(p, ref_ids, -1)
    ref_w = ref_w / ref_w.sum(-1, keepdims=True)
    assert np.array_equal(ids.numpy(), ref_ids)
    assert np.allclose(w.numpy(), ref_w, rtol=1e-6, atol=1e-7)
    w2, _ = route(torch.from_numpy(logits), 4, False)
    assert np.allclose(w2.numpy(), np.take_along_axis(p, ref_ids, -1), rtol=1e-6, atol=1e-7)
    experts, pairs = sort_pairs(ids)
    flat = ref_ids.reshape(-1)
    assert np.array_equal(experts.numpy(), np.sort(flat, kind="stable"))
    assert np.array_equal(flat[pairs.numpy()], experts.numpy())          # pair indices in expert order
    assert sorted(pairs.tolist()) == list(range(flat.size))


def test_decoder_refuses_positions_beyond_max_pos():
    """The host-side bound of the decoder harness: claiming positions past max_pos raises before anything is launched
    (the KV cache and the rotary tables hold max_pos positions)."""
    import types

    import pytest

    from candle_b200.decoder import DecoderConfig, LlamaShapedDecoder
    stub = types.SimpleNamespace(cfg=DecoderConfig.tiny(), _pos_host=0)
    LlamaShapedDecoder._claim_positions(stub, 100)
    LlamaShapedDecoder._claim_positions(stub, 28)
    assert stub._pos_host == 128 == stub.cfg.max_pos
    with pytest.raises(ValueError, match="max_pos"):
        LlamaShapedDecoder._claim_positions(stub, 1)
    assert stub._pos_host == 128
    stub2 = types.SimpleNamespace(cfg=DecoderConfig.tiny(), _pos_host=0)
    with pytest.raises(ValueError, match="max_pos"):
        LlamaShapedDecoder.generate(stub2, __import__("torch").zeros((1, 120), dtype=__import__("torch").int64), 10)
