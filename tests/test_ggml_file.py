"""The legacy GGML container reader (candle_b200/ggml_file.py) against files written here byte by byte after the layout
the reference reads (candle-core/src/quantized/ggml_file.rs:44-60, 78-117, 191-266).  The reference holds no test file
for this format; the cases follow its reader statement by statement."""
import struct

import numpy as np
import pytest

from candle_b200.capi import CandleQError
from candle_b200.ggml_file import Content
from candle_b200.quantized import GgmlDType

MAGIC = {"ggjt": 0x67676a74, "ggmf": 0x67676d66, "ggml": 0x67676d6c, "ggla": 0x67676c61}


def _file(magic, version, vocab, tensors, align32):
    out = bytearray(struct.pack("<I", MAGIC[magic]))
    if version is not None:
        out += struct.pack("<I", version)
    out += struct.pack("<7I", len(vocab), 64, 256, 4, 2, 16, 2)
    for word, score in vocab:
        out += struct.pack("<I", len(word)) + word + struct.pack("<f", score)
    for name, dtype, dims, data in tensors:
        nb = name.encode()
        out += struct.pack("<3I", len(dims), len(nb), int(dtype))
        out += struct.pack(f"<{len(dims)}I", *reversed(dims))          # innermost first
        out += nb
        if align32:
            out += b"\0" * ((32 - len(out) % 32) % 32)
        out += data
    return bytes(out)


def _blocks(rng, dtype, dims):
    n = int(np.prod(dims))
    return rng.integers(0, 256, size=n // dtype.block_size() * dtype.type_size(), dtype=np.uint8).tobytes()


@pytest.mark.parametrize("magic,version,label,align", [("ggml", None, "GgmlUnversioned", False), ("ggmf", 1, "GgmfV1", False),
                                                       ("ggjt", 1, "GgjtV1", True), ("ggjt", 3, "GgjtV3", True)])
def test_reads_every_container_version(magic, version, label, align, tmp_path):
    rng = np.random.default_rng(3)
    vocab = [(b"<s>", 0.0), (b"\xe2\x96\x81the", -3.5), (b"", 1.25)]
    t1, t2 = _blocks(rng, GgmlDType.Q4_0, (8, 64)), _blocks(rng, GgmlDType.Q6K, (2, 3, 256))
    norm = np.arange(5, dtype=np.float32).tobytes()
    data = _file(magic, version, vocab, [("tok_embeddings.weight", GgmlDType.Q4_0, (8, 64), t1),
                                         ("layers.0.w", GgmlDType.Q6K, (2, 3, 256), t2), ("norm.weight", GgmlDType.F32, (5,), norm)], align)
    path = tmp_path / "m.bin"
    path.write_bytes(data)
    for source in (path, data, open(path, "rb")):
        c = Content.read(source)
        assert c.magic == label
        hp = c.hparams
        assert (hp.n_vocab, hp.n_embd, hp.n_mult, hp.n_head, hp.n_layer, hp.n_rot, hp.ftype) == (3, 64, 256, 4, 2, 16, 2)
        assert [w for w, _ in c.vocab] == [b"<s>", b"\xe2\x96\x81the", b""] and [s for _, s in c.vocab] == [0.0, -3.5, 1.25]
        assert set(c.tensors) == {"tok_embeddings.weight", "layers.0.w", "norm.weight"}
        t = c.tensors["layers.0.w"]
        assert (t.ggml_dtype, t.shape, t.data) == (GgmlDType.Q6K, (2, 3, 256), t2)
        assert c.tensors["tok_embeddings.weight"].data == t1 and c.tensors["norm.weight"].data == norm
        got = c.remove("norm.weight")
        assert got.shape == (5,) and "norm.weight" not in c.tensors
        with pytest.raises(CandleQError, match="cannot find tensor with name 'norm.weight'"):
            c.remove("norm.weight")


def test_rejects_what_the_reference_rejects():
    with pytest.raises(CandleQError, match="unknown magic 12345678"):
        Content.read(struct.pack("<I", 0x12345678))
    with pytest.raises(CandleQError, match="unsupported magic/version Ggjt/7"):
        Content.read(struct.pack("<II", MAGIC["ggjt"], 7))
    with pytest.raises(CandleQError, match="unsupported magic/version Ggla/1"):
        Content.read(struct.pack("<II", MAGIC["ggla"], 1))
    good = _file("ggjt", 3, [(b"a", 0.0)], [("w", GgmlDType.Q4K, (3, 100), b"\0" * 168)], True)   # 300 elements: not whole blocks (300 * 144 / 256 bytes are read first)
    with pytest.raises(CandleQError, match="Error creating tensor w: the number of elements 300 is not divisible by the block size 256"):
        Content.read(good)
    short = _file("ggjt", 3, [(b"a", 0.0)], [("w", GgmlDType.Q4K, (2, 256), b"\0" * 100)], True)
    with pytest.raises(CandleQError, match="failed to fill whole buffer"):
        Content.read(short)
    with pytest.raises(CandleQError, match="failed to fill whole buffer"):
        Content.read(_file("ggml", None, [(b"abc", 1.0)], [], False)[:-2])


@pytest.mark.gpu
def test_remove_uploads_the_tensor(cuda_dev):
    rng = np.random.default_rng(4)
    t1 = _blocks(rng, GgmlDType.Q8_0, (4, 64))
    c = Content.read(_file("ggjt", 2, [], [("w", GgmlDType.Q8_0, (4, 64), t1)], True), device=cuda_dev)
    q = c.remove("w")
    assert q.shape == (4, 64) and q.dtype == GgmlDType.Q8_0 and q.data() == t1
