"""GGUF reader (csrc/host/gguf.cpp) against files written here byte by byte after the format the reference reads and
writes (candle-core/src/quantized/gguf_file.rs:470-640): versions, all value types, nested arrays, alignment, reversed
dimensions, and the errors the reference raises for malformed files."""
import struct

import numpy as np
import pytest

from candle_b200.capi import CandleQError
from candle_b200.gguf_file import Content
from candle_b200.quantized import GgmlDType

T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<B", T_U64: "<Q",
       T_I64: "<q", T_F64: "<d"}


def _len(n, version):
    return struct.pack("<I" if version == 1 else "<Q", n)


def _string(s, version):
    b = s.encode()
    return _len(len(b), version) + b


def _value(vt, v, version):
    if vt == T_STR:
        return _string(v, version)
    if vt == T_ARR:
        et, items = v
        return struct.pack("<I", et) + _len(len(items), version) + b"".join(_value(et, it, version) for it in items)
    return struct.pack(FMT[vt], v)


def write_gguf(path, metadata, tensors, version=3, alignment=32, magic=0x46554747):
    """metadata: [(key, type, value)]; tensors: [(name, ggml dtype id, dims outermost-first, bytes)]."""
    out = struct.pack("<II", magic, version) + _len(len(tensors), version) + _len(len(metadata), version)
    for key, vt, v in metadata:
        out += _string(key, version) + struct.pack("<I", vt) + _value(vt, v, version)
    offset, blobs = 0, []
    for name, dt, dims, data in tensors:
        out += _string(name, version) + struct.pack("<I", len(dims))
        out += b"".join(struct.pack("<I" if version == 1 else "<Q", d) for d in reversed(dims))
        out += struct.pack("<IQ", dt, offset)
        padded = data + b"\0" * (-len(data) % alignment)
        blobs.append(padded)
        offset += len(padded)
    out += b"\0" * (-len(out) % alignment)
    with open(path, "wb") as f:
        f.write(out + b"".join(blobs))
    return len(out)


def _blocks(rng, dtype: GgmlDType, n, k):
    return rng.integers(0, 256, size=n * k // dtype.block_size() * dtype.type_size(), dtype=np.uint8).tobytes()


@pytest.mark.parametrize("version", [1, 2, 3])
def test_reads_header_metadata_and_tensor_infos(lib, tmp_path, version):
    rng = np.random.default_rng(version)
    w1, w2 = _blocks(rng, GgmlDType.Q4K, 8, 512), _blocks(rng, GgmlDType.Q6K, 3, 256)
    norm = np.arange(64, dtype=np.float32).tobytes()
    meta = [("general.architecture", T_STR, "llama"), ("llama.block_count", T_U32, 32), ("a.u8", T_U8, 200), ("a.i8", T_I8, -5),
            ("a.u16", T_U16, 65000), ("a.i16", T_I16, -300), ("a.i32", T_I32, -70000), ("a.f32", T_F32, 1e-5), ("a.bool", T_BOOL, 1),
            ("a.u64", T_U64, 2 ** 60 + 1), ("a.i64", T_I64, -2 ** 40), ("a.f64", T_F64, 0.1),
            ("tokens", T_ARR, (T_STR, ["<s>", "a\"b", "tab\t"])), ("nested", T_ARR, (T_ARR, [(T_I32, [1, -2]), (T_I32, [])])),
            ("padded\0\0", T_STR, "x\0")]
    data_start = write_gguf(tmp_path / "m.gguf", meta, [("blk.0.attn_q.weight", 12, (8, 512), w1), ("output.weight", 14, (3, 256), w2),
                                                      ("norm.weight", 0, (64,), norm)], version=version)
    c = Content.read(tmp_path / "m.gguf")
    assert c.magic == version and c.tensor_data_offset == data_start
    md = c.metadata
    assert md["general.architecture"] == "llama" and md["llama.block_count"] == 32
    assert (md["a.u8"], md["a.i8"], md["a.u16"], md["a.i16"], md["a.i32"]) == (200, -5, 65000, -300, -70000)
    assert md["a.bool"] is True and md["a.u64"] == 2 ** 60 + 1 and md["a.i64"] == -2 ** 40 and md["a.f64"] == 0.1
    assert np.float32(md["a.f32"]) == np.float32(1e-5)
    assert md["tokens"] == ["<s>", "a\"b", "tab\t"] and md["nested"] == [[1, -2], []]
    assert md["padded"] == "x"                                   # trailing NULs are dropped from strings
    q = c.tensor_infos["blk.0.attn_q.weight"]
    assert (q.ggml_dtype, q.shape, q.offset, q.nbytes) == (GgmlDType.Q4K, (8, 512), 0, len(w1))
    o = c.tensor_infos["output.weight"]
    assert (o.ggml_dtype, o.shape, o.nbytes) == (GgmlDType.Q6K, (3, 256), len(w2)) and o.offset % 32 == 0
    assert c.tensor_infos["norm.weight"].shape == (64,)
    assert c.tensor_bytes("output.weight").tobytes() == w2
    assert np.array_equal(c.tensor_bytes("norm.weight").view(np.float32), np.arange(64, dtype=np.float32))
    with pytest.raises(CandleQError, match="cannot find tensor info for nope"):
        c.tensor_bytes("nope")
    c.close()


def test_alignment_key_moves_the_tensor_data(lib, tmp_path):
    w = bytes(range(144))
    start = write_gguf(tmp_path / "a.gguf", [("general.alignment", T_U32, 64)], [("w", 12, (1, 256), w)], alignment=64)
    c = Content.read(tmp_path / "a.gguf")
    assert c.tensor_data_offset == start and start % 64 == 0 and c.tensor_bytes("w").tobytes() == w


def test_rejects_malformed_files(lib, tmp_path):
    p = tmp_path / "bad.gguf"
    write_gguf(p, [], [], magic=0x12345678)
    with pytest.raises(CandleQError, match="unknown magic 0x12345678"):
        Content.read(p)
    write_gguf(p, [], [], version=7)
    with pytest.raises(CandleQError, match="unsupported magic/version"):
        Content.read(p)
    p.write_bytes(struct.pack("<IIQQ", 0x46554747, 3, 1 << 40, 0))                 # absurd tensor count
    with pytest.raises(CandleQError, match="exceeds max"):
        Content.read(p)
    p.write_bytes(struct.pack("<IIQQ", 0x46554747, 3, 1000, 1000))                 # counts that cannot fit
    with pytest.raises(CandleQError, match="needs at least"):
        Content.read(p)
    p.write_bytes(struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1 << 20) + b"ab" + b"\0" * 32)   # string too long
    with pytest.raises(CandleQError, match="exceeds remaining file bytes"):
        Content.read(p)
    p.write_bytes(struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + _string("k", 3) + struct.pack("<I", 99) + b"\0" * 32)
    with pytest.raises(CandleQError, match="unrecognized value-type"):
        Content.read(p)
    write_gguf(p, [], [("w", 12, (1, 2, 3, 4, 256), b"")])                       # five dimensions
    with pytest.raises(CandleQError, match="dimensions, max is 4"):
        Content.read(p)
    write_gguf(p, [], [("w", 12, (3, 100), b"")])                               # not a whole number of blocks
    with pytest.raises(CandleQError, match="not divisible by the block size 256"):
        Content.read(p)
    write_gguf(p, [], [("w", 99, (1, 256), b"")])
    with pytest.raises(CandleQError, match="unknown dtype for tensor 99"):
        Content.read(p)
    write_gguf(p, [], [("w", 12, (4, 256), b"\0" * 100)])                        # data shorter than the shape says
    c = Content.read(p)
    with pytest.raises(CandleQError, match="only .* remaining in file"):
        c.tensor_bytes("w")


@pytest.mark.gpu
def test_tensor_upload_and_row_shards(lib, oracle, cuda_dev, tmp_path):
    import torch
    from candle_b200.quantized import QMatMul, QTensor
    from helpers import make_case
    n, k = 64, 1024
    _, x, wq = make_case(oracle, 12, k, n, 2, seed=4)
    write_gguf(tmp_path / "w.gguf", [("general.name", T_STR, "t")], [("pad", 0, (3,), b"\1" * 12), ("w", 12, (n, k), wq.tobytes())])
    c = Content.read(tmp_path / "w.gguf")
    qt = c.tensor("w", cuda_dev)
    assert qt.shape == (n, k) and qt.dtype == GgmlDType.Q4K and qt.data() == wq.tobytes()
    xd = torch.from_numpy(x).to(cuda_dev)
    full = QMatMul.from_qtensor(qt).forward(xd)
    assert torch.equal(full, QMatMul.from_qtensor(QTensor.from_data(wq.reshape(-1), GgmlDType.Q4K, (n, k), cuda_dev)).forward(xd))
    parts = [QMatMul.from_qtensor(c.tensor("w", cuda_dev, rows=(r * 16, 16))).forward(xd) for r in range(4)]
    assert torch.equal(torch.cat(parts, dim=1), full)
    with pytest.raises(CandleQError, match="row range outside the tensor"):
        c.tensor("w", cuda_dev, rows=(60, 16))


def test_reads_a_file_written_by_the_gguf_package(lib, tmp_path):
    """Interoperability with an independent writer (the `gguf` Python package of the llama.cpp project), when installed."""
    gguf = pytest.importorskip("gguf")
    path = str(tmp_path / "pkg.gguf")
    w = gguf.GGUFWriter(path, "llama")
    w.add_block_count(2)
    w.add_context_length(4096)
    w.add_token_list(["<s>", "</s>", "hello"])
    norm = np.linspace(0, 1, 32, dtype=np.float32)
    q8 = np.random.default_rng(0).integers(0, 256, size=(4, 64 // 32 * 34), dtype=np.uint8)
    w.add_tensor("blk.0.attn_norm.weight", norm)
    w.add_tensor("blk.0.ffn_down.weight", q8, raw_shape=(4, 64 // 32 * 34), raw_dtype=gguf.GGMLQuantizationType.Q8_0)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    c = Content.read(path)
    assert c.magic == 3 and c.metadata["general.architecture"] == "llama" and c.metadata["llama.block_count"] == 2
    assert c.metadata["tokenizer.ggml.tokens"] == ["<s>", "</s>", "hello"]
    assert np.array_equal(c.tensor_bytes("blk.0.attn_norm.weight").view(np.float32), norm)
    info = c.tensor_infos["blk.0.ffn_down.weight"]
    assert info.ggml_dtype == GgmlDType.Q8_0 and info.shape == (4, 64) and c.tensor_bytes("blk.0.ffn_down.weight").tobytes() == q8.tobytes()


def test_write_round_trips_through_the_reader_and_the_gguf_package(lib, tmp_path):
    """`gguf_file.write` (the reference's `gguf_file::write`): every value type, nested and empty arrays, tensors of
    several block formats with 32-byte padding between them; read back by this library's reader and, when installed, by
    the independent `gguf` package."""
    from candle_b200.gguf_file import HostTensor, Value, write
    rng = np.random.default_rng(11)
    w1, w2 = _blocks(rng, GgmlDType.Q4K, 8, 512), _blocks(rng, GgmlDType.Q8_0, 5, 96)       # 5 * 3 * 34 = 510 bytes: padded to 512
    norm = np.arange(7, dtype=np.float32).tobytes()
    meta = [("general.architecture", Value("string", "llama")), ("llama.block_count", Value("u32", 32)), ("a.u8", Value("u8", 200)),
            ("a.i8", Value("i8", -5)), ("a.u16", Value("u16", 65000)), ("a.i16", Value("i16", -300)), ("a.i32", Value("i32", -70000)),
            ("a.f32", Value("f32", 0.5)), ("a.bool", Value("bool", True)), ("a.u64", Value("u64", 2 ** 60 + 1)),
            ("a.i64", Value("i64", -2 ** 40)), ("a.f64", Value("f64", 0.1)),
            ("tokens", Value("array", [Value("string", s) for s in ("<s>", "a\"b", "tab\t")])),
            ("nested", Value("array", [Value("array", [Value("i32", 1), Value("i32", -2)]), Value("array", [])])),
            ("empty", Value("array", []))]
    tensors = [("blk.0.attn_q.weight", HostTensor(GgmlDType.Q4K, (8, 512), w1)), ("blk.0.ffn_down.weight", HostTensor(GgmlDType.Q8_0, (5, 96), w2)),
               ("norm.weight", HostTensor(GgmlDType.F32, (7,), norm))]
    path = tmp_path / "written.gguf"
    with open(path, "wb") as f:
        write(f, meta, tensors)
    raw = path.read_bytes()
    assert raw[:8] == struct.pack("<II", 0x46554747, 2) and len(raw) % 32 == 0
    c = Content.read(path)
    assert c.magic == 2 and c.tensor_data_offset % 32 == 0
    md = c.metadata
    assert md["general.architecture"] == "llama" and md["llama.block_count"] == 32 and md["a.bool"] is True
    assert (md["a.u8"], md["a.i8"], md["a.u16"], md["a.i16"], md["a.i32"], md["a.f32"]) == (200, -5, 65000, -300, -70000, 0.5)
    assert md["a.u64"] == 2 ** 60 + 1 and md["a.i64"] == -2 ** 40 and md["a.f64"] == 0.1
    assert md["tokens"] == ["<s>", "a\"b", "tab\t"] and md["nested"] == [[1, -2], []] and md["empty"] == []
    q, d, nw = c.tensor_infos["blk.0.attn_q.weight"], c.tensor_infos["blk.0.ffn_down.weight"], c.tensor_infos["norm.weight"]
    assert (q.ggml_dtype, q.shape, q.offset) == (GgmlDType.Q4K, (8, 512), 0)
    assert (d.ggml_dtype, d.shape, d.offset) == (GgmlDType.Q8_0, (5, 96), len(w1))
    assert (nw.ggml_dtype, nw.shape, nw.offset) == (GgmlDType.F32, (7,), len(w1) + 512)
    assert c.tensor_bytes("blk.0.attn_q.weight").tobytes() == w1 and c.tensor_bytes("blk.0.ffn_down.weight").tobytes() == w2
    assert c.tensor_bytes("norm.weight").tobytes() == norm
    c.close()
    with pytest.raises(CandleQError, match="multiple value-types"):
        with open(tmp_path / "bad.gguf", "wb") as f:
            write(f, [("x", Value("array", [Value("u8", 1), Value("i8", 1)]))], [])
    with pytest.raises(CandleQError, match="do not match shape"):
        with open(tmp_path / "bad.gguf", "wb") as f:
            write(f, [], [("w", HostTensor(GgmlDType.Q4K, (2, 256), b"\0" * 100))])
    gguf = pytest.importorskip("gguf")
    r = gguf.GGUFReader(str(path))
    assert int(r.fields["llama.block_count"].parts[-1][0]) == 32
    by_name = {t.name: t for t in r.tensors}
    assert bytes(by_name["blk.0.ffn_down.weight"].data.tobytes()) == w2
    assert bytes(by_name["blk.0.attn_q.weight"].data.tobytes()) == w1
    assert by_name["norm.weight"].data.tobytes() == norm
