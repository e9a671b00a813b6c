"""ctypes/numpy front end of the CPU oracle (``candle_q_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py``.  The shipped package never imports this module.

The C file restates candle's CPU quantizers / vec_dot / matmul
(candle-core/src/quantized/k_quants.rs, utils.rs, avx.rs) and the arithmetic of its CUDA
kernels (candle-kernels/src/mmvq_gguf.cu, quantized.cu, mmq_gguf/mmq_quantize.cu).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libcandle_q_oracle.so")

# GGML type ids (candle-core/src/quantized/mod.rs:300-342)
Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q2K, Q3K, Q4K, Q5K, Q6K, Q8K = 2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15
TYPE_SIZE = {Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34, Q8_1: 36, Q2K: 84, Q3K: 110, Q4K: 144, Q5K: 176, Q6K: 210, Q8K: 292}
BLOCK_SIZE = {Q4_0: 32, Q4_1: 32, Q5_0: 32, Q5_1: 32, Q8_0: 32, Q8_1: 32, Q2K: 256, Q3K: 256, Q4K: 256, Q5K: 256, Q6K: 256, Q8K: 256}
NAMES = {"q4_0": Q4_0, "q4_1": Q4_1, "q5_0": Q5_0, "q5_1": Q5_1, "q8_0": Q8_0, "q8_1": Q8_1, "q2k": Q2K, "q3k": Q3K, "q4k": Q4K, "q5k": Q5K, "q6k": Q6K, "q8k": Q8K,
         "q2_k": Q2K, "q3_k": Q3K, "q4_k": Q4K, "q5_k": Q5K, "q6_k": Q6K, "q8_k": Q8K}
# dot-product accumulation orders of cqo_vec_dot
SCALAR, SIMD_ORDER, SIMD_HW = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile (gcc); returns the path of the shared library."""
    src = os.path.join(_HERE, "candle_q_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libcandle_q_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        vp, i32, i64, f32p = C.c_void_p, C.c_int, C.c_int64, C.c_void_p
        L.cqo_quantize.argtypes = [i32, f32p, vp, i64]
        L.cqo_quantize_rows.argtypes = [i32, f32p, vp, i64, i64]
        L.cqo_dequantize.argtypes = [i32, vp, f32p, i64]
        L.cqo_vec_dot.argtypes = [i32, i32, i64, vp, vp]
        L.cqo_vec_dot.restype = C.c_float
        L.cqo_matmul.argtypes = [i32, i32, i64, i64, i64, f32p, vp, f32p, i32]
        L.cqo_cpu_block_dots.argtypes = [i32, i64, i64, vp, vp, vp, vp]
        L.cqo_cuda_quantize_q8_1.argtypes = [f32p, vp, i32, i32, i32]
        L.cqo_cuda_mmvq.argtypes = [i32, vp, vp, f32p, i32, i32, i32, i32, i32, i32]
        L.cqo_cuda_block_dots.argtypes = [i32, i64, i64, vp, vp, vp, vp]
        L.cqo_cuda_quantize_mmq_q8_1.argtypes = [i32, f32p, vp, i64, i64, i64]
        L.cqo_cuda_mmq.argtypes = [i32, vp, vp, f32p, i64, i64, i64]
        L.cqo_num_cores.restype = i32
        L.cqo_have_avx2.restype = i32
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32)


def num_cores() -> int:
    return int(lib().cqo_num_cores())


def row_bytes(dtype: int, k: int) -> int:
    assert k % BLOCK_SIZE[dtype] == 0, (dtype, k)
    return k // BLOCK_SIZE[dtype] * TYPE_SIZE[dtype]


def quantize(dtype: int, x) -> np.ndarray:
    """Reference CPU quantizer (``GgmlType::from_float``).  x[..., k] f32 -> uint8 [rows, row_bytes]."""
    x = _f32(x)
    k = x.shape[-1]
    rows = x.size // k
    out = np.zeros((rows, row_bytes(dtype, k)), dtype=np.uint8)
    if rows > 1:
        lib().cqo_quantize_rows(dtype, _p(x), _p(out), rows, k)
    else:
        lib().cqo_quantize(dtype, _p(x), _p(out), k)
    return out


def dequantize(dtype: int, blocks: np.ndarray, k: int) -> np.ndarray:
    """``GgmlType::to_float`` for rows of `k` elements."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    rows = blocks.size // row_bytes(dtype, k)
    out = np.empty((rows, k), dtype=np.float32)
    lib().cqo_dequantize(dtype, _p(blocks), _p(out), rows * k)
    return out


def vec_dot(dtype: int, w_row: np.ndarray, act_row: np.ndarray, k: int, mode: int = SCALAR) -> float:
    w_row = np.ascontiguousarray(w_row, dtype=np.uint8)
    act_row = np.ascontiguousarray(act_row, dtype=np.uint8)
    return float(lib().cqo_vec_dot(dtype, mode, k, _p(w_row), _p(act_row)))


def vec_dot_type(dtype: int) -> int:
    return int(lib().cqo_vec_dot_type(dtype))


def matmul(dtype: int, lhs, w_blocks: np.ndarray, n: int, mode: int = SIMD_ORDER, nthreads: int = 0) -> np.ndarray:
    """``k_quants::matmul``: lhs f32 [m, k] x quantized W [n, k] -> f32 [m, n]."""
    lhs = _f32(lhs)
    m, k = lhs.shape
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8)
    assert w_blocks.size == n * row_bytes(dtype, k)
    dst = np.empty((m, n), dtype=np.float32)
    lib().cqo_matmul(dtype, mode, m, k, n, _p(lhs), _p(w_blocks), _p(dst), nthreads)
    return dst


def cpu_block_dots(dtype: int, w_blocks: np.ndarray, act_blocks: np.ndarray, k: int, n: int):
    """Integer per-block dot products of the CPU path, (dots[n, k/blk], min_dots[n, k/blk])."""
    nb = k // BLOCK_SIZE[dtype]
    out = np.zeros((n, nb), dtype=np.int32)
    outm = np.zeros((n, nb), dtype=np.int32)
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8)
    act_blocks = np.ascontiguousarray(act_blocks, dtype=np.uint8)
    lib().cqo_cpu_block_dots(dtype, k, n, _p(w_blocks), _p(act_blocks), _p(out), _p(outm))
    return out, outm


# ---- CUDA semantics -----------------------------------------------------------------------

def pad(p: int, q: int) -> int:
    return (p + q - 1) // q * q


def cuda_quantize_q8_1(x, k_padded: int | None = None) -> np.ndarray:
    """``quantize_q8_1`` kernel: x f32 [rows, k] -> uint8 [rows, k_padded/32 * 36]."""
    x = _f32(x)
    rows, k = x.shape
    if k_padded is None:
        k_padded = pad(k, 512)
    out = np.zeros((rows, k_padded // 32 * 36), dtype=np.uint8)
    lib().cqo_cuda_quantize_q8_1(_p(x), _p(out), k, k_padded, rows)
    return out


def cuda_mmvq(dtype: int, w_blocks: np.ndarray, q8_1: np.ndarray, k: int, n: int, fma: bool = True) -> np.ndarray:
    """Reference MMVQ kernel, thread-by-thread: returns f32 [b, n]."""
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8)
    q8_1 = np.ascontiguousarray(q8_1, dtype=np.uint8)
    b = q8_1.shape[0]
    stride_col_y = q8_1.shape[1] // 36
    dst = np.empty((b, n), dtype=np.float32)
    lib().cqo_cuda_mmvq(dtype, _p(w_blocks), _p(q8_1), _p(dst), k, n, stride_col_y, n, b, int(fma))
    return dst


def cuda_block_dots(dtype: int, w_blocks: np.ndarray, q8_1_row: np.ndarray, k: int, n: int):
    nb = k // BLOCK_SIZE[dtype]
    out = np.zeros((n, nb), dtype=np.int32)
    outm = np.zeros((n, nb), dtype=np.int32)
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8)
    q8_1_row = np.ascontiguousarray(q8_1_row, dtype=np.uint8)
    lib().cqo_cuda_block_dots(dtype, k, n, _p(w_blocks), _p(q8_1_row), _p(out), _p(outm))
    return out, outm


def cuda_quantize_mmq_q8_1(x, layout: str, k_padded: int | None = None) -> np.ndarray:
    """``quantize_mmq_q8_1``: x f32 [tokens, k] -> uint8 [k_padded/128, tokens, 144]; layout 'D4', 'DS4' or 'D2S6'."""
    x = _f32(x)
    tokens, k = x.shape
    if k_padded is None:
        k_padded = pad(pad(k, 512), 128)
    out = np.zeros((k_padded // 128, tokens, 144), dtype=np.uint8)
    lib().cqo_cuda_quantize_mmq_q8_1({"D4": 0, "DS4": 1, "D2S6": 2}[layout], _p(x), _p(out), k, k_padded, tokens)
    return out


def cuda_mmq(dtype: int, w_blocks: np.ndarray, y_mmq: np.ndarray, k: int, n: int) -> np.ndarray:
    """Matmul over the ``block_q8_1_mmq`` scratch (uint8 [k_padded/128, tokens, 144]) -> f32 [tokens, n]."""
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8)
    y_mmq = np.ascontiguousarray(y_mmq, dtype=np.uint8)
    tokens = y_mmq.shape[1]
    out = np.zeros((tokens, n), dtype=np.float32)
    lib().cqo_cuda_mmq(dtype, _p(w_blocks), _p(y_mmq), _p(out), k, n, tokens)
    return out


def f32_to_bf16_bits(x) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 (as uint16 bit patterns)."""
    u = _f32(x).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
