"""Python face of the host objects: ``GgmlDType``, ``QTensor``, ``QMatMul``.

Mirrors the names and behaviour of candle-core/src/quantized/mod.rs (``GgmlDType`` :281-421, ``QTensor``
:59-66 and :505-562, ``QMatMul`` :807-852 and ``Module::forward`` :1020-1043) and of candle-pyo3's
``QTensor.matmul_t`` (candle-pyo3/src/lib.rs:1276-1280).  All arithmetic happens in
``libcandle_q_b200.so``; torch only supplies device memory and the current stream.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Sequence

import numpy as np
import torch

from . import capi
from .capi import CandleQError


class GgmlDType(enum.IntEnum):
    """GGML tensor types with their ids in GGUF files (mod.rs:300-342)."""
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2K = 10
    Q3K = 11
    Q4K = 12
    Q5K = 13
    Q6K = 14
    Q8K = 15
    BF16 = 30

    @classmethod
    def from_u32(cls, u: int) -> "GgmlDType":
        try:
            return cls(u)
        except ValueError:
            raise CandleQError(f"unknown dtype for tensor {u}") from None

    def type_size(self) -> int:
        """Bytes per block (mod.rs:387-406)."""
        return _TYPE_SIZE[self]

    def block_size(self) -> int:
        """Elements per block (mod.rs:409-421)."""
        if self in (GgmlDType.F32, GgmlDType.F16, GgmlDType.BF16):
            return 1
        if self in (GgmlDType.Q4_0, GgmlDType.Q4_1, GgmlDType.Q5_0, GgmlDType.Q5_1, GgmlDType.Q8_0, GgmlDType.Q8_1):
            return 32
        return 256


_TYPE_SIZE = {
    GgmlDType.F32: 4, GgmlDType.F16: 2, GgmlDType.BF16: 2, GgmlDType.Q4_0: 18, GgmlDType.Q4_1: 20,
    GgmlDType.Q5_0: 22, GgmlDType.Q5_1: 24, GgmlDType.Q8_0: 34, GgmlDType.Q8_1: 36, GgmlDType.Q2K: 84,
    GgmlDType.Q3K: 110, GgmlDType.Q4K: 144, GgmlDType.Q5K: 176, GgmlDType.Q6K: 210, GgmlDType.Q8K: 292,
}

_ELEM = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}


def set_activation_mode(cpu_exact: bool) -> None:
    """False (default): Q8_1 activations, the arithmetic of candle's CUDA kernels.
    True: activations quantized exactly like candle's CPU path (Q8_0 / Q8_K)."""
    capi.lib().cqh_set_act_mode(1 if cpu_exact else 0)


def quantize_blocks(src, dtype: GgmlDType, imatrix=None) -> bytes:
    """f32 values -> GGUF blocks in host memory, with the reference's CPU ``from_float`` arithmetic (k_quants.rs); the ten
    GGUF block formats.  Uses no device.  ``src``: a numpy array or CPU tensor whose last dimension is a multiple of the block
    size.  With ``imatrix`` (one importance value per element of the last dimension) the importance-weighted
    ``from_float_imatrix`` runs instead (Q2K, Q3K, Q4K, Q5K, Q6K)."""
    dtype = GgmlDType(dtype)
    x = np.ascontiguousarray(src.detach().cpu().numpy() if isinstance(src, torch.Tensor) else src, dtype=np.float32)
    dims, nd = _dims(x.shape)
    out = np.empty(x.size // dtype.block_size() * dtype.type_size() if x.ndim and x.shape[-1] % dtype.block_size() == 0 else 0,
                   dtype=np.uint8)
    if imatrix is None:
        capi.hcheck(capi.lib().cqh_quantize_f32(int(dtype), x.ctypes.data, dims, nd, out.ctypes.data, out.size), "quantize_blocks")
    else:
        im = np.ascontiguousarray(imatrix, dtype=np.float32).reshape(-1)
        capi.hcheck(capi.lib().cqh_quantize_imatrix_f32(int(dtype), x.ctypes.data, dims, nd, im.ctypes.data, im.size,
                                                         out.ctypes.data, out.size), "quantize_blocks")
    return out.tobytes()


def _dims(shape: Sequence[int]):
    arr = (C.c_int64 * len(shape))(*[int(d) for d in shape])
    return arr, len(shape)


class QTensor:
    """A quantized tensor resident on one CUDA device."""

    def __init__(self, handle: int, dtype: GgmlDType, shape: tuple[int, ...], device: torch.device, keep=None):
        self._h = C.c_void_p(handle)
        self._dtype = dtype
        self._shape = tuple(int(d) for d in shape)
        self._device = device
        self._keep = keep   # backing tensor of a non-owning view

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                capi.lib().cqh_qtensor_free(h)
            except Exception:
                pass

    @classmethod
    def from_data(cls, data, dtype: GgmlDType, shape: Sequence[int], device="cuda:0") -> "QTensor":
        """Upload GGUF blocks held in host memory (``QStorage::from_data`` + ``load_quantized``,
        mod.rs:94-133, cuda.rs:989-1008)."""
        dtype = GgmlDType(dtype)
        device = torch.device(device)
        if isinstance(data, torch.Tensor):
            data = data.detach().cpu().contiguous().numpy()
        buf = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if isinstance(data, (bytes, bytearray, memoryview))
                                   else np.asarray(data).view(np.uint8).reshape(-1))
        dims, nd = _dims(shape)
        h = C.c_void_p()
        capi.hcheck(capi.lib().cqh_qtensor_load(int(dtype), buf.ctypes.data, buf.size, dims, nd,
                                                 device.index or 0, C.byref(h)), "QTensor.from_data")
        return cls(h.value, dtype, tuple(shape), device)

    @classmethod
    def quantize_onto(cls, src: torch.Tensor, dtype: GgmlDType, device="cuda:0") -> "QTensor":
        """``QTensor::quantize_onto`` (mod.rs:645-671): quantizes a tensor held on the CPU with the reference's CPU
        ``from_float`` arithmetic and puts the blocks on ``device``.  Built for the ten GGUF block formats (Q4_0 ... Q6K)."""
        dtype = GgmlDType(dtype)
        if src.device.type != "cpu":
            raise CandleQError("`quantize_onto` expects a `src` to be on the cpu, got cuda.")
        device = torch.device(device)
        x = src.detach().to(torch.float32).contiguous()
        dims, nd = _dims(tuple(x.shape))
        h = C.c_void_p()
        capi.hcheck(capi.lib().cqh_qtensor_quantize_onto(int(dtype), x.data_ptr(), dims, nd, device.index or 0, C.byref(h)),
                    "QTensor.quantize_onto")
        return cls(h.value, dtype, tuple(x.shape), device)

    @classmethod
    def quantize_imatrix_onto(cls, src: torch.Tensor, imatrix_weights, dtype: GgmlDType, device="cuda:0") -> "QTensor":
        """``QTensor::quantize_imatrix_onto`` (mod.rs:601-642): as ``quantize_onto`` with one importance value per element of
        the last dimension (``from_float_imatrix``; Q2K, Q3K, Q4K, Q5K, Q6K)."""
        dtype = GgmlDType(dtype)
        if src.device.type != "cpu":
            raise CandleQError("`quantize_onto` expects a `src` to be on the cpu, got cuda.")
        device = torch.device(device)
        x = src.detach().to(torch.float32).contiguous()
        im = np.ascontiguousarray(imatrix_weights, dtype=np.float32).reshape(-1)
        dims, nd = _dims(tuple(x.shape))
        h = C.c_void_p()
        capi.hcheck(capi.lib().cqh_qtensor_quantize_imatrix_onto(int(dtype), x.data_ptr(), dims, nd, im.ctypes.data, im.size,
                                                                  device.index or 0, C.byref(h)), "QTensor.quantize_imatrix_onto")
        return cls(h.value, dtype, tuple(x.shape), device)

    @classmethod
    def quantize_imatrix(cls, src: torch.Tensor, imatrix_weights, dtype: GgmlDType) -> "QTensor":
        """``QTensor::quantize_imatrix`` (mod.rs:564-598); the result lives on ``src``'s CUDA device."""
        if not src.is_cuda:
            raise CandleQError("QTensor.quantize_imatrix: this library holds quantized tensors on CUDA devices only; "
                               "use quantize_imatrix_onto(src, imatrix, dtype, device) for a tensor on the cpu")
        return cls.quantize_imatrix_onto(src.detach().to("cpu", torch.float32), imatrix_weights, dtype, src.device)

    @classmethod
    def quantize(cls, src: torch.Tensor, dtype: GgmlDType) -> "QTensor":
        """``QTensor::quantize`` (mod.rs:543-562): the quantized tensor lives on ``src``'s device, which must be a CUDA
        device here.  As in the reference's CUDA storage (cuda.rs:704-725) the values are brought to the host, quantized
        there and the blocks uploaded; this is a load-time step."""
        if not src.is_cuda:
            raise CandleQError("QTensor.quantize: this library holds quantized tensors on CUDA devices only; "
                               "use quantize_onto(src, dtype, device) for a tensor on the cpu")
        return cls.quantize_onto(src.detach().to("cpu", torch.float32), dtype, src.device)

    @classmethod
    def from_device_blocks(cls, blocks: torch.Tensor, dtype: GgmlDType, shape: Sequence[int]) -> "QTensor":
        """Non-owning view of GGUF blocks already on the device (``blocks``: contiguous uint8 CUDA tensor)."""
        dtype = GgmlDType(dtype)
        if not blocks.is_cuda or blocks.dtype != torch.uint8 or not blocks.is_contiguous():
            raise CandleQError("from_device_blocks expects a contiguous uint8 CUDA tensor")
        dims, nd = _dims(shape)
        h = C.c_void_p()
        capi.hcheck(capi.lib().cqh_qtensor_wrap(int(dtype), blocks.data_ptr(), blocks.numel(), dims, nd,
                                                 blocks.device.index or 0, C.byref(h)), "QTensor.from_device_blocks")
        return cls(h.value, dtype, tuple(shape), blocks.device, keep=blocks)

    @property
    def shape(self) -> tuple[int, ...]:
        return self._shape

    @property
    def dtype(self) -> GgmlDType:
        return self._dtype

    @property
    def device(self) -> torch.device:
        return self._device

    def rank(self) -> int:
        return len(self._shape)

    def storage_size_in_bytes(self) -> int:
        n = 1
        for d in self._shape:
            n *= d
        return n // self._dtype.block_size() * self._dtype.type_size()

    def device_ptr(self) -> int:
        return int(capi.lib().cqh_qtensor_device_ptr(self._h))

    def data(self) -> bytes:
        """The canonical GGUF bytes (``QTensor::data``, mod.rs:754-756)."""
        out = np.empty(self.storage_size_in_bytes(), dtype=np.uint8)
        capi.hcheck(capi.lib().cqh_qtensor_data(self._h, out.ctypes.data, out.size), "QTensor.data")
        return out.tobytes()

    def indexed_moe_forward(self, x: torch.Tensor, ids: torch.Tensor, zero_init: bool = False) -> torch.Tensor:
        """``QTensor::indexed_moe_forward`` (mod.rs:758-784): self is [experts, n, k]; x f32 [batch, topk or 1, k];
        ids u32/i32 [batch, topk] -> f32 [batch, topk, n].  Ids outside [0, experts) are skipped; with `zero_init` their
        output rows read as zero (an expert-parallel rank passes ids shifted by its first expert)."""
        if self.rank() != 3:
            raise CandleQError("indexed_moe_forward expects a rank-3 [experts, n, k] tensor")
        if not x.is_cuda or x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 3:
            raise CandleQError("indexed_moe_forward expects a contiguous f32 CUDA tensor [batch, topk or 1, k]")
        batch, x_dim1, k = x.shape
        if k != self._shape[2]:
            raise CandleQError(f"mismatch on matmul dim {list(self._shape)} {list(x.shape)}")
        ids32 = ids.to(torch.int32).contiguous()
        topk = ids32.shape[1]
        out = (torch.zeros if zero_init else torch.empty)((batch, topk, self._shape[1]), dtype=torch.float32, device=x.device)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        with torch.cuda.device(x.device):
            capi.hcheck(capi.lib().cqh_indexed_moe_forward(self._h, x.data_ptr(), x_dim1, ids32.data_ptr(), batch, topk,
                                                            out.data_ptr(), stream))
        return out

    def indexed_moe_forward_q8_1(self, act: torch.Tensor, x_dim1: int, ids: torch.Tensor, zero_init: bool = False) -> torch.Tensor:
        """`indexed_moe_forward` from activations a fused producer already stored as Q8_1 containers: `act` uint8
        [batch * x_dim1, pad(k, 512) / 32 * 36].  No quantize launch; f32 [batch, topk, n]."""
        if self.rank() != 3:
            raise CandleQError("indexed_moe_forward expects a rank-3 [experts, n, k] tensor")
        k = self._shape[2]
        row_bytes = capi.pad(k, 512) // 32 * 36
        ids32 = ids.to(torch.int32).contiguous()
        batch, topk = ids32.shape
        if not act.is_cuda or act.dtype != torch.uint8 or not act.is_contiguous() or tuple(act.shape) != (batch * x_dim1, row_bytes):
            raise CandleQError(f"indexed_moe_forward_q8_1 expects a contiguous uint8 CUDA tensor [{batch * x_dim1}, {row_bytes}]")
        out = (torch.zeros if zero_init else torch.empty)((batch, topk, self._shape[1]), dtype=torch.float32, device=act.device)
        stream = torch.cuda.current_stream(act.device).cuda_stream
        with torch.cuda.device(act.device):
            capi.hcheck(capi.lib().cqh_indexed_moe_forward_q8_1(self._h, act.data_ptr(), x_dim1, ids32.data_ptr(), batch, topk,
                                                                 out.data_ptr(), stream))
        return out

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """``QTensor::dequantize`` / ``dequantize_f16`` (mod.rs:689-710): the tensor as f32 (f16, bf16) on its device."""
        if dtype not in _ELEM:
            raise CandleQError(f"Expected f32/f16/bf16, got {dtype}")
        out = torch.empty(self._shape, dtype=dtype, device=self._device)
        stream = torch.cuda.current_stream(self._device).cuda_stream
        with torch.cuda.device(self._device):
            capi.hcheck(capi.lib().cqh_qtensor_dequantize(self._h, out.data_ptr(), _ELEM[dtype], stream), "QTensor.dequantize")
        return out

    def embedding(self, ids: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """``QTensor::embedding`` (mod.rs:712-748): rows `ids` of a [rows, hidden] tensor -> [*ids.shape, hidden]."""
        if self.rank() != 2:
            raise CandleQError("embedding expects a rank-2 [rows, hidden] quantized tensor")
        flat = ids.to(device=self._device, dtype=torch.int64).reshape(-1)
        if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= self._shape[0]):
            bad = int(flat[(flat < 0) | (flat >= self._shape[0])][0])
            raise CandleQError(f"embedding id {bad} is out of range for {self._shape[0]} rows")
        ids32 = flat.to(torch.int32).contiguous()
        out = torch.empty((*ids.shape, self._shape[1]), dtype=dtype, device=self._device)
        stream = torch.cuda.current_stream(self._device).cuda_stream
        with torch.cuda.device(self._device):
            capi.hcheck(capi.lib().cqh_qtensor_embedding(self._h, ids32.data_ptr(), ids32.numel(), out.data_ptr(), _ELEM[dtype], stream),
                        "QTensor.embedding")
        return out

    def matmul_t(self, xs: torch.Tensor) -> torch.Tensor:
        """xs @ self.T, as candle-pyo3's ``QTensor.matmul_t``."""
        return QMatMul.from_qtensor(self).forward(xs)


def _env_switch(name: str) -> bool:
    """The reference's reading of its switches (mod.rs:814-834): set, not empty and not "0"."""
    import os
    v = os.environ.get(name)
    return v is not None and v != "" and v != "0"


class QMatMul:
    """y = x . W^T.  The three variants of the reference's ``QMatMul`` enum (mod.rs:807-852, 1020-1043):

    * ``kind == "QTensor"``   - W stays quantized and the product runs in this library's kernels;
    * ``kind == "Tensor"``    - W de-quantized to a dense f32 tensor: always for GGUF tensors stored as F32 / F16 / BF16
      (norm vectors, sometimes whole matrices), and for every tensor when ``CANDLE_DEQUANTIZE_ALL`` is set;
    * ``kind == "TensorF16"`` - W de-quantized to f16 when ``CANDLE_DEQUANTIZE_ALL_F16`` is set; inputs are cast to f16
      for the product and the result back to the input type.

    The two dense variants multiply with the tensor library's GEMM, as the reference does with its own."""

    def __init__(self, qtensor: QTensor, _dense: torch.Tensor | None = None, _kind: str = "QTensor"):
        if qtensor.rank() != 2 and _dense is None:
            raise CandleQError("QMatMul expects a rank-2 quantized tensor")
        self.qtensor = qtensor
        self.dense = _dense
        self.kind = _kind

    @classmethod
    def from_qtensor(cls, qtensor: QTensor) -> "QMatMul":
        """``QMatMul::from_arc`` (mod.rs:837-852); the switches are read at every call, not cached per thread."""
        plain = qtensor.dtype in (GgmlDType.F32, GgmlDType.F16, GgmlDType.BF16)
        if plain or _env_switch("CANDLE_DEQUANTIZE_ALL"):
            return cls(qtensor, qtensor.dequantize(torch.float32), "Tensor")
        if _env_switch("CANDLE_DEQUANTIZE_ALL_F16"):
            return cls(qtensor, qtensor.dequantize(torch.float16), "TensorF16")
        return cls(qtensor)

    def dequantize_f16(self) -> torch.Tensor:
        """``QMatMul::dequantize_f16`` (mod.rs:858-864)."""
        if self.kind == "QTensor":
            return self.qtensor.dequantize(torch.float16)
        return self.dense.to(torch.float16)

    def _forward_dense(self, xs: torch.Tensor, out: torch.Tensor | None) -> torch.Tensor:
        w = self.dense
        if self.kind == "TensorF16":
            y = torch.matmul(xs.to(torch.float16), w.t()).to(xs.dtype)
        else:
            y = torch.matmul(xs, w.t().to(xs.dtype) if w.dtype != xs.dtype else w.t())
        if out is not None:
            out.copy_(y)
            return out
        return y

    def forward(self, xs: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if not xs.is_cuda:
            raise CandleQError("QMatMul.forward needs a CUDA tensor: this build has no CPU path")
        if xs.dtype not in _ELEM:
            raise CandleQError(f"Expected f32/f16/bf16, got {xs.dtype}")
        if self.kind != "QTensor":
            return self._forward_dense(xs, out)
        if not xs.is_contiguous():
            raise CandleQError("input tensor is not contiguous")
        n = self.qtensor.shape[0]
        if out is None:
            out = torch.empty((*xs.shape[:-1], n), dtype=xs.dtype, device=xs.device)
        dims, nd = _dims(xs.shape)
        stream = torch.cuda.current_stream(xs.device).cuda_stream
        with torch.cuda.device(xs.device):
            capi.hcheck(capi.lib().cqh_qmatmul_forward(self.qtensor._h, xs.data_ptr(), _ELEM[xs.dtype], dims, nd,
                                                        out.data_ptr(), stream))
        return out

    def forward_host(self, xs: torch.Tensor, out: torch.Tensor, stream: int | None = None) -> torch.Tensor:
        """x . W^T for activations and results in HOST memory (pinned for asynchronous copies): upload, multiply and
        copy back in one library call; the copy-back overlaps the next call.  Call `host_flush()` and synchronise the
        stream before reading `out`."""
        if self.kind != "QTensor":
            raise CandleQError("forward_host needs the quantized variant")
        if xs.is_cuda or out.is_cuda or xs.dtype not in _ELEM or out.dtype != xs.dtype:
            raise CandleQError("forward_host takes CPU tensors of one f32 / f16 / bf16 type")
        if not xs.is_contiguous() or not out.is_contiguous():
            raise CandleQError("input tensor is not contiguous")
        n = self.qtensor.shape[0]
        if tuple(out.shape) != (*xs.shape[:-1], n):
            raise CandleQError(f"forward_host: output shape {tuple(out.shape)} does not match {(*xs.shape[:-1], n)}")
        dims, nd = _dims(xs.shape)
        dev = self.qtensor.device
        st = torch.cuda.current_stream(dev).cuda_stream if stream is None else stream
        with torch.cuda.device(dev):
            capi.hcheck(capi.lib().cqh_qmatmul_forward_host(self.qtensor._h, xs.data_ptr(), _ELEM[xs.dtype], dims, nd, out.data_ptr(), st))
        return out

    def host_flush(self, stream: int | None = None) -> None:
        """Make the stream wait for every copy-back of `forward_host` still in flight on this tensor's device."""
        dev = self.qtensor.device
        st = torch.cuda.current_stream(dev).cuda_stream if stream is None else stream
        capi.hcheck(capi.lib().cqh_qmatmul_host_flush(dev.index or 0, st))

    def forward_q8_1(self, act: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """The GEMV alone: `act` holds Q8_1 containers, uint8 [rows, pad(k, 512) / 32 * 36], made by a fused producer
        (or the stand-alone quantizer).  Returns f32 [rows, n]."""
        k = self.qtensor.shape[1]
        row_bytes = capi.pad(k, 512) // 32 * 36
        if not act.is_cuda or act.dtype != torch.uint8 or not act.is_contiguous() or act.dim() != 2 or act.shape[1] != row_bytes:
            raise CandleQError(f"forward_q8_1 expects a contiguous uint8 CUDA tensor [rows, {row_bytes}]")
        rows, n = act.shape[0], self.qtensor.shape[0]
        if out is None:
            out = torch.empty((rows, n), dtype=torch.float32, device=act.device)
        stream = torch.cuda.current_stream(act.device).cuda_stream
        with torch.cuda.device(act.device):
            capi.hcheck(capi.lib().cqh_qmatmul_forward_q8_1(self.qtensor._h, act.data_ptr(), rows, out.data_ptr(), stream))
        return out

    def forward_q8_1_pair(self, other: "QMatMul", act: torch.Tensor):
        """`self` and `other` applied to the same Q8_1 containers; one launch when a single row meets a (Q4_K, Q6_K)
        pair of equal K, two otherwise.  Returns (f32 [rows, n_self], f32 [rows, n_other])."""
        rows = act.shape[0]
        if not act.is_cuda or act.dtype != torch.uint8 or not act.is_contiguous() or act.dim() != 2:
            raise CandleQError("forward_q8_1_pair expects a contiguous uint8 CUDA tensor of Q8_1 containers")
        out_a = torch.empty((rows, self.qtensor.shape[0]), dtype=torch.float32, device=act.device)
        out_b = torch.empty((rows, other.qtensor.shape[0]), dtype=torch.float32, device=act.device)
        stream = torch.cuda.current_stream(act.device).cuda_stream
        with torch.cuda.device(act.device):
            capi.hcheck(capi.lib().cqh_qmatmul_forward_q8_1_pair(self.qtensor._h, other.qtensor._h, act.data_ptr(), rows,
                                                                 out_a.data_ptr(), out_b.data_ptr(), stream))
        return out_a, out_b

    __call__ = forward
