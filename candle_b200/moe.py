"""``moe_gemm_gguf`` as in candle-nn/src/moe.rs:169-337: grouped expert GEMV over sorted (token, expert) pairs.

    gate = moe_gemm_gguf(xs, gate_experts, None, sorted_token_ids, expert_ids, topk, is_prefill)
    down = moe_gemm_gguf(h,  down_experts, topk_weights, sorted_token_ids, expert_ids, topk, is_prefill)

`weights` is a rank-3 QTensor [experts, n, k].  Decode calls take f32 activations, prefill calls f16 / bf16
(the reference casts before its prefill kernel, moe.rs:310-333); the output is always f32 [pairs, n].
"""
from __future__ import annotations

import torch

from . import capi
from .capi import CandleQError
from .quantized import GgmlDType, QTensor

# gguf_dtype codes of candle-kernels/src/ffi.rs:36
_CODE = {GgmlDType.Q8_0: 0, GgmlDType.Q4K: 1, GgmlDType.Q2K: 2, GgmlDType.Q3K: 3, GgmlDType.Q5K: 4, GgmlDType.Q6K: 5}


def moe_gemm_gguf(xs: torch.Tensor, weights: QTensor, topk_weights: torch.Tensor | None, sorted_token_ids: torch.Tensor,
                  expert_ids: torch.Tensor, topk: int, is_prefill: bool = False, zero_init: bool = False) -> torch.Tensor:
    """zero_init: start from a zeroed output (pairs whose expert id is out of range are skipped and would otherwise
    be left uninitialised) - what an expert-parallel rank needs before the pair outputs are summed across ranks."""
    if weights.rank() != 3:
        raise CandleQError("moe_gemm_gguf expects expert weights of rank 3 [experts, n, k]")
    if weights.dtype not in _CODE:
        raise CandleQError(f"moe_gemm_gguf: unsupported quantized dtype {weights.dtype.name}")
    num_experts, n, k = weights.shape
    if xs.dim() != 2 or xs.shape[1] != k or not xs.is_cuda or not xs.is_contiguous():
        raise CandleQError(f"moe_gemm_gguf: input must be a contiguous CUDA matrix [rows, {k}]")
    size_m = sorted_token_ids.numel()
    rows_in = xs.shape[0]
    if topk_weights is None and rows_in * topk != size_m or topk_weights is not None and rows_in != size_m:
        raise CandleQError("moe_gemm_gguf: input rows do not match the number of (token, expert) pairs")
    sti = sorted_token_ids.to(torch.int32).contiguous()
    eid = expert_ids.to(torch.int32).contiguous()
    tw = None if topk_weights is None else topk_weights.to(torch.float32).contiguous().view(-1)
    out = (torch.zeros if zero_init else torch.empty)((size_m, n), dtype=torch.float32, device=xs.device)
    L = capi.lib()
    stream = torch.cuda.current_stream(xs.device).cuda_stream
    with torch.cuda.device(xs.device):
        if is_prefill:
            if xs.dtype not in (torch.float16, torch.bfloat16):
                raise CandleQError("moe_gemm_gguf prefill takes f16 or bf16 activations")
            L.moe_gemm_gguf_prefill(xs.data_ptr(), weights.device_ptr(), sti.data_ptr(), eid.data_ptr(),
                                    tw.data_ptr() if tw is not None else None, out.data_ptr(), num_experts, topk, size_m, n, k,
                                    0 if xs.dtype == torch.float16 else 1, _CODE[weights.dtype], stream)
        else:
            if xs.dtype != torch.float32:
                raise CandleQError("moe_gemm_gguf decode takes f32 activations")
            L.moe_gemm_gguf(xs.data_ptr(), weights.device_ptr(), sti.data_ptr(), eid.data_ptr(),
                            tw.data_ptr() if tw is not None else None, out.data_ptr(), num_experts, topk, size_m, n, k,
                            _CODE[weights.dtype], stream)
    capi.check("moe_gemm_gguf")
    return out


def moe_prefill_gemm(xs: torch.Tensor, weights: QTensor, topk_weights: torch.Tensor | None, sorted_token_ids: torch.Tensor,
                     expert_ids: torch.Tensor, topk: int, zero_init: bool = False) -> torch.Tensor:
    """The grouped tensor-core GEMM (``cq_moe_prefill_gemm``) with the argument meaning of ``moe_gemm_gguf``; xs may be f32,
    f16 or bf16.  Q4_K / Q6_K experts only."""
    if weights.rank() != 3 or weights.dtype not in (GgmlDType.Q4K, GgmlDType.Q6K):
        raise CandleQError("moe_prefill_gemm expects Q4K or Q6K expert weights of rank 3 [experts, n, k]")
    num_experts, n, k = weights.shape
    if xs.dim() != 2 or xs.shape[1] != k or not xs.is_cuda or not xs.is_contiguous():
        raise CandleQError(f"moe_prefill_gemm: input must be a contiguous CUDA matrix [rows, {k}]")
    elem = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}.get(xs.dtype)
    if elem is None:
        raise CandleQError(f"Expected f32/f16/bf16, got {xs.dtype}")
    size_m = sorted_token_ids.numel()
    if topk_weights is None and xs.shape[0] * topk != size_m or topk_weights is not None and xs.shape[0] != size_m:
        raise CandleQError("moe_prefill_gemm: input rows do not match the number of (token, expert) pairs")
    sti, eid = sorted_token_ids.to(torch.int32).contiguous(), expert_ids.to(torch.int32).contiguous()
    tw = None if topk_weights is None else topk_weights.to(torch.float32).contiguous().view(-1)
    out = (torch.zeros if zero_init else torch.empty)((size_m, n), dtype=torch.float32, device=xs.device)
    L = capi.lib()
    scratch = torch.empty(L.cq_moe_prefill_scratch_bytes(size_m, num_experts, k), dtype=torch.uint8, device=xs.device)
    with torch.cuda.device(xs.device):
        L.cq_moe_prefill_gemm(int(weights.dtype), xs.data_ptr(), elem, weights.device_ptr(), sti.data_ptr(), eid.data_ptr(),
                              tw.data_ptr() if tw is not None else None, out.data_ptr(), scratch.data_ptr(), num_experts, topk, size_m,
                              n, k, torch.cuda.current_stream(xs.device).cuda_stream)
    capi.check("moe_prefill_gemm")
    return out
