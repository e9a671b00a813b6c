"""ctypes binding of libcandle_q_b200.so (the C ABI declared in include/candle_q_b200.h).

Loading fails loudly when the shared library has not been built: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libcandle_q_b200.so")

# GGML type ids / element kinds / activation encodings (include/candle_q_b200.h)
Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 2, 3, 6, 7, 8, 10, 11, 12, 13, 14
F32, F16, BF16 = 0, 1, 2
ACT_Q8_1, ACT_Q8_0, ACT_Q8_K = 0, 1, 2
MAX_PEERS = 8      # CQ_MAX_PEERS

TYPE_SIZE = {Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34, Q2_K: 84, Q3_K: 110, Q4_K: 144, Q5_K: 176, Q6_K: 210}
BLOCK_ELEMS = {Q4_0: 32, Q4_1: 32, Q5_0: 32, Q5_1: 32, Q8_0: 32, Q2_K: 256, Q3_K: 256, Q4_K: 256, Q5_K: 256, Q6_K: 256}
TYPE_NAME = {Q4_0: "q4_0", Q4_1: "q4_1", Q5_0: "q5_0", Q5_1: "q5_1", Q8_0: "q8_0", Q2_K: "q2_k", Q3_K: "q3_k", Q4_K: "q4_k", Q5_K: "q5_k", Q6_K: "q6_k"}
ELEM_NAME = {F32: "f32", F16: "f16", BF16: "bf16"}

STATUS = {0: "ok", 1: "bad argument", 2: "unsupported", 3: "CUDA error", 4: "device-side timeout"}


class CandleQError(RuntimeError):
    pass


_lib = None


def lib() -> C.CDLL:
    """The loaded shared library.  Raises if it is missing (build it with candle_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CandleQError(
                f"{LIB_PATH} is missing: build it with `python -m candle_b200.build` "
                "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for this path.")
        L = C.CDLL(LIB_PATH)
        vp, i32 = C.c_void_p, C.c_int
        L.cq_last_status.restype = i32
        L.cq_last_cuda_error.restype = i32
        L.cq_last_message.restype = C.c_char_p
        L.cq_version.restype = C.c_char_p
        L.cq_quantize_act.argtypes = [vp, i32, vp, i32, i32, i32, i32, vp]
        L.cq_mmvq.argtypes = [i32, i32, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        L.cq_block_dots.argtypes = [i32, i32, vp, vp, vp, vp, i32, i32, vp]
        L.cq_mmvq_plan.argtypes = [i32, i32, i32, i32, i32, C.POINTER(i32)]
        L.cq_mmvq_plan.restype = i32
        L.cq_device_timeout_flag.restype = i32
        L.cq_prefill_scratch_bytes.argtypes = [i32, i32]
        L.cq_prefill_scratch_bytes.restype = C.c_size_t
        L.cq_prefill_quantize.argtypes = [vp, i32, vp, i32, i32, vp]
        L.cq_prefill_gemm.argtypes = [i32, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        L.cq_prefill_timeout_flag.restype = i32
        L.cq_prefill32_scratch_bytes.argtypes = [i32, i32]
        L.cq_prefill32_scratch_bytes.restype = C.c_size_t
        L.cq_prefill32_quantize.argtypes = [vp, i32, vp, i32, i32, vp]
        L.cq_prefill32_gemm.argtypes = [i32, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        L.cq_prefill32_timeout_flag.restype = i32
        i64 = C.c_int64
        L.moe_gemm_gguf.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64]
        L.moe_gemm_gguf_prefill.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i64]
        L.cq_moe_gemv_sorted.argtypes = [i32, i32, vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        L.cq_indexed_moe_forward.argtypes = [i32, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp]
        L.cq_moe_timeout_flag.restype = i32
        L.cq_moe_prefill_scratch_bytes.argtypes = [i32, i32, i32]
        L.cq_moe_prefill_scratch_bytes.restype = C.c_size_t
        L.cq_moe_prefill_gemm.argtypes = [i32, vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        L.cq_mmq_timeout_flag.restype = i32
        for lay in ("D4", "DS4", "D2S6"):
            getattr(L, f"launch_mmq_quantize_q8_1_{lay}").argtypes = [vp, vp, vp, i32, i64, i64, i64, i64, i64, i64, i64, i64, vp]
        for t in TYPE_NAME.values():
            getattr(L, f"launch_mmq_gguf_{t}").argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i32, i32, i64, i32, vp]
        L.cq_attention_f32.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, C.c_float, i32, vp]
        L.cq_rms_norm_f32.argtypes = [vp, vp, vp, i32, i32, C.c_float, vp]
        L.cq_add_rms_norm_f32.argtypes = [vp, vp, vp, vp, i32, i32, C.c_float, vp]
        L.cq_rope_store_kv_f32.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp]
        L.cq_silu_mul_f32.argtypes = [vp, vp, i32, i32, vp]
        L.cq_peer_gather_words.argtypes = [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        L.cq_peer_gather_stage_bytes.argtypes = [i32, i32, i32]
        L.cq_peer_gather_stage_bytes.restype = C.c_size_t
        L.cq_peer_exchange_rows.argtypes = [vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, vp]
        L.cq_peer_exchange_rows.restype = None
        L.cq_peer_exchange_stage_bytes.argtypes = [i32, i32]
        L.cq_peer_exchange_stage_bytes.restype = C.c_size_t
        L.cq_peer_gather_set_limit_clocks.argtypes = [C.c_longlong]
        L.cq_peer_gather_timeout_flag.restype = i32
        L.cq_add_rms_norm_q8_1.argtypes = [vp, vp, vp, vp, i32, i32, i32, C.c_float, vp]
        L.cq_silu_mul_q8_1.argtypes = [vp, vp, i32, i32, i32, vp]
        L.cq_attention_q8_1.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, C.c_float, i32, i32, vp]
        L.cq_set_pdl.argtypes = [i32]
        L.cq_glue_position_overflow_flag.restype = i32
        L.cq_moe_route_f32.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
        L.cq_moe_router_f32.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        L.cq_moe_router_f32.restype = None
        L.cq_moe_weighted_sum_f32.argtypes = [vp, vp, vp, i32, i32, i32, vp]
        L.cq_moe_weighted_sum_f32.restype = None
        L.cq_qknorm_rope_store_kv_f32.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32,
                                                  C.c_float, i32, vp]
        L.cq_attention_split_scratch_floats.argtypes = [i32, i32, i32, i32]
        L.cq_attention_split_scratch_floats.restype = C.c_size_t
        L.cq_attention_split.argtypes = [vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, C.c_float, i32, i32, vp]
        L.cq_rope_attention_split.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, C.c_float,
                                              i32, i32, i32, i32, vp]
        L.cq_rope_attention_split.restype = None
        L.cq_set_mma_min_batch.argtypes = [i32]
        L.cq_set_mma_kernel.argtypes = [i32]
        L.cq_set_cluster_split.argtypes = [i32]
        L.cq_set_cluster_split.restype = None
        L.cq_qmatmul_decode_static.argtypes = [i32, vp, vp, i32, vp, i32, i32, i32, vp]
        for el in ELEM_NAME.values():
            getattr(L, f"launch_mmvq_gguf_quantize_q8_1_{el}").argtypes = [vp, vp, i32, i32, i32, vp]
            for t in TYPE_NAME.values():
                getattr(L, f"launch_mmvq_gguf_{t}_{el}_plain").argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp]
        i64p, sz = C.POINTER(C.c_int64), C.c_size_t
        L.cqh_last_error.restype = C.c_char_p
        L.cqh_qtensor_load.argtypes = [i32, vp, sz, i64p, i32, i32, C.POINTER(vp)]
        L.cqh_qtensor_wrap.argtypes = [i32, vp, sz, i64p, i32, i32, C.POINTER(vp)]
        L.cqh_quantize_f32.argtypes = [i32, vp, i64p, i32, vp, sz]
        L.cqh_qtensor_quantize_onto.argtypes = [i32, vp, i64p, i32, i32, C.POINTER(vp)]
        L.cqh_quantize_imatrix_f32.argtypes = [i32, vp, i64p, i32, vp, C.c_int64, vp, sz]
        L.cqh_qtensor_quantize_imatrix_onto.argtypes = [i32, vp, i64p, i32, vp, C.c_int64, i32, C.POINTER(vp)]
        L.cqh_qtensor_free.argtypes = [vp]
        L.cqh_qtensor_free.restype = None
        L.cqh_qtensor_data.argtypes = [vp, vp, sz]
        L.cqh_qtensor_device_ptr.argtypes = [vp]
        L.cqh_qtensor_device_ptr.restype = vp
        L.cqh_qmatmul_forward.argtypes = [vp, vp, i32, i64p, i32, vp, vp]
        L.cqh_qmatmul_forward_host.argtypes = [vp, vp, i32, i64p, i32, vp, vp]
        L.cqh_qmatmul_forward_host_sharded.argtypes = [vp, vp, i32, i64p, i32, vp, vp, vp, i32, i32, vp]
        L.cqh_qmatmul_host_flush.argtypes = [i32, vp]
        L.cqh_set_act_mode.argtypes = [i32]
        L.cqh_qtensor_dequantize.argtypes = [vp, vp, i32, vp]
        L.cqh_qtensor_embedding.argtypes = [vp, vp, i64, vp, i32, vp]
        L.cq_dequantize.argtypes = [i32, vp, vp, i32, i64, i64, vp]
        L.cq_get_rows.argtypes = [i32, vp, vp, vp, i32, i64, i64, i64, vp]
        L.cq_get_rows_bad_id.restype = i32
        L.cq_convert_plain.argtypes = [i32, vp, vp, i32, i64, vp]
        L.cqh_qmatmul_forward_q8_1.argtypes = [vp, vp, i32, vp, vp]
        L.cqh_qmatmul_forward_q8_1_pair.argtypes = [vp, vp, vp, i32, vp, vp, vp]
        L.cq_mmvq_pair_q4k_q6k.argtypes = [vp, i32, vp, vp, i32, vp, vp, i32, i32, vp]
        L.cq_mmvq_pair_q4k_q6k.restype = i32
        L.cqh_indexed_moe_forward.argtypes = [vp, vp, i32, vp, i32, i32, vp, vp]
        L.cqh_indexed_moe_forward_q8_1.argtypes = [vp, vp, i32, vp, i32, i32, vp, vp]
        L.cq_add_rms_norm_f32_q8_1.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, C.c_float, vp]
        L.cq_add_rms_norm_f32_q8_1.restype = None
        L.cqh_get_act_mode.restype = i32
        L.cqh_workspace_reserve.argtypes = [i32, sz]
        u64 = C.c_uint64
        L.cqh_gguf_last_error.restype = C.c_char_p
        L.cqh_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.cqh_gguf_close.argtypes = [vp]
        L.cqh_gguf_close.restype = None
        L.cqh_gguf_version.argtypes = [vp]
        L.cqh_gguf_tensor_data_offset.argtypes = [vp]
        L.cqh_gguf_tensor_data_offset.restype = u64
        L.cqh_gguf_tensor_count.argtypes = [vp]
        L.cqh_gguf_tensor_count.restype = i64
        L.cqh_gguf_metadata_json.argtypes = [vp]
        L.cqh_gguf_metadata_json.restype = C.c_char_p
        L.cqh_gguf_find_tensor.argtypes = [vp, C.c_char_p]
        L.cqh_gguf_find_tensor.restype = i64
        L.cqh_gguf_tensor_info.argtypes = [vp, i64, C.POINTER(C.c_char_p), C.POINTER(i32), i64p, C.POINTER(i32), C.POINTER(u64),
                                           C.POINTER(u64)]
        L.cqh_gguf_read_tensor.argtypes = [vp, i64, vp, u64]
        L.cqh_gguf_load_tensor.argtypes = [vp, i64, i32, i64, i64, C.POINTER(vp)]
        _lib = L
    return _lib


def hcheck(rc: int, what: str = "") -> None:
    """Raise the error text of a failed cqh_* call."""
    if rc != 0:
        raise CandleQError(f"{what}: {lib().cqh_last_error().decode()}" if what else lib().cqh_last_error().decode())


def check(what: str = "") -> None:
    """Raise if the library recorded a failure since the last clear."""
    L = lib()
    st = L.cq_last_status()
    if st != 0:
        msg = L.cq_last_message().decode()
        L.cq_clear_status()
        raise CandleQError(f"{what}: {STATUS.get(st, st)}: {msg}")


def pad(p: int, q: int) -> int:
    return (p + q - 1) // q * q
