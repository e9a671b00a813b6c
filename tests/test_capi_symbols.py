"""The C-ABI library loads on a CPU-only box and exports every function include/*.h declares."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        src = open(h).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        src = re.sub(r"#define CQ_DECL_\w+\(name\).*?\n(?:.*\\\n)*.*\n", "", src)
        for m in re.finditer(r"CQ_DECL_\w+\((\w+)\);", src):
            names.add(m.group(1))
        for m in re.finditer(r"^\s*(?:const\s+)?(?:void|int|char|size_t|int64_t|uint64_t)\s*\*?\s*(\w+)\s*\(", src, flags=re.M):
            names.add(m.group(1))
    return sorted(names)


def test_header_declares_the_reference_symbols():
    names = declared_functions()
    for t in ("q4_0", "q4_1", "q5_0", "q5_1", "q8_0", "q2_k", "q3_k", "q4_k", "q5_k", "q6_k"):
        for e in ("f32", "f16", "bf16"):
            assert f"launch_mmvq_gguf_{t}_{e}_plain" in names     # candle-kernels/src/ffi.rs:61-393
    for e in ("f32", "f16", "bf16"):
        assert f"launch_mmvq_gguf_quantize_q8_1_{e}" in names     # candle-kernels/src/ffi.rs:396-419
    for lay in ("D4", "DS4", "D2S6"):
        assert f"launch_mmq_quantize_q8_1_{lay}" in names         # candle-kernels/src/ffi.rs:424-468
    for t in ("q4_0", "q4_1", "q5_0", "q5_1", "q8_0", "q2_k", "q3_k", "q4_k", "q5_k", "q6_k"):
        assert f"launch_mmq_gguf_{t}" in names                    # candle-kernels/src/ffi.rs:471-630
    assert "moe_gemm_gguf" in names and "moe_gemm_gguf_prefill" in names      # candle-kernels/src/ffi.rs:25-56


def test_library_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_status_channel_without_gpu(lib):
    lib.cq_clear_status()
    assert lib.cq_last_status() == 0
    # argument validation happens before any CUDA call: null pointers are rejected, nothing is launched
    lib.cq_mmvq(12, 0, 0, None, None, None, 256, 4, 16, 4, 1, None)
    assert lib.cq_last_status() == 1
    assert b"null" in lib.cq_last_message()
    lib.cq_clear_status()
    lib.launch_mmvq_gguf_quantize_q8_1_f32(None, None, 256, 512, 1, None)
    assert lib.cq_last_status() == 1
    lib.cq_clear_status()
    assert lib.cq_version().startswith(b"candle_q_b200")
