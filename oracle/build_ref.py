"""Build the reference's own CUDA kernels for this path, unmodified, for sm_100a - test and benchmark infrastructure only.

candle's quantized GEMV (candle-kernels/src/mmvq_gguf.cu) and its tiled int8 prompt GEMM (candle-kernels/src/mmq_gguf/
mmq_quantize.cu + the per-format instance files) are self-contained CUDA sources with `extern "C"` launchers - the very
symbols candle-kernels/src/ffi.rs binds.  They are compiled where they lie in the reference checkout (nothing is copied)
into shared libraries under oracle/_ref/, which is ignored by git and travels with the built libraries:

    oracle/_ref/libcandle_ref_mmvq.so   launch_mmvq_gguf_*_plain, launch_mmvq_gguf_quantize_q8_1_*
    oracle/_ref/libcandle_ref_mmq.so    launch_mmq_quantize_q8_1_*, launch_mmq_gguf_* (the ten GGUF block formats)
    oracle/_ref/libcandle_ref_moe.so    moe_gemm_gguf, moe_gemm_gguf_prefill (candle-kernels/src/moe/moe_gguf.cu, moe_wmma_gguf.cu)

tests/test_gpu_reference_kernels.py compares this library's kernels and the oracle with them on the same GPU; bench.py
times them beside its own numbers (`reference_cuda`).  Nothing in the product loads them.

    python oracle/build_ref.py [path of the candle checkout]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MMVQ = os.path.join(OUT, "libcandle_ref_mmvq.so")
MMQ = os.path.join(OUT, "libcandle_ref_mmq.so")
MOE = os.path.join(OUT, "libcandle_ref_moe.so")
MMQ_FORMATS = ("q4_0", "q4_1", "q5_0", "q5_1", "q8_0", "q2_k", "q3_k", "q4_k", "q5_k", "q6_k")


_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-Xcompiler", "-fPIC"]


def _nvcc(out: str, sources: list[str], verbose: bool) -> None:
    """One shared library from `sources`; several sources are compiled side by side (the per-format MMQ instances take
    most of a minute each), then linked."""
    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)

    if len(sources) == 1:
        run(["nvcc"] + _FLAGS + ["-shared", "-o", out] + sources)
        return
    import concurrent.futures
    import tempfile
    with tempfile.TemporaryDirectory(dir=OUT) as tmp:
        objs = [os.path.join(tmp, os.path.splitext(os.path.basename(s))[0] + ".o") for s in sources]
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 1)) as pool:
            list(pool.map(lambda so: run(["nvcc"] + _FLAGS + ["-c", "-o", so[1], so[0]]), zip(sources, objs)))
        run(["nvcc"] + _FLAGS + ["-shared", "-o", out] + objs)


def build(reference_root: str, verbose: bool = False, force: bool = False) -> list[str]:
    """Compiles what is missing (or everything with `force`); returns the libraries that exist afterwards."""
    src = os.path.join(reference_root, "candle-kernels", "src")
    if not os.path.isfile(os.path.join(src, "mmvq_gguf.cu")):
        raise FileNotFoundError(f"no candle-kernels/src/mmvq_gguf.cu under {reference_root}")
    os.makedirs(OUT, exist_ok=True)
    if force or not os.path.isfile(MMVQ):
        _nvcc(MMVQ, [os.path.join(src, "mmvq_gguf.cu")], verbose)
    if force or not os.path.isfile(MMQ):
        mmq = os.path.join(src, "mmq_gguf")
        _nvcc(MMQ, [os.path.join(mmq, "mmq_quantize.cu")] + [os.path.join(mmq, f"mmq_instance_{f}.cu") for f in MMQ_FORMATS], verbose)
    if force or not os.path.isfile(MOE):
        moe = os.path.join(src, "moe")
        _nvcc(MOE, [os.path.join(moe, "moe_gguf.cu"), os.path.join(moe, "moe_wmma_gguf.cu")], verbose)
    return [p for p in (MMVQ, MMQ, MOE) if os.path.isfile(p)]


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CANDLE_REFERENCE_ROOT", "")
    if not root:
        raise SystemExit("usage: python oracle/build_ref.py <path of the candle checkout>")
    for lib in build(root, verbose=True, force="--force" in sys.argv):
        print("built", lib)
