#!/usr/bin/env python
"""Benchmark of the quantized-matmul decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("gemv_sweep_llama3_8b"): one step is one pass over the Llama-3-8B
projection shapes (K->N: 4096->4096, 4096->1024, 4096->14336, 14336->4096, 4096->128256) x {Q4_K, Q6_K,
Q8_0} x batch {1, 2, 4, 8}: 60 activation-quantize + GEMV pairs.  Weights are seeded synthetic GGUF blocks
(candle_b200/synth.py), activations N(0, 1).

Metric: achieved HBM bandwidth in GB/s = algorithmic bytes of the step (weights once + f32 activations in +
f32 outputs, per GEMV) / device time of the step.
  value     : inputs resident in HBM, the step replayed as one CUDA graph, CUDA-event timed.
  e2e       : the same step through the host-buffer entry point (QMatMul.forward_host = cqh_qmatmul_forward_host):
              activations start in pinned host memory and results end in pinned host memory; upload, quantize, GEMV and
              copy-back are inside the timed region (with several GPUs: copy, QMatMul.forward, gather, copy).
  roofline  : the GEMV kernels alone (no quantize launches), CUDA-event timed in this run.
  cpu_baseline : the reference's CPU algorithm (oracle port, AVX2, host threads = physical cores) on the same sweep.
Further objects of the same JSON line (reported beside the headline, not part of `value`):
  sustained   : the same graph replayed for at least a second.
  gemv_cases  : GB/s of every (format, shape, batch) GEMV launch on its own (L2 flushed before each launch).
  int8_peak   : an int8 library GEMM 8192^3 measured in this process: the denominator of the prompt kernel's fraction.
  prefill     : prompt-phase GEMM, Q4_K 4096->14336 and 14336->4096, M = 128 .. 8192 tokens, f32 and bf16 inputs: useful
                TOP/s of the tcgen05 kernel, of the whole forward (quantize + GEMM), and of the reference's own two-call
                protocol (launch_mmq_quantize_q8_1_DS4 + launch_mmq_gguf_q4_k) served by this library.
  prefill_block_formats : the Q8_0 / Q4_0 prompt kernel at 2048 tokens on the same shapes, and the two-call protocol beside it.
  moe         : Qwen3-30B-A3B-shaped mixture-of-experts decoder (tokens/s) and the grouped expert GEMM (TOP/s).
  decode      : Llama-3-8B-shaped Q4_K_M decoder, tokens/s at batch 1 and 8.

With N > 1 GPUs (torchrun) every weight matrix is sharded by output rows over the ranks (column-parallel);
each rank runs its slice and the slices are all-gathered by one kernel over NVLink peer memory (csrc/peer_gather.cu).
Total work is fixed: "strong" scaling.

`--impl reference` times the reference's CPU implementation of the path (the oracle port) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096), (4096, 128256)]   # (K, N)
TYPE_NAMES = ["Q4K", "Q6K", "Q8_0"]
BATCHES = [1, 2, 4, 8]
BYTES_PER_ELEM = {"Q4K": 144 / 256, "Q6K": 210 / 256, "Q8_0": 34 / 32, "Q4_0": 18 / 32}
METRIC = "qmatmul_gemv_hbm_bandwidth"
UNIT = "GB/s"


def gemv_bytes(tname: str, k: int, n: int, b: int) -> float:
    """Algorithmic bytes of one GEMV: weights once, f32 activations in, f32 outputs out."""
    return n * k * BYTES_PER_ELEM[tname] + b * k * 4 + b * n * 4


# dram__bytes_read + dram__bytes_write over algorithmic bytes, one ncu-captured launch per (format, K, N, rows)
# (profiles/gemv_sweep_dram_traffic.md).  Batches 2 and 4 take the figure of batch 1 (same kernel family).
DRAM_TRAFFIC_RATIO = {
    ("Q4K", 4096, 4096, 1): 0.998,
    ("Q4K", 4096, 4096, 8): 0.979,
    ("Q4K", 4096, 1024, 1): 0.998,
    ("Q4K", 4096, 1024, 8): 0.958,
    ("Q4K", 4096, 14336, 1): 0.998,
    ("Q4K", 4096, 14336, 8): 0.984,
    ("Q4K", 14336, 4096, 1): 0.999,
    ("Q4K", 14336, 4096, 8): 0.987,
    ("Q4K", 4096, 128256, 1): 1.0,
    ("Q4K", 4096, 128256, 8): 0.994,
    ("Q6K", 4096, 4096, 1): 0.999,
    ("Q6K", 4096, 4096, 8): 0.986,
    ("Q6K", 4096, 1024, 1): 0.999,
    ("Q6K", 4096, 1024, 8): 0.973,
    ("Q6K", 4096, 14336, 1): 0.999,
    ("Q6K", 4096, 14336, 8): 0.989,
    ("Q6K", 14336, 4096, 1): 0.999,
    ("Q6K", 14336, 4096, 8): 0.991,
    ("Q6K", 4096, 128256, 1): 1.001,
    ("Q6K", 4096, 128256, 8): 1.024,
    ("Q8_0", 4096, 4096, 1): 0.999,
    ("Q8_0", 4096, 4096, 8): 0.988,
    ("Q8_0", 4096, 1024, 1): 0.999,
    ("Q8_0", 4096, 1024, 8): 0.975,
    ("Q8_0", 4096, 14336, 1): 0.999,
    ("Q8_0", 4096, 14336, 8): 0.992,
    ("Q8_0", 14336, 4096, 1): 0.999,
    ("Q8_0", 14336, 4096, 8): 0.993,
    ("Q8_0", 4096, 128256, 1): 1.0,
    ("Q8_0", 4096, 128256, 8): 0.998,
}


def step_traffic_bytes(world: int = 1) -> float:
    """DRAM bytes of one step and GPU from the measured per-launch ratios."""
    tot = 0.0
    for b in BATCHES:
        for t in TYPE_NAMES:
            for (k, n) in SHAPES:
                tot += gemv_bytes(t, k, n // world, b) * DRAM_TRAFFIC_RATIO[(t, k, n, 8 if b == 8 else 1)]
    return tot


def step_bytes(batches=BATCHES) -> float:
    return sum(gemv_bytes(t, k, n, b) for b in batches for t in TYPE_NAMES for (k, n) in SHAPES)


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.lines: list[str] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()      # the exact process started above
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        hi = [v for v in sm if v >= 0.5 * (mx[0] if mx else 0)] or sm
        return {"sm_mhz": hi[len(hi) // 2] if hi else None, "sm_max_mhz": mx[0] if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU algorithm (oracle port) on the host cores
# --------------------------------------------------------------------------------------------------
def host_cpu_info():
    """(model name, physical cores, logical cores) of the host, from /proc/cpuinfo."""
    model, phys, logical = "unknown", set(), 0
    try:
        pid = cid = None
        for ln in open("/proc/cpuinfo"):
            if ln.startswith("model name") and model == "unknown":
                model = ln.split(":", 1)[1].strip()
            elif ln.startswith("processor"):
                logical += 1
            elif ln.startswith("physical id"):
                pid = ln.split(":", 1)[1].strip()
            elif ln.startswith("core id"):
                cid = ln.split(":", 1)[1].strip()
                phys.add((pid, cid))
    except OSError:
        pass
    logical = logical or (os.cpu_count() or 1)
    return model, (len(phys) or logical), logical


def cpu_threads():
    """Threads of the CPU legs: the physical cores, the reference's default (candle-core/src/utils.rs:312-325)."""
    return max(1, host_cpu_info()[1])


def cpu_sample_setup(seed=0):
    """The CPU legs run the benchmark's own sweep: the fifteen full matrices (the 128256-row head included) at batch
    1, 2, 4 and 8 - the same config as the GPU arm.  Block bytes are random with plausible f16 scales (throughput does
    not depend on the values)."""
    import numpy as np
    from oracle import oracle as O
    rng = np.random.default_rng(seed)
    items = []
    for t in TYPE_NAMES:
        dt = getattr(O, t)
        for (k, n) in SHAPES:
            rb = O.row_bytes(dt, k)
            w = rng.integers(0, 256, size=(n, rb), dtype=np.uint8)
            blk = w.reshape(n * (k // O.BLOCK_SIZE[dt]), O.TYPE_SIZE[dt])
            for off in ({O.Q4K: (0, 2), O.Q6K: (208,), O.Q8_0: (0,)}[dt]):
                blk[:, off:off + 2] = np.full((blk.shape[0],), 1e-3, dtype=np.float16).view(np.uint8).reshape(-1, 2)
            xs = {b: rng.standard_normal((b, k)).astype(np.float32) for b in BATCHES}
            items.append((t, dt, k, n, w, xs))
    nbytes = sum(gemv_bytes(t, k, n, b) for (t, _, k, n, _, _) in items for b in BATCHES)
    return items, nbytes


def cpu_sample_run(items, nthreads):
    from oracle import oracle as O
    mode = O.SIMD_HW if O.lib().cqo_have_avx2() else O.SIMD_ORDER
    for b in BATCHES:
        for (_, dt, k, n, w, xs) in items:
            O.matmul(dt, xs[b], w, n, mode=mode, nthreads=nthreads)


SAMPLE_DESC = ("one full pass of the sweep: the 15 (type, shape) matrices at batch 1, 2, 4 and 8, full sizes; "
               "k_quants::matmul restated in C with AVX2 dots, one thread per physical core")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    items, nbytes = cpu_sample_setup()
    nthreads = cpu_threads()
    model, phys, logical = host_cpu_info()
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_sample_run(items, nthreads)
    steps = max(1, min(args.steps, 8))      # a pass takes about a second of CPU time: bound the run to a few minutes
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_sample_run(items, nthreads)
    dt = (time.perf_counter() - t0) / steps
    val = nbytes / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 dot products, f32 accumulation", "data": "synthetic",
        "config": {"workload": "gemv_sweep_llama3_8b", "types": TYPE_NAMES, "shapes_k_n": SHAPES, "batches": BATCHES},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": nthreads, "kind": "port", "sample": SAMPLE_DESC,
                         "cpu_model": model, "physical_cores": phys, "logical_cores": logical},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


class IsolatedTimer:
    """Time of one launch on its own: a CUDA graph of five {L2 flush (a 256 MB fill), launch} pairs minus a graph of the
    five flushes alone, best of three replays each.  Launch latency that a neighbour would hide in a stream is included."""

    def __init__(self, dev):
        import torch
        self.torch, self.dev = torch, dev
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.side = torch.cuda.Stream(device=dev)
        self.t_flush = self._graph_ms(lambda: None)

    def _graph_ms(self, launch):
        torch = self.torch

        def body():
            for i in range(5):
                self.flush.fill_(i)
                launch()
        with torch.cuda.stream(self.side):
            body()
            self.side.synchronize()
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gph, stream=self.side):
                body()
            best = float("inf")
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.side)
                gph.replay()
                e1.record(self.side)
                self.side.synchronize()
                best = min(best, e0.elapsed_time(e1))
        return best

    def ms(self, launch) -> float:
        return max((self._graph_ms(launch) - self.t_flush) / 5.0, 1e-4)


def token_hash(toks) -> str:
    """SHA-256 of the generated token ids (order-sensitive, unlike a sum)."""
    import hashlib
    import torch
    return hashlib.sha256(torch.stack(toks).to(torch.int64).cpu().numpy().tobytes()).hexdigest()[:16]


def measure_int8_peak(dev):
    """int8 x int8 -> int32 library GEMM 8192^3 (torch._int_mm, cuBLASLt) in this process: best of 10 launches and the
    mean of a 2 s back-to-back loop.  It is the denominator of the prompt kernel's fraction; 4500 TOP/s is the nominal
    dense int8 figure of the part."""
    import torch
    n = 8192
    try:
        a = torch.randint(-127, 127, (n, n), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 127, (n, n), dtype=torch.int8, device=dev).t()      # column-major right operand
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch._int_mm(a, b); e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(2000.0 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        sus = e0.elapsed_time(e1) / reps
        ops = 2.0 * n * n * n
        return {"burst_tops": ops / best / 1e9, "sustained_tops": ops / sus / 1e9, "nominal_tops": 4500.0,
                "how": "torch._int_mm int8 8192^3 (library GEMM): best of 10 launches; mean of a 2 s back-to-back loop"}
    except Exception as e:      # no int8 library GEMM in this build
        return {"burst_tops": None, "sustained_tops": None, "nominal_tops": 4500.0, "how": f"torch._int_mm unavailable: {e}"}


def _time_launches(fn, iters):
    """Mean CUDA-event time in ms of `iters` back-to-back calls of fn(i) after two warm-up calls."""
    import torch
    fn(0); fn(1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def measure_prefill(dev, rank, world, peak_tops):
    """Benchmark configuration 3 (prompt GEMM): Q4_K 4096->14336 and 14336->4096, M = 128, 512, 2048, 8192 tokens, f32 and bf16 activations;
    the output dimension is sharded over `world` ranks.  Per case the useful rate 2*M*N*K / t of (a) the tcgen05 GEMM
    alone, (b) QMatMul.forward (activation tiles + GEMM), (c) for f32: the reference's two-call protocol served by this
    library (launch_mmq_quantize_q8_1_DS4 + launch_mmq_gguf_q4_k).  Weights rotate through four copies so that
    consecutive launches do not find them in L2."""
    import torch
    import torch.distributed as dist
    from candle_b200 import capi
    from candle_b200.quantized import GgmlDType, QMatMul, QTensor
    from candle_b200.synth import random_blocks
    L = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    ref_mmq = _load_reference_mmq()
    out = []
    for (k, n) in ((4096, 14336), (14336, 4096)):
        n_l = n // world
        ws = [random_blocks(GgmlDType.Q4K, n_l, k, seed=7 + 10 * i + rank, device=dev) for i in range(4)]
        mms = [QMatMul.from_qtensor(QTensor.from_device_blocks(w, GgmlDType.Q4K, (n_l, k))) for w in ws]
        for m in (128, 512, 2048, 8192):
            ops = 2.0 * m * n * k          # whole job, all ranks
            iters = 20 if m <= 2048 else 8
            for tdt, ename, ecode in ((torch.float32, "f32", capi.F32), (torch.bfloat16, "bf16", capi.BF16)):
                x = torch.randn((m, k), device=dev, generator=torch.Generator(device=dev).manual_seed(m + k)).to(tdt)
                y = torch.empty((m, n_l), dtype=tdt, device=dev)
                scratch = torch.empty(L.cq_prefill_scratch_bytes(m, k), dtype=torch.uint8, device=dev)
                L.cq_prefill_quantize(x.data_ptr(), ecode, scratch.data_ptr(), k, m, st)
                t_gemm = _time_launches(lambda i: L.cq_prefill_gemm(12, ws[i % 4].data_ptr(), scratch.data_ptr(), y.data_ptr(), ecode,
                                                                     k, n_l, m, n_l, st), iters)
                t_fwd = _time_launches(lambda i: mms[i % 4].forward(x, out=y), iters)
                row = {"k": k, "n": n, "m": m, "in": ename, "gemm_ms": t_gemm, "forward_ms": t_fwd}
                if ename == "f32":      # the drop-in route: the reference's own scratch and entry points
                    kp = capi.pad(k, 512)
                    mmq_scratch = torch.empty(((kp // 128) * m + 128) * 144, dtype=torch.uint8, device=dev)
                    fixup = torch.empty(4 << 20, dtype=torch.float32, device=dev)
                    y32 = torch.empty((m, n_l), dtype=torch.float32, device=dev)

                    def dropin(i):
                        L.launch_mmq_quantize_q8_1_DS4(x.data_ptr(), None, mmq_scratch.data_ptr(), 0, k, k, 0, 0, kp, m, 1, 1, st)
                        L.launch_mmq_gguf_q4_k(fixup.data_ptr(), ws[i % 4].data_ptr(), mmq_scratch.data_ptr(), y32.data_ptr(), k, n_l, m,
                                               k // 256, n_l, 1000, 148, 232448, 32, st)
                    row["dropin_mmq_ms"] = _time_launches(dropin, 3 if m >= 2048 else 6)
                    if ref_mmq is not None and world == 1:      # the reference's tiled int8 mma.sync GEMM itself, same two calls
                        def reference_pair(i):
                            ref_mmq.launch_mmq_quantize_q8_1_DS4(x.data_ptr(), None, mmq_scratch.data_ptr(), 0, k, k, 0, 0, kp, m, 1, 1, st)
                            ref_mmq.launch_mmq_gguf_q4_k(fixup.data_ptr(), ws[i % 4].data_ptr(), mmq_scratch.data_ptr(), y32.data_ptr(), k, n_l, m,
                                                         k // 256, n_l, 1000, 148, 232448, 32, st)
                        row["reference_cuda_mmq_ms"] = _time_launches(reference_pair, 6)
                        row["reference_cuda_mmq_tops"] = ops / row["reference_cuda_mmq_ms"] / 1e9
                    del mmq_scratch, fixup, y32
                capi.check("prefill bench")
                t = torch.tensor([row["gemm_ms"], row["forward_ms"], row.get("dropin_mmq_ms", 0.0)], device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                row["gemm_ms"], row["forward_ms"] = float(t[0]), float(t[1])
                row["gemm_tops"] = ops / row["gemm_ms"] / 1e9
                row["forward_tops"] = ops / row["forward_ms"] / 1e9
                if "dropin_mmq_ms" in row:
                    row["dropin_mmq_ms"] = float(t[2])
                    row["dropin_mmq_tops"] = ops / row["dropin_mmq_ms"] / 1e9
                # what the tensor pipe executes: per 256-element super-block nine K = 32 steps of N = 128 (two operand planes
                # of 64 weight rows, plus the block-sums step) where four steps of one plane would be the useful product
                row["gemm_issued_tops"] = row["gemm_tops"] * 2.25
                if peak_tops:
                    row["gemm_frac_of_int8_peak"] = row["gemm_tops"] / (peak_tops * world)
                    row["gemm_issued_frac_of_int8_peak"] = row["gemm_issued_tops"] / (peak_tops * world)
                out.append(row)
                del x, y, scratch
        del ws, mms
        torch.cuda.empty_cache()
    assert L.cq_prefill_timeout_flag() == 0, "a prefill launch gave up a bounded wait"
    return out


def measure_prefill_block_formats(dev, peak_tops):
    """The prompt kernel of the 32-element block formats (Q8_0, Q4_0) on the same two shapes at 2048 tokens, f32 inputs:
    useful TOP/s of QMatMul.forward, and of the reference's two-call protocol (GEMV passes) beside it."""
    import torch
    from candle_b200 import capi
    from candle_b200.quantized import GgmlDType, QMatMul, QTensor
    from candle_b200.synth import random_blocks
    L = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    res = []
    m = 2048
    for tname, lay in (("Q8_0", "D4"), ("Q4_0", "DS4")):
        for (k, n) in ((4096, 14336), (14336, 4096)):
            ws = [random_blocks(GgmlDType[tname], n, k, seed=3 + i, device=dev) for i in range(3)]
            mms = [QMatMul.from_qtensor(QTensor.from_device_blocks(w, GgmlDType[tname], (n, k))) for w in ws]
            x = torch.randn((m, k), device=dev)
            y = torch.empty((m, n), device=dev)
            t_fwd = _time_launches(lambda i: mms[i % 3].forward(x, out=y), 10)
            kp = capi.pad(k, 512)
            mmq_scratch = torch.empty(((kp // 128) * m + 128) * 144, dtype=torch.uint8, device=dev)
            fixup = torch.empty(4 << 20, dtype=torch.float32, device=dev)

            def dropin(i):
                getattr(L, f"launch_mmq_quantize_q8_1_{lay}")(x.data_ptr(), None, mmq_scratch.data_ptr(), 0, k, k, 0, 0, kp, m, 1, 1, st)
                getattr(L, f"launch_mmq_gguf_{tname.lower()}")(fixup.data_ptr(), ws[i % 3].data_ptr(), mmq_scratch.data_ptr(), y.data_ptr(), k, n, m,
                                                               k // 32, n, 1000, 148, 232448, 32, st)
            t_drop = _time_launches(dropin, 3)
            capi.check("block-format prefill bench")
            ops = 2.0 * m * n * k
            row = {"type": tname, "k": k, "n": n, "m": m, "forward_ms": t_fwd, "forward_tops": ops / t_fwd / 1e9, "dropin_mmq_ms": t_drop,
                   "dropin_mmq_tops": ops / t_drop / 1e9}
            if peak_tops:
                row["forward_frac_of_int8_peak"] = row["forward_tops"] / peak_tops
            res.append(row)
            del ws, mms, x, y, mmq_scratch, fixup
            torch.cuda.empty_cache()
    assert L.cq_prefill32_timeout_flag() == 0, "a block-format prefill launch gave up a bounded wait"
    return res


def measure_moe_gemm(dev):
    """The grouped expert GEMM at the Qwen3-30B-A3B shape: 1024 tokens x top-8 = 8192 (token, expert) pairs over 128
    Q4_K experts, gate|up (2048 -> 1536) and down (768 -> 2048); useful TOP/s = 2 * pairs * n * k / t."""
    import torch
    from candle_b200.moe import moe_prefill_gemm
    from candle_b200.quantized import GgmlDType, QTensor
    from candle_b200.synth import random_blocks
    tokens, topk, experts = 1024, 8, 128
    g = torch.Generator(device=dev).manual_seed(11)
    ids = torch.stack([torch.randperm(experts, device=dev, generator=g)[:topk] for _ in range(tokens)]).to(torch.int32)
    expert_ids, pairs = torch.sort(ids.reshape(-1), stable=True)
    res = []
    for name, n, k, per_pair in (("gate_up", 1536, 2048, False), ("down", 2048, 768, True)):
        w = QTensor.from_device_blocks(random_blocks(GgmlDType.Q4K, experts * n, k, seed=5, device=dev).reshape(-1), GgmlDType.Q4K,
                                       (experts, n, k))
        x = torch.randn((tokens * topk if per_pair else tokens, k), device=dev, generator=g)
        tw = torch.ones(tokens * topk, device=dev) if per_pair else None
        ms = _time_launches(lambda i: moe_prefill_gemm(x, w, tw, pairs, expert_ids, topk), 10)
        res.append({"matmul": name, "pairs": tokens * topk, "n": n, "k": k, "ms": ms, "useful_tops": 2.0 * tokens * topk * n * k / ms / 1e9})
        del w, x
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    from candle_b200 import capi
    from candle_b200.quantized import GgmlDType, QMatMul
    from candle_b200.synth import random_qtensor

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    L = capi.lib()

    # ---- resident inputs: each rank holds rows [rank*N/g, (rank+1)*N/g) of every matrix
    mats = {}
    for ti, t in enumerate(TYPE_NAMES):
        for si, (k, n) in enumerate(SHAPES):
            assert n % world == 0
            qt = random_qtensor(GgmlDType[t], n // world, k, seed=1000 * ti + 10 * si + rank, device=dev)
            mats[(t, k, n)] = QMatMul.from_qtensor(qt)
    xs = {(k, b): torch.randn((b, k), device=dev, generator=torch.Generator(device=dev).manual_seed(k + b))
          for (k, _) in SHAPES for b in BATCHES}
    outs = {(n, b): torch.empty((b, n // world), device=dev) for (_, n) in SHAPES for b in BATCHES}
    gather = None
    if world > 1:       # one kernel over NVLink peer memory per gather (falls back to the NCCL collective with CQ_PEER_GATHER=0)
        from candle_b200.parallel import make_gatherer
        gather = make_gatherer(None, world, dev)
    gather_kind = "peer-memory gather kernel" if type(gather).__name__ == "PeerGatherer" else "NCCL all-gather"
    order = [(b, t, k, n) for b in BATCHES for t in TYPE_NAMES for (k, n) in SHAPES]
    total_bytes = step_bytes()

    def step_full():
        for (b, t, k, n) in order:
            mats[(t, k, n)].forward(xs[(k, b)], out=outs[(n, b)])
            if world > 1:
                gather(outs[(n, b)])

    # pre-quantized activations for the GEMV-only (roofline) pass
    kp = {k: capi.pad(k, 512) for (k, _) in SHAPES}
    q8 = {}
    for (k, b), x in xs.items():
        y = torch.empty((b, kp[k] // 32 * 36), dtype=torch.uint8, device=dev)
        L.cq_quantize_act(x.data_ptr(), capi.F32, y.data_ptr(), k, kp[k], b, capi.ACT_Q8_1, torch.cuda.current_stream().cuda_stream)
        q8[(k, b)] = y
    capi.check("bench setup")

    def step_gemv_only():
        s = torch.cuda.current_stream().cuda_stream
        for (b, t, k, n) in order:
            L.cq_mmvq(int(GgmlDType[t]), capi.ACT_Q8_1, capi.F32, mats[(t, k, n)].qtensor.device_ptr(), q8[(k, b)].data_ptr(),
                      outs[(n, b)].data_ptr(), k, n // world, kp[k] // 32, n // world, b, s)

    def timed(fn, steps, warmup, use_graph):
        """CUDA-event time of `steps` calls of fn after `warmup` calls; barrier + synchronize on both sides."""
        side = torch.cuda.Stream(device=dev)
        graph = None
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 3)):
                fn()
            side.synchronize()
            if use_graph:
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        fn()
                    graph.replay()
                    side.synchronize()
                except Exception:       # capture refused (e.g. a collective that cannot be recorded): launch eagerly
                    graph = None
                    torch.cuda.synchronize()
        graphed.append(graph is not None)
        run = graph.replay if graph is not None else fn
        with torch.cuda.stream(side):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(steps):
                run()
            e1.record(side)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    use_graph = True           # the gathers of the sharded run are kernels of this library (or NCCL calls) and are recorded as well
    graphed = []
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(step_full, args.steps, args.warmup, use_graph)
    # the same step for at least a second (the K-step region above lasts tens of milliseconds): clocks are sampled here too
    sus_steps = max(args.steps, int(1100.0 / max(ms_step, 1e-3)) + 1)
    ms_sustained = timed(step_full, sus_steps, 1, use_graph)
    clocks = sampler.stop() if rank == 0 else None
    ms_gemv = timed(step_gemv_only, args.steps, args.warmup, use_graph)
    ms_gemv_sustained = timed(step_gemv_only, sus_steps, 1, use_graph)
    if gather is not None and hasattr(gather, "check"):
        gather.check()          # a gather that gave up its bounded wait would have timed garbage

    # ---- every GEMV launch on its own (IsolatedTimer: L2 flushed before each launch)
    timer = IsolatedTimer(dev)
    per_case = {}
    for (b, t, k, n) in order:
        def one(b=b, t=t, k=k, n=n):
            L.cq_mmvq(int(GgmlDType[t]), capi.ACT_Q8_1, capi.F32, mats[(t, k, n)].qtensor.device_ptr(), q8[(k, b)].data_ptr(),
                      outs[(n, b)].data_ptr(), k, n // world, kp[k] // 32, n // world, b, torch.cuda.current_stream().cuda_stream)
        per_case.setdefault(t, {}).setdefault(f"{k}x{n}", {})[str(b)] = round(gemv_bytes(t, k, n // world, b) / timer.ms(one) / 1e6, 1)
    del timer
    capi.check("per-case sweep")

    # ---- e2e: host activations -> device, QMatMul.forward, result -> host, all inside the timed region
    h_x = {key: x.cpu().pin_memory() for key, x in xs.items()}
    h_y = {key: torch.empty((key[1], key[0]), dtype=torch.float32).pin_memory() for key in
           {(n, b) for (_, n) in SHAPES for b in BATCHES}}
    d_x = {key: torch.empty_like(x) for key, x in xs.items()}
    h2d = sum(b * k * 4 for (b, _, k, _) in order)
    d2h = sum(b * n * 4 for (b, _, _, n) in order)

    host_fwd = None
    if world > 1:
        from candle_b200.parallel import ShardedHostForward
        host_fwd = ShardedHostForward(gather, dev)

    def step_e2e():
        if world == 1:      # host buffers in, host buffers out: one library call per matmul, copy-backs overlap the next call
            last = None
            for (b, t, k, n) in order:
                last = mats[(t, k, n)]
                last.forward_host(h_x[(k, b)], h_y[(n, b)])
            last.host_flush()
            return
        for (b, t, k, n) in order:      # several GPUs: the same overlap around the shard's product and the all-gather
            host_fwd(mats[(t, k, n)], h_x[(k, b)], h_y[(n, b)])
        host_fwd.flush()

    ms_e2e = timed(step_e2e, args.steps, args.warmup, False)
    if gather is not None and hasattr(gather, "check"):
        gather.check()

    # ---- the reference's own CUDA kernels on this GPU (oracle/build_ref.py), the same step: quantize + `_plain` GEMV
    reference_cuda = None
    ref_lib = _load_reference_mmvq() if world == 1 else None
    if ref_lib is not None:
        tags = {"Q4K": "q4_k", "Q6K": "q6_k", "Q8_0": "q8_0"}
        ref_q8 = {key: torch.empty_like(v) for key, v in q8.items()}

        def step_reference():
            s_ = torch.cuda.current_stream().cuda_stream
            for (b, t, k, n) in order:
                ref_lib.launch_mmvq_gguf_quantize_q8_1_f32(xs[(k, b)].data_ptr(), ref_q8[(k, b)].data_ptr(), k, kp[k], b, s_)
                getattr(ref_lib, f"launch_mmvq_gguf_{tags[t]}_f32_plain")(mats[(t, k, n)].qtensor.device_ptr(), ref_q8[(k, b)].data_ptr(),
                                                                          outs[(n, b)].data_ptr(), k, n, kp[k] // 32, n, b, s_)
        ms_ref = timed(step_reference, max(3, args.steps // 4), 3, True)
        reference_cuda = {"what": "candle-kernels/src/mmvq_gguf.cu compiled unmodified for sm_100a, the same 60 quantize + GEMV pairs, "
                                  "CUDA graph replay", "value": total_bytes / ms_ref / 1e6, "unit": UNIT, "ms_per_step": ms_ref}
        del ref_q8

    # free the sweep's buffers before the other measurements
    del mats, xs, outs, q8, h_x, h_y, d_x
    gather = None
    torch.cuda.empty_cache()
    def extra(fn):
        """One of the additional measurements: a failure in it (a bounded wait that gave up, out of memory) is reported in
        its place instead of taking the headline down.  Its checks come after its last collective, so the ranks stay in
        step; they agree on the outcome before going on."""
        err, out = None, None
        try:
            out = fn()
        except Exception as e:      # noqa: BLE001 - reported in the JSON line
            err = f"{type(e).__name__}: {e}"
            L.cq_peer_gather_clear_timeout()
            L.cq_clear_status()
            torch.cuda.empty_cache()
        if world > 1:
            bad = torch.tensor([1 if err else 0], device=dev)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
            if int(bad.item()) and err is None:
                err = "failed on another rank"
        return {"error": err} if err else out

    int8_peak = extra(lambda: measure_int8_peak(dev)) if not args.no_prefill else None
    prefill = prefill_b32 = None
    if not args.no_prefill:
        peak_i8 = int8_peak.get("burst_tops") if isinstance(int8_peak, dict) else None
        prefill = extra(lambda: measure_prefill(dev, rank, world, peak_i8))
        prefill_b32 = extra(lambda: measure_prefill_block_formats(dev, peak_i8)) if world == 1 else None
    decode = None
    if not args.no_decode:
        decode = [extra(lambda b=b: decode_tok_s(dev, rank, world, b)) for b in (1, 8)]
    moe = None
    if not args.no_moe:
        moe = {"model": "Qwen3-30B-A3B-shaped, experts Q4_K, attention and head Q6_K, random weights", "prompt": 1024, "steps": 128,
               "parallelism": f"expert parallel x{world}" if world > 1 else "single GPU",
               "runs": [extra(lambda b=b: moe_decode_tok_s(dev, rank, world, b, 1024, 128)) for b in (1, 8)]}
        if world == 1:
            moe["grouped_gemm"] = extra(lambda: measure_moe_gemm(dev))

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak_gbs()
    value = total_bytes / ms_step / 1e6
    gemv_gbs = total_bytes / ms_gemv / 1e6
    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 dot products, f32 accumulation", "data": "synthetic",
        "config": {"workload": "gemv_sweep_llama3_8b", "types": TYPE_NAMES, "shapes_k_n": SHAPES, "batches": BATCHES,
                   "gemv_per_step": len(order), "bytes_per_step": total_bytes,
                   "l2": "1.6 GB of distinct weights are streamed between two uses of the same matrix (L2 is 126 MB)",
                   "parallelism": f"column-parallel x{world} + {gather_kind}" if world > 1 else "single GPU",
                   "launch": "CUDA graph replay" if graphed and graphed[0] else "eager launches"},
        "frac_of_8TBps_nominal_per_gpu": value / world / 8000.0,
        "gpu_launches": 2 * len(order) * args.steps,
        "sustained": {"value": total_bytes / ms_sustained / 1e6, "unit": UNIT, "steps": sus_steps, "ms_per_step": ms_sustained,
                      "gemv_only_GBps": total_bytes / ms_gemv_sustained / 1e6},
        "gemv_cases": {"unit": "GB/s per launch (algorithmic bytes, this rank's shard): graph of 5 {256 MB L2 flush, launch} pairs minus the flushes",
                       "by_type_shape_batch": per_case},
        "reference_cuda": reference_cuda,
        "int8_peak": int8_peak,
        "prefill": prefill,
        "prefill_block_formats": prefill_b32,
        "moe": moe,
        "e2e": {"value": total_bytes / ms_e2e / 1e6, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e},
        "roofline": {"bound": "hbm", "achieved": gemv_gbs / world, "peak": peak, "unit": "GB/s",
                     "frac": gemv_gbs / world / peak, "traffic": step_traffic_bytes(world),
                     "traffic_source": "bytes per step and GPU: every launch's algorithmic bytes x the dram__bytes_read+write / "
                                       "algorithmic ratio of that (format, shape) in a one-launch ncu capture at 1 and 8 rows "
                                       "(profiles/gemv_sweep_dram_traffic.md: 0.96 - 1.02; rows 2 and 4 take the 1-row ratio)",
                     "peak_source": peak_src,
                     "kernel": "gemv_staged_kernel / gemv_mma_kernel / gemv_mma2_kernel (all 60 GEMV launches of the step, quantize launches excluded)",
                     "ms_per_step": ms_gemv, "per_gpu": True},
        "clocks": clocks,
        "decode": {"model": "Llama-3-8B-shaped, Q4_K_M mix, random weights", "prompt": 512, "steps": 256,
                   "parallelism": f"row-sharded projections x{world}, all-gather", "runs": decode},
    }
    if world == 1:
        items, nbytes = cpu_sample_setup()
        nthreads = cpu_threads()
        model, phys, logical = host_cpu_info()
        cpu_sample_run(items, nthreads)
        t0 = time.perf_counter()
        reps = 0
        while reps < 2 or (time.perf_counter() - t0 < 10 and reps < 20):
            cpu_sample_run(items, nthreads)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        result["cpu_baseline"] = {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": nthreads, "kind": "port",
                                  "sample": SAMPLE_DESC + f"; {reps} passes", "cpu_model": model, "physical_cores": phys,
                                  "logical_cores": logical}
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


def run_case(args):
    """One GEMV case, a few launches, per-launch CUDA-event times: the small command the ncu captures profile.
    --case TYPE:K:N:B, e.g. Q4K:4096:128256:1."""
    import torch
    from candle_b200 import capi
    from candle_b200.quantized import GgmlDType
    from candle_b200.synth import random_blocks
    t, k, n, b = args.case.split(":")
    k, n, b = int(k), int(n), int(b)
    dev = torch.device("cuda:0")
    L = capi.lib()
    if args.mma_min_batch is not None:
        L.cq_set_mma_min_batch(args.mma_min_batch)
    if args.mma_kernel is not None:
        L.cq_set_mma_kernel(args.mma_kernel)
    if args.no_pdl:
        L.cq_set_pdl(0)
    ncopies = max(2, min(16, int(300e6 // (n * k * BYTES_PER_ELEM[t])) + 1))     # rotate through > L2 of weights
    ws = [random_blocks(GgmlDType[t], n, k, seed=i, device=dev) for i in range(ncopies)]
    x = torch.randn((b, k), device=dev)
    kp = capi.pad(k, 512)
    y = torch.empty((b, kp // 32 * 36), dtype=torch.uint8, device=dev)
    out = torch.empty((b, n), device=dev)
    s = torch.cuda.current_stream().cuda_stream
    L.cq_quantize_act(x.data_ptr(), capi.F32, y.data_ptr(), k, kp, b, capi.ACT_Q8_1, s)
    times = []
    for i in range(args.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        L.cq_mmvq(int(GgmlDType[t]), capi.ACT_Q8_1, capi.F32, ws[i % ncopies].data_ptr(), y.data_ptr(), out.data_ptr(),
                  k, n, kp // 32, n, b, s)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    capi.check("case")
    nbytes = gemv_bytes(t, k, n, b)
    best = min(times[1:]) if len(times) > 1 else times[0]
    iso_us = IsolatedTimer(dev).ms(lambda: L.cq_mmvq(int(GgmlDType[t]), capi.ACT_Q8_1, capi.F32, ws[0].data_ptr(), y.data_ptr(), out.data_ptr(),
                                                      k, n, kp // 32, n, b, torch.cuda.current_stream().cuda_stream)) * 1e3
    plan = (__import__("ctypes").c_int * 4)()
    L.cq_mmvq_plan(int(GgmlDType[t]), capi.ACT_Q8_1, k, n, b, plan)
    print(json.dumps({"case": args.case, "plan_kernel_rows_grid_threads": list(plan), "us": [round(v, 1) for v in times],
                      "algorithmic_bytes": nbytes, "best_GBps": round(nbytes / best / 1e3, 1),
                      "isolated_us": round(iso_us, 2), "isolated_GBps": round(nbytes / iso_us / 1e3, 1)}))


def run_traffic_sweep(args):
    """Profiling helper: every (format, shape) GEMV of the sweep once at batch 1 and once at batch 8, in a fixed order that
    is printed as JSON - the launch list an `ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum
    -k regex:gemv_` capture of this command maps onto, one captured launch per printed case (--traffic-types limits the
    formats so that a capture stays small)."""
    import torch
    from candle_b200 import capi
    from candle_b200.quantized import GgmlDType
    from candle_b200.synth import random_blocks
    dev = torch.device("cuda:0")
    L = capi.lib()
    s = torch.cuda.current_stream().cuda_stream
    cases = []
    for t in args.traffic_types.split(","):
        for (k, n) in SHAPES:
            w = random_blocks(GgmlDType[t], n, k, seed=1, device=dev)
            kp = capi.pad(k, 512)
            for b in (1, 8):
                x = torch.randn((b, k), device=dev)
                y = torch.empty((b, kp // 32 * 36), dtype=torch.uint8, device=dev)
                out = torch.empty((b, n), device=dev)
                L.cq_quantize_act(x.data_ptr(), capi.F32, y.data_ptr(), k, kp, b, capi.ACT_Q8_1, s)
                L.cq_mmvq(int(GgmlDType[t]), capi.ACT_Q8_1, capi.F32, w.data_ptr(), y.data_ptr(), out.data_ptr(), k, n, kp // 32, n, b, s)
                torch.cuda.synchronize()
                plan = (__import__("ctypes").c_int * 4)()
                L.cq_mmvq_plan(int(GgmlDType[t]), capi.ACT_Q8_1, k, n, b, plan)
                cases.append({"type": t, "k": k, "n": n, "b": b, "algorithmic_bytes": gemv_bytes(t, k, n, b), "plan": list(plan)})
            del w
    capi.check("traffic sweep")
    print(json.dumps({"traffic_sweep": cases}))


def run_prefill_case(args):
    """One prefill GEMM case: --prefill-case M:K:N (--prefill-type Q4K | Q6K), a few launches with CUDA-event times
    (profiling helper)."""
    import torch
    from candle_b200 import capi
    from candle_b200.quantized import GgmlDType
    from candle_b200.synth import random_blocks
    m, k, n = (int(v) for v in args.prefill_case.split(":"))
    dev = torch.device("cuda:0")
    L = capi.lib()
    wt = GgmlDType[args.prefill_type]
    block32 = wt in (GgmlDType.Q8_0, GgmlDType.Q4_0)        # the block-format kernel (prefill_b32.cu)
    scratch_bytes, quantize, gemm = ((L.cq_prefill32_scratch_bytes, L.cq_prefill32_quantize, L.cq_prefill32_gemm) if block32 else
                                     (L.cq_prefill_scratch_bytes, L.cq_prefill_quantize, L.cq_prefill_gemm))
    w = random_blocks(wt, n, k, seed=1, device=dev)
    x = torch.randn((m, k), device=dev)
    scratch = torch.empty(scratch_bytes(m, k), dtype=torch.uint8, device=dev)
    out = torch.empty((m, n), device=dev)
    s = torch.cuda.current_stream().cuda_stream
    quantize(x.data_ptr(), capi.F32, scratch.data_ptr(), k, m, s)
    times = []
    for _ in range(args.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gemm(int(wt), w.data_ptr(), scratch.data_ptr(), out.data_ptr(), capi.F32, k, n, m, n, s)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    capi.check("prefill case")
    best = min(times[1:]) if len(times) > 1 else times[0]
    print(json.dumps({"prefill_case": args.prefill_case, "type": args.prefill_type, "ms": times, "useful_TOPS": 2.0 * m * n * k / best / 1e9}))


def moe_decode_tok_s(dev, rank, world, batch, prompt_len=1024, steps=256, use_graph=True):
    """Qwen3-30B-A3B-shaped mixture-of-experts decoder (experts Q4_K, attention and head Q6_K, random
    weights), expert parallel over `world` ranks: random prompt, then greedy decoding."""
    import torch
    import torch.distributed as dist
    from candle_b200.moe_decoder import MoeDecoderConfig, MoeShapedDecoder
    cfg = MoeDecoderConfig.qwen3_30b_a3b()
    m = MoeShapedDecoder(cfg, dev, rank=rank, world=world, batch=batch, seed=1)
    prompt = torch.randint(0, cfg.vocab, (batch, prompt_len), device=dev, generator=torch.Generator(device=dev).manual_seed(3))
    m.forward(prompt[:, :min(prompt_len, 64)])      # grows the activation workspace before anything is recorded
    graphed = m.capture_decode_step() if use_graph else False
    m.reset()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record()
    tok = m.forward(prompt)
    e1.record()
    toks = [tok]
    for _ in range(steps - 1):
        tok = m.decode_step(tok).clone()
        toks.append(tok)
    e2.record()
    torch.cuda.synchronize()
    t_prompt, t_dec = e0.elapsed_time(e1), e1.elapsed_time(e2)
    if world > 1:
        t = torch.tensor([t_prompt, t_dec], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_prompt, t_dec = float(t[0]), float(t[1])
    m.check()
    checksum = token_hash(toks)
    del m
    torch.cuda.empty_cache()
    return {"batch": batch, "decode_tok_s": batch * (steps - 1) / t_dec * 1e3, "ms_per_step": t_dec / (steps - 1),
            "prompt_tok_s": batch * prompt_len / t_prompt * 1e3, "cuda_graph": bool(graphed), "token_hash": checksum,
            "active_weight_bytes_per_token": cfg.active_weight_bytes_per_token(), "experts_per_rank": cfg.experts // world}


def run_dequant_case(args):
    """De-quantize one tensor: --dequant-case TYPE:N:K, a few launches with CUDA-event times (profiling helper).
    Bytes = GGUF blocks read + f32 written."""
    import torch
    from candle_b200.quantized import GgmlDType, QTensor
    from candle_b200.synth import random_blocks
    t, n, k = args.dequant_case.split(":")
    n, k = int(n), int(k)
    dev = torch.device("cuda:0")
    blocks = random_blocks(GgmlDType[t], n, k, seed=1, device=dev)
    qt = QTensor.from_device_blocks(blocks, GgmlDType[t], (n, k))
    times = []
    for _ in range(args.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = qt.dequantize()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
        del out
    nbytes = blocks.numel() + 4.0 * n * k
    best = min(times[1:]) if len(times) > 1 else times[0]
    print(json.dumps({"dequant_case": args.dequant_case, "us": times, "bytes": nbytes, "best_GBps": nbytes / best / 1e3}))


def _load_reference_mmvq():
    """The reference's MMVQ kernels built by oracle/build_ref.py, or None (a baseline timed beside, never the product path)."""
    import ctypes as C
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "libcandle_ref_mmvq.so")
    if not os.path.isfile(path):
        return None
    try:
        lib = C.CDLL(path)
    except OSError:
        return None
    vp, i32 = C.c_void_p, C.c_int
    lib.launch_mmvq_gguf_quantize_q8_1_f32.argtypes, lib.launch_mmvq_gguf_quantize_q8_1_f32.restype = [vp, vp, i32, i32, i32, vp], None
    for tag in ("q4_k", "q6_k", "q8_0", "q4_0"):
        f = getattr(lib, f"launch_mmvq_gguf_{tag}_f32_plain")
        f.argtypes, f.restype = [vp, vp, vp, i32, i32, i32, i32, i32, vp], None
    return lib


def _load_reference_mmq():
    import ctypes as C
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "libcandle_ref_mmq.so")
    if not os.path.isfile(path):
        return None
    try:
        lib = C.CDLL(path)
    except OSError:
        return None
    vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
    for layout in ("D4", "DS4"):
        f = getattr(lib, f"launch_mmq_quantize_q8_1_{layout}")
        f.argtypes, f.restype = [vp, vp, vp, i32, i64, i64, i64, i64, i64, i64, i64, i64, vp], None
    for tag in ("q4_k", "q6_k", "q8_0", "q4_0"):
        f = getattr(lib, f"launch_mmq_gguf_{tag}")
        f.argtypes, f.restype = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i32, i32, i64, i32, vp], None
    return lib


def decode_tok_s(dev, rank, world, batch, prompt_len=512, steps=256, use_graph=True, fuse_rope=None):
    """Llama-3-8B-shaped Q4_K_M decoder, random prompt of `prompt_len` ids (seed 2), `steps` greedy
    tokens.  Returns (decode tokens/s over all sequences, prompt tokens/s, token checksum)."""
    import torch
    import torch.distributed as dist
    from candle_b200.decoder import DecoderConfig, LlamaShapedDecoder
    cfg = DecoderConfig.llama3_8b()
    m = LlamaShapedDecoder(cfg, dev, rank=rank, world=world, batch=batch, seed=1)
    if fuse_rope is not None:
        m.fuse_rope = fuse_rope
    prompt = torch.randint(0, cfg.vocab, (batch, prompt_len), device=dev, generator=torch.Generator(device=dev).manual_seed(2))
    m.forward(prompt)          # grows the activation workspace to its final size before anything is recorded
    graphed = m.capture_decode_step() if use_graph else False
    m.reset()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record()
    tok = m.forward(prompt)
    e1.record()
    toks = [tok]
    for _ in range(steps - 1):
        tok = m.decode_step(tok).clone()
        toks.append(tok)
    e2.record()
    torch.cuda.synchronize()
    t_prompt, t_dec = e0.elapsed_time(e1), e1.elapsed_time(e2)
    if world > 1:
        t = torch.tensor([t_prompt, t_dec], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_prompt, t_dec = float(t[0]), float(t[1])
    m.check()
    checksum = token_hash(toks)
    del m
    torch.cuda.empty_cache()
    return {"batch": batch, "decode_tok_s": batch * (steps - 1) / t_dec * 1e3, "ms_per_step": t_dec / (steps - 1),
            "prompt_tok_s": batch * prompt_len / t_prompt * 1e3, "cuda_graph": bool(graphed), "token_hash": checksum,
            "weight_bytes_per_token": cfg.weight_bytes_per_token(),
            "weight_stream_GBps": cfg.weight_bytes_per_token() / (t_dec / (steps - 1)) / 1e6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--decode-case", default=None, help="profile helper: BATCH:PROMPT:STEPS, runs only the decoder measurement")
    ap.add_argument("--no-fuse-rope", action="store_true", help="with --decode-case: rope + KV store as a launch of its own")
    ap.add_argument("--no-graph", action="store_true", help="with --decode-case: launch decode steps eagerly")
    ap.add_argument("--mma-min-batch", type=int, default=None, help="with --case: rows from which the tensor-core GEMV is used (9: never)")
    ap.add_argument("--mma-kernel", type=int, default=None, help="with --case: 1 only the CTA-shared tensor-core GEMV, 2 the warp-private one")
    ap.add_argument("--cluster-split", type=int, default=None, help="with --case / --decode-case: 0 never, 1 default rule, 2 always "
                    "(thread-block clusters for the split form of the warp-private tensor-core GEMV)")
    ap.add_argument("--no-pdl", action="store_true", help="with --case: plain launches instead of programmatic dependent launches")
    ap.add_argument("--tune", default=None, help="with --decode-case: RB:CTAS_PER_SM forced for every GEMV (experiment hook)")
    ap.add_argument("--moe-decode-case", default=None, help="BATCH:PROMPT:STEPS, runs the mixture-of-experts decoder measurement "
                    "(under torchrun: expert parallel)")
    ap.add_argument("--dequant-case", default=None, help="profile helper: TYPE:N:K, de-quantizes one tensor to f32")
    ap.add_argument("--no-decode", action="store_true", help="skip the Llama-3-8B-shaped decode measurement")
    ap.add_argument("--no-prefill", action="store_true", help="skip the int8 peak and prompt-phase GEMM measurements")
    ap.add_argument("--no-moe", action="store_true", help="skip the mixture-of-experts measurements")
    ap.add_argument("--prefill-case", default=None, help="profile helper: M:K:N, runs the Q4_K prefill GEMM --iters times")
    ap.add_argument("--prefill-type", default="Q4K", choices=["Q4K", "Q6K", "Q8_0", "Q4_0"], help="weight format of --prefill-case")
    ap.add_argument("--case", default=None, help="profile helper: TYPE:K:N:B, runs that GEMV --iters times")
    ap.add_argument("--traffic-sweep", action="store_true", help="profile helper: each (format, shape) GEMV once at batch 1 and 8")
    ap.add_argument("--traffic-types", default="Q4K,Q6K,Q8_0", help="with --traffic-sweep: comma-separated formats")
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    if args.cluster_split is not None:
        from candle_b200 import capi as _capi
        _capi.lib().cq_set_cluster_split(args.cluster_split)
    if args.decode_case:
        import torch
        b_, p_, s_ = (int(v) for v in args.decode_case.split(":"))
        if args.tune:       # needs a library built with -DCQ_EXPERIMENT
            import ctypes
            from candle_b200 import capi
            rb_, cps_ = (int(v) for v in args.tune.split(":"))
            fn = getattr(capi.lib(), "cq_set_tuning", None)
            if fn is None:
                raise SystemExit("--tune needs an experiment build of the library (nvcc -DCQ_EXPERIMENT)")
            fn(ctypes.c_int(rb_), ctypes.c_int(cps_))
        torch.cuda.set_device(0)
        print(json.dumps(decode_tok_s(torch.device("cuda:0"), 0, 1, b_, p_, s_, use_graph=not args.no_graph,
                                      fuse_rope=False if args.no_fuse_rope else None)))
    elif args.traffic_sweep:
        run_traffic_sweep(args)
    elif args.prefill_case:
        run_prefill_case(args)
    elif args.moe_decode_case:
        import torch
        import torch.distributed as dist
        b_, p_, s_ = (int(v) for v in args.moe_decode_case.split(":"))
        world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        res = moe_decode_tok_s(torch.device(f"cuda:{local}"), rank, world, b_, p_, s_, use_graph=not args.no_graph)
        if rank == 0:
            print(json.dumps(dict(res, n_gpus=world)))
        if world > 1:
            dist.destroy_process_group()
    elif args.dequant_case:
        run_dequant_case(args)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
