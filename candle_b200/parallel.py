"""Column-parallel sharding of quantized projections inside one NVLink/NVSwitch box.

Every weight row of W[N, K] is an independent unit (a GGUF block never spans rows), so each rank keeps a
contiguous range of rows, computes y[:, rows] with the ordinary kernels and the slices are all-gathered.
The per-element summation order does not depend on the shard count, so results are bit-identical for any
world size - which K-sharding followed by an all-reduce (the scheme of candle's only multi-GPU example,
candle-examples/examples/llama_multiprocess/model.rs:13-137) cannot give.

On CUDA the exchange runs as one kernel of this library over NVLink peer memory (`PeerGatherer`, csrc/peer_gather.cu);
`Gatherer` (a library all-gather) is the portable form and what the CPU tests with the gloo backend exercise.
"""
from __future__ import annotations

import ctypes
import os
import sys

import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int, unit: int = 1) -> tuple[int, int]:
    """Contiguous row range [start, start + count) of rank `rank`; `unit` rows stay together (e.g. one head)."""
    if n % (world * unit) != 0:
        raise ValueError(f"{n} rows cannot be split into {world} shards of whole units of {unit}")
    count = n // world
    return rank * count, count


def shard_block_rows(blocks, n: int, world: int, rank: int, unit: int = 1):
    """Slice the rows of a [n, row_bytes] block matrix (numpy or torch) for `rank`."""
    start, count = shard_rows(n, world, rank, unit)
    return blocks[start:start + count]


class Gatherer:
    """All-gather of column slices [rows, n_local] -> [rows, n_local * world], rank-major along the last dimension.

    Buffers are allocated once per shape so that the call can sit inside a CUDA graph."""

    def __init__(self, group=None, world: int | None = None):
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self._bufs: dict = {}

    def __call__(self, local: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return local
        rows, n_local = local.shape
        key = (rows, n_local, local.dtype, local.device)
        if key not in self._bufs:
            self._bufs[key] = (torch.empty((self.world * rows, n_local), dtype=local.dtype, device=local.device),
                               torch.empty((rows, self.world * n_local), dtype=local.dtype, device=local.device))
        stacked, full = self._bufs[key]
        dist.all_gather_into_tensor(stacked, local.contiguous(), group=self.group)
        if rows == 1:       # rank-major slices of a single row are already the gathered row
            return stacked.view(1, self.world * n_local)
        full.view(rows, self.world, n_local).copy_(stacked.view(self.world, rows, n_local).permute(1, 0, 2))
        return full


class PeerGatherer(Gatherer):
    """The same gather as one kernel over peer memory: every rank stores its slice, word by word together with an epoch
    tag, into staging areas of all other ranks and picks up what they stored here (`cq_peer_gather_words`).  The staging
    areas live in symmetric memory (`torch.distributed._symmetric_memory`: one CUDA virtual-memory allocation per rank,
    mapped by all); they are made on first use of a shape, which is a collective step, so shapes must first occur
    outside CUDA-graph capture and in the same order on all ranks.  Every shape has two areas and the kernel picks one by
    the parity of its device-side epoch counter, so two consecutive gathers never store into the same area - in eager
    runs and across the replays of a CUDA graph (two result buffers alternate on the host so that back-to-back gathers
    of one shape return different tensors).  When a rank would send more than `MAX_SENT_WORDS` 32-bit words in total (prompts, the
    vocabulary slice of a large batch on many ranks) the library all-gather is used: the slot protocol doubles the bytes
    on the link and is built for latency, not bandwidth."""

    MAX_SENT_WORDS = 1 << 18     # slice words x (world - 1)

    def __init__(self, group=None, world: int | None = None):
        super().__init__(group, world)
        import torch.distributed._symmetric_memory as symm_mem
        from . import capi
        self._symm, self._capi = symm_mem, capi
        g = group if group is not None else dist.group.WORLD
        self._group_name = g.group_name
        self.rank = dist.get_rank(g)
        if self.world > capi.MAX_PEERS:
            raise ValueError(f"at most {capi.MAX_PEERS} ranks")
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._keep = []
        self._state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._slots: dict = {}
        self._last = None

    def _new_slot(self, rows: int, n_local: int, dtype, row_exchange: bool = False):
        lib = self._capi.lib()
        nbytes = lib.cq_peer_exchange_stage_bytes(rows, n_local) if row_exchange else lib.cq_peer_gather_stage_bytes(rows, n_local, self.world)
        stage = self._symm.empty((nbytes,), dtype=torch.uint8, device=self.device)
        hdl = self._symm.rendezvous(stage, group=self._group_name)
        stage.zero_()
        self._keep.append((stage, hdl))
        return [int(p) for p in hdl.buffer_ptrs]

    def __call__(self, local: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return local
        if local.dim() != 2:
            raise ValueError("peer gather takes a 2-d tensor")
        if local.numel() * local.element_size() * (self.world - 1) > 4 * self.MAX_SENT_WORDS:
            self._last = None       # a library collective in between orders the accesses like any other gather
            return super().__call__(local)
        dtype = local.dtype
        if local.element_size() != 4:       # e.g. rows of Q8_1 containers (uint8, 36 bytes each): move them as 32-bit words
            if (local.shape[1] * local.element_size()) % 4 != 0:
                raise ValueError("peer gather: rows must be whole 32-bit words")
            local = local.contiguous().view(torch.int32)
        elif local.stride(1) != 1:
            local = local.contiguous()
        rows, n_local = local.shape
        key = (rows, n_local, local.dtype)
        entry = self._ensure(key)
        if self._last == key:
            entry[1] ^= 1       # back-to-back gathers of one shape return different result tensors
        self._last = key
        full, ptrs = entry[0][entry[1]], entry[2]
        self._capi.lib().cq_peer_gather_words(local.data_ptr(), local.stride(0), ptrs, full.data_ptr(), self._state.data_ptr(),
                                               rows, n_local, self.world * n_local, self.rank, self.world,
                                               torch.cuda.current_stream().cuda_stream)
        return full if full.dtype == dtype else full.view(dtype)

    def _ensure(self, key):
        """The staging areas and result buffers of a gather shape (rows, n_local, dtype), made on first use - a collective
        step, outside CUDA-graph capture."""
        if key not in self._slots:
            rows, n_local, dtype = key
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("a new gather shape inside CUDA-graph capture: run the step once before capturing")
            areas = [self._new_slot(rows, n_local, dtype) for _ in range(2)]      # even / odd epochs
            ptrs = (ctypes.c_void_p * (2 * self._capi.MAX_PEERS))()
            for e in range(2):
                for p, a in enumerate(areas[e]):
                    ptrs[e * self._capi.MAX_PEERS + p] = a
            outs = [torch.empty((rows, self.world * n_local), dtype=dtype, device=self.device) for _ in range(2)]
            self._slots[key] = [outs, 0, ptrs]
            torch.cuda.synchronize()
            dist.barrier(group=self.group)      # nobody stores into a staging area before its owner has zeroed it
        return self._slots[key]

    def forward_host(self, mm, h_x: torch.Tensor, h_y: torch.Tensor) -> bool:
        """`mm.forward` of this rank's row shard on f32 activations in pinned host memory, the gather of the slices and the
        copy-back of the gathered rows into `h_y`, as ONE library call (uploads and copy-backs on the library's own
        streams, see `QMatMul.forward_host`; join with `mm.host_flush()`).  False when the slice is too large for the
        slot protocol: the caller then uses `ShardedHostForward`."""
        rows = h_x.numel() // h_x.shape[-1]
        n_local = mm.qtensor.shape[0]
        if h_x.dtype != torch.float32 or h_y.dtype != torch.float32 or rows * n_local * 4 * (self.world - 1) > 4 * self.MAX_SENT_WORDS:
            return False
        entry = self._ensure((rows, n_local, torch.float32))
        self._last = None
        dims = (ctypes.c_int64 * h_x.dim())(*[int(d) for d in h_x.shape])
        self._capi.hcheck(self._capi.lib().cqh_qmatmul_forward_host_sharded(
            mm.qtensor._h, h_x.data_ptr(), 0, dims, h_x.dim(), h_y.data_ptr(), entry[2], self._state.data_ptr(), self.rank, self.world,
            torch.cuda.current_stream().cuda_stream), "forward_host_sharded")
        return True

    def exchange_rows(self, local: torch.Tensor, owner: torch.Tensor, n_owned: int):
        """Rows of `local` [rows, n] (4-byte elements) that each belong to one rank - this rank owns row j iff
        0 <= owner[j] < n_owned (`owner`: int32 [rows] on the device) - as one kernel over peer memory: every rank ends up
        with all rows.  Returns None when the buffer is too large for the slot protocol (the caller then uses a library
        collective); the staging areas of a shape are made on first use, outside CUDA-graph capture."""
        if self.world == 1:
            return local
        if local.dim() != 2 or local.element_size() != 4 or not local.is_contiguous():
            raise ValueError("peer row exchange takes a contiguous 2-d tensor of 4-byte elements")
        if owner.dtype != torch.int32 or owner.numel() != local.shape[0] or not owner.is_contiguous():
            raise ValueError("peer row exchange: owner must be a contiguous int32 tensor with one entry per row")
        if local.numel() * (self.world - 1) > self.MAX_SENT_WORDS * self.world:
            self._last = None
            return None
        rows, n = local.shape
        key = (rows, n, local.dtype, "rows")
        if key not in self._slots:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("a new exchange shape inside CUDA-graph capture: run the step once before capturing")
            areas = [self._new_slot(rows, n, local.dtype, True) for _ in range(2)]
            ptrs = (ctypes.c_void_p * (2 * self._capi.MAX_PEERS))()
            for e in range(2):
                for p, a in enumerate(areas[e]):
                    ptrs[e * self._capi.MAX_PEERS + p] = a
            outs = [torch.empty((rows, n), dtype=local.dtype, device=self.device) for _ in range(2)]
            self._slots[key] = [outs, 0, ptrs]
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        entry = self._slots[key]
        if self._last == key:
            entry[1] ^= 1
        self._last = key
        full, ptrs = entry[0][entry[1]], entry[2]
        self._capi.lib().cq_peer_exchange_rows(local.data_ptr(), owner.data_ptr(), int(n_owned), ptrs, full.data_ptr(),
                                                self._state.data_ptr(), rows, n, self.rank, self.world,
                                                torch.cuda.current_stream().cuda_stream)
        return full

    def check(self) -> None:
        """Raises if any gather so far gave up waiting for another rank (synchronises the device)."""
        if self._capi.lib().cq_peer_gather_timeout_flag() != 0:
            raise RuntimeError("peer gather: a bounded wait for another rank gave up")


class ShardedHostForward:
    """`QMatMul.forward` of a row shard for callers whose activations and results live in pinned HOST memory, one process
    per GPU: upload on an upload stream, the shard's product and the all-gather on the caller's stream, the copy-back of the
    gathered rows on a copy stream - so that the copies of one call overlap the arithmetic of its neighbours, as
    `QMatMul.forward_host` does on a single GPU.  A ring of four staging slots; `flush()` joins the copy stream.
    The host activations must be complete when the call is made."""

    SLOTS = 4

    def __init__(self, gather: Gatherer, device):
        self.gather, self.device = gather, torch.device(device)
        self.up, self.down = torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device)
        self._slots = [{"x": None, "free": None} for _ in range(self.SLOTS)]
        self._next = 0
        self._result_events: dict = {}      # gathered-result shape -> copy-back events of its last two uses

    def __call__(self, mm, h_x: torch.Tensor, h_y: torch.Tensor) -> None:
        one_call = getattr(self.gather, "forward_host", None)
        if one_call is not None and one_call(mm, h_x, h_y):
            self._flush_mm = mm
            return
        sl = self._slots[self._next]
        self._next = (self._next + 1) % self.SLOTS
        main = torch.cuda.current_stream(self.device)
        if sl["free"] is not None:      # the product that read this slot's activations is over
            self.up.wait_event(sl["free"])
        need = h_x.numel() * h_x.element_size()
        if sl["x"] is None or sl["x"].numel() < need:
            torch.cuda.synchronize(self.device)
            sl["x"] = torch.empty(max(need, 1 << 16), dtype=torch.uint8, device=self.device)
        d_x = sl["x"][:need].view(h_x.dtype).view(h_x.shape)
        with torch.cuda.stream(self.up):
            d_x.copy_(h_x, non_blocking=True)
            ev_up = torch.cuda.Event()
            ev_up.record(self.up)
        main.wait_event(ev_up)
        y = mm.forward(d_x)
        # the gatherer alternates two result buffers per shape: their last copy-backs must be over before one is rewritten
        key = (tuple(y.shape), y.dtype)
        for ev in self._result_events.get(key, ()):
            main.wait_event(ev)
        full = self.gather(y)
        done = torch.cuda.Event()
        done.record(main)
        self.down.wait_event(done)
        with torch.cuda.stream(self.down):
            h_y.copy_(full, non_blocking=True)
            ev_dn = torch.cuda.Event()
            ev_dn.record(self.down)
        sl["free"] = done
        self._result_events[key] = (self._result_events.get(key, ()) + (ev_dn,))[-2:]

    def flush(self) -> None:
        """The caller's stream waits for every copy-back in flight: synchronise it and the host results are complete."""
        torch.cuda.current_stream(self.device).wait_stream(self.down)
        mm = getattr(self, "_flush_mm", None)
        if mm is not None:
            mm.host_flush()


def make_gatherer(group=None, world: int | None = None, device=None) -> Gatherer:
    """`PeerGatherer` on CUDA with more than one rank (unless CQ_PEER_GATHER=0), else the library all-gather."""
    w = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
    on_cuda = device is not None and torch.device(device).type == "cuda"
    if w > 1 and on_cuda and os.environ.get("CQ_PEER_GATHER", "1") != "0":
        ok = 1
        try:
            pg = PeerGatherer(group, w)
            pg(torch.zeros((1, 8), device=device))      # first staging area: the step that needs peer mappings to work
            pg.check()
        except Exception as e:      # no peer access between these GPUs, or an older torch: every rank must learn of it
            ok = 0
            try:        # a probe that gave up leaves the device flag set: clear it so later checks see only their own gathers
                from . import capi
                capi.lib().cq_peer_gather_clear_timeout()
                capi.lib().cq_clear_status()
            except Exception:
                pass
            print(f"candle_b200: peer-memory gather unavailable ({type(e).__name__}: {e}); using the library all-gather",
                  file=sys.stderr)
        flag = torch.tensor([ok], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 1:
            return pg
    return Gatherer(group, w)


def argmax_sharded(local_logits: torch.Tensor, vocab_start: int, gather: Gatherer) -> torch.Tensor:
    """Greedy token over a vocabulary sharded by rows: gather (max, global index) pairs and break ties towards the
    lowest global index, which is what argmax over the whole row returns."""
    mx = local_logits.max(dim=-1).values
    ar = torch.arange(local_logits.shape[-1], device=local_logits.device)
    idx = torch.where(local_logits == mx.unsqueeze(-1), ar, ar.new_full((), 1 << 40)).min(dim=-1).values   # first maximum
    pair = torch.stack([mx, (idx + vocab_start).to(mx.dtype)], dim=-1)      # indices < 2^24 are exact in f32
    allp = gather(pair)                                                      # [rows, 2 * world]
    allp = allp.view(allp.shape[0], -1, 2)
    best = allp[..., 0].max(dim=-1, keepdim=True).values
    cand = torch.where(allp[..., 0] == best, allp[..., 1], torch.full_like(allp[..., 1], float("inf")))
    return cand.min(dim=-1).values.to(torch.int64)
