"""Llama-shaped decoder harness: a caller of ``QMatMul::forward`` with the shape of Llama-3-8B (32 layers, d = 4096, 32 query / 8 KV heads of 128,
FFN 14336, vocabulary 128256).

Structure and call order follow candle-transformers/src/models/quantized_llama.rs:178-262, 568-596 (f32 residual
stream, RMSNorm eps 1e-5, interleaved RoPE, f32 KV cache, GQA attention, SwiGLU, logits for the last position)
and the greedy loop of candle-examples/examples/quantized/main.rs:616-690.  Weights are random GGUF blocks
(candle_b200/synth.py) in the Q4_K_M mix: Q6_K for attn_v, ffn_down and the output head, Q4_K elsewhere.

Tensor parallelism: every projection is sharded by output rows (whole heads for q/k/v) and its output slices are
all-gathered; nothing is ever reduced across ranks, so a token sequence is bit-identical at 1, 2, 4 and 8 GPUs.
Glue (norm with the pending residual add, RoPE with the KV-cache store, SwiGLU) is one small f32 kernel per step
(csrc/glue.cu); attention is ``cq_attention_f32``, whose summation order does not depend on how many heads a rank
owns.  q and k of a layer come from one stacked projection, gate and up from another.
Weights are generated in eight row pieces with seeds that do not depend on the world size.
"""
from __future__ import annotations

import dataclasses
import math

import torch

from . import capi
from .parallel import Gatherer, argmax_sharded, make_gatherer
from .quantized import GgmlDType, QMatMul, QTensor
from .synth import random_blocks

PIECES = 8   # finest shard granularity; rank r of g holds pieces [r * 8 / g, (r + 1) * 8 / g)


@dataclasses.dataclass
class DecoderConfig:
    layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    max_pos: int = 1024

    @staticmethod
    def llama3_8b() -> "DecoderConfig":
        return DecoderConfig()

    @staticmethod
    def tiny() -> "DecoderConfig":
        return DecoderConfig(layers=2, d_model=1024, n_heads=8, n_kv_heads=8, head_dim=128, ffn=2048, vocab=4096, max_pos=128)

    def weight_bytes_per_token(self) -> int:
        """Bytes of quantized weights one decoded token streams (whole model, all ranks together)."""
        q4, q6 = 144 / 256, 210 / 256
        d, kv = self.d_model, self.n_kv_heads * self.head_dim
        per_layer = (d * d + kv * d + d * d + 2 * self.ffn * d) * q4 + (kv * d + d * self.ffn) * q6
        return int(self.layers * per_layer + self.vocab * d * q6)


def _sharded_blocks(dtype: GgmlDType, n: int, k: int, seed: int, rank: int, world: int, device) -> torch.Tensor:
    """GGUF blocks of this rank's rows of a [n, k] projection, generated piece by piece."""
    per = PIECES // world
    piece_rows = n // PIECES
    return torch.cat([random_blocks(dtype, piece_rows, k, seed * 16 + p, device) for p in range(rank * per, (rank + 1) * per)], dim=0)


def _sharded_matmul(dtype: GgmlDType, k: int, parts, rank: int, world: int, device) -> QMatMul:
    """One QMatMul over the local rows of one or several projections of the same block format that read the same
    input (`parts`: (rows, seed) pairs).  A GEMV row never depends on its neighbours, so stacking projections does
    not change any output bit; it only saves launches and activation quantizations."""
    blocks = torch.cat([_sharded_blocks(dtype, n, k, seed, rank, world, device) for n, seed in parts], dim=0).contiguous()
    rows = sum(n for n, _ in parts) // world
    return QMatMul.from_qtensor(QTensor.from_device_blocks(blocks, dtype, (rows, k)))


class _Layer:
    pass


class LlamaShapedDecoder:
    def __init__(self, cfg: DecoderConfig, device, rank: int = 0, world: int = 1, batch: int = 1, seed: int = 0, group=None):
        if PIECES % world or cfg.n_kv_heads % world or cfg.vocab % PIECES or cfg.ffn % PIECES:
            raise ValueError("world size must divide 8 and the head / vocabulary / ffn sizes")
        self.cfg, self.device, self.rank, self.world, self.batch = cfg, torch.device(device), rank, world, batch
        self.gather = make_gatherer(group, world, self.device)
        d, hd = cfg.d_model, cfg.head_dim
        self.hq_l, self.hkv_l = cfg.n_heads // world, cfg.n_kv_heads // world
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        self.tok_embd = torch.randn((cfg.vocab, d), device=self.device, generator=g) * 0.02      # de-quantized at load in the reference
        self.layers = []
        for li in range(cfg.layers):
            L = _Layer()
            s = seed * 100003 + li * 16
            L.attn_norm = 1.0 + 0.1 * torch.randn(d, device=self.device, generator=g)
            L.ffn_norm = 1.0 + 0.1 * torch.randn(d, device=self.device, generator=g)
            mm = lambda dtype, k, parts: _sharded_matmul(dtype, k, parts, rank, world, self.device)
            L.wqk = mm(GgmlDType.Q4K, d, [(cfg.n_heads * hd, s + 1), (cfg.n_kv_heads * hd, s + 2)])    # [q heads | k heads]
            L.wv = mm(GgmlDType.Q6K, d, [(cfg.n_kv_heads * hd, s + 3)])
            # wo is small (9 MB at the Llama-3-8B shape): every rank keeps all of it and computes the whole projection
            # from the gathered attention output - cheaper than a slice plus a second exchange, and the same bits
            L.wo = _sharded_matmul(GgmlDType.Q4K, cfg.n_heads * hd, [(d, s + 4)], 0, 1, self.device)
            L.gate_up = mm(GgmlDType.Q4K, d, [(cfg.ffn, s + 5), (cfg.ffn, s + 6)])                     # [gate | up]
            L.down = mm(GgmlDType.Q6K, cfg.ffn, [(d, s + 7)])
            L.k_cache = torch.zeros((batch, self.hkv_l, cfg.max_pos, hd), device=self.device)
            L.v_cache = torch.zeros((batch, self.hkv_l, cfg.max_pos, hd), device=self.device)
            self.layers.append(L)
        self.out_norm = 1.0 + 0.1 * torch.randn(d, device=self.device, generator=g)
        self.output = _sharded_matmul(GgmlDType.Q6K, d, [(cfg.vocab, seed * 100003 + 999983)], rank, world, self.device)
        self.vocab_start = rank * (cfg.vocab // world)
        # RoPE tables (quantized_llama.rs:540-556): theta_i = base^(-2i/d), angle = pos * theta_i
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=self.device, dtype=torch.float32) / hd))
        ang = torch.arange(cfg.max_pos, device=self.device, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.pos = torch.zeros(1, dtype=torch.int32, device=self.device)       # cache position of the next token
        self._pos_host = 0      # host copy of pos: positions are checked against max_pos before anything is launched
        self._graph = None
        self.fuse_quantize = True       # decode steps: producers store Q8_1 containers directly
        self.fuse_rope = True           # decode steps: rotary embedding + cache update inside the attention launch
        self._att_scratch = None        # split-context attention: partial results and arrival counters
        self.tap = None                 # tests set a dict here: forward() then records copies of its intermediate tensors
        if world > 1:       # ranks build their shards at different speeds: line up before the first gather, whose polls are bounded
            import torch.distributed as dist
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)

    def _rec(self, key: str, t: torch.Tensor) -> None:
        """Record a copy of an intermediate tensor when a test has set `self.tap` to a dict (no-op otherwise)."""
        if self.tap is not None:
            self.tap[key] = t.detach().clone()

    # ---- glue -------------------------------------------------------------------------------------------------
    def _norm(self, x: torch.Tensor, delta, w: torch.Tensor) -> torch.Tensor:
        """RMSNorm of x (after x += delta, in place, when a pending residual is given)."""
        out = torch.empty_like(x)
        st = torch.cuda.current_stream(self.device).cuda_stream
        if delta is None:
            capi.lib().cq_rms_norm_f32(x.data_ptr(), w.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], self.cfg.rms_eps, st)
        else:
            capi.lib().cq_add_rms_norm_f32(x.data_ptr(), delta.data_ptr(), w.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1],
                                           self.cfg.rms_eps, st)
        return out

    def _norm_q8(self, x: torch.Tensor, delta, w: torch.Tensor) -> torch.Tensor:
        """The same normalisation, stored as the Q8_1 containers the next matmul reads."""
        R, d = x.shape
        out = torch.empty((R, d // 32 * 36), dtype=torch.uint8, device=self.device)
        capi.lib().cq_add_rms_norm_q8_1(x.data_ptr(), None if delta is None else delta.data_ptr(), w.data_ptr(), out.data_ptr(),
                                        R, d, d, self.cfg.rms_eps, torch.cuda.current_stream(self.device).cuda_stream)
        return out

    def _attention(self, qk: torch.Tensor, L, B: int, T: int, out: torch.Tensor, q8: bool) -> None:
        """Causal attention of the rotated queries in `qk` over the layer's cache.  Up to 64 queries the context is
        split over several CTAs per head (a different, equally fixed order of additions), else one CTA per head;
        the choice depends on (B, T) only, so it is the same at every tensor-parallel width."""
        cfg, lib, hd = self.cfg, capi.lib(), self.cfg.head_dim
        st = torch.cuda.current_stream(self.device).cuda_stream
        q_stride = (self.hq_l + self.hkv_l) * hd
        scale = 1.0 / math.sqrt(hd)
        blocks = self.hq_l * hd // 32
        if B * T <= 64:
            if self._att_scratch is None:
                n = lib.cq_attention_split_scratch_floats(64, 1, self.hq_l, cfg.max_pos)
                self._att_scratch = (torch.empty(n, dtype=torch.float32, device=self.device),
                                     torch.zeros(64 * self.hq_l, dtype=torch.int32, device=self.device))
            scratch, counters = self._att_scratch
            lib.cq_attention_split(qk.data_ptr(), L.k_cache.data_ptr(), L.v_cache.data_ptr(), out.data_ptr(), 1 if q8 else 0,
                                   self.pos.data_ptr(), scratch.data_ptr(), counters.data_ptr(), B, T, self.hq_l, self.hkv_l, hd,
                                   cfg.max_pos, scale, q_stride, blocks, st)
        elif q8:
            lib.cq_attention_q8_1(qk.data_ptr(), L.k_cache.data_ptr(), L.v_cache.data_ptr(), out.data_ptr(), self.pos.data_ptr(),
                                  B, T, self.hq_l, self.hkv_l, hd, cfg.max_pos, scale, q_stride, blocks, st)
        else:
            lib.cq_attention_f32(qk.data_ptr(), L.k_cache.data_ptr(), L.v_cache.data_ptr(), out.data_ptr(), self.pos.data_ptr(),
                                 B, T, self.hq_l, self.hkv_l, hd, cfg.max_pos, scale, q_stride, st)

    def _rope_attention(self, qk: torch.Tensor, v: torch.Tensor, L, B: int, out: torch.Tensor, q8: bool, li: int) -> None:
        """One query per sequence: rotary embedding of q and the new key, the cache update and the attention as one launch
        (the bits of `cq_rope_store_kv_f32` followed by `_attention`)."""
        cfg, lib, hd = self.cfg, capi.lib(), self.cfg.head_dim
        st = torch.cuda.current_stream(self.device).cuda_stream
        q_cols, kv_cols = self.hq_l * hd, self.hkv_l * hd
        stride = q_cols + kv_cols
        if self._att_scratch is None:
            n = lib.cq_attention_split_scratch_floats(64, 1, self.hq_l, cfg.max_pos)
            self._att_scratch = (torch.empty(n, dtype=torch.float32, device=self.device),
                                 torch.zeros(64 * self.hq_l, dtype=torch.int32, device=self.device))
        scratch, counters = self._att_scratch
        q_rot = torch.empty_like(qk) if self.tap is not None else None
        lib.cq_rope_attention_split(qk.data_ptr(), qk.data_ptr() + 4 * q_cols, v.data_ptr(), None if q_rot is None else q_rot.data_ptr(),
                                    self.cos.data_ptr(), self.sin.data_ptr(), L.k_cache.data_ptr(), L.v_cache.data_ptr(),
                                    out.data_ptr(), 1 if q8 else 0, self.pos.data_ptr(), scratch.data_ptr(), counters.data_ptr(),
                                    B, self.hq_l, self.hkv_l, hd, cfg.max_pos, 1.0 / math.sqrt(hd), stride, stride, kv_cols,
                                    q_cols // 32, st)
        if q_rot is not None:
            self._rec(f"{li}.q_rot", q_rot)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens: int64 [B, T] at cache positions pos .. pos+T-1.  Returns the greedy next token [B] and advances pos.

        Up to 8 rows (decode steps) every activation that only feeds a matmul is produced directly as Q8_1 containers
        and the matmuls skip their quantize launch; the containers are the bytes the stand-alone quantizer would
        make, so tokens do not depend on which path ran."""
        cfg, B, T = self.cfg, tokens.shape[0], tokens.shape[1]
        self._claim_positions(T)
        hd, R, lib = cfg.head_dim, B * T, capi.lib()
        st = torch.cuda.current_stream(self.device).cuda_stream
        q_cols, kv_cols = self.hq_l * hd, self.hkv_l * hd
        f_l = cfg.ffn // self.world
        fused = self.fuse_quantize and R <= 8 and lib.cqh_get_act_mode() == 0 and cfg.d_model % 512 == 0 and cfg.ffn % 512 == 0 and \
            (cfg.n_heads * hd) % 512 == 0
        u8 = dict(dtype=torch.uint8, device=self.device)
        f32 = dict(dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            x = self.tok_embd.index_select(0, tokens.reshape(-1))                       # [R, d], private to this call
            delta = None                                                                # residual not yet added to x
            for li, L in enumerate(self.layers):
                self._rec(f"{li}.x_in", x)
                if delta is not None:
                    self._rec(f"{li}.delta_in", delta)
                if fused:
                    h = self._norm_q8(x, delta, L.attn_norm)
                    qk, v = L.wqk.forward_q8_1_pair(L.wv, h)
                else:
                    h = self._norm(x, delta, L.attn_norm)
                    qk, v = L.wqk.forward(h), L.wv.forward(h)                           # [R, q_cols + kv_cols], [R, kv_cols]
                self._rec(f"{li}.h_attn", h), self._rec(f"{li}.qk", qk), self._rec(f"{li}.v", v)
                # rope + KV store inside the attention kernel: one sequence only - with more, the fused kernel's registers
                # cost more than the launch saves (B200, 512-token context: 533 / 530 tok/s at b=1, 1812 / 1903 at b=8)
                one_launch = self.fuse_rope and T == 1 and B == 1 and hd == 128
                if not one_launch:
                    lib.cq_rope_store_kv_f32(qk.data_ptr(), qk.data_ptr() + 4 * q_cols, v.data_ptr(), self.cos.data_ptr(),
                                             self.sin.data_ptr(), self.pos.data_ptr(), L.k_cache.data_ptr(), L.v_cache.data_ptr(),
                                             B, T, self.hq_l, self.hkv_l, hd, cfg.max_pos, q_cols + kv_cols, q_cols + kv_cols,
                                             kv_cols, st)
                    self._rec(f"{li}.q_rot", qk)
                if fused:
                    att = torch.empty((R, q_cols // 32 * 36), **u8)
                    if one_launch:
                        self._rope_attention(qk, v, L, B, att, True, li)
                    else:
                        self._attention(qk, L, B, T, att, True)
                    delta = L.wo.forward_q8_1(self.gather(att))
                    h = self._norm_q8(x, delta, L.ffn_norm)
                    gu = L.gate_up.forward_q8_1(h)                                      # [R, 2 * f_l]
                    a = torch.empty((R, f_l // 32 * 36), **u8)
                    lib.cq_silu_mul_q8_1(gu.data_ptr(), a.data_ptr(), R, f_l, f_l, st)
                    delta = self.gather(L.down.forward_q8_1(self.gather(a)))
                else:
                    att = torch.empty((R, q_cols), **f32)
                    if one_launch:
                        self._rope_attention(qk, v, L, B, att, False, li)
                    else:
                        self._attention(qk, L, B, T, att, False)
                    self._rec(f"{li}.att", att)
                    delta = L.wo.forward(self.gather(att))
                    self._rec(f"{li}.x_mid", x), self._rec(f"{li}.wo", delta)
                    h = self._norm(x, delta, L.ffn_norm)
                    gu = L.gate_up.forward(h)
                    a = torch.empty((R, f_l), **f32)
                    lib.cq_silu_mul_f32(gu.data_ptr(), a.data_ptr(), R, f_l, st)
                    self._rec(f"{li}.h_ffn", h), self._rec(f"{li}.gu", gu), self._rec(f"{li}.act", a)
                    delta = self.gather(L.down.forward(self.gather(a)))
                    self._rec(f"{li}.down", delta)
            self._rec("final.x_in", x), self._rec("final.delta_in", delta)
            h = (self._norm_q8 if fused else self._norm)(x, delta, self.out_norm)
            capi.check("decoder glue")
            self._rec("final.h", h)
            last = h.view(B, T, -1)[:, -1, :].contiguous()
            logits = self.output.forward_q8_1(last) if fused else self.output.forward(last)     # [B, vocab / world]
            self.last_logits = logits       # this rank's vocabulary slice, last position (read by tests)
            tok = argmax_sharded(logits, self.vocab_start, self.gather)
            self.pos += T
        return tok

    # ---- greedy loop ------------------------------------------------------------------------------------------
    def _claim_positions(self, t: int) -> None:
        """Host-side bound on cache positions: raises before anything is launched when `t` more tokens would run past
        the KV cache and the rotary tables (both hold cfg.max_pos positions)."""
        if self._pos_host + t > self.cfg.max_pos:
            raise ValueError(f"position {self._pos_host} + {t} tokens exceeds max_pos = {self.cfg.max_pos}")
        self._pos_host += t

    def check(self) -> None:
        """Raises if a device-side check tripped since the last call: a peer gather that gave up waiting for another
        rank, or a rope / KV-store launch that met a position beyond the cache (synchronises the device)."""
        chk = getattr(getattr(self, "gather", None), "check", None)
        if chk is not None:
            chk()
        if capi.lib().cq_glue_position_overflow_flag() != 0:
            capi.lib().cq_clear_status()
            raise RuntimeError("a decode step ran past max_pos: tokens after that point are invalid")

    def reset(self):
        self.pos.zero_()
        self._pos_host = 0

    def capture_decode_step(self) -> bool:
        """Record one decode step (T = 1) as a CUDA graph.  Returns False when capture is not possible
        (then decode_step launches eagerly)."""
        self._tok_in = torch.zeros((self.batch, 1), dtype=torch.int64, device=self.device)
        saved, saved_host = self.pos.clone(), self._pos_host
        try:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))     # _tok_in and every earlier write are visible
            with torch.cuda.stream(side):
                for _ in range(2):                      # warm-up: allocations, attributes, workspace growth
                    self.forward(self._tok_in)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    self._tok_out = self.forward(self._tok_in)
            self._graph = graph
            ok = True
        except Exception:
            self._graph = None
            ok = False
        torch.cuda.synchronize(self.device)
        self.pos.copy_(saved)
        self._pos_host = saved_host
        return ok

    def decode_step(self, tok: torch.Tensor) -> torch.Tensor:
        if self._graph is None:
            return self.forward(tok.view(self.batch, 1))
        self._claim_positions(1)        # the replayed step advances the device-side position
        self._tok_in.copy_(tok.view(self.batch, 1))
        self._graph.replay()
        return self._tok_out

    def generate(self, prompt: torch.Tensor, steps: int) -> torch.Tensor:
        """Greedy decoding: prompt int64 [B, Tp] -> generated tokens [B, steps]."""
        if prompt.shape[1] + max(steps - 1, 0) > self.cfg.max_pos:
            raise ValueError(f"prompt of {prompt.shape[1]} tokens plus {steps} steps exceeds max_pos = {self.cfg.max_pos}")
        self.reset()
        tok = self.forward(prompt)
        outs = [tok]
        for _ in range(steps - 1):
            tok = self.decode_step(tok).clone()
            outs.append(tok)
        self.check()
        return torch.stack(outs, dim=1)
