"""Mixture-of-experts decoder harness: a caller of the expert-indexed matmuls with the shape of Qwen3-30B-A3B
(48 layers, d = 2048, 32 query / 4 KV heads of 128, 128 experts of width 768, 8 per token).

Structure follows candle-transformers/src/models/quantized_qwen3_moe.rs:168-218, 295-304, 398-421 and
candle-transformers/src/fused_moe.rs:222-301: f32 residual stream, RMSNorm, q/k/v projections, per-head RMSNorm of q
and k, non-interleaved RoPE, GQA attention over an f32 KV cache, output projection; then router -> softmax -> top-8 ->
renormalise -> expert gate/up -> SwiGLU -> expert down -> weighted sum.  Weights are random GGUF blocks: experts Q4_K,
attention and the output head Q6_K.  Deviation from the reference model: attention runs in f32 (the reference casts q,
k, v to its --dtype, bf16 by default, for the attention matmuls only).

Parallelism: the experts of a layer are split contiguously over the ranks (expert parallel); attention, router and head
are replicated.  A rank passes expert ids shifted by its first expert, pairs routed elsewhere are skipped and stay
zero, and the pair outputs are summed across ranks - one value plus zeros per element, exact in any order - so tokens
are bit-identical for any number of ranks.
"""
from __future__ import annotations

import dataclasses
import math

import torch
import torch.distributed as dist

from . import capi
from .decoder import LlamaShapedDecoder
from .moe import moe_prefill_gemm
from .quantized import GgmlDType, QMatMul, QTensor
from .synth import random_blocks


@dataclasses.dataclass
class MoeDecoderConfig:
    layers: int = 48
    d_model: int = 2048
    n_heads: int = 32
    n_kv_heads: int = 4
    head_dim: int = 128
    experts: int = 128
    experts_per_tok: int = 8
    expert_ffn: int = 768
    vocab: int = 151936
    rope_theta: float = 1000000.0
    rms_eps: float = 1e-6
    max_pos: int = 2048
    norm_topk_prob: bool = True

    @staticmethod
    def qwen3_30b_a3b() -> "MoeDecoderConfig":
        return MoeDecoderConfig()

    @staticmethod
    def tiny() -> "MoeDecoderConfig":
        return MoeDecoderConfig(layers=2, d_model=512, n_heads=4, n_kv_heads=2, experts=16, experts_per_tok=4, expert_ffn=256,
                                vocab=2048, max_pos=128)

    def active_weight_bytes_per_token(self) -> int:
        q4, q6 = 144 / 256, 210 / 256
        d, hq, hkv = self.d_model, self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        att = ((hq + 2 * hkv) * d + d * hq) * q6
        moe = self.experts_per_tok * 3 * self.expert_ffn * d * q4
        return int(self.layers * (att + moe) + self.vocab * d * q6)


class _Layer:
    pass


def _qmm(dtype, n, k, seed, device):
    return QMatMul.from_qtensor(QTensor.from_device_blocks(random_blocks(dtype, n, k, seed, device), dtype, (n, k)))


class MoeShapedDecoder:
    def __init__(self, cfg: MoeDecoderConfig, device, rank: int = 0, world: int = 1, batch: int = 1, seed: int = 0, group=None):
        if cfg.experts % world:
            raise ValueError("the world size must divide the number of experts")
        self.cfg, self.device, self.rank, self.world, self.batch, self.group = cfg, torch.device(device), rank, world, batch, group
        d, hd, f = cfg.d_model, cfg.head_dim, cfg.expert_ffn
        self.e_local = cfg.experts // world
        self.e0 = rank * self.e_local
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        rnd = lambda *shape, scale=1.0: torch.randn(shape, device=self.device, generator=g) * scale
        self.tok_embd = rnd(cfg.vocab, d, scale=0.02)
        qkv_rows = (cfg.n_heads + 2 * cfg.n_kv_heads) * hd
        self.layers = []
        for li in range(cfg.layers):
            L = _Layer()
            s = seed * 100003 + li * 64
            L.attn_norm, L.ffn_norm = 1.0 + 0.1 * rnd(d), 1.0 + 0.1 * rnd(d)
            L.q_norm, L.k_norm = 1.0 + 0.1 * rnd(hd), 1.0 + 0.1 * rnd(hd)
            L.wqkv = _qmm(GgmlDType.Q6K, qkv_rows, d, s + 1, self.device)            # [q heads | k heads | v heads]
            L.wo = _qmm(GgmlDType.Q6K, d, cfg.n_heads * hd, s + 2, self.device)
            L.router = rnd(cfg.experts, d, scale=0.05)
            # expert e of the layer is generated from a seed that does not depend on the world size
            gu = torch.stack([random_blocks(GgmlDType.Q4K, 2 * f, d, (s + 3) * 4096 + e, self.device)
                              for e in range(self.e0, self.e0 + self.e_local)])
            dn = torch.stack([random_blocks(GgmlDType.Q4K, d, f, (s + 4) * 4096 + e, self.device)
                              for e in range(self.e0, self.e0 + self.e_local)])
            L.gate_up = QTensor.from_device_blocks(gu.reshape(-1), GgmlDType.Q4K, (self.e_local, 2 * f, d))    # rows [gate | up]
            L.down = QTensor.from_device_blocks(dn.reshape(-1), GgmlDType.Q4K, (self.e_local, d, f))
            L.k_cache = torch.zeros((batch, cfg.n_kv_heads, cfg.max_pos, hd), device=self.device)
            L.v_cache = torch.zeros((batch, cfg.n_kv_heads, cfg.max_pos, hd), device=self.device)
            self.layers.append(L)
        self.out_norm = 1.0 + 0.1 * rnd(d)
        self.output = _qmm(GgmlDType.Q6K, cfg.vocab, d, seed * 100003 + 999983, self.device)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=self.device, dtype=torch.float32) / hd))
        ang = torch.arange(cfg.max_pos, device=self.device, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().contiguous(), ang.sin().contiguous()
        self.pos = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._pos_host = 0      # host copy of pos: positions are checked against max_pos before anything is launched
        self._graph = None
        self._att_scratch = None
        self._router_counters = None    # arrival counters of the one-launch router
        self.fuse_quantize = True       # decode steps: norm and attention store Q8_1 containers directly
        self.tap = None                 # tests set a dict here: forward() then records copies of its intermediate tensors
        self.hq_l, self.hkv_l = cfg.n_heads, cfg.n_kv_heads      # attention is replicated: every rank owns all heads
        if world > 1:       # the peer-memory exchange of expert outputs (library collectives when peers cannot be mapped)
            from .parallel import make_gatherer
            self.gather = make_gatherer(group, world, self.device)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)

    # the norm and attention helpers are those of the dense harness
    _norm = LlamaShapedDecoder._norm
    _rec = LlamaShapedDecoder._rec
    reset = LlamaShapedDecoder.reset
    check = LlamaShapedDecoder.check
    _claim_positions = LlamaShapedDecoder._claim_positions
    capture_decode_step = LlamaShapedDecoder.capture_decode_step
    decode_step = LlamaShapedDecoder.decode_step
    generate = LlamaShapedDecoder.generate

    _norm_q8 = LlamaShapedDecoder._norm_q8

    def _attention(self, qkv, L, B, T, out, q8: bool = False):
        """`q8` (at most 64 queries): the result goes out as the Q8_1 containers the next matmul reads."""
        cfg, lib, hd = self.cfg, capi.lib(), self.cfg.head_dim
        st = torch.cuda.current_stream(self.device).cuda_stream
        stride = (cfg.n_heads + 2 * cfg.n_kv_heads) * hd
        scale = 1.0 / math.sqrt(hd)
        if B * T <= 64:
            if self._att_scratch is None:
                n = lib.cq_attention_split_scratch_floats(64, 1, cfg.n_heads, cfg.max_pos)
                self._att_scratch = (torch.empty(n, dtype=torch.float32, device=self.device),
                                     torch.zeros(64 * cfg.n_heads, dtype=torch.int32, device=self.device))
            scratch, counters = self._att_scratch
            lib.cq_attention_split(qkv.data_ptr(), L.k_cache.data_ptr(), L.v_cache.data_ptr(), out.data_ptr(), 1 if q8 else 0,
                                   self.pos.data_ptr(), scratch.data_ptr(), counters.data_ptr(), B, T, cfg.n_heads, cfg.n_kv_heads, hd,
                                   cfg.max_pos, scale, stride, cfg.n_heads * hd // 32, st)
        elif q8:
            raise ValueError("Q8_1 attention output is for at most 64 queries")
        else:
            lib.cq_attention_f32(qkv.data_ptr(), L.k_cache.data_ptr(), L.v_cache.data_ptr(), out.data_ptr(), self.pos.data_ptr(),
                                 B, T, cfg.n_heads, cfg.n_kv_heads, hd, cfg.max_pos, scale, stride, st)

    def _moe(self, h: torch.Tensor, L, key: str = "", h8: torch.Tensor | None = None) -> torch.Tensor:
        """fused_moe.rs:222-301 for rows h [R, d] -> [R, d].  `key`: prefix of the recorded intermediates (tests).
        `h8` (decode steps): the same rows as Q8_1 containers - the expert matmuls then run without quantize launches."""
        cfg, lib = self.cfg, capi.lib()
        R, k, f = h.shape[0], cfg.experts_per_tok, cfg.expert_ffn
        st = torch.cuda.current_stream(self.device).cuda_stream
        ids = torch.empty((R, k), dtype=torch.int32, device=self.device)
        w = torch.empty((R, k), dtype=torch.float32, device=self.device)
        small = R <= 64 and cfg.d_model % 4 == 0       # a decode step: logits + routing, and the slot sum, as one launch each
        if small:
            if self._router_counters is None:
                self._router_counters = torch.zeros(64, dtype=torch.int32, device=self.device)
            logits = torch.empty((R, cfg.experts), dtype=torch.float32, device=self.device)
            lib.cq_moe_router_f32(h.data_ptr(), L.router.data_ptr(), logits.data_ptr(), ids.data_ptr(), w.data_ptr(),
                                  self._router_counters.data_ptr(), R, cfg.experts, cfg.d_model, k, 1 if cfg.norm_topk_prob else 0, st)
        else:
            logits = torch.nn.functional.linear(h, L.router)
            lib.cq_moe_route_f32(logits.data_ptr(), ids.data_ptr(), w.data_ptr(), R, cfg.experts, k, 1 if cfg.norm_topk_prob else 0, st)
        self._rec(key + "router_logits", logits), self._rec(key + "ids", ids), self._rec(key + "route_w", w)
        local = ids - self.e0 if self.world > 1 else ids           # other ranks' experts fall outside [0, e_local): skipped
        zero = self.world > 1
        a = torch.empty((R, k, f), dtype=torch.float32, device=self.device)
        # The switch between the two arithmetics (Q8_1 GEMV below it, Q8_K tensor-core GEMM above) depends on the MODEL's expert
        # count, not on how many experts this rank holds: the same step must take the same path at every world size.
        if R * k >= max(64, 4 * cfg.experts):     # prompt: pairs sorted by expert, grouped GEMM on the tensor cores
            experts, pairs = torch.sort(local.reshape(-1), stable=True)
            gu = moe_prefill_gemm(h, L.gate_up, None, pairs, experts, k, zero_init=zero)          # [R * k, 2f]
            lib.cq_silu_mul_f32(gu.data_ptr(), a.data_ptr(), R * k, f, st)
            y = moe_prefill_gemm(a.view(R * k, f), L.down, torch.ones(R * k, device=self.device), pairs, experts, k,
                                 zero_init=zero).view(R, k, -1)
        elif h8 is not None and f % 32 == 0:
            gu = L.gate_up.indexed_moe_forward_q8_1(h8, 1, local, zero_init=zero)                 # [R, k, 2f]
            fp = capi.pad(f, 512)
            a8 = torch.empty((R * k, fp // 32 * 36), dtype=torch.uint8, device=self.device)
            lib.cq_silu_mul_q8_1(gu.data_ptr(), a8.data_ptr(), R * k, f, fp, st)
            y = L.down.indexed_moe_forward_q8_1(a8, k, local, zero_init=zero)                     # [R, k, d]
            a = a8
        else:
            gu = L.gate_up.indexed_moe_forward(h.view(R, 1, -1), local, zero_init=zero)           # [R, k, 2f]
            lib.cq_silu_mul_f32(gu.data_ptr(), a.data_ptr(), R * k, f, st)
            y = L.down.indexed_moe_forward(a, local, zero_init=zero)                              # [R, k, d]
        self._rec(key + "gu", gu.view(R, k, 2 * f)), self._rec(key + "act", a), self._rec(key + "down", y)
        if self.world > 1:
            # every (token, slot) row of y was computed by the rank that holds its expert: all-gather by slot, then the
            # slot-order sum below.  Few rows: one peer-memory kernel; many: an all-reduce (one value plus zeros: exact).
            got = None
            xr = getattr(getattr(self, "gather", None), "exchange_rows", None)
            if xr is not None:
                got = xr(y.view(R * k, -1), local.reshape(-1).contiguous(), self.e_local)
            if got is None:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            else:
                y = got.view(R, k, -1)
        if small:
            y = y.contiguous()
            out = torch.empty((R, y.shape[-1]), dtype=torch.float32, device=self.device)
            lib.cq_moe_weighted_sum_f32(y.data_ptr(), w.data_ptr(), out.data_ptr(), R, k, y.shape[-1], st)
            return out
        return (y * w.unsqueeze(-1)).sum(dim=1)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens int64 [B, T] at cache positions pos .. pos+T-1 -> greedy next token [B]; advances pos."""
        cfg, B, T = self.cfg, tokens.shape[0], tokens.shape[1]
        self._claim_positions(T)
        hd, R, lib = cfg.head_dim, B * T, capi.lib()
        st = torch.cuda.current_stream(self.device).cuda_stream
        q_cols, kv_cols = cfg.n_heads * hd, cfg.n_kv_heads * hd
        stride = q_cols + 2 * kv_cols
        fused = self.fuse_quantize and R <= 8 and lib.cqh_get_act_mode() == 0 and cfg.d_model % 512 == 0 and q_cols % 512 == 0
        with torch.cuda.device(self.device):
            x = self.tok_embd.index_select(0, tokens.reshape(-1))
            delta = None
            for li, L in enumerate(self.layers):
                self._rec(f"{li}.x_in", x)
                if delta is not None:
                    self._rec(f"{li}.delta_in", delta)
                if fused:       # decode steps: the producers store Q8_1 containers, the matmuls skip their quantize launch
                    h = self._norm_q8(x, delta, L.attn_norm)
                    qkv = L.wqkv.forward_q8_1(h)
                else:
                    h = self._norm(x, delta, L.attn_norm)
                    qkv = L.wqkv.forward(h)                                                       # [R, stride]
                self._rec(f"{li}.h_attn", h), self._rec(f"{li}.qkv", qkv)
                base = qkv.data_ptr()
                lib.cq_qknorm_rope_store_kv_f32(base, base + 4 * q_cols, base + 4 * (q_cols + kv_cols), L.q_norm.data_ptr(),
                                                L.k_norm.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), self.pos.data_ptr(),
                                                L.k_cache.data_ptr(), L.v_cache.data_ptr(), B, T, cfg.n_heads, cfg.n_kv_heads, hd,
                                                cfg.max_pos, stride, stride, stride, cfg.rms_eps, 1, st)
                self._rec(f"{li}.q_rot", qkv)
                if fused:
                    att = torch.empty((R, q_cols // 32 * 36), dtype=torch.uint8, device=self.device)
                    self._attention(qkv, L, B, T, att, q8=True)
                    delta = L.wo.forward_q8_1(att)
                else:
                    att = torch.empty((R, q_cols), dtype=torch.float32, device=self.device)
                    self._attention(qkv, L, B, T, att)
                    delta = L.wo.forward(att)
                self._rec(f"{li}.att", att)
                self._rec(f"{li}.x_mid", x), self._rec(f"{li}.wo", delta)
                if fused and R * cfg.experts_per_tok < max(64, 4 * cfg.experts):     # f32 rows for the router, Q8_1 for the experts
                    h = torch.empty_like(x)
                    h8 = torch.empty((R, cfg.d_model // 32 * 36), dtype=torch.uint8, device=self.device)
                    lib.cq_add_rms_norm_f32_q8_1(x.data_ptr(), delta.data_ptr(), L.ffn_norm.data_ptr(), h.data_ptr(), h8.data_ptr(),
                                                 R, cfg.d_model, cfg.d_model, cfg.rms_eps, st)
                    delta = self._moe(h, L, f"{li}.", h8)
                else:
                    h = self._norm(x, delta, L.ffn_norm)
                    delta = self._moe(h, L, f"{li}.")
                self._rec(f"{li}.h_ffn", h), self._rec(f"{li}.moe", delta)
            self._rec("final.x_in", x), self._rec("final.delta_in", delta)
            h = self._norm(x, delta, self.out_norm)
            capi.check("moe decoder glue")
            self._rec("final.h", h)
            last = h.view(B, T, cfg.d_model)[:, -1, :].contiguous()
            logits = self.output.forward(last)
            self.last_logits = logits       # last position (read by tests)
            # first maximum, as argmax over the row
            mx = logits.max(dim=-1, keepdim=True).values
            ar = torch.arange(logits.shape[-1], device=self.device)
            tok = torch.where(logits == mx, ar, ar.new_full((), 1 << 40)).min(dim=-1).values
            self.pos += T
        return tok
