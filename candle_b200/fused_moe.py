"""``FusedMoeGGUF``: routing plus the three grouped expert matmuls of a quantized mixture-of-experts block.

Mirrors candle-transformers/src/fused_moe.rs:222-301 (``FusedMoeGGUF::forward``): router logits -> softmax -> the
``num_experts_per_tok`` largest weights per token (optionally renormalised) -> (token, expert) pairs sorted by expert ->
``moe_gemm_gguf`` for gate and up, ``up * act(gate)``, ``moe_gemm_gguf`` for down with the routing weights applied ->
sum over the token's experts.  The router is a dense f32 linear layer (candle de-quantizes it at load); routing itself is
a handful of small tensor operations; everything heavy goes through the expert-indexed GEMV of libcandle_q_b200.

Expert parallelism: a rank may own a contiguous range of experts.  Pairs routed elsewhere write nothing (the kernels
skip expert ids outside their range), every pair is produced by exactly one rank, so summing the pair outputs across
ranks adds one value and zeros - exact in any order - and the result has the same bits for any number of ranks.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .capi import CandleQError
from .moe import moe_gemm_gguf
from .quantized import QTensor


def route(router_logits: torch.Tensor, num_experts_per_tok: int, norm_topk_prob: bool):
    """fused_moe.rs:233-247: softmax over experts, the top-k of each token (descending), optional renormalisation.
    Returns (topk_weights f32 [tokens, k], topk_ids int64 [tokens, k])."""
    weights = torch.softmax(router_logits.to(torch.float32), dim=-1)
    order = torch.argsort(weights, dim=-1, descending=True, stable=True)
    topk_ids = order[:, :num_experts_per_tok].contiguous()
    topk_weights = weights.gather(-1, topk_ids)
    if norm_topk_prob:
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
    return topk_weights, topk_ids


def sort_pairs(topk_ids: torch.Tensor):
    """fused_moe.rs:249-260: the flattened (token, slot) pairs sorted by expert id.
    Returns (expert_ids int32 [pairs] ascending, sorted_token_ids int32 [pairs] = pair indices in that order)."""
    expert_ids, sorted_token_ids = torch.sort(topk_ids.reshape(-1), stable=True)
    return expert_ids.to(torch.int32), sorted_token_ids.to(torch.int32)


class FusedMoeGGUF:
    def __init__(self, gate: torch.Tensor, gate_experts: QTensor, up_experts: QTensor, down_experts: QTensor,
                 num_experts_per_tok: int, norm_topk_prob: bool = True, prefill_dtype: torch.dtype = torch.bfloat16,
                 expert_offset: int = 0, group=None, world: int = 1):
        """gate: router weight f32 [num_experts, hidden].  *_experts: rank-3 QTensors [local experts, n, k] holding the
        experts [expert_offset, expert_offset + local experts) of the layer."""
        for w in (gate_experts, up_experts, down_experts):
            if w.rank() != 3:
                raise CandleQError("FusedMoeGGUF expects expert weights of rank 3 [experts, n, k]")
        if gate_experts.shape != up_experts.shape or down_experts.shape[1] != gate_experts.shape[2] or \
                down_experts.shape[2] != gate_experts.shape[1]:
            raise CandleQError("FusedMoeGGUF: expert weight shapes do not fit together")
        self.gate, self.gate_experts, self.up_experts, self.down_experts = gate, gate_experts, up_experts, down_experts
        self.num_experts_per_tok, self.norm_topk_prob, self.prefill_dtype = num_experts_per_tok, norm_topk_prob, prefill_dtype
        self.expert_offset, self.group, self.world = expert_offset, group, world

    def forward(self, xs: torch.Tensor, is_prefill: bool) -> torch.Tensor:
        batch, seq_len, hidden = xs.shape
        original_dtype = xs.dtype
        x = xs.reshape(-1, hidden).to(torch.float32).contiguous()
        num_tokens, k = x.shape[0], self.num_experts_per_tok
        topk_weights, topk_ids = route(torch.nn.functional.linear(x, self.gate), k, self.norm_topk_prob)
        expert_ids, sorted_token_ids = sort_pairs(topk_ids)
        local_ids = expert_ids - self.expert_offset          # ids outside [0, local experts) are skipped by the kernels
        xin = x.to(self.prefill_dtype) if is_prefill else x  # the reference casts for its prefill kernel (moe.rs:310-333)
        zero = self.world > 1                                 # pairs of other ranks must read as zero
        gate = moe_gemm_gguf(xin, self.gate_experts, None, sorted_token_ids, local_ids, k, is_prefill, zero_init=zero)
        up = moe_gemm_gguf(xin, self.up_experts, None, sorted_token_ids, local_ids, k, is_prefill, zero_init=zero)
        down_in = up * torch.nn.functional.silu(gate)         # [pairs, intermediate]
        if is_prefill:
            down_in = down_in.to(self.prefill_dtype)
        ys = moe_gemm_gguf(down_in, self.down_experts, topk_weights, sorted_token_ids, local_ids, k, is_prefill, zero_init=zero)
        if self.world > 1:
            dist.all_reduce(ys, op=dist.ReduceOp.SUM, group=self.group)      # one value plus zeros per element: exact
        ys = ys.reshape(num_tokens, k, hidden).sum(dim=1)
        return ys.to(original_dtype).reshape(batch, seq_len, hidden)
