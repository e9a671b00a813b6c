"""The two decoder harnesses against a CPU forward of the same model, step by step through whole forward passes.

The other decoder tests compare the harness with itself (graph vs eager, tensor-parallel vs one GPU, fused vs unfused
producers); a systematic glue error - RoPE pairing, the grouped-query head map, a KV-cache position, the expert routing -
would pass all of them.  Here a two-layer model of each kind runs a prompt and several greedy steps on the GPU in
CPU-exact activation mode while recording every intermediate tensor (`model.tap`), and a numpy forward - written from
the reference models, its matmuls the oracle's restatement of the reference's CPU `k_quants::matmul` on the weights read
back from the device - recomputes every step from the GPU's inputs OF THAT STEP:

    norm -> q/k/v projections -> rotary embedding + KV-cache store -> attention over the cache -> output projection ->
    residual + norm -> (gate|up, SwiGLU, down) or (router, top-k, expert gate|up, SwiGLU, expert down, weighted slot sum)
    ... -> final norm -> vocabulary head -> greedy token.

Every step must agree within 1e-3 (max |a - ref| / max |ref|; measured around 1e-7).  The check is per step rather than on
the final logits of a free-running CPU model because activation quantization is a step function: a difference of one
f32 unit in the last place before a matmul can flip one rounded int8 value, which moves that row's outputs by about 1e-3
and then spreads - two correct implementations that order their f32 additions differently drift apart by about 1e-2
within two layers (observed here), which says nothing about either.  Re-synchronising at every step keeps the comparison
exact and still walks the whole data flow, the cache positions of the decode steps included.

The numpy forward follows the reference models, not the harness code:
  dense: candle-transformers/src/models/quantized_llama.rs:178-262, 568-596 (interleaved RoPE, f32 KV cache, repeat_kv);
  MoE  : candle-transformers/src/models/quantized_qwen3_moe.rs:168-218, 295-421 and fused_moe.rs:222-301 (per-head RMSNorm
         of q and k, non-interleaved RoPE, softmax -> top-k -> renormalise, sum over the slots in slot order).
No reference test pins the MoE index semantics (parity unpinned by the reference for those rows); the oracle for them is
this per-expert composition of pinned dots.
"""
import numpy as np
import pytest
import torch

from candle_b200.decoder import DecoderConfig, LlamaShapedDecoder
from candle_b200.moe_decoder import MoeDecoderConfig, MoeShapedDecoder
from candle_b200.quantized import set_activation_mode
from helpers import rel_err

pytestmark = pytest.mark.gpu
F = np.float32
TOL = 1e-3


def _blocks(qt):
    """GGUF bytes of a device tensor as uint8 [rows, row_bytes] (rows = product of the leading dims)."""
    raw = np.frombuffer(qt.data(), dtype=np.uint8)
    rows = int(np.prod(qt.shape[:-1]))
    return raw.reshape(rows, -1).copy()


def _rms_norm(x, w, eps):
    ms = (x.astype(F) ** 2).mean(axis=-1, keepdims=True, dtype=F)
    return (x / np.sqrt(ms + F(eps))).astype(F) * w


def _rope_interleaved(x, cos, sin):
    """x [T, H, D]: pairs (2i, 2i+1) rotated by the angle of position t (candle's rope_i)."""
    x0, x1 = x[..., 0::2], x[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    out = np.empty_like(x)
    out[..., 0::2] = x0 * c - x1 * s
    out[..., 1::2] = x0 * s + x1 * c
    return out


def _rope_neox(x, cos, sin):
    """x [T, H, D]: pairs (i, i + D/2) (candle's rope)."""
    h = x.shape[-1] // 2
    x0, x1 = x[..., :h], x[..., h:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=-1).astype(F)


def _attention(q, kc, vc, pos0):
    """q [T, Hq, D] at positions pos0.., caches [Hkv, ctx, D] already holding positions < pos0 + T.  Causal softmax
    attention with query head h reading KV head h // (Hq / Hkv) (repeat_kv)."""
    T, hq, D = q.shape
    rep = hq // kc.shape[0]
    out = np.zeros((T, hq, D), dtype=F)
    for t in range(T):
        n_ctx = pos0 + t + 1
        for h in range(hq):
            k, v = kc[h // rep, :n_ctx], vc[h // rep, :n_ctx]
            sc = (k @ q[t, h]).astype(F) / F(np.sqrt(D))
            p = np.exp(sc - sc.max())
            out[t, h] = (p / p.sum()) @ v
    return out


def _silu_mul(g, u):
    return (g / (1.0 + np.exp(-g))).astype(F) * u


class _Lockstep:
    """Shared machinery: the reference KV caches, the tap dictionary of the running forward, the comparison."""

    def __init__(self, model, oracle):
        self.m, self.O, self.cfg = model, oracle, model.cfg
        c = self.cfg
        self.embd = model.tok_embd.cpu().numpy()
        self.cos, self.sin = model.cos.cpu().numpy(), model.sin.cpu().numpy()
        self.kc = [[np.zeros((c.n_kv_heads, c.max_pos, c.head_dim), dtype=F) for _ in range(model.batch)] for _ in model.layers]
        self.vc = [[np.zeros((c.n_kv_heads, c.max_pos, c.head_dim), dtype=F) for _ in range(model.batch)] for _ in model.layers]
        self.pos = 0
        self.worst = 0.0
        self.checked = 0

    def mm(self, dtype, x, w):
        return self.O.matmul(dtype, np.ascontiguousarray(x, dtype=F), w, w.shape[0])

    def same(self, what, got, ref):
        got = got.cpu().numpy() if torch.is_tensor(got) else got
        e = rel_err(got.reshape(ref.shape), ref)
        self.worst = max(self.worst, e)
        self.checked += 1
        assert e <= TOL, f"{what}: {e:.3e}"

    def caches_and_attention(self, li, tap, q_rot, k_rot, v, B, T, hq, hkv, hd):
        """KV store at positions pos..pos+T-1 of the reference caches, the device caches compared over the whole filled
        range, then attention of the GPU's rotated queries over the reference caches."""
        L = self.m.layers[li]
        att_ref = np.zeros((B, T, hq * hd), dtype=F)
        for b in range(B):
            self.kc[li][b][:, self.pos:self.pos + T] = k_rot[b].transpose(1, 0, 2)
            self.vc[li][b][:, self.pos:self.pos + T] = v[b].transpose(1, 0, 2)
            att_ref[b] = _attention(q_rot[b], self.kc[li][b], self.vc[li][b], self.pos).reshape(T, hq * hd)
        n = self.pos + T
        self.same(f"layer {li} k cache", L.k_cache[:, :, :n], np.stack([self.kc[li][b][:, :n] for b in range(B)]))
        self.same(f"layer {li} v cache", L.v_cache[:, :, :n], np.stack([self.vc[li][b][:, :n] for b in range(B)]))
        self.same(f"layer {li} attention", tap[f"{li}.att"], att_ref.reshape(B * T, -1))


class _DenseRef(_Lockstep):
    def __init__(self, model, oracle):
        super().__init__(model, oracle)
        self.w = [dict(wqk=_blocks(L.wqk.qtensor), wv=_blocks(L.wv.qtensor), wo=_blocks(L.wo.qtensor), gate_up=_blocks(L.gate_up.qtensor),
                       down=_blocks(L.down.qtensor), attn_norm=L.attn_norm.cpu().numpy(), ffn_norm=L.ffn_norm.cpu().numpy())
                  for L in model.layers]
        self.out_norm, self.output = model.out_norm.cpu().numpy(), _blocks(model.output.qtensor)

    def check(self, tokens, tap):
        """Every step of one forward pass of `tokens` [B, T] from the recorded tensors; returns the reference logits."""
        c, O = self.cfg, self.O
        B, T = tokens.shape
        hd, hq, hkv = c.head_dim, c.n_heads, c.n_kv_heads
        cos, sin = self.cos[self.pos:self.pos + T], self.sin[self.pos:self.pos + T]
        np_ = lambda k: tap[k].cpu().numpy()
        self.same("embedding", tap["0.x_in"], self.embd[tokens.reshape(-1)])
        for li, W in enumerate(self.w):
            x = np_(f"{li}.x_in") + (np_(f"{li}.delta_in") if f"{li}.delta_in" in tap else 0)
            self.same(f"layer {li} attn norm", tap[f"{li}.h_attn"], _rms_norm(x, W["attn_norm"], c.rms_eps))
            h = np_(f"{li}.h_attn")
            self.same(f"layer {li} wq|wk", tap[f"{li}.qk"], self.mm(O.Q4K, h, W["wqk"]))
            self.same(f"layer {li} wv", tap[f"{li}.v"], self.mm(O.Q6K, h, W["wv"]))
            qk, v = np_(f"{li}.qk"), np_(f"{li}.v").reshape(B, T, hkv, hd)
            q_rot = np.stack([_rope_interleaved(qk[b * T:(b + 1) * T, :hq * hd].reshape(T, hq, hd), cos, sin) for b in range(B)])
            k_rot = np.stack([_rope_interleaved(qk[b * T:(b + 1) * T, hq * hd:].reshape(T, hkv, hd), cos, sin) for b in range(B)])
            self.same(f"layer {li} rope q", tap[f"{li}.q_rot"][:, :hq * hd], q_rot.reshape(B * T, -1))
            q_gpu = np_(f"{li}.q_rot")[:, :hq * hd].reshape(B, T, hq, hd)
            self.caches_and_attention(li, tap, q_gpu, k_rot, v, B, T, hq, hkv, hd)
            self.same(f"layer {li} wo", tap[f"{li}.wo"], self.mm(O.Q4K, np_(f"{li}.att"), W["wo"]))
            self.same(f"layer {li} residual", tap[f"{li}.x_mid"], x)
            x = np_(f"{li}.x_mid") + np_(f"{li}.wo")
            self.same(f"layer {li} ffn norm", tap[f"{li}.h_ffn"], _rms_norm(x, W["ffn_norm"], c.rms_eps))
            self.same(f"layer {li} gate|up", tap[f"{li}.gu"], self.mm(O.Q4K, np_(f"{li}.h_ffn"), W["gate_up"]))
            gu = np_(f"{li}.gu")
            self.same(f"layer {li} swiglu", tap[f"{li}.act"], _silu_mul(gu[:, :c.ffn], gu[:, c.ffn:]))
            self.same(f"layer {li} down", tap[f"{li}.down"], self.mm(O.Q6K, np_(f"{li}.act"), W["down"]))
        x = np_("final.x_in") + np_("final.delta_in")
        self.same("final norm", tap["final.h"], _rms_norm(x, self.out_norm, c.rms_eps))
        last = np_("final.h").reshape(B, T, -1)[:, -1]
        logits = self.mm(O.Q6K, last, self.output)
        self.same("logits", self.m.last_logits, logits)
        self.pos += T
        return logits


class _MoeRef(_Lockstep):
    def __init__(self, model, oracle):
        super().__init__(model, oracle)
        c = self.cfg
        self.w = [dict(attn_norm=L.attn_norm.cpu().numpy(), ffn_norm=L.ffn_norm.cpu().numpy(), q_norm=L.q_norm.cpu().numpy(),
                       k_norm=L.k_norm.cpu().numpy(), wqkv=_blocks(L.wqkv.qtensor), wo=_blocks(L.wo.qtensor), router=L.router.cpu().numpy(),
                       gate_up=_blocks(L.gate_up).reshape(c.experts, 2 * c.expert_ffn, -1), down=_blocks(L.down).reshape(c.experts, c.d_model, -1))
                  for L in model.layers]
        self.out_norm, self.output = model.out_norm.cpu().numpy(), _blocks(model.output.qtensor)

    def check(self, tokens, tap):
        c, O = self.cfg, self.O
        B, T = tokens.shape
        hd, hq, hkv, f, k = c.head_dim, c.n_heads, c.n_kv_heads, c.expert_ffn, c.experts_per_tok
        cos, sin = self.cos[self.pos:self.pos + T], self.sin[self.pos:self.pos + T]
        np_ = lambda key: tap[key].cpu().numpy()
        self.same("embedding", tap["0.x_in"], self.embd[tokens.reshape(-1)])
        for li, W in enumerate(self.w):
            x = np_(f"{li}.x_in") + (np_(f"{li}.delta_in") if f"{li}.delta_in" in tap else 0)
            self.same(f"layer {li} attn norm", tap[f"{li}.h_attn"], _rms_norm(x, W["attn_norm"], c.rms_eps))
            self.same(f"layer {li} wqkv", tap[f"{li}.qkv"], self.mm(O.Q6K, np_(f"{li}.h_attn"), W["wqkv"]))
            qkv = np_(f"{li}.qkv")
            q = qkv[:, :hq * hd].reshape(B, T, hq, hd)
            kk = qkv[:, hq * hd:(hq + hkv) * hd].reshape(B, T, hkv, hd)
            v = qkv[:, (hq + hkv) * hd:].reshape(B, T, hkv, hd)
            q_rot = np.stack([_rope_neox(_rms_norm(q[b], W["q_norm"], c.rms_eps), cos, sin) for b in range(B)])
            k_rot = np.stack([_rope_neox(_rms_norm(kk[b], W["k_norm"], c.rms_eps), cos, sin) for b in range(B)])
            self.same(f"layer {li} q norm + rope", tap[f"{li}.q_rot"][:, :hq * hd], q_rot.reshape(B * T, -1))
            q_gpu = np_(f"{li}.q_rot")[:, :hq * hd].reshape(B, T, hq, hd)
            self.caches_and_attention(li, tap, q_gpu, k_rot, v, B, T, hq, hkv, hd)
            self.same(f"layer {li} wo", tap[f"{li}.wo"], self.mm(O.Q6K, np_(f"{li}.att"), W["wo"]))
            x = np_(f"{li}.x_mid") + np_(f"{li}.wo")
            self.same(f"layer {li} ffn norm", tap[f"{li}.h_ffn"], _rms_norm(x, W["ffn_norm"], c.rms_eps))
            h = np_(f"{li}.h_ffn")
            # router: f32 linear -> softmax -> top-k (descending, lowest index among equals) -> renormalise
            logits = (h @ W["router"].T).astype(F)
            self.same(f"layer {li} router logits", tap[f"{li}.router_logits"], logits)
            lg = np_(f"{li}.router_logits")
            p = np.exp(lg - lg.max(axis=-1, keepdims=True))
            p = (p / p.sum(axis=-1, keepdims=True)).astype(F)
            ids_gpu, w_gpu = np_(f"{li}.ids"), np_(f"{li}.route_w")
            for r in range(B * T):
                ids = np.argsort(-p[r], kind="stable")[:k]
                # two probabilities closer than f32 rounding may swap places: compare ids only where the order is clear
                gaps = np.abs(np.diff(np.sort(p[r])[::-1][:k + 1]))
                if gaps.min() > 1e-6:
                    assert np.array_equal(ids_gpu[r], ids), f"layer {li} row {r}: experts {ids_gpu[r]} vs {ids}"
                pw = p[r][ids_gpu[r]]
                assert rel_err(w_gpu[r], pw / pw.sum() if c.norm_topk_prob else pw) <= TOL
            # experts: per (row, slot) pair, from the GPU's ids, step by step
            gu_gpu, act_gpu = np_(f"{li}.gu"), np_(f"{li}.act")
            gu_ref = np.stack([np.stack([self.mm(O.Q4K, h[r:r + 1], W["gate_up"][ids_gpu[r, s]])[0] for s in range(k)]) for r in range(B * T)])
            self.same(f"layer {li} expert gate|up", gu_gpu, gu_ref)
            self.same(f"layer {li} expert swiglu", act_gpu, _silu_mul(gu_gpu[..., :f], gu_gpu[..., f:]))
            dn_ref = np.stack([np.stack([self.mm(O.Q4K, act_gpu[r, s][None, :], W["down"][ids_gpu[r, s]])[0] for s in range(k)]) for r in range(B * T)])
            self.same(f"layer {li} expert down", tap[f"{li}.down"], dn_ref)
            dn = np_(f"{li}.down")
            acc = np.zeros((B * T, c.d_model), dtype=F)
            for s in range(k):      # slot order, as sum(D::Minus2)
                acc = acc + dn[:, s] * w_gpu[:, s:s + 1]
            self.same(f"layer {li} slot sum", tap[f"{li}.moe"], acc)
        x = np_("final.x_in") + np_("final.delta_in")
        self.same("final norm", tap["final.h"], _rms_norm(x, self.out_norm, c.rms_eps))
        last = np_("final.h").reshape(B, T, -1)[:, -1]
        logits = self.mm(O.Q6K, last, self.output)
        self.same("logits", self.m.last_logits, logits)
        self.pos += T
        return logits


def _run(model, ref, prompt, steps):
    """Prompt, then `steps` greedy decode steps; every forward pass is checked step by step and its token against the
    arg-max of the reference logits (where the two best logits are not within rounding of each other)."""
    model.reset()
    toks = prompt
    for step in range(steps + 1):
        model.tap = {}
        tok = model.forward(toks)
        logits = ref.check(toks.cpu().numpy(), model.tap)
        top2 = np.sort(logits, axis=-1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 1e-4 * np.abs(logits).max()
        assert np.array_equal(tok.cpu().numpy()[clear], logits.argmax(axis=-1)[clear]), f"greedy token differs at step {step}"
        toks = tok.view(-1, 1)
    model.tap = None
    model.check()
    assert ref.checked > 20 * (steps + 1)
    return ref.worst


@pytest.mark.parametrize("prompt_len", [19, 50])
def test_dense_decoder_matches_cpu_forward(oracle, cuda_dev, prompt_len):
    """prompt_len 19: 38 rows, split-context attention; 50: 100 rows, one CTA per (sequence, head, query).  Both prompts
    run the tcgen05 prompt kernels, the decode steps the GEMV; 8 query heads share 2 KV heads."""
    cfg = DecoderConfig(layers=2, d_model=512, n_heads=8, n_kv_heads=2, head_dim=128, ffn=1024, vocab=1024, max_pos=64)
    m = LlamaShapedDecoder(cfg, cuda_dev, batch=2, seed=3)
    prompt = torch.randint(0, cfg.vocab, (2, prompt_len), device=cuda_dev, generator=torch.Generator(device=cuda_dev).manual_seed(2))
    set_activation_mode(True)       # the reference's CPU arithmetic (Q8_K activations) in every matmul
    try:
        worst = _run(m, _DenseRef(m, oracle), prompt, steps=5)
    finally:
        set_activation_mode(False)
    assert worst <= 1e-5            # far inside the bar: every step differs by f32 summation order only


@pytest.mark.parametrize("prompt_len", [5, 40])
def test_moe_decoder_matches_cpu_forward(oracle, cuda_dev, prompt_len):
    """prompt_len 5: 10 rows x 4 slots stay below the grouped-GEMM threshold (expert-indexed GEMV); 40: the prompt runs
    through the grouped tensor-core GEMM.  Decode steps use the expert-indexed GEMV in both."""
    cfg = MoeDecoderConfig(layers=2, d_model=512, n_heads=4, n_kv_heads=2, experts=16, experts_per_tok=4, expert_ffn=256,
                           vocab=1024, max_pos=64)
    m = MoeShapedDecoder(cfg, cuda_dev, batch=2, seed=4)
    prompt = torch.randint(0, cfg.vocab, (2, prompt_len), device=cuda_dev, generator=torch.Generator(device=cuda_dev).manual_seed(3))
    set_activation_mode(True)
    try:
        worst = _run(m, _MoeRef(m, oracle), prompt, steps=4)
    finally:
        set_activation_mode(False)
    assert worst <= 1e-5
