"""Tensor-parallel decoder for the Muse-Glimmer block: batched prefill and greedy / sampled decode with
one rank per GPU.

The block (reference: ``neuralfn/csrc/native_gpt2/resident_glimmer_cuda.cpp:3100-3498``, template
``neuralfn/torch_templates.py:493-790``): centred RMS norm -> fused q | k | v | gate projection ->
weightless per-head QK norm, query scale, rotary embedding on sliding-window layers only (every fourth
layer is global and position-free) -> attention -> sigmoid gate -> output projection -> post-norm ->
residual; the same sandwich around a SwiGLU MLP. Sliding-window layers keep a ring cache of ``window``
positions, global layers the whole context.

Sharding over W ranks: query / gate heads and the MLP width are split; a KV head is kept by every rank
whose query heads read it (with 2 KV heads on 8 ranks each is replicated four times), so attention never
crosses ranks. Per layer a decode step is 4 skinny GEMMs, one decode-attention launch (QK norm, rotary
and cache append fused), a gate, a SwiGLU and two fused all-reduce launches that also apply the
post-norm, the residual add and the next layer's input norm (``nfn_allreduce_sandwich_norm``). Prefill
runs one sequence at a time with the sequence-parallel fused collective GEMMs (all-gather -> GEMM,
GEMM -> reduce-scatter). CPU ranks (gloo) run the same schedule through PyTorch, which is how the sharding
is tested against the unsharded restatement ``glimmer_reference_logits``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel.tp import TensorParallelContext
from .tp_decode import TPLlamaDecoder

__all__ = ["GlimmerTPConfig", "TPGlimmerDecoder", "random_glimmer_params", "glimmer_reference_logits"]


@dataclass
class GlimmerTPConfig:
    n_layer: int = 48
    d_model: int = 6656
    n_head: int = 32
    n_kv_head: int = 2
    head_dim: int = 128
    d_ff: int = 24576
    vocab_size: int = 202048
    window: int = 4096
    global_every: int = 4          # layers l with (l + 1) % global_every == 0 are global and position-free
    rope_theta: float = 500000.0
    q_scale: float = 3.87
    norm_eps: float = 1e-5
    post_norm_eps: float = 1e-8
    qk_norm_eps: float = 1e-5
    logit_softcap: float = 30.0
    output_multiplier: float = 0.19611613513818404
    vocab_pad_to: int = 64
    rope_convention: str = "hf"

    @property
    def padded_vocab(self) -> int:
        p = self.vocab_pad_to
        return (self.vocab_size + p - 1) // p * p

    def is_local(self, layer: int) -> bool:
        return self.global_every <= 0 or (layer + 1) % self.global_every != 0

    @classmethod
    def from_spec(cls, spec, **over) -> "GlimmerTPConfig":
        """From a ``build_muse_glimmer_spec`` / ``glimmer_benchmark_shape`` model spec."""
        bs = spec.block_spec
        kw = dict(n_layer=spec.num_layers, d_model=spec.model_dim, n_head=bs.num_heads, n_kv_head=bs.num_kv_heads or bs.num_heads,
                  head_dim=bs.head_dim, d_ff=bs.intermediate_size, vocab_size=spec.vocab_size, window=bs.window_size,
                  global_every=len(bs.layer_attention_pattern) or 0, rope_theta=bs.rope_theta, q_scale=bs.q_scale_factor,
                  norm_eps=bs.norm_eps, post_norm_eps=bs.post_norm_eps, qk_norm_eps=bs.qk_norm_eps, logit_softcap=spec.logit_softcap,
                  output_multiplier=spec.output_multiplier)
        kw.update(over)
        return cls(**kw)


LAYER_KEYS = ("attn_norm", "wq", "wk", "wv", "wg", "wo", "post_attn_norm", "mlp_norm", "w_gate", "w_up", "w_down", "post_mlp_norm")


def random_glimmer_params(cfg: GlimmerTPConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    """Unsharded fp32 weights of a (small) configuration, for tests."""
    g = torch.Generator().manual_seed(seed)
    C, hd, H, Hkv, Fd, Vp = cfg.d_model, cfg.head_dim, cfg.n_head, cfg.n_kv_head, cfg.d_ff, cfg.padded_vocab
    r = lambda *s, std=0.05: torch.randn(*s, generator=g) * std  # noqa: E731
    p = {"embed": r(Vp, C, std=0.5), "head": r(Vp, C, std=0.2), "final_norm": 1 + r(C, std=0.1)}
    for l in range(cfg.n_layer):
        p.update({f"layers.{l}.attn_norm": r(C, std=0.1), f"layers.{l}.wq": r(H * hd, C), f"layers.{l}.wk": r(Hkv * hd, C),
                  f"layers.{l}.wv": r(Hkv * hd, C), f"layers.{l}.wg": r(H * hd, C), f"layers.{l}.wo": r(C, H * hd),
                  f"layers.{l}.post_attn_norm": r(C, std=0.1), f"layers.{l}.mlp_norm": r(C, std=0.1), f"layers.{l}.w_gate": r(Fd, C),
                  f"layers.{l}.w_up": r(Fd, C), f"layers.{l}.w_down": r(C, Fd), f"layers.{l}.post_mlp_norm": r(C, std=0.1)})
    return p


def _crms(x: torch.Tensor, w: torch.Tensor | None, eps: float, centered: bool = True) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * (1.0 + w.float() if centered else w.float())
    return y.to(x.dtype)


def _rope_tables(T: int, hd: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
    ang = torch.outer(torch.arange(T, device=device, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


def _rot(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotary embedding (HF convention): t [..., T, hd], cos / sin [T, hd / 2]."""
    a, b = t[..., :t.size(-1) // 2], t[..., t.size(-1) // 2:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)


def glimmer_reference_logits(cfg: GlimmerTPConfig, p: dict[str, torch.Tensor], tokens: torch.Tensor) -> torch.Tensor:
    """Unsharded fp32 forward of tokens [B, T] -> logits [B, T, vocab] (soft-capped). Full recompute, no cache."""
    B, T = tokens.shape
    C, hd, H, Hkv = cfg.d_model, cfg.head_dim, cfg.n_head, cfg.n_kv_head
    x = _crms(p["embed"].float()[tokens], None, cfg.norm_eps)
    cos, sin = _rope_tables(T, hd, cfg.rope_theta, x.device)
    pos = torch.arange(T)
    for l in range(cfg.n_layer):
        w = {k: p[f"layers.{l}.{k}"].float() for k in LAYER_KEYS}
        h = _crms(x, w["attn_norm"], cfg.norm_eps)
        q = (h @ w["wq"].T).view(B, T, H, hd).transpose(1, 2)
        k = (h @ w["wk"].T).view(B, T, Hkv, hd).transpose(1, 2)
        v = (h @ w["wv"].T).view(B, T, Hkv, hd).transpose(1, 2)
        gate = torch.sigmoid(h @ w["wg"].T)
        q, k = _crms(q, None, cfg.qk_norm_eps) * cfg.q_scale, _crms(k, None, cfg.qk_norm_eps)
        local = cfg.is_local(l)
        if local:
            q, k = _rot(q, cos, sin), _rot(k, cos, sin)
        mask = pos[None, :] <= pos[:, None]
        if local and cfg.window > 0:
            mask = mask & (pos[None, :] > pos[:, None] - cfg.window)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=H != Hkv)
        a = a.transpose(1, 2).reshape(B, T, H * hd) * gate
        x = x + _crms(a @ w["wo"].T, w["post_attn_norm"], cfg.post_norm_eps)
        h = _crms(x, w["mlp_norm"], cfg.norm_eps)
        m = (F.silu(h @ w["w_gate"].T) * (h @ w["w_up"].T)) @ w["w_down"].T
        x = x + _crms(m, w["post_mlp_norm"], cfg.post_norm_eps)
    x = _crms(x, p["final_norm"], cfg.norm_eps, centered=False)
    logits = (x @ p["head"].float().T)[..., :cfg.vocab_size] * cfg.output_multiplier
    if cfg.logit_softcap > 0:
        logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
    return logits


class TPGlimmerDecoder(TPLlamaDecoder):
    """Same driving interface as ``TPLlamaDecoder`` (``prefill`` / ``step`` / ``generate`` / ``set_sampling`` /
    CUDA-graph decode); the layer schedule is the Glimmer block's."""

    def __init__(self, cfg: GlimmerTPConfig, tp: TensorParallelContext, *, max_batch: int, max_seq: int, full_params: dict | None = None,
                 seed: int = 1234, use_graph: bool = False) -> None:
        W, r = tp.world, tp.rank
        if cfg.n_head % W or cfg.d_ff % W or cfg.padded_vocab % (8 * W):
            raise ValueError("query heads, d_ff and the padded vocabulary must divide by the TP size")
        if cfg.n_kv_head >= W:
            if cfg.n_kv_head % W:
                raise ValueError("KV heads must divide by the TP size (or the TP size by the KV heads)")
            self.Hkv, self.kv0 = cfg.n_kv_head // W, r * (cfg.n_kv_head // W)
        else:
            if W % cfg.n_kv_head:
                raise ValueError("the TP size must be a multiple of the KV heads when it exceeds them")
            self.Hkv, self.kv0 = 1, r * cfg.n_kv_head // W      # replicated: this rank's query heads all read KV head kv0
        self.cfg, self.tp, self.B, self.cap = cfg, tp, max_batch, max_seq
        dev = self.dev = tp.device
        self.cuda = dev.type == "cuda"
        self.dtype = torch.bfloat16 if self.cuda else torch.float32
        self.Hq, self.Fl, self.Vl = cfg.n_head // W, cfg.d_ff // W, cfg.padded_vocab // W
        hd, C = cfg.head_dim, cfg.d_model
        self.q_cols, self.kv_cols = self.Hq * hd, self.Hkv * hd
        self.gate_off = self.q_cols + 2 * self.kv_cols
        if full_params is not None:
            self._shard(full_params)
        else:
            self._random_shards(seed)
        # ring caches of `window` positions on sliding-window layers, the whole context on global ones
        self.caps = [min(cfg.window, max_seq) if (cfg.is_local(l) and cfg.window > 0) else max_seq for l in range(cfg.n_layer)]
        self.k_cache = [torch.zeros(max_batch, self.Hkv, c, hd, dtype=self.dtype, device=dev) for c in self.caps]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        self.lengths = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.cos, self.sin = _rope_tables(max_seq, hd, cfg.rope_theta, dev)
        self.x = torch.zeros(max_batch, C, dtype=self.dtype, device=dev)
        self.tokens = torch.zeros(max_batch, dtype=torch.int64, device=dev)
        self.last_logits = None
        self.sampling = None
        self._draws = 0
        self.use_graph = bool(use_graph and self.cuda)
        self._graph = None
        self._graph_ok = True
        self._fused_calls_per_step = 2 * cfg.n_layer + (1 if W > 1 else 0)
        if self.cuda:
            from ..ops.infer import DecodeAttentionWorkspace
            self._ws = DecodeAttentionWorkspace(max_batch, self.Hq, self.Hkv, hd, dev)
            self._gemm_ws = torch.empty(32 << 20, dtype=torch.uint8, device=dev)
            self._zero_pos = torch.zeros(max_seq, dtype=torch.int32, device=dev)

    # -------------------------------------------------------------------------------- weights --
    def _shard(self, p: dict[str, torch.Tensor]) -> None:
        cfg, W, r, hd = self.cfg, self.tp.world, self.tp.rank, self.cfg.head_dim
        to = lambda t: t.to(self.dev, self.dtype).contiguous()  # noqa: E731
        self.embed, self.norm = to(p["embed"]), to(p["final_norm"])
        self.head = to(p["head"][r * self.Vl:(r + 1) * self.Vl])
        q0, q1 = r * self.Hq * hd, (r + 1) * self.Hq * hd
        k0, k1 = self.kv0 * hd, (self.kv0 + self.Hkv) * hd
        f0, f1 = r * self.Fl, (r + 1) * self.Fl
        self.layers = []
        for l in range(cfg.n_layer):
            g = lambda k: p[f"layers.{l}.{k}"]  # noqa: E731
            self.layers.append({
                "attn_norm": to(g("attn_norm")), "post_attn_norm": to(g("post_attn_norm")), "mlp_norm": to(g("mlp_norm")),
                "post_mlp_norm": to(g("post_mlp_norm")),
                "wqkvg": to(torch.cat([g("wq")[q0:q1], g("wk")[k0:k1], g("wv")[k0:k1], g("wg")[q0:q1]], 0)),
                "wo": to(g("wo")[:, q0:q1]), "w_gate_up": to(torch.cat([g("w_gate")[f0:f1], g("w_up")[f0:f1]], 0)),
                "w_down": to(g("w_down")[:, f0:f1])})

    def _random_shards(self, seed: int) -> None:
        cfg, dev, hd, C = self.cfg, self.dev, self.cfg.head_dim, self.cfg.d_model
        shared = torch.Generator(device=dev).manual_seed(seed)
        own = torch.Generator(device=dev).manual_seed(seed * 7919 + 1 + self.tp.rank)

        def rnd(shape, gen, std=0.02):
            return torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, std, generator=gen).to(self.dtype)

        self.embed = rnd((cfg.padded_vocab, C), shared, 1.0)
        self.head = rnd((self.Vl, C), own)
        self.norm = torch.ones(C, dtype=self.dtype, device=dev)
        zeros = lambda: torch.zeros(C, dtype=self.dtype, device=dev)  # noqa: E731  (centred norms: weight 0 = identity scale)
        rs = 0.02 / (2 * cfg.n_layer) ** 0.5
        self.layers = [{"attn_norm": zeros(), "post_attn_norm": zeros(), "mlp_norm": zeros(), "post_mlp_norm": zeros(),
                        "wqkvg": rnd(((2 * self.Hq + 2 * self.Hkv) * hd, C), own), "wo": rnd((C, self.Hq * hd), own, rs),
                        "w_gate_up": rnd((2 * self.Fl, C), own), "w_down": rnd((C, self.Fl), own, rs)} for _ in range(cfg.n_layer)]

    # ----------------------------------------------------------------------- building blocks --
    def _qk_prepare(self, qkvg: torch.Tensor, T: int, local: bool, positions: torch.Tensor | None = None) -> None:
        """In place on packed rows: weightless QK norm, query scale, rotary embedding on local layers."""
        cfg, hd = self.cfg, self.cfg.head_dim
        if self.cuda:
            from ..ops.infer import qk_norm_rope_forward
            pos = positions if local else self._zero_pos[:qkvg.shape[0]]      # position 0 everywhere = no rotation
            qk_norm_rope_forward(qkvg, T=T, n_q_heads=self.Hq, n_kv_heads=self.Hkv, head_dim=hd, cos=self.cos, sin=self.sin,
                                 convention=cfg.rope_convention, positions=pos, eps=cfg.qk_norm_eps, q_scale=cfg.q_scale)
            return
        n = qkvg.shape[0]
        q = _crms(qkvg[:, :self.q_cols].view(n, self.Hq, hd), None, cfg.qk_norm_eps) * cfg.q_scale
        k = _crms(qkvg[:, self.q_cols:self.q_cols + self.kv_cols].view(n, self.Hkv, hd), None, cfg.qk_norm_eps)
        if local:
            pos = positions.long() if positions is not None else torch.arange(n) % T
            cos, sin = self.cos[pos][:, None], self.sin[pos][:, None]
            q, k = _rot(q, cos, sin), _rot(k, cos, sin)
        qkvg[:, :self.q_cols] = q.reshape(n, -1)
        qkvg[:, self.q_cols:self.q_cols + self.kv_cols] = k.reshape(n, -1)

    def _attend_one(self, qkvg: torch.Tensor, l: int) -> torch.Tensor:
        cfg, hd, local = self.cfg, self.cfg.head_dim, self.cfg.is_local(l)
        if self.cuda:
            from ..ops.infer import decode_attention, sigmoid_gate_inplace
            a = decode_attention(qkvg, self.k_cache[l], self.v_cache[l], self.lengths, n_q_heads=self.Hq, n_kv_heads=self.Hkv, head_dim=hd,
                                 workspace=self._ws, cos=self.cos if local else None, sin=self.sin if local else None,
                                 convention=cfg.rope_convention, qk_norm=True, eps=cfg.qk_norm_eps, scale=hd ** -0.5 * cfg.q_scale)
            return sigmoid_gate_inplace(a, qkvg[:, self.gate_off:])
        B = qkvg.shape[0]
        qkvg = qkvg.clone()
        pos = (self.lengths[:B] - 1)
        self._qk_prepare(qkvg, 1, local, positions=pos)
        q = qkvg[:, :self.q_cols].view(B, self.Hq, hd)
        k = qkvg[:, self.q_cols:self.q_cols + self.kv_cols].view(B, self.Hkv, hd)
        v = qkvg[:, self.q_cols + self.kv_cols:self.gate_off].view(B, self.Hkv, hd)
        cap, rows = self.caps[l], torch.arange(B)
        slot = pos.long() % cap
        self.k_cache[l][rows, :, slot] = k
        self.v_cache[l][rows, :, slot] = v
        rep = self.Hq // self.Hkv
        kk, vv = self.k_cache[l][:B].repeat_interleave(rep, 1), self.v_cache[l][:B].repeat_interleave(rep, 1)
        s = torch.einsum("bhd,bhtd->bht", q, kk) * hd ** -0.5
        live = torch.arange(cap)[None, :] < self.lengths[:B, None].clamp(max=cap)     # a ring holds min(len, cap) entries
        s = s.masked_fill(~live[:, None, :], float("-inf"))
        a = torch.einsum("bht,bhtd->bhd", s.softmax(-1), vv).reshape(B, self.q_cols)
        return a * torch.sigmoid(qkvg[:, self.gate_off:])

    def _reduce_sandwich(self, partial: torch.Tensor, sym, post_w: torch.Tensor, next_w: torch.Tensor | None) -> torch.Tensor:
        cfg = self.cfg
        return self.tp.allreduce_resid_norm(partial, sym, resid=self.x[:partial.shape[0]], norm_weight=next_w, eps=cfg.norm_eps,
                                            centered=True, post_weight=post_w, post_eps=cfg.post_norm_eps)

    def _pick(self, h: torch.Tensor) -> torch.Tensor:
        if self.sampling is None:
            return super()._pick(h)          # multiplier and soft-cap are monotonic: the arg-max is unchanged
        cfg = self.cfg
        logits = self._mm(h, self.head).float() * cfg.output_multiplier
        if cfg.logit_softcap > 0:
            logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
        logits = logits.to(self.dtype)
        self.last_logits = logits
        off = self.tp.rank * self.Vl
        if self.tp.rank == self.tp.world - 1 and cfg.padded_vocab != cfg.vocab_size:
            logits[:, cfg.vocab_size - off:] = -30000.0
        return self._sample(logits)

    # ------------------------------------------------------------------------------- prefill --
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] (B = max_batch, the same on every rank, T divisible by W). Sequences are
        prefilled one after another (each is one sequence-parallel pass); returns the first generated tokens."""
        cfg, tp = self.cfg, self.tp
        B, T = tokens.shape
        W = tp.world
        if B != self.B or T > self.cap or T % W:
            raise ValueError("prefill wants max_batch rows, T <= max_seq and T divisible by the TP size")
        fused = tp.impl == "fused"
        if fused and (T // W) % 128:
            tp.impl = "nccl"                 # short prompts: library collectives around the plain GEMM for this pass
            self._graph_ok = W == 1
        try:
            last = torch.stack([self._prefill_one(b, tokens[b]) for b in range(B)])      # [B, C] final-layer rows
        finally:
            if fused:
                tp.impl = "fused"
        self.lengths.fill_(T)
        nxt = self._pick(_crms(last, self.norm, cfg.norm_eps, centered=False))
        self.tokens.copy_(nxt)
        return nxt.clone()

    def _prefill_one(self, slot: int, toks: torch.Tensor) -> torch.Tensor:
        cfg, tp, hd = self.cfg, self.tp, self.cfg.head_dim
        T, W = toks.numel(), tp.world
        rows, lo = T // W, tp.rank * (T // W)
        x = _crms(self.embed[toks.to(self.dev)[lo:lo + rows].long()], None, cfg.norm_eps)        # this rank's rows of the residual stream
        positions = torch.arange(T, device=self.dev, dtype=torch.int32)
        for l, p in enumerate(self.layers):
            local = cfg.is_local(l)
            qkvg = tp.column_linear(_crms(x, p["attn_norm"], cfg.norm_eps), p["wqkvg"])                # [T, local columns]
            self._qk_prepare(qkvg, T, local, positions=positions)
            q, k = qkvg[:, :self.q_cols], qkvg[:, self.q_cols:self.q_cols + self.kv_cols]
            v = qkvg[:, self.q_cols + self.kv_cols:self.gate_off]
            window = cfg.window if (local and cfg.window > 0) else 0
            if self.cuda:
                from ..ops import kernels as K
                from ..ops.infer import kv_cache_write, sigmoid_gate_inplace
                a, _ = K.attention_forward(q, k, v, B=1, T=T, n_q_heads=self.Hq, n_kv_heads=self.Hkv, head_dim=hd, causal=True,
                                           window=window, scale=hd ** -0.5, need_lse=False)
                kv_cache_write(qkvg, self.k_cache[l][slot], self.v_cache[l][slot], n_q_heads=self.Hq, n_kv_heads=self.Hkv, head_dim=hd)
                sigmoid_gate_inplace(a, qkvg[:, self.gate_off:])
            else:
                q4, k4, v4 = (t.reshape(1, T, -1, hd).transpose(1, 2) for t in (q, k, v))
                pos = torch.arange(T)
                mask = pos[None, :] <= pos[:, None]
                if window:
                    mask = mask & (pos[None, :] > pos[:, None] - window)
                a = F.scaled_dot_product_attention(q4, k4, v4, attn_mask=mask, enable_gqa=self.Hq != self.Hkv, scale=hd ** -0.5)
                a = a.transpose(1, 2).reshape(T, self.q_cols) * torch.sigmoid(qkvg[:, self.gate_off:])
                cap = self.caps[l]
                keep = torch.arange(max(0, T - cap), T)                                        # a ring keeps the last `cap` positions
                self.k_cache[l][slot][:, keep % cap] = k4[0][:, keep]
                self.v_cache[l][slot][:, keep % cap] = v4[0][:, keep]
            x = self._post_add(tp.row_linear(a, p["wo"]), p["post_attn_norm"], x)
            gu = tp.column_linear(_crms(x, p["mlp_norm"], cfg.norm_eps), p["w_gate_up"])
            if self.cuda:
                from ..ops.infer import swiglu_forward
                g = swiglu_forward(gu, self.Fl)
            else:
                g = F.silu(gu[:, :self.Fl]) * gu[:, self.Fl:]
            x = self._post_add(tp.row_linear(g, p["w_down"]), p["post_mlp_norm"], x)
        # the sequence's last row lives on the last rank: every rank contributes its candidate, zero elsewhere
        mine = x[-1:].clone() if tp.rank == W - 1 else torch.zeros(1, cfg.d_model, dtype=x.dtype, device=x.device)
        if W == 1:
            return mine[0]
        if tp.impl == "fused":
            buf, sym = tp.partial_buffer(1, cfg.d_model)
            buf.copy_(mine)
            return tp.allreduce_resid_norm(buf, sym)[0].clone()
        y = mine.float()
        dist.all_reduce(y, group=tp.group)
        return y.to(x.dtype)[0]

    def _post_add(self, branch: torch.Tensor, post_w: torch.Tensor, resid: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if self.cuda:
            from ..ops.infer import rmsnorm_residual
            return rmsnorm_residual(branch.contiguous(), post_w, resid, eps=cfg.post_norm_eps, centered=True)
        return resid + _crms(branch, post_w, cfg.post_norm_eps)

    # -------------------------------------------------------------------------------- decode --
    def _step_body(self) -> None:
        cfg, B = self.cfg, self.B
        self.lengths += 1
        self.x.copy_(_crms(self.embed[self.tokens], None, cfg.norm_eps))
        h = _crms(self.x, self.layers[0]["attn_norm"], cfg.norm_eps)
        for l, p in enumerate(self.layers):
            a = self._attend_one(self._mm(h, p["wqkvg"]), l)
            part, sym = self._partial(B)
            h = self._reduce_sandwich(self._mm(a, p["wo"], out=part), sym, p["post_attn_norm"], p["mlp_norm"])
            gu = self._mm(h, p["w_gate_up"])
            if self.cuda:
                from ..ops.infer import swiglu_forward
                g = swiglu_forward(gu, self.Fl)
            else:
                g = F.silu(gu[:, :self.Fl]) * gu[:, self.Fl:]
            part, sym = self._partial(B)
            last = l + 1 == cfg.n_layer
            h = self._reduce_sandwich(self._mm(g, p["w_down"], out=part), sym, p["post_mlp_norm"],
                                      None if last else self.layers[l + 1]["attn_norm"])
        # after the last layer `h` is the residual stream itself; the final norm is not centred
        self.tokens.copy_(self._pick(_crms(h, self.norm, cfg.norm_eps, centered=False)))
