"""Llama-family dense transformer over the sm_100a kernel library: RMSNorm, rotary
embeddings, grouped-query attention (optional sliding window, optional weightless per-head
QK norm), SwiGLU MLP, tied or untied head, fused cross-entropy (soft-cap / z-loss).

Same design as ``models.gpt2``: flat bf16 parameter / gradient buffers, explicit forward and
backward (no autograd tape) so a whole optimizer step is one CUDA graph, fp32 PyTorch oracle
(``reference_forward``) for the tests. Parameter names match the resident inference
engine's Llama layout (``tok_embeddings``, ``layers.N.{attn_norm,wqkv,wo,ffn_norm,w_gate_up,
w_down}``, ``norm``, ``lm_head``), so trained weights load into it unchanged.

Reference model family: ``build_llama_spec`` and the Llama-style presets
(``neuralfn/config.py:950-1100``), native trainer family ``llama`` in
``csrc/native_train/missing_native_train.cpp``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .gpt2 import FlatLayout, ParamSpec

__all__ = ["LlamaConfig", "llama_param_specs", "init_llama_params_", "LlamaEngine", "llama_reference_forward"]


@dataclass
class LlamaConfig:
    n_layer: int = 16
    n_head: int = 16
    n_kv_head: int = 4
    d_model: int = 1024
    d_ff: int = 2816
    vocab_size: int = 32000
    max_seq_len: int = 2048
    rope_theta: float = 10000.0
    rope_convention: str = "hf"
    norm_eps: float = 1e-5
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    tie_embeddings: bool = False
    window: int = 0                 # sliding window of every layer (0 = full causal)
    logit_softcap: float = 0.0
    z_loss: float = 0.0
    vocab_pad_to: int = 128
    head_dim_override: int = 0
    # pipeline-parallel stage view: this engine owns layers [pp_layer_begin, pp_layer_end); the first
    # stage also owns the embedding, the last one the final norm and the head (0 / 0 = whole model)
    pp_layer_begin: int = 0
    pp_layer_end: int = 0
    pp_first: bool = True
    pp_last: bool = True

    @property
    def layer_range(self) -> range:
        return range(self.pp_layer_begin, self.pp_layer_end or self.n_layer)

    @property
    def head_dim(self) -> int:
        return self.head_dim_override or self.d_model // self.n_head

    @property
    def padded_vocab(self) -> int:
        p = self.vocab_pad_to
        return (self.vocab_size + p - 1) // p * p

    @property
    def qkv_dim(self) -> int:
        return (self.n_head + 2 * self.n_kv_head) * self.head_dim

    # hooks used by trainers.dense_gpt.DenseGPTTrainer
    def param_specs(self) -> list[ParamSpec]:
        return llama_param_specs(self)

    def init_params_(self, layout: FlatLayout, master: torch.Tensor, seed: int) -> None:
        init_llama_params_(self, layout, master, seed)

    def make_engine(self, layout, params, grads, batch: int, seq: int) -> "LlamaEngine":
        return LlamaEngine(self, layout, params, grads, batch, seq)


def llama_param_specs(cfg: LlamaConfig) -> list[ParamSpec]:
    C, F_, Vp, hd = cfg.d_model, cfg.d_ff, cfg.padded_vocab, cfg.head_dim
    if cfg.tie_embeddings and not (cfg.pp_first and cfg.pp_last):
        raise ValueError("tied embeddings need the first and the last pipeline stage on one rank")
    specs = [ParamSpec("tok_embeddings", (Vp, C), True, "normal")] if cfg.pp_first else []
    for l in cfg.layer_range:
        p = f"layers.{l}."
        specs += [ParamSpec(p + "attn_norm", (C,), False, "ones"),
                  ParamSpec(p + "wqkv", (cfg.qkv_dim, C), True, "normal"),
                  ParamSpec(p + "wo", (C, cfg.n_head * hd), True, "resid"),
                  ParamSpec(p + "ffn_norm", (C,), False, "ones"),
                  ParamSpec(p + "w_gate_up", (2 * F_, C), True, "normal"),
                  ParamSpec(p + "w_down", (C, F_), True, "resid")]
    if cfg.pp_last:
        specs.append(ParamSpec("norm", (C,), False, "ones"))
        if not cfg.tie_embeddings:
            specs.append(ParamSpec("lm_head", (Vp, C), True, "normal"))
    return specs


def init_llama_params_(cfg: LlamaConfig, layout: FlatLayout, master: torch.Tensor, seed: int = 1337) -> None:
    gen = torch.Generator(device=master.device)
    gen.manual_seed(seed)
    master.zero_()
    for s in layout.order:
        v = layout.view(master, s.name)
        if s.init == "normal":
            v.normal_(0.0, 0.02, generator=gen)
        elif s.init == "resid":
            v.normal_(0.0, 0.02 / math.sqrt(2 * cfg.n_layer), generator=gen)
        elif s.init == "ones":
            v.fill_(1.0)
    if cfg.pp_first:
        layout.view(master, "tok_embeddings")[cfg.vocab_size:].zero_()
    if cfg.pp_last and not cfg.tie_embeddings:
        layout.view(master, "lm_head")[cfg.vocab_size:].zero_()


def _rope_ref(x, cos, sin, sign):
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    return torch.cat((a * cos - sign * b * sin, b * cos + sign * a * sin), dim=-1)


def llama_reference_forward(cfg: LlamaConfig, params: dict[str, torch.Tensor], tokens: torch.Tensor,
                            targets: torch.Tensor | None = None):
    """Plain PyTorch restatement (any dtype/device). Returns (loss, logits[B, T, V])."""
    B, T = tokens.shape
    C, Hq, Hkv, hd = cfg.d_model, cfg.n_head, cfg.n_kv_head, cfg.head_dim
    dev = tokens.device
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
    cos, sin = ang.cos().float().to(dev)[None, :, None], ang.sin().float().to(dev)[None, :, None]
    sign = 1.0 if cfg.rope_convention == "hf" else -1.0

    def rms(v, w, eps):
        return (v.float() * torch.rsqrt(v.float().pow(2).mean(-1, keepdim=True) + eps)).to(v.dtype) * w

    x = params["tok_embeddings"][tokens]
    for l in range(cfg.n_layer):
        p = f"layers.{l}."
        qkv = F.linear(rms(x, params[p + "attn_norm"], cfg.norm_eps), params[p + "wqkv"])
        q = qkv[..., :Hq * hd].reshape(B, T, Hq, hd)
        k = qkv[..., Hq * hd:(Hq + Hkv) * hd].reshape(B, T, Hkv, hd)
        v = qkv[..., (Hq + Hkv) * hd:].reshape(B, T, Hkv, hd)
        if cfg.qk_norm:
            q = q * torch.rsqrt(q.float().pow(2).mean(-1, keepdim=True) + cfg.qk_norm_eps).to(q.dtype)
            k = k * torch.rsqrt(k.float().pow(2).mean(-1, keepdim=True) + cfg.qk_norm_eps).to(k.dtype)
        q, k = _rope_ref(q, cos, sin, sign).to(q.dtype), _rope_ref(k, cos, sin, sign).to(k.dtype)
        k = k.repeat_interleave(Hq // Hkv, dim=2)
        v = v.repeat_interleave(Hq // Hkv, dim=2)
        i, j = torch.arange(T, device=dev)[:, None], torch.arange(T, device=dev)[None, :]
        mask = j <= i
        if cfg.window > 0:
            mask = mask & (i - j < cfg.window)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask)
        x = x + F.linear(a.transpose(1, 2).reshape(B, T, Hq * hd), params[p + "wo"])
        gu = F.linear(rms(x, params[p + "ffn_norm"], cfg.norm_eps), params[p + "w_gate_up"])
        x = x + F.linear(F.silu(gu[..., :cfg.d_ff]) * gu[..., cfg.d_ff:], params[p + "w_down"])
    x = rms(x, params["norm"], cfg.norm_eps)
    head = params["tok_embeddings"] if cfg.tie_embeddings else params["lm_head"]
    logits = F.linear(x, head)[..., :cfg.vocab_size].float()
    if cfg.logit_softcap > 0:
        logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
    loss = None
    if targets is not None:
        lse = torch.logsumexp(logits, -1)
        nll = lse - logits.gather(-1, targets.long()[..., None]).squeeze(-1)
        loss = (nll + cfg.z_loss * lse.pow(2)).mean()
    return loss, logits


class LlamaEngine:
    """Forward/backward over preallocated buffers (CUDA only); optimizer lives in ``parallel.dp``."""

    def __init__(self, cfg: LlamaConfig, layout: FlatLayout, params: torch.Tensor, grads: torch.Tensor, batch: int, seq: int) -> None:
        from ..ops import infer as I
        from ..ops import kernels as K
        from ..ops.gemm import gemm
        self.K, self.I, self.gemm = K, I, gemm
        self.cfg, self.layout, self.B, self.T = cfg, layout, batch, seq
        if seq > cfg.max_seq_len:
            raise ValueError("sequence longer than max_seq_len")
        if cfg.head_dim not in (64, 128):
            raise ValueError("head_dim must be 64 or 128")
        self.params, self.grads = params, grads
        self.p, self.g = layout.views(params), layout.views(grads)
        dev = params.device
        N, C, Fd, Q = batch * seq, cfg.d_model, cfg.d_ff, cfg.qkv_dim
        A = cfg.n_head * cfg.head_dim
        bf, f32 = torch.bfloat16, torch.float32
        e = lambda *s, dtype=bf: torch.empty(*s, device=dev, dtype=dtype)  # noqa: E731
        self.cos, self.sin = I.rope_tables(seq, cfg.head_dim, cfg.rope_theta, device=dev)
        self.x0 = e(N, C)
        self.acts = [dict(n1=e(N, C), r1=e(N, dtype=f32), qkv=e(N, Q),
                          qk_rstd=e(N, cfg.n_head + cfg.n_kv_head, dtype=f32) if cfg.qk_norm else None,
                          att=e(N, A), lse=e(batch, cfg.n_head, seq, dtype=f32), x1=e(N, C), n2=e(N, C), r2=e(N, dtype=f32),
                          gu=e(N, 2 * Fd), h=e(N, Fd), x2=e(N, C)) for _ in cfg.layer_range]
        self.layers = list(cfg.layer_range)
        self.nf, self.rf = e(N, C), e(N, dtype=f32)
        self.mean_scratch = e(N, dtype=f32)  # RMS norms have no mean; the kernel wrapper wants a buffer
        self.logits = e(N, cfg.padded_vocab)
        self.row_loss = e(N, dtype=f32)
        self.loss = torch.zeros(1, device=dev, dtype=f32)
        self.d_a, self.d_b, self.d_n = e(N, C), e(N, C), e(N, C)
        self.d_h, self.d_gu = e(N, Fd), e(N, 2 * Fd)
        self.d_qkv, self.d_att = e(N, Q), e(N, A)
        self.delta = e(batch, cfg.n_head, seq, dtype=f32)
        self.dq_accum = e(N, A, dtype=f32)
        self.scratch = e(max(64 * 2 * max(2 * Fd, Q, C), K.norm_fused_rows() * 3 * C), dtype=f32)
        self.ws = e(32 * 1024 * 1024, dtype=f32)
        self.tokens = torch.zeros(N, device=dev, dtype=torch.int32)
        self.tok_sorted = torch.zeros(N, device=dev, dtype=torch.int32)      # stable sort of the batch's tokens: the token-embedding gradient
        self.tok_order = torch.zeros(N, device=dev, dtype=torch.int64)       # sums equal tokens in row order (bitwise reproducible)
        self.targets = torch.zeros(N, device=dev, dtype=torch.int32)

    def _views(self, t):
        cfg = self.cfg
        q_end, k_end = cfg.n_head * cfg.head_dim, (cfg.n_head + cfg.n_kv_head) * cfg.head_dim
        return t[:, :q_end], t[:, q_end:k_end], t[:, k_end:]

    def forward(self, *, compute_grad_logits: bool = True, grad_scale: float | None = None) -> torch.Tensor:
        K, I, gemm, cfg, p = self.K, self.I, self.gemm, self.cfg, self.p
        B, T, N = self.B, self.T, self.B * self.T
        Hq, Hkv, hd = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        if cfg.pp_first:
            K.embedding_forward(self.tokens, p["tok_embeddings"], None, T=T, out=self.x0)
        x = self.x0  # later stages: filled by the pipeline runtime with the previous stage's output
        for l, a in zip(self.layers, self.acts):
            pre = f"layers.{l}."
            K.norm_forward(x, p[pre + "attn_norm"], None, eps=cfg.norm_eps, mode=K.NORM_RMS, mean=self.mean_scratch,out=a["n1"], rstd=a["r1"])
            gemm(a["n1"], p[pre + "wqkv"], out=a["qkv"])
            if cfg.qk_norm:
                K.qk_norm_forward(a["qkv"], Hq, Hkv, hd, eps=cfg.qk_norm_eps, rstd=a["qk_rstd"])
            I.rope_inplace(a["qkv"], T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=self.cos, sin=self.sin,
                           convention=cfg.rope_convention)
            q, k, v = self._views(a["qkv"])
            K.attention_forward(q, k, v, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, causal=True, window=cfg.window,
                                out=a["att"], lse=a["lse"])
            gemm(a["att"], p[pre + "wo"], resid=x, out=a["x1"])
            K.norm_forward(a["x1"], p[pre + "ffn_norm"], None, eps=cfg.norm_eps, mode=K.NORM_RMS, mean=self.mean_scratch,out=a["n2"], rstd=a["r2"])
            gemm(a["n2"], p[pre + "w_gate_up"], out=a["gu"])
            I.swiglu_forward(a["gu"], cfg.d_ff, out=a["h"])
            gemm(a["h"], p[pre + "w_down"], resid=a["x1"], out=a["x2"])
            x = a["x2"]
        if not cfg.pp_last:
            return x  # hand to the next stage
        K.norm_forward(x, p["norm"], None, eps=cfg.norm_eps, mode=K.NORM_RMS, mean=self.mean_scratch,out=self.nf, rstd=self.rf)
        head = p["tok_embeddings"] if cfg.tie_embeddings else p["lm_head"]
        if cfg.logit_softcap > 0:
            gemm(self.nf, head, act="tanh_cap", act_param=cfg.logit_softcap, out=self.logits)
        else:
            gemm(self.nf, head, out=self.logits)
        K.cross_entropy(self.logits, self.targets, vocab=cfg.vocab_size, cap=cfg.logit_softcap, z_coef=cfg.z_loss,
                        grad_scale=(1.0 / N if grad_scale is None else grad_scale), loss_scale=1.0 / N,
                        write_grad=compute_grad_logits, row_loss=self.row_loss, mean_loss=self.loss)
        return self.loss

    def backward(self) -> None:
        K, I, gemm, cfg, p, g = self.K, self.I, self.gemm, self.cfg, self.p, self.g
        B, T = self.B, self.T
        Hq, Hkv, hd = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        sc, ws = self.scratch, self.ws
        dx, spare = self.d_a, self.d_b  # later stages: d_a was filled with the next stage's input gradient
        if cfg.pp_last:
            head_name = "tok_embeddings" if cfg.tie_embeddings else "lm_head"
            gemm(self.logits, p[head_name], b_mn=True, out=self.d_n)
            gemm(self.logits, self.nf, a_mn=True, b_mn=True, out=g[head_name])
            x_last = self.acts[-1]["x2"] if self.acts else self.x0
            K.norm_backward(self.d_n, x_last, p["norm"], None, self.rf, g["norm"], None, sc, mode=K.NORM_RMS, out=dx)
        if cfg.pp_first and not cfg.tie_embeddings:
            g["tok_embeddings"].zero_()
        for i in range(len(self.layers) - 1, -1, -1):
            a, l = self.acts[i], self.layers[i]
            pre = f"layers.{l}."
            x_in = self.acts[i - 1]["x2"] if i > 0 else self.x0
            # MLP: x2 = w_down(swiglu(w_gate_up(n2))) + x1
            gemm(dx, p[pre + "w_down"], b_mn=True, out=self.d_h)
            gemm(dx, a["h"], a_mn=True, b_mn=True, workspace=ws, out=g[pre + "w_down"])
            I.swiglu_backward(a["gu"], self.d_h, cfg.d_ff, out=self.d_gu)
            gemm(self.d_gu, p[pre + "w_gate_up"], b_mn=True, out=self.d_n)
            gemm(self.d_gu, a["n2"], a_mn=True, b_mn=True, workspace=ws, out=g[pre + "w_gate_up"])
            K.norm_backward(self.d_n, a["x1"], p[pre + "ffn_norm"], None, a["r2"], g[pre + "ffn_norm"], None, sc, mode=K.NORM_RMS, dresid=dx, out=spare)
            dx, spare = spare, dx
            # attention: x1 = wo(att) + x
            gemm(dx, p[pre + "wo"], b_mn=True, out=self.d_att)
            gemm(dx, a["att"], a_mn=True, b_mn=True, workspace=ws, out=g[pre + "wo"])
            q, k, v = self._views(a["qkv"])
            dq, dk, dv = self._views(self.d_qkv)
            K.attention_backward(self.d_att, q, k, v, a["att"], a["lse"], B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd,
                                 causal=True, window=cfg.window, dq=dq, dk=dk, dv=dv, delta=self.delta, dq_accum=self.dq_accum)
            I.rope_inplace(self.d_qkv, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=self.cos, sin=self.sin,
                           convention=cfg.rope_convention, backward=True)
            if cfg.qk_norm:
                # the norm backward needs the normalised (pre-rotation) q/k: undo the rotation of the saved copy
                I.rope_inplace(a["qkv"], T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=self.cos, sin=self.sin,
                               convention=cfg.rope_convention, backward=True)
                K.qk_norm_backward(self.d_qkv, a["qkv"], a["qk_rstd"], Hq, Hkv, hd)
            gemm(self.d_qkv, p[pre + "wqkv"], b_mn=True, out=self.d_n)
            gemm(self.d_qkv, a["n1"], a_mn=True, b_mn=True, workspace=ws, out=g[pre + "wqkv"])
            K.norm_backward(self.d_n, x_in, p[pre + "attn_norm"], None, a["r1"], g[pre + "attn_norm"], None, sc, mode=K.NORM_RMS, dresid=dx, out=spare)
            dx, spare = spare, dx
        self.d_input = dx  # gradient w.r.t. this stage's input (sent to the previous stage)
        if cfg.pp_first:
            st_, od_ = K.sort_tokens(self.tokens, self.tok_sorted, self.tok_order)
            K.embedding_backward(dx, self.tokens, g["tok_embeddings"], None, B=B, T=T, sorted_tokens=st_, order=od_)

    def set_batch(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        self.tokens.copy_(tokens.reshape(-1), non_blocking=True)
        self.targets.copy_(targets.reshape(-1), non_blocking=True)

    def logits_view(self) -> torch.Tensor:
        return self.logits.view(self.B, self.T, -1)[..., :self.cfg.vocab_size]
