"""Tensor stages, part 3b: self-contained attention blocks (projections included) and
KV-cache helpers: causal self-attention with QK RMS + gain, fused causal attention,
multi-head latent attention, DFlash block attention, KV read/write, PCA and int8 KV
compression. Reference: ``neuralfn/torch_backend.py:428-596,1817-2010,2536-2585``."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .stages_attention import (apply_rotary_emb, apply_rotary_emb_hf, apply_rotary_interleaved,
                               rope_inv_freq, rope_tables)
from .stages_core import stage


def _heads(x: Tensor, n: int, d: int) -> Tensor:
    b, t, _ = x.shape
    return x.reshape(b, t, n, d).transpose(1, 2)


class _ProjectedAttention(nn.Module):
    def __init__(self, model_dim: int, num_heads: int, num_kv_heads: int, rope_base: float) -> None:
        super().__init__()
        if model_dim % num_heads:
            raise ValueError("model_dim must be divisible by num_heads")
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.head_dim = model_dim // num_heads
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for rotary embeddings")
        kv = num_kv_heads * self.head_dim
        self.q_proj = nn.Linear(model_dim, model_dim, bias=False)
        self.k_proj = nn.Linear(model_dim, kv, bias=False)
        self.v_proj = nn.Linear(model_dim, kv, bias=False)
        self.out_proj = nn.Linear(model_dim, model_dim, bias=False)
        for lin in (self.q_proj, self.k_proj, self.v_proj, self.out_proj):
            nn.init.normal_(lin.weight, std=0.02)
        self.register_buffer("inv_freq", rope_inv_freq(self.head_dim, rope_base), persistent=False)

    def _qkv(self, x: Tensor):
        q = _heads(self.q_proj(x), self.num_heads, self.head_dim)
        k = _heads(self.k_proj(x), self.num_kv_heads, self.head_dim)
        v = _heads(self.v_proj(x), self.num_kv_heads, self.head_dim)
        return q, k, v

    def _rope(self, q: Tensor, k: Tensor):
        cos, sin = rope_tables(torch.arange(q.size(2), device=q.device), self.inv_freq, q.dtype)
        return apply_rotary_emb(q, cos, sin), apply_rotary_emb(k, cos, sin)

    def _merge(self, y: Tensor) -> Tensor:
        b, h, t, d = y.shape
        return self.out_proj(y.transpose(1, 2).reshape(b, t, h * d))


@stage("causal_self_attention")
class CausalSelfAttentionStage(_ProjectedAttention):
    """q/k RMS-normalised, legacy RoPE, learnable per-head q gain, causal SDPA."""

    def __init__(self, model_dim, num_heads, num_kv_heads, rope_base, qk_gain_init) -> None:
        super().__init__(model_dim, num_heads, num_kv_heads, rope_base)
        self.q_gain = nn.Parameter(torch.full((num_heads,), float(qk_gain_init)))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["num_heads"]), int(cfg["num_kv_heads"]),
                   float(cfg["rope_base"]), float(cfg["qk_gain_init"]))

    def forward(self, x: Tensor) -> Tensor:
        from .kernel_bridge import attention
        q, k, v = self._qkv(x)
        q = F.rms_norm(q, (q.size(-1),))
        k = F.rms_norm(k, (k.size(-1),))
        q, k = self._rope(q, k)
        q = q * self.q_gain.to(q.dtype)[None, :, None, None]
        return self._merge(attention(q, k, v, causal=True))


@stage("fused_causal_attention")
class FusedCausalAttentionStage(_ProjectedAttention):
    def __init__(self, model_dim, num_heads, num_kv_heads, rope_base=10000.0, dropout_p=0.0) -> None:
        super().__init__(model_dim, num_heads, num_kv_heads, rope_base)
        self.dropout_p = float(dropout_p)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["num_heads"]), int(cfg.get("num_kv_heads", cfg["num_heads"])),
                   float(cfg.get("rope_base", 10000.0)), float(cfg.get("dropout_p", 0.0)))

    def forward(self, x: Tensor) -> Tensor:
        from .kernel_bridge import attention
        q, k, v = self._qkv(x)
        q, k = self._rope(q, k)
        return self._merge(attention(q, k, v, causal=True, dropout_p=self.dropout_p if self.training else 0.0))


@stage("multi_latent_attention")
class MLAStage(nn.Module):
    """Multi-head latent attention: low-rank joint KV latent, decoupled RoPE on a split of head_dim."""

    def __init__(self, model_dim: int, num_heads: int, kv_lora_rank: int | None = None,
                 qk_rope_dim: int | None = None, rope_base: float = 10000.0, dropout_p: float = 0.0) -> None:
        super().__init__()
        if model_dim % num_heads:
            raise ValueError("model_dim must be divisible by num_heads")
        hd = model_dim // num_heads
        rope = qk_rope_dim if qk_rope_dim is not None else max(hd // 2, 2)
        rope = max(rope - rope % 2, 2)
        if hd - rope <= 0:
            raise ValueError("qk_rope_dim must be smaller than head_dim")
        rank = kv_lora_rank if kv_lora_rank is not None else max(2 * hd, model_dim // 2)
        self.num_heads, self.head_dim, self.rope_dim, self.nope_dim = num_heads, hd, rope, hd - rope
        self.kv_lora_rank, self.dropout_p = rank, float(dropout_p)
        self.q_proj = nn.Linear(model_dim, num_heads * hd, bias=False)
        self.kv_a = nn.Linear(model_dim, rank + rope, bias=False)
        self.kv_b = nn.Linear(rank, num_heads * (self.nope_dim + hd), bias=False)
        self.out_proj = nn.Linear(num_heads * hd, model_dim, bias=False)
        for lin in (self.q_proj, self.kv_a, self.kv_b, self.out_proj):
            nn.init.normal_(lin.weight, std=0.02)
        self.register_buffer("inv_freq", rope_inv_freq(rope, rope_base), persistent=False)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["num_heads"]), cfg.get("kv_lora_rank"), cfg.get("qk_rope_dim"),
                   float(cfg.get("rope_base", 10000.0)), float(cfg.get("dropout_p", 0.0)))

    def forward(self, x: Tensor) -> Tensor:
        b, t, _ = x.shape
        h = self.num_heads
        q = self.q_proj(x).view(b, t, h, self.head_dim)
        q_nope, q_rope = q.split([self.nope_dim, self.rope_dim], dim=-1)
        kv_c, k_rope = self.kv_a(x).split([self.kv_lora_rank, self.rope_dim], dim=-1)
        kv = self.kv_b(F.rms_norm(kv_c, (self.kv_lora_rank,))).view(b, t, h, self.nope_dim + self.head_dim)
        k_nope, v = kv.split([self.nope_dim, self.head_dim], dim=-1)
        cos, sin = rope_tables(torch.arange(t, device=x.device), self.inv_freq, q.dtype)
        q_rope = apply_rotary_emb(q_rope.transpose(1, 2), cos, sin)
        k_rope = apply_rotary_emb(k_rope.unsqueeze(2).expand(b, t, h, self.rope_dim).transpose(1, 2), cos, sin)
        qf = torch.cat([q_nope.transpose(1, 2), q_rope], dim=-1)
        kf = torch.cat([k_nope.transpose(1, 2), k_rope], dim=-1)
        y = F.scaled_dot_product_attention(qf, kf, v.transpose(1, 2), is_causal=True,
                                           dropout_p=self.dropout_p if self.training else 0.0)
        return self.out_proj(y.transpose(1, 2).reshape(b, t, h * self.head_dim))


@stage("dflash_attention")
class DFlashAttentionStage(nn.Module):
    """Block-drafting attention: keys/values are the shared-projection of [context ; block]
    hidden states, q/k carry learned RMS weights, RoPE uses explicit positions, and the mask
    is supplied by the caller (bidirectional within +-window inside a block)."""

    def __init__(self, model_dim: int, num_heads: int, num_kv_heads: int, head_dim: int, window_size: int,
                 rope_base: float = 500000.0, norm_eps: float = 1e-5, convention: str = "hf",
                 bias: bool = False, dropout_p: float = 0.0) -> None:
        super().__init__()
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.window_size, self.norm_eps, self.convention = int(window_size), float(norm_eps), convention
        self.dropout_p = float(dropout_p)
        self.q_proj = nn.Linear(model_dim, num_heads * head_dim, bias=bias)
        self.k_proj = nn.Linear(model_dim, num_kv_heads * head_dim, bias=bias)
        self.v_proj = nn.Linear(model_dim, num_kv_heads * head_dim, bias=bias)
        self.o_proj = nn.Linear(num_heads * head_dim, model_dim, bias=bias)
        for lin in (self.q_proj, self.k_proj, self.v_proj, self.o_proj):
            nn.init.normal_(lin.weight, std=0.02)
        self.q_norm = nn.Parameter(torch.ones(head_dim))
        self.k_norm = nn.Parameter(torch.ones(head_dim))
        self.register_buffer("inv_freq", rope_inv_freq(head_dim, rope_base), persistent=False)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["num_heads"]), int(cfg["num_kv_heads"]), int(cfg["head_dim"]),
                   int(cfg["window_size"]), float(cfg.get("rope_base", 500000.0)), float(cfg.get("norm_eps", 1e-5)),
                   str(cfg.get("convention", "hf")), bool(cfg.get("bias", False)), float(cfg.get("dropout_p", 0.0)))

    def _rope(self, x: Tensor, positions: Tensor) -> Tensor:
        # positions: [B, T]
        freqs = positions.to(self.inv_freq.dtype).unsqueeze(-1) * self.inv_freq.to(x.device)
        cos, sin = freqs.cos().to(x.dtype).unsqueeze(1), freqs.sin().to(x.dtype).unsqueeze(1)
        if self.convention == "interleaved":
            return apply_rotary_interleaved(x, cos, sin)
        return (apply_rotary_emb_hf if self.convention == "hf" else apply_rotary_emb)(x, cos, sin)

    def default_mask(self, q_pos: Tensor, kv_pos: Tensor) -> Tensor:
        """Bidirectional visibility within +-window: [B, 1, Tq, Tk] bool."""
        d = q_pos.unsqueeze(-1) - kv_pos.unsqueeze(-2)
        return (d.abs() < self.window_size).unsqueeze(1)

    def forward(self, block_hidden: Tensor, context_hidden: Tensor, block_positions: Tensor,
                context_positions: Tensor, attention_mask: Tensor | None = None) -> Tensor:
        b, tq, _ = block_hidden.shape
        kv_in = torch.cat([context_hidden, block_hidden], dim=1)
        kv_pos = torch.cat([context_positions, block_positions], dim=1)
        q = _heads(self.q_proj(block_hidden), self.num_heads, self.head_dim)
        k = _heads(self.k_proj(kv_in), self.num_kv_heads, self.head_dim)
        v = _heads(self.v_proj(kv_in), self.num_kv_heads, self.head_dim)
        q = F.rms_norm(q, (self.head_dim,), self.q_norm.to(q.dtype), self.norm_eps)
        k = F.rms_norm(k, (self.head_dim,), self.k_norm.to(k.dtype), self.norm_eps)
        q, k = self._rope(q, block_positions), self._rope(k, kv_pos)
        mask = attention_mask if attention_mask is not None else self.default_mask(block_positions, kv_pos)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=self.num_heads != self.num_kv_heads,
                                           dropout_p=self.dropout_p if self.training else 0.0)
        return self.o_proj(y.transpose(1, 2).reshape(b, tq, self.num_heads * self.head_dim))


# ---------------------------------------------------------------------------- KV helpers --
@stage("kv_cache_read")
class KVCacheReadStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, new: Tensor, cache: Tensor | None = None) -> Tensor:
        return new if cache is None or cache.numel() == 0 else torch.cat([cache.to(new.dtype), new], dim=-2)


@stage("kv_cache_write")
class KVCacheWriteStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, full: Tensor) -> Tensor:
        return full.detach()


@stage("kv_pca_encode")
class KVPCAEncodeStage(nn.Module):
    def __init__(self, head_dim: int, compressed_dim: int) -> None:
        super().__init__()
        self.proj = nn.Linear(head_dim, compressed_dim, bias=False)
        nn.init.orthogonal_(self.proj.weight)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["head_dim"]), int(cfg["compressed_dim"]))

    def forward(self, x: Tensor) -> Tensor:
        return self.proj(x)


@stage("kv_pca_decode")
class KVPCADecodeStage(nn.Module):
    def __init__(self, head_dim: int, compressed_dim: int) -> None:
        super().__init__()
        self.proj = nn.Linear(compressed_dim, head_dim, bias=False)
        nn.init.orthogonal_(self.proj.weight)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["head_dim"]), int(cfg["compressed_dim"]))

    def forward(self, x: Tensor) -> Tensor:
        return self.proj(x)


@stage("kv_quant_pack")
class KVQuantPackStage(nn.Module):
    """int8 per-token quantisation: returns (int8 codes, fp scale per token)."""

    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, x: Tensor):
        scale = x.detach().abs().amax(dim=-1, keepdim=True).clamp(min=1e-8) / 127.0
        return torch.round(x / scale).clamp(-127, 127).to(torch.int8), scale


@stage("kv_quant_unpack")
class KVQuantUnpackStage(nn.Module):
    def __init__(self, head_dim: int = 64) -> None:
        super().__init__()
        self.head_dim = head_dim

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("head_dim", 64)))

    def forward(self, codes: Tensor, scale: Tensor) -> Tensor:
        return codes.to(scale.dtype) * scale
