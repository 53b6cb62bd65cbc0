"""Tensor stages, part 3: attention building blocks.

Head reshapes, rotary embeddings (both conventions and linear / NTK / YaRN scaling),
QK gain, the SDPA core and its masked variants (sliding window, block sparse, streaming
sinks, native sparse), differential attention, the fused causal / MLA / DFlash blocks and
the KV-cache helpers. Semantics follow ``neuralfn/torch_backend.py:279-340,428-596,
1728-2010,2236-2401,2536-2585``.

Tensors between these stages are ``[B, H, T, D]``. On CUDA the SDPA core, sliding-window
attention and RoPE go to the sm_100a kernels via ``kernel_bridge``.
"""
from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .stages_core import stage


# ------------------------------------------------------------------------------ rotary --
def rope_inv_freq(dim: int, base: float, scaling: dict[str, Any] | None = None) -> Tensor:
    idx = torch.arange(0, dim, 2, dtype=torch.float32)
    inv = 1.0 / (base ** (idx / dim))
    if not scaling:
        return inv
    kind = str(scaling.get("type", scaling.get("rope_type", "linear"))).lower()
    factor = float(scaling.get("factor", 1.0)) or 1.0
    if kind in ("linear", "pi"):
        return inv / factor
    if kind in ("ntk", "ntk-aware", "dynamic"):
        return 1.0 / ((base * factor ** (dim / max(dim - 2, 1))) ** (idx / dim))
    if kind == "yarn":
        orig = float(scaling.get("original_max_position", scaling.get("original_max_position_embeddings", 2048)))
        fast, slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))

        def corr(n_rot: float) -> float:
            return dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(base))

        low = max(math.floor(corr(fast)), 0)
        high = min(math.ceil(corr(slow)), dim // 2 - 1)
        if high <= low:
            high = low + 1
        ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0.0, 1.0)
        return inv * (1.0 - ramp) + (inv / factor) * ramp
    return inv


def rope_tables(positions: Tensor, inv_freq: Tensor, dtype: torch.dtype) -> tuple[Tensor, Tensor]:
    freqs = torch.outer(positions.to(inv_freq.dtype), inv_freq.to(positions.device))
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def apply_rotary_emb(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """"legacy" convention: half-split pairs rotated by the negative angle."""
    half = x.size(-1) // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat((x1 * cos + x2 * sin, x2 * cos - x1 * sin), dim=-1)


def apply_rotary_emb_hf(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """"hf" convention (rotate_half): half-split pairs rotated by the positive angle."""
    half = x.size(-1) // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def apply_rotary_interleaved(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Adjacent (even, odd) pairs rotated by the positive angle (GGUF layout)."""
    x1, x2 = x[..., 0::2], x[..., 1::2]
    out = torch.stack((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
    return out.flatten(-2)


@stage("reshape_heads")
class ReshapeHeadsStage(nn.Module):
    def __init__(self, num_heads: int) -> None:
        super().__init__()
        self.num_heads = int(num_heads)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["num_heads"]))

    def forward(self, x: Tensor) -> Tensor:
        b, t, w = x.shape
        if w % self.num_heads:
            raise ValueError("Last tensor dimension must be divisible by num_heads")
        return x.reshape(b, t, self.num_heads, w // self.num_heads).transpose(1, 2)


@stage("merge_heads")
class MergeHeadsStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, x: Tensor) -> Tensor:
        b, h, t, d = x.shape
        return x.transpose(1, 2).reshape(b, t, h * d)


@stage("repeat_kv")
class RepeatKVStage(nn.Module):
    def __init__(self, num_heads: int, num_kv_heads: int) -> None:
        super().__init__()
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        self.repeats = num_heads // num_kv_heads

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["num_heads"]), int(cfg["num_kv_heads"]))

    def forward(self, x: Tensor) -> Tensor:
        return x if self.repeats == 1 else x.repeat_interleave(self.repeats, dim=1)


@stage("rotary_embedding")
class RotaryEmbeddingStage(nn.Module):
    def __init__(self, head_dim: int, rope_base: float, rope_scaling: dict[str, Any] | None = None,
                 convention: str = "legacy") -> None:
        super().__init__()
        if head_dim % 2:
            raise ValueError("head_dim must be even for rotary embeddings")
        if convention not in {"legacy", "hf"}:
            raise ValueError("rotary convention must be 'legacy' or 'hf'")
        self.register_buffer("inv_freq", rope_inv_freq(head_dim, rope_base, rope_scaling), persistent=False)
        self.convention = convention

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["head_dim"]), float(cfg["rope_base"]), cfg.get("rope_scaling"),
                   str(cfg.get("convention", "legacy")))

    def forward(self, q: Tensor, k: Tensor):
        pos = torch.arange(q.size(2), device=q.device)
        cos, sin = rope_tables(pos, self.inv_freq, q.dtype)
        fn = apply_rotary_emb_hf if self.convention == "hf" else apply_rotary_emb
        return fn(q, cos, sin), fn(k, cos, sin)


@stage("qk_gain")
class QKGainStage(nn.Module):
    def __init__(self, num_heads: int, qk_gain_init: float = 1.0) -> None:
        super().__init__()
        self.q_gain = nn.Parameter(torch.full((num_heads,), float(qk_gain_init)))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["num_heads"]), float(cfg.get("qk_gain_init", 1.0)))

    def forward(self, q: Tensor) -> Tensor:
        return q * self.q_gain.to(q.dtype)[None, :, None, None]


# --------------------------------------------------------------------------- SDPA core --
def sparse_attention_mask(seq_q: int, seq_k: int, *, is_causal: bool, window: int | None, num_sinks: int,
                          block: int | None, compress_stride: int | None, device, dtype) -> Tensor:
    """Additive mask [seq_q, seq_k]: allowed = causal & (window | sinks | same block | strided).
    Queries are right-aligned to the keys (KV-cache compatible). Window W = keys q-W+1 .. q."""
    i = torch.arange(seq_q, device=device).unsqueeze(1) + (seq_k - seq_q)
    j = torch.arange(seq_k, device=device).unsqueeze(0)
    causal = (j <= i) if is_causal else torch.ones(seq_q, seq_k, dtype=torch.bool, device=device)
    rules = []
    if window is not None and window > 0:
        rules.append(j > i - window)
    if num_sinks and num_sinks > 0:
        rules.append((j < num_sinks).expand(seq_q, seq_k))
    if block is not None and block > 0:
        rules.append(i // block == j // block)
    if compress_stride is not None and compress_stride > 1:
        rules.append((j % compress_stride == 0).expand(seq_q, seq_k))
    keep = torch.ones(seq_q, seq_k, dtype=torch.bool, device=device)
    if rules:
        keep = rules[0]
        for r in rules[1:]:
            keep = keep | r
    return torch.zeros(seq_q, seq_k, dtype=dtype, device=device).masked_fill(~(causal & keep), float("-inf"))


@stage("scaled_dot_product_attention")
class ScaledDotProductAttentionStage(nn.Module):
    def __init__(self, is_causal: bool = True, backend: str = "sdpa", dropout_p: float = 0.0) -> None:
        super().__init__()
        self.is_causal, self.backend, self.dropout_p = bool(is_causal), backend, float(dropout_p)

    @classmethod
    def from_config(cls, cfg):
        return cls(bool(cfg.get("is_causal", True)), str(cfg.get("backend", "sdpa")), float(cfg.get("dropout_p", 0.0)))

    def forward(self, q: Tensor, k: Tensor, v: Tensor) -> Tensor:
        from .kernel_bridge import attention
        drop = self.dropout_p if self.training else 0.0
        return attention(q, k, v, causal=self.is_causal, window=0, dropout_p=drop, math_path=self.backend == "math")


class _MaskedSDPAStage(nn.Module):
    def __init__(self, *, is_causal: bool, dropout_p: float) -> None:
        super().__init__()
        self.is_causal, self.dropout_p = bool(is_causal), float(dropout_p)

    def _rules(self) -> dict[str, Any]:
        raise NotImplementedError

    def forward(self, q: Tensor, k: Tensor, v: Tensor) -> Tensor:
        rules = self._rules()
        drop = self.dropout_p if self.training else 0.0
        only_window = (rules["window"] and not rules["num_sinks"] and not rules["block"]
                       and not rules["compress_stride"] and q.size(-2) == k.size(-2))
        if only_window:
            from .kernel_bridge import attention
            return attention(q, k, v, causal=self.is_causal, window=int(rules["window"]), dropout_p=drop)
        mask = sparse_attention_mask(q.size(-2), k.size(-2), is_causal=self.is_causal, device=q.device,
                                     dtype=q.dtype, **rules)
        return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=drop, is_causal=False,
                                              enable_gqa=q.size(1) != k.size(1))


@stage("sliding_window_attention")
class SlidingWindowAttentionStage(_MaskedSDPAStage):
    def __init__(self, window_size: int = 256, is_causal: bool = True, dropout_p: float = 0.0) -> None:
        super().__init__(is_causal=is_causal, dropout_p=dropout_p)
        self.window_size = int(window_size)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("window_size", 256)), bool(cfg.get("is_causal", True)), float(cfg.get("dropout_p", 0.0)))

    def _rules(self):
        return {"window": self.window_size, "num_sinks": 0, "block": None, "compress_stride": None}


@stage("block_sparse_attention")
class BlockSparseAttentionStage(_MaskedSDPAStage):
    def __init__(self, sparse_block_size: int = 64, num_sinks: int = 0, is_causal: bool = True,
                 dropout_p: float = 0.0) -> None:
        super().__init__(is_causal=is_causal, dropout_p=dropout_p)
        self.sparse_block_size, self.num_sinks = int(sparse_block_size), int(num_sinks)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("sparse_block_size", 64)), int(cfg.get("num_sinks", 0)),
                   bool(cfg.get("is_causal", True)), float(cfg.get("dropout_p", 0.0)))

    def _rules(self):
        return {"window": None, "num_sinks": self.num_sinks, "block": self.sparse_block_size, "compress_stride": None}


@stage("streaming_attention_sinks")
class StreamingAttentionSinksStage(_MaskedSDPAStage):
    def __init__(self, window_size: int = 256, num_sinks: int = 4, is_causal: bool = True,
                 dropout_p: float = 0.0) -> None:
        super().__init__(is_causal=is_causal, dropout_p=dropout_p)
        self.window_size, self.num_sinks = int(window_size), int(num_sinks)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("window_size", 256)), int(cfg.get("num_sinks", 4)),
                   bool(cfg.get("is_causal", True)), float(cfg.get("dropout_p", 0.0)))

    def _rules(self):
        return {"window": self.window_size, "num_sinks": self.num_sinks, "block": None, "compress_stride": None}


@stage("native_sparse_attention")
class NativeSparseAttentionStage(_MaskedSDPAStage):
    """Deterministic NSA stand-in: local window + sink tokens + every ``compress_stride``-th key."""

    def __init__(self, window_size: int = 128, sparse_block_size: int = 64, num_sinks: int = 0,
                 compress_stride: int = 16, is_causal: bool = True, dropout_p: float = 0.0) -> None:
        super().__init__(is_causal=is_causal, dropout_p=dropout_p)
        self.window_size, self.num_sinks, self.compress_stride = int(window_size), int(num_sinks), int(compress_stride)
        self.sparse_block_size = int(sparse_block_size)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("window_size", 128)), int(cfg.get("sparse_block_size", 64)),
                   int(cfg.get("num_sinks", 0)), int(cfg.get("compress_stride", 16)),
                   bool(cfg.get("is_causal", True)), float(cfg.get("dropout_p", 0.0)))

    def _rules(self):
        return {"window": self.window_size, "num_sinks": self.num_sinks, "block": None,
                "compress_stride": self.compress_stride}


@stage("differential_attention")
class DifferentialAttentionStage(nn.Module):
    """Two softmax maps on the two halves of head_dim, a1 - lambda * a2, head RMS, * (1 - lambda_init)."""

    def __init__(self, lambda_init: float = 0.8, is_causal: bool = True, dropout_p: float = 0.0,
                 eps: float = 1e-5) -> None:
        super().__init__()
        self.is_causal, self.dropout_p, self.eps = bool(is_causal), float(dropout_p), float(eps)
        self.lambda_param = nn.Parameter(torch.tensor(float(lambda_init)))
        self.lambda_init = float(lambda_init)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("lambda_init", 0.8)), bool(cfg.get("is_causal", True)), float(cfg.get("dropout_p", 0.0)))

    def forward(self, q: Tensor, k: Tensor, v: Tensor) -> Tensor:
        d = q.size(-1)
        if d % 2:
            raise ValueError("differential attention requires an even head_dim")
        h = d // 2
        drop = self.dropout_p if self.training else 0.0
        gqa = q.size(1) != k.size(1)
        a1 = F.scaled_dot_product_attention(q[..., :h], k[..., :h], v, dropout_p=drop, is_causal=self.is_causal,
                                            enable_gqa=gqa)
        a2 = F.scaled_dot_product_attention(q[..., h:], k[..., h:], v, dropout_p=drop, is_causal=self.is_causal,
                                            enable_gqa=gqa)
        out = a1 - self.lambda_param.to(a1.dtype) * a2
        return F.rms_norm(out, (out.size(-1),), eps=self.eps) * (1.0 - self.lambda_init)
