"""Tensor stages, part 1: embeddings, heads, norms, residuals, linears, adapters.

Every ``module_type`` a graph node may name is registered here (or in the sibling
``stages_*`` modules) through ``@stage``; ``build_module(module_type, config)``
instantiates it. Semantics and config keys follow the reference stage catalogue
(``neuralfn/torch_backend.py:343-1097,2404-2530,3311-3920``) so graphs interchange.

On CUDA the hot stages route to the sm_100a kernel library through
``neuralfn_b200.tensor.kernel_bridge`` (autograd functions around the C ABI); on CPU
they run as plain PyTorch, which is also the oracle the kernel tests compare against.
"""
from __future__ import annotations

import math
from typing import Any, Callable

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

STAGE_REGISTRY: dict[str, Callable[[dict[str, Any]], nn.Module]] = {}


def stage(*names: str):
    """Register ``factory(cfg) -> nn.Module`` (or a class with ``from_config``) under module types."""
    def deco(obj):
        factory = obj.from_config if hasattr(obj, "from_config") else obj
        for n in names:
            STAGE_REGISTRY[n] = factory
        return obj
    return deco


def build_module(module_type: str, module_config: dict[str, Any] | None = None, tile_cuda_config: Any = None) -> nn.Module:
    """Instantiate the stage registered for ``module_type`` from its JSON config."""
    from . import (stages_attention, stages_attention_blocks, stages_linear, stages_losses,  # noqa: F401
                   stages_moe, stages_misc, stages_semantic, stages_vision)
    cfg = dict(module_config or {})
    cfg["__module_type__"] = module_type
    try:
        factory = STAGE_REGISTRY[module_type]
    except KeyError:
        raise ValueError(f"Unknown torch module type: {module_type!r}") from None
    return factory(cfg)


# ----------------------------------------------------------------- embeddings / heads --
@stage("token_embedding")
class TokenEmbeddingStage(nn.Module):
    """tokens -> (hidden, weight). The weight is a second output so a tied head can consume it."""

    def __init__(self, vocab_size: int, model_dim: int) -> None:
        super().__init__()
        self.embedding = nn.Embedding(vocab_size, model_dim)
        nn.init.normal_(self.embedding.weight, std=0.02)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["vocab_size"]), int(cfg["model_dim"]))

    def forward(self, tokens: Tensor):
        return self.embedding(tokens.long()), self.embedding.weight


@stage("absolute_position_embedding")
class AbsolutePositionEmbeddingStage(nn.Module):
    def __init__(self, max_seq_len: int, model_dim: int) -> None:
        super().__init__()
        self.embedding = nn.Embedding(max_seq_len, model_dim)
        nn.init.normal_(self.embedding.weight, std=0.02)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("max_seq_len", 1024)), int(cfg["model_dim"]))

    def forward(self, x: Tensor) -> Tensor:
        pos = torch.arange(x.size(1), device=x.device)
        return x + self.embedding(pos).unsqueeze(0).to(x.dtype)


@stage("tied_lm_head")
class TiedLMHeadStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, x: Tensor, weight: Tensor) -> Tensor:
        return F.linear(x, weight.to(x.dtype))


@stage("lm_head")
class LMHeadStage(nn.Module):
    def __init__(self, model_dim: int, vocab_size: int) -> None:
        super().__init__()
        self.proj = nn.Linear(model_dim, vocab_size, bias=False)
        nn.init.normal_(self.proj.weight, std=0.02)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["vocab_size"]))

    def forward(self, x: Tensor) -> Tensor:
        return self.proj(x)


@stage("logit_softcap")
class LogitSoftcapStage(nn.Module):
    def __init__(self, softcap: float) -> None:
        super().__init__()
        self.softcap = float(softcap)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg["softcap"]))

    def forward(self, logits: Tensor) -> Tensor:
        return self.softcap * torch.tanh(logits / self.softcap) if self.softcap > 0 else logits


@stage("tensor_scale")
class TensorScaleStage(nn.Module):
    def __init__(self, scale: float = 1.0) -> None:
        super().__init__()
        self.scale = float(scale)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("scale", 1.0)))

    def forward(self, x: Tensor) -> Tensor:
        return x * self.scale


@stage("loss_scale")
class LossScaleStage(TensorScaleStage):
    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("coef", 1.0)))


# ------------------------------------------------------------------------------ norms --
@stage("rms_norm")
class RMSNormStage(nn.Module):
    """RMSNorm with optional weight; ``centered`` stores w with effective scale 1 + w (zero init)."""

    def __init__(self, model_dim: int | None = None, eps: float = 1e-6, centered: bool = False,
                 force_float32: bool = False) -> None:
        super().__init__()
        self.eps, self.centered, self.force_float32 = float(eps), bool(centered), bool(force_float32)
        if model_dim is not None:
            init = torch.zeros(int(model_dim)) if centered else torch.ones(int(model_dim))
            self.weight = nn.Parameter(init)
        else:
            self.register_parameter("weight", None)

    @classmethod
    def from_config(cls, cfg):
        md = cfg.get("model_dim")
        return cls(None if md is None else int(md), float(cfg.get("eps", 1e-6)),
                   bool(cfg.get("centered", False)), bool(cfg.get("force_float32", False)))

    def forward(self, x: Tensor) -> Tensor:
        from .kernel_bridge import rms_norm
        return rms_norm(x, self.weight, self.eps, self.centered, self.force_float32)


@stage("layer_norm")
class LayerNormStage(nn.Module):
    def __init__(self, model_dim: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.norm = nn.LayerNorm(model_dim, eps=eps)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), float(cfg.get("eps", 1e-5)))

    def forward(self, x: Tensor) -> Tensor:
        from .kernel_bridge import layer_norm
        return layer_norm(x, self.norm.weight, self.norm.bias, self.norm.eps)


@stage("dyt")
class DyTStage(nn.Module):
    """Dynamic Tanh: gamma * tanh(alpha * x) + beta."""

    def __init__(self, model_dim: int, alpha_init: float = 1.0) -> None:
        super().__init__()
        self.alpha = nn.Parameter(torch.tensor(float(alpha_init)))
        self.gamma = nn.Parameter(torch.ones(model_dim))
        self.beta = nn.Parameter(torch.zeros(model_dim))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), float(cfg.get("alpha_init", 1.0)))

    def forward(self, x: Tensor) -> Tensor:
        return self.gamma.to(x.dtype) * torch.tanh(self.alpha.to(x.dtype) * x) + self.beta.to(x.dtype)


@stage("group_norm")
class GroupNormStage(nn.Module):
    def __init__(self, model_dim: int, num_groups: int = 1, eps: float = 1e-5) -> None:
        super().__init__()
        self.norm = nn.GroupNorm(num_groups, model_dim, eps=eps)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg.get("num_groups", 1)), float(cfg.get("eps", 1e-5)))

    def forward(self, x: Tensor) -> Tensor:
        shape = x.shape
        y = self.norm(x.reshape(-1, shape[-1], 1).float()).to(x.dtype)
        return y.reshape(shape)


@stage("qk_norm")
class QKNormStage(nn.Module):
    """Weightless RMS over head_dim applied to q and k ([B, H, T, D])."""

    def __init__(self, eps: float = 1e-6, force_float32: bool = False) -> None:
        super().__init__()
        self.eps, self.force_float32 = float(eps), bool(force_float32)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("eps", 1e-6)), bool(cfg.get("force_float32", False)))

    def _norm(self, t: Tensor) -> Tensor:
        src = t.float() if self.force_float32 else t
        return (src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + self.eps)).to(t.dtype)

    def forward(self, q: Tensor, k: Tensor):
        return self._norm(q), self._norm(k)


# -------------------------------------------------------------------------- residuals --
@stage("residual_add")
class ResidualAddStage(nn.Module):
    """x + scale * delta with a learnable per-channel scale."""

    def __init__(self, dim: int, init_scale: float = 1.0) -> None:
        super().__init__()
        self.scale = nn.Parameter(torch.full((dim,), float(init_scale)))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["dim"]), float(cfg.get("init_scale", 1.0)))

    def forward(self, x: Tensor, delta: Tensor) -> Tensor:
        return x + self.scale.to(delta.dtype) * delta


@stage("residual_mix")
class ResidualMixStage(nn.Module):
    def __init__(self, dim: int, primary_init: float = 1.0, skip_init: float = 0.0) -> None:
        super().__init__()
        self.primary = nn.Parameter(torch.full((dim,), float(primary_init)))
        self.skip = nn.Parameter(torch.full((dim,), float(skip_init)))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["dim"]), float(cfg.get("primary_init", 1.0)), float(cfg.get("skip_init", 0.0)))

    def forward(self, x: Tensor, skip: Tensor) -> Tensor:
        return self.primary.to(x.dtype) * x + self.skip.to(x.dtype) * skip


@stage("manifold_hyper_connection")
class ManifoldHyperConnectionStage(nn.Module):
    """Norm-preserving residual mix: sqrt(1 - beta^2) * residual + beta * delta."""

    def __init__(self, dim: int, beta_init: float = 0.1) -> None:
        super().__init__()
        self.beta_raw = nn.Parameter(torch.full((dim,), math.atanh(min(max(beta_init, 1e-4), 0.999))))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["dim"]), float(cfg.get("beta_init", 0.1)))

    def forward(self, x: Tensor, delta: Tensor) -> Tensor:
        beta = torch.tanh(self.beta_raw).to(x.dtype)
        return torch.sqrt(1.0 - beta * beta) * x + beta * delta
