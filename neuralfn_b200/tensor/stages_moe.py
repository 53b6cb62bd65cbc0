"""Tensor stages, part 4: mixture-of-experts routing and expert FFNs.

router logits -> [aux-free bias] -> top-k (softmax | sigmoid | sqrt-softplus, renormalised)
-> expert dispatch (SwiGLU experts, weights [E, d, h], [E, h, d], [E, d, h]) -> combine,
plus the density load-balance loss ``E * sum_e mean(softmax)_e^2`` and (extension) the
router z-loss ``mean(logsumexp(logits)^2)``. Reference: ``neuralfn/torch_backend.py:2593-2955``.

The dispatch is dropless. Tokens are sorted by expert once (permute), every expert runs as
one grouped GEMM over its contiguous slice, and results are scattered back weighted - the
same permute/grouped-GEMM/combine shape that the expert-parallel kernels implement across
GPUs (``neuralfn_b200.parallel.ep``).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .stages_core import stage

import os as _os

_FORCE_TORCH_MOE = _os.environ.get("NFN_B200_FORCE_TORCH", "") == "1"


class RoutingStatsMixin:
    """Running telemetry of a router: per-expert load, mean routing entropy, top-1 share."""

    def _init_routing_stats(self, num_experts: int, top_k: int) -> None:
        self._rs_experts, self._rs_top_k = int(num_experts), int(top_k)
        self.last_routing_stats: dict | None = None
        self._rs_accum: list[dict] = []

    @torch.no_grad()
    def _update_routing_stats(self, scores: Tensor, routing_weights: Tensor, routing_indices: Tensor) -> None:
        e = self._rs_experts
        idx = routing_indices.reshape(-1)
        load = torch.bincount(idx, minlength=e).float()
        load = load / load.sum().clamp(min=1.0)
        p = scores.float().reshape(-1, scores.size(-1))
        p = p / p.sum(-1, keepdim=True).clamp(min=1e-12)
        ent = -(p * p.clamp(min=1e-12).log()).sum(-1).mean()
        self.last_routing_stats = {
            "expert_load": load.tolist(), "load_max": float(load.max()), "load_min": float(load.min()),
            "router_entropy": float(ent), "top1_weight_mean": float(routing_weights[..., 0].float().mean()),
            "num_experts": e, "top_k": self._rs_top_k}

    def reset_routing_accum(self) -> None:
        self._rs_accum = []

    def add_to_routing_accum(self) -> None:
        if self.last_routing_stats is not None:
            self._rs_accum.append(self.last_routing_stats)

    def merged_routing_stats(self) -> dict | None:
        if not self._rs_accum:
            return self.last_routing_stats
        n = len(self._rs_accum)
        load = [sum(s["expert_load"][i] for s in self._rs_accum) / n for i in range(self._rs_experts)]
        return {"expert_load": load, "load_max": max(load), "load_min": min(load),
                "router_entropy": sum(s["router_entropy"] for s in self._rs_accum) / n,
                "top1_weight_mean": sum(s["top1_weight_mean"] for s in self._rs_accum) / n,
                "num_experts": self._rs_experts, "top_k": self._rs_top_k, "micro_batches": n}


@stage("router_logits")
class RouterLogitsStage(nn.Module):
    def __init__(self, model_dim: int, experts: int) -> None:
        super().__init__()
        self.gate = nn.Linear(model_dim, experts, bias=False)
        nn.init.normal_(self.gate.weight, std=0.02)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["experts"]))

    def forward(self, x: Tensor) -> Tensor:
        return self.gate(x)


@stage("auxfree_load_balancing")
class AuxFreeBalancingStage(nn.Module):
    """Detached per-expert bias added before top-k; nudged by sign(1/E - realised load) each step."""

    def __init__(self, experts: int, top_k: int = 2, bias_lr: float = 0.001) -> None:
        super().__init__()
        self.experts = int(experts)
        self.top_k = max(min(int(top_k), self.experts), 1)
        self.bias_lr = float(bias_lr)
        self.register_buffer("expert_bias", torch.zeros(self.experts))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["experts"]), int(cfg.get("top_k", 2)), float(cfg.get("bias_lr", 0.001)))

    def forward(self, logits: Tensor) -> Tensor:
        biased = logits + self.expert_bias.to(logits.dtype)
        if self.training:
            with torch.no_grad():
                idx = torch.topk(biased.reshape(-1, self.experts), self.top_k, dim=-1).indices.reshape(-1)
                counts = torch.bincount(idx, minlength=self.experts).float()
                load = counts / counts.sum().clamp(min=1.0)
                self.expert_bias += self.bias_lr * torch.sign(1.0 / self.experts - load)
        return biased


def route_scores(logits: Tensor, score_fn: str) -> Tensor:
    if score_fn == "sqrt_softplus":
        return torch.sqrt(F.softplus(logits.float()).clamp_min(1e-12)).to(logits.dtype)
    if score_fn == "sigmoid":
        return torch.sigmoid(logits)
    return F.softmax(logits, dim=-1)


@stage("topk_route")
class TopKRouteStage(RoutingStatsMixin, nn.Module):
    def __init__(self, top_k: int, experts: int = 8, score_fn: str = "softmax") -> None:
        super().__init__()
        self.top_k, self.score_fn = int(top_k), str(score_fn or "softmax")
        self._init_routing_stats(experts, top_k)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["top_k"]), int(cfg.get("experts", 8)), str(cfg.get("score_fn", "softmax")))

    def forward(self, logits: Tensor):
        scores = route_scores(logits, self.score_fn)
        w, idx = torch.topk(scores, self.top_k, dim=-1)
        w = w / w.sum(dim=-1, keepdim=True)
        self._update_routing_stats(scores, w, idx)
        return w.to(logits.dtype), idx


def moe_hidden_dim(model_dim: int, mlp_mult: float, multiple_of: int | None) -> int:
    if not math.isfinite(float(mlp_mult)) or mlp_mult <= 0:
        raise ValueError("mlp_mult must be finite and positive")
    hidden = max(1, int(model_dim * float(mlp_mult)))
    if multiple_of:
        m = int(multiple_of)
        if m < 0:
            raise ValueError("multiple_of must be non-negative")
        hidden = m * ((hidden + m - 1) // m)
    return hidden


def grouped_swiglu_experts(x_flat: Tensor, w1: Tensor, w2: Tensor, w3: Tensor, weights: Tensor,
                           indices: Tensor) -> Tensor:
    """Dropless MoE FFN on flattened tokens: sort the (token, k) assignments by expert, run every
    expert on its contiguous slice, scatter-add the weighted results back."""
    n, d = x_flat.shape
    top_k = indices.shape[-1]
    experts = w1.shape[0]
    if x_flat.is_cuda and not _FORCE_TORCH_MOE:
        # CUDA + bf16 (directly or under bf16 autocast): grouped tcgen05 GEMMs with native backward
        from ..ops.moe import moe_experts, moe_experts_native_ok
        cast = torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16
        xb, a1, a2, a3 = ((t.to(torch.bfloat16) for t in (x_flat, w1, w2, w3)) if cast else (x_flat, w1, w2, w3))
        if moe_experts_native_ok(xb, a1, a2, a3, indices):
            return moe_experts(xb, a1, a2, a3, weights, indices).to(x_flat.dtype if not cast else torch.bfloat16)
    flat_e = indices.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    token_of = (order // top_k)
    counts = torch.bincount(flat_e, minlength=experts)
    xs = x_flat[token_of]
    ws = weights.reshape(-1)[order].unsqueeze(-1).to(x_flat.dtype)
    outs = torch.empty_like(xs)
    start = 0
    for e, c in enumerate(counts.tolist()):
        if c == 0:
            continue
        seg = xs[start:start + c]
        h = F.silu(seg @ w1[e].to(seg.dtype)) * (seg @ w3[e].to(seg.dtype))
        outs[start:start + c] = h @ w2[e].to(seg.dtype)
        start += c
    out = torch.zeros_like(x_flat)
    out.index_add_(0, token_of, outs * ws)
    return out


@stage("expert_dispatch")
class ExpertDispatchStage(nn.Module):
    def __init__(self, model_dim: int, experts: int, mlp_mult: float = 4.0, multiple_of: int | None = None,
                 hidden_dim: int | None = None) -> None:
        super().__init__()
        hidden = hidden_dim or moe_hidden_dim(model_dim, mlp_mult, multiple_of)
        self.w1 = nn.Parameter(torch.empty(experts, model_dim, hidden))
        self.w2 = nn.Parameter(torch.empty(experts, hidden, model_dim))
        self.w3 = nn.Parameter(torch.empty(experts, model_dim, hidden))
        for w in (self.w1, self.w2, self.w3):
            nn.init.normal_(w, std=0.02)
        self.experts = experts

    @classmethod
    def from_config(cls, cfg):
        mo = cfg.get("multiple_of")
        return cls(int(cfg["model_dim"]), int(cfg["experts"]), float(cfg.get("mlp_mult", 4.0)),
                   int(mo) if mo is not None else None, cfg.get("hidden_dim"))

    def forward(self, x: Tensor, routing_weights: Tensor, routing_indices: Tensor) -> Tensor:
        b, t, d = x.shape
        out = grouped_swiglu_experts(x.reshape(-1, d), self.w1, self.w2, self.w3,
                                     routing_weights.reshape(-1, routing_weights.shape[-1]),
                                     routing_indices.reshape(-1, routing_indices.shape[-1]))
        return out.reshape(b, t, d)


@stage("expert_combine")
class ExpertCombineStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, x: Tensor) -> Tensor:
        return x


@stage("broadcast_expert_routes")
class BroadcastExpertRoutesStage(nn.Module):
    """Batch-level routes [B, k] (or [B, 1, k]) broadcast over the sequence axis of ``hidden``."""

    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, hidden: Tensor, expert_weights: Tensor, expert_indices: Tensor):
        if hidden.ndim != 3:
            raise ValueError("broadcast_expert_routes expects hidden shaped [batch, seq, dim]")
        b, t, _ = hidden.shape

        def widen(r: Tensor) -> Tensor:
            if r.ndim == 1:
                r = r.unsqueeze(0)
            if r.ndim == 2:
                r = r.unsqueeze(1)
            if r.ndim != 3 or r.size(0) != b:
                raise ValueError("broadcast_expert_routes expects routes shaped [batch, top_k] or [batch, seq, top_k]")
            if r.size(1) == 1:
                r = r.expand(b, t, r.size(-1))
            elif r.size(1) != t:
                raise ValueError("broadcast_expert_routes sequence axis must be 1 or match hidden seq_len")
            return r.contiguous()

        return widen(expert_weights).to(hidden.dtype), widen(expert_indices.long())


@stage("load_balance_loss")
class LoadBalanceLossStage(nn.Module):
    """E * sum_e density_e^2 with density = mean softmax probability of expert e."""

    def __init__(self, experts: int) -> None:
        super().__init__()
        self.experts = int(experts)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["experts"]))

    def forward(self, router_logits: Tensor, routing_weights: Tensor, routing_indices: Tensor):
        density = F.softmax(router_logits, dim=-1).mean(dim=(0, 1))
        return self.experts * (density * density).sum(), router_logits


@stage("router_z_loss")
class RouterZLossStage(nn.Module):
    """mean(logsumexp(router_logits)^2) - keeps router logits small (not in the reference catalogue)."""

    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, router_logits: Tensor) -> Tensor:
        return torch.logsumexp(router_logits.float(), dim=-1).pow(2).mean()


@stage("aux_loss_add")
class AuxLossAddStage(nn.Module):
    def __init__(self, coef: float) -> None:
        super().__init__()
        self.coef = float(coef)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg["coef"]))

    def forward(self, main_loss: Tensor, aux_loss: Tensor) -> Tensor:
        return main_loss + self.coef * aux_loss
