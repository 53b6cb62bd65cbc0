"""Mixture-of-experts Llama for training with expert parallelism inside data parallelism.

Every rank holds a full copy of the dense tensors (embedding, attention projections, routers, norms,
head) and ``E / W`` experts of every layer, and trains on its own batch. A block is RMSNorm ->
rotary GQA attention -> residual -> RMSNorm -> router (softmax | sigmoid | sqrt-softplus scores,
top-k, renormalised) -> ``expert_parallel_ffn`` -> residual. The loss is token cross-entropy plus
the density balance loss ``coef * E * sum_e mean(scores)_e^2`` and the router z-loss
``coef * mean(logsumexp(logits)^2)``, both averaged over the layers.

Gradients: dense tensors are averaged over the group after the backward pass; an expert's gradient
already collects the rows of every rank on its owner and is divided by W to stay the gradient of
the same mean loss. Parameters live in one flat bf16 buffer (experts first) with a flat gradient
buffer, so ``FlatAdamWTrainer`` (fp32 master weights + the fused flat AdamW kernel, clipping by
the group-wide norm) drives it like the tensor-parallel Llama.

Reference counterparts: the standard-MoE family (``nfn_mixllama_native_train``, selector
``moe|mixllama|mixllama_fast``) with ``topk_route`` / ``moe_swiglu_*`` / ``moe_router_aux_*``
(``kernels.cu:12612-12862, 15028-15072, 22194-22237``), single GPU, dense expert tensors; the
router z-loss is an extension (the reference has none).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..models.gpt2 import FlatLayout, ParamSpec
from ..tensor import kernel_bridge as KB
from ..tensor.stages_moe import route_scores
from .ep_train import expert_parallel_ffn
from .tp_llama import TPLlamaTrainer as FlatAdamWTrainer

__all__ = ["MoELlamaConfig", "EPMoELlama", "FlatAdamWTrainer", "moe_llama_reference_loss"]


@dataclass
class MoELlamaConfig:
    n_layer: int = 4
    n_head: int = 8
    n_kv_head: int = 4
    d_model: int = 512
    n_experts: int = 8
    top_k: int = 2
    expert_hidden: int = 1024
    vocab_size: int = 32000
    max_seq_len: int = 2048
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    score_fn: str = "softmax"
    balance_coef: float = 0.01
    router_z_coef: float = 1e-3
    vocab_pad_to: int = 128

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head

    @property
    def padded_vocab(self) -> int:
        p = self.vocab_pad_to
        return (self.vocab_size + p - 1) // p * p


def moe_llama_param_specs(cfg: MoELlamaConfig, world: int) -> list[ParamSpec]:
    if cfg.n_experts % world:
        raise ValueError(f"{cfg.n_experts} experts do not divide over {world} ranks")
    C, hd, El, h = cfg.d_model, cfg.head_dim, cfg.n_experts // world, cfg.expert_hidden
    specs = []
    for l in range(cfg.n_layer):
        p = f"layers.{l}."
        specs += [ParamSpec(p + "w1", (El, C, h), True, "normal"), ParamSpec(p + "w2", (El, h, C), True, "resid"), ParamSpec(p + "w3", (El, C, h), True, "normal")]
    specs += [ParamSpec("tok_embeddings", (cfg.padded_vocab, C), True, "normal"), ParamSpec("lm_head", (cfg.padded_vocab, C), True, "normal")]
    for l in range(cfg.n_layer):
        p = f"layers.{l}."
        specs += [ParamSpec(p + "wqkv", ((cfg.n_head + 2 * cfg.n_kv_head) * hd, C), True, "normal"), ParamSpec(p + "wo", (C, cfg.n_head * hd), True, "resid"),
                  ParamSpec(p + "router", (cfg.n_experts, C), True, "normal")]
    for l in range(cfg.n_layer):
        specs += [ParamSpec(f"layers.{l}.attn_norm", (C,), False, "ones"), ParamSpec(f"layers.{l}.ffn_norm", (C,), False, "ones")]
    specs.append(ParamSpec("norm", (C,), False, "ones"))
    return specs


def _is_expert(name: str) -> bool:
    return name.endswith((".w1", ".w2", ".w3"))


def _forward_loss(cfg: MoELlamaConfig, p: dict, tokens: torch.Tensor, targets: torch.Tensor, ffn, dtype) -> torch.Tensor:
    """Shared by the parallel model and the single-process oracle; ``ffn(l, h, w, idx)`` runs the experts."""
    B, T = tokens.shape
    M, hd, Hq, Hkv, E = B * T, cfg.head_dim, cfg.n_head, cfg.n_kv_head, cfg.n_experts
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
    cos, sin = ang.cos().float().to(tokens.device).contiguous(), ang.sin().float().to(tokens.device).contiguous()
    x = F.embedding(tokens.reshape(-1).long(), p["tok_embeddings"])
    balance = x.new_zeros((), dtype=torch.float32)
    zloss = x.new_zeros((), dtype=torch.float32)
    for l in range(cfg.n_layer):
        q_ = f"layers.{l}."
        qkv = KB.linear(KB.rms_norm(x, p[q_ + "attn_norm"], cfg.norm_eps), p[q_ + "wqkv"])
        qkv = KB.rope_packed_qkv(qkv.contiguous(), T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=cos, sin=sin, convention="hf")
        a = KB.attention_packed_qkv(qkv, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, causal=True)
        x = x + KB.linear(a, p[q_ + "wo"])
        h = KB.rms_norm(x, p[q_ + "ffn_norm"], cfg.norm_eps)
        logits = KB.linear(h, p[q_ + "router"]).float()
        scores = route_scores(logits, cfg.score_fn)
        w, idx = torch.topk(scores, cfg.top_k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        balance = balance + E * torch.softmax(logits, -1).mean(0).pow(2).sum()
        zloss = zloss + torch.logsumexp(logits, -1).pow(2).mean()
        x = x + ffn(l, h, w, idx).to(x.dtype)
    x = KB.rms_norm(x, p["norm"], cfg.norm_eps)
    logits = KB.linear(x, p["lm_head"])
    if cfg.padded_vocab != cfg.vocab_size:
        pad = torch.zeros(cfg.padded_vocab, dtype=logits.dtype, device=logits.device)
        pad[cfg.vocab_size:] = -30000.0
        logits = logits + pad
    ce = KB.token_cross_entropy(logits, targets.reshape(-1))
    return ce + cfg.balance_coef * balance / cfg.n_layer + cfg.router_z_coef * zloss / cfg.n_layer


class EPMoELlama:
    def __init__(self, cfg: MoELlamaConfig, device, group=None, *, dtype=None, seed: int = 1337) -> None:
        self.cfg, self.group = cfg, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        dev = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        self.layout = FlatLayout(moe_llama_param_specs(cfg, self.world))
        self.n_sharded = self.layout.offsets["tok_embeddings"]  # expert tensors come first
        self.params = torch.zeros(self.layout.n_total, dtype=self.dtype, device=dev)
        self.grads = torch.zeros_like(self.params)
        self.p = {}
        gviews = self.layout.views(self.grads)
        for name, view in self.layout.views(self.params).items():
            view.requires_grad_(True)
            view.main_grad = gviews[name]
            self.p[name] = view
        self.init_(seed)

    @torch.no_grad()
    def init_(self, seed: int) -> None:
        """Dense tensors from a stream all ranks share; every expert from a stream keyed by its
        GLOBAL index, so the model does not depend on how many ranks hold it."""
        cfg, El = self.cfg, self.cfg.n_experts // self.world
        rs = 0.02 / math.sqrt(2 * cfg.n_layer)
        shared = torch.Generator().manual_seed(seed)
        for s in self.layout.order:
            v = self.p[s.name]
            if s.init == "ones":
                v.fill_(1.0)
            elif _is_expert(s.name):
                layer, which = int(s.name.split(".")[1]), s.name.rsplit(".", 1)[1]
                for j in range(El):
                    e = self.rank * El + j
                    g = torch.Generator().manual_seed(seed * 1000003 + layer * 4099 + e * 7 + {"w1": 1, "w2": 2, "w3": 3}[which])
                    v[j].copy_(torch.empty(s.shape[1:]).normal_(0.0, rs if s.init == "resid" else 0.02, generator=g))
            else:
                v.copy_(torch.empty(s.shape).normal_(0.0, rs if s.init == "resid" else 0.02, generator=shared))
        for name in ("tok_embeddings", "lm_head"):
            self.p[name][cfg.vocab_size:].zero_()

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """This rank's loss over ITS batch [B, T] (cross-entropy + router losses)."""
        p, cfg = self.p, self.cfg

        exchange = self._exchange(tokens.numel())

        def ffn(l, h, w, idx):
            q_ = f"layers.{l}."
            if exchange is not None:
                from .ep_fused_train import fused_expert_parallel_ffn
                return fused_expert_parallel_ffn(h, w, idx, p[q_ + "w1"], p[q_ + "w2"], p[q_ + "w3"], exchange)
            return expert_parallel_ffn(h, w, idx, p[q_ + "w1"], p[q_ + "w2"], p[q_ + "w3"], cfg.n_experts, self.group)

        return _forward_loss(cfg, p, tokens, targets, ffn, self.dtype)

    def _exchange(self, n_tokens: int):
        """Peer-memory exchange buffers for the expert rows (CUDA bf16, up to 8 ranks); None selects the library
        all-to-all (``NFN_EP_EXCHANGE=nccl``, CPU, other dtypes). Built once for the largest batch seen."""
        import os
        cfg = self.cfg
        dev = self.params.device
        if (dev.type != "cuda" or self.dtype != torch.bfloat16 or self.world > 8 or os.environ.get("NFN_EP_EXCHANGE", "peer") == "nccl"
                or cfg.d_model % 64 or cfg.expert_hidden % 64):
            return None
        ex = getattr(self, "_peer_exchange", None)
        if ex is None or ex.T < n_tokens:
            from .ep_fused_train import PeerExchange
            factor = float(os.environ.get("NFN_EP_CAPACITY_FACTOR", self.world))
            ex = self._peer_exchange = PeerExchange(cfg.n_experts, cfg.top_k, cfg.d_model, n_tokens, dev, self.group, capacity_factor=factor)
        return ex

    def backward(self, loss: torch.Tensor) -> None:
        self.grads.zero_()
        for v in self.p.values():
            v.grad = None
        loss.backward()
        with torch.no_grad():
            for v in self.p.values():
                if v.grad is not None:
                    v.main_grad.copy_(v.grad)
                    v.grad = None
            if self.world > 1:
                dist.all_reduce(self.grads[self.n_sharded:], group=self.group)
                self.grads.mul_(1.0 / self.world)  # dense: average of the ranks; experts: owner's sum over ranks / W

    def reduce_loss(self, mine: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(mine, group=self.group)
            mine /= self.world
        return mine

    def grad_norm(self) -> torch.Tensor:
        s = torch.linalg.vector_norm(self.grads[:self.n_sharded], dtype=torch.float32) ** 2
        if self.world > 1:
            dist.all_reduce(s, group=self.group)
        return torch.sqrt(s + torch.linalg.vector_norm(self.grads[self.n_sharded:], dtype=torch.float32) ** 2)

    def full_state(self) -> dict[str, torch.Tensor]:
        """Unsharded fp32 parameters on the host (expert tensors gathered over the group)."""
        out = {}
        for name, v in self.p.items():
            t = v.detach().float()
            if _is_expert(name) and self.world > 1:
                parts = [torch.empty_like(t) for _ in range(self.world)]
                dist.all_gather(parts, t.contiguous(), group=self.group)
                t = torch.cat(parts, 0)
            out[name] = t.cpu()
        return out


def moe_llama_reference_loss(cfg: MoELlamaConfig, params: dict[str, torch.Tensor], tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Single-process oracle on unsharded parameters (all experts local)."""
    from ..tensor.stages_moe import grouped_swiglu_experts

    def ffn(l, h, w, idx):
        q_ = f"layers.{l}."
        return grouped_swiglu_experts(h, params[q_ + "w1"], params[q_ + "w2"], params[q_ + "w3"], w, idx)

    return _forward_loss(cfg, params, tokens, targets, ffn, torch.float32)
