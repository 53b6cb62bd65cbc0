"""Tensor stages, part 6: data-source stubs, frozen sibling graphs, sequence-model
alternatives (Mamba-style, TTT, universal transformer / ACT), JEPA, masked diffusion,
byte-patch tokenisation. Reference: ``neuralfn/torch_backend.py:1149-1227,1579-1640,
1699-1727,2982-3190,6376-6410,7168``."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .stages_core import stage


# ------------------------------------------------------------------ data-source stubs --
class _PassThroughSource(nn.Module):
    """Source nodes are resolved by the trainer into input roles; at run time they pass
    their already-materialised batch tensors through."""

    def __init__(self, **cfg) -> None:
        super().__init__()
        self.source_config = dict(cfg)

    @classmethod
    def from_config(cls, cfg):
        return cls(**{k: v for k, v in cfg.items() if not k.startswith("__")})

    def forward(self, *args: Tensor):
        return args[0] if len(args) == 1 else tuple(args)


for _name in ("dataset_source", "semantic_data_source", "sft_dataset_source", "dpo_dataset_source",
              "ppo_rollout_source"):
    stage(_name)(type(f"{_name.title().replace('_', '')}Stage", (_PassThroughSource,), {}))


class _FrozenGraphStage(nn.Module):
    """A frozen sibling graph loaded from its own graph JSON + weights file (reference model
    for DPO/PPO, reward model for PPO). The topology digest stored with the weights must
    match the graph."""

    def __init__(self, graph_path: str = "", weights_path: str = "", **extra) -> None:
        super().__init__()
        self.graph_path, self.weights_path = str(graph_path), str(weights_path)
        self.extra = extra
        self._compiled = None

    def _ensure_loaded(self, device):
        if self._compiled is not None:
            return self._compiled
        if not self.graph_path or not self.weights_path:
            raise ValueError(f"{type(self).__name__} requires graph and weights paths to be set")
        from ..serialization import load_graph
        from ..inference import graph_topology_sha256, load_pt_checkpoint
        from .compiler import CompiledTorchGraph
        graph = load_graph(self.graph_path)
        state, meta = load_pt_checkpoint(self.weights_path, map_location=device or "cpu")
        digest = str(meta.get("graph_topology_sha256", ""))
        if digest and digest != graph_topology_sha256(graph):
            raise ValueError("frozen graph weights were saved for a different graph topology")
        view = self._inference_view(graph)
        if view is None:
            compiled = CompiledTorchGraph(graph)
            compiled.load_state_dict(state, strict=True)
        else:
            # a training root (tokens, targets, ... -> loss): run the same trunk and head without the loss nodes
            compiled = CompiledTorchGraph(view)
            result = compiled.load_state_dict(state, strict=False)
            if result.missing_keys:
                raise ValueError(f"frozen graph weights lack {len(result.missing_keys)} tensors of the inference view, "
                                 f"first: {result.missing_keys[0]}")
        for p in compiled.parameters():
            p.requires_grad = False
        compiled.train(False)
        compiled.to(device)
        object.__setattr__(self, "_compiled", compiled)  # keep it out of the parent's state_dict
        return compiled

    def _inference_view(self, graph):
        """None when ``graph`` already maps this stage's inputs to its output; else the graph to run instead."""
        return None

    @staticmethod
    def _training_spec(graph):
        """The model spec stored in a training root that takes more than the token input, else None."""
        if len(graph.input_node_ids) <= 1 or not (graph.torch_config or {}).get("template_spec"):
            return None
        from ..torch_templates_roots import build_model_spec_from_config
        return build_model_spec_from_config(graph.torch_config)

    def _call(self, compiled, tokens: Tensor):
        return compiled(tokens)

    @torch.no_grad()
    def forward(self, tokens: Tensor) -> Tensor:
        out = self._call(self._ensure_loaded(tokens.device), tokens)
        return out[0] if isinstance(out, (tuple, list)) else out


@stage("reference_forward")
class ReferenceForwardStage(_FrozenGraphStage):
    @classmethod
    def from_config(cls, cfg):
        return cls(str(cfg.get("ref_graph_path", "")), str(cfg.get("ref_weights_path", "")),
                   vocab_size=int(cfg.get("vocab_size", 256)), model_dim=int(cfg.get("model_dim", 128)))

    def _inference_view(self, graph):
        spec = self._training_spec(graph)
        if spec is None:
            return None
        from ..torch_templates_roots import build_model_stage_graph
        return build_model_stage_graph(spec, with_loss=False)


@stage("reward_forward")
class RewardForwardStage(_FrozenGraphStage):
    @classmethod
    def from_config(cls, cfg):
        return cls(str(cfg.get("reward_graph_path", "")), str(cfg.get("reward_weights_path", "")),
                   model_dim=int(cfg.get("model_dim", 128)))

    def _inference_view(self, graph):
        spec = self._training_spec(graph)
        if spec is None:
            return None
        from ..torch_templates_roots import build_reward_scoring_graph
        return build_reward_scoring_graph(spec)

    def _call(self, compiled, tokens: Tensor):
        if compiled._expected_flat_inputs == 2:      # the scoring view: every position counts, the head reads the last one
            return compiled(tokens, torch.ones(tokens.shape, device=tokens.device))
        return compiled(tokens)


# ------------------------------------------------------------ sequence-model variants --
@stage("mamba")
class MambaStage(nn.Module):
    """Simplified selective-state block (no scan): in-proj -> causal depthwise conv -> SiLU ->
    input-dependent gate -> out-proj."""

    def __init__(self, model_dim: int, d_state: int = 16, d_conv: int = 4, expand: int = 2) -> None:
        super().__init__()
        inner = expand * model_dim
        self.in_proj = nn.Linear(model_dim, 2 * inner, bias=False)
        self.conv = nn.Conv1d(inner, inner, d_conv, groups=inner, padding=d_conv - 1)
        self.x_proj = nn.Linear(inner, d_state, bias=False)
        self.dt_proj = nn.Linear(d_state, inner, bias=True)
        self.out_proj = nn.Linear(inner, model_dim, bias=False)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg.get("d_state", 16)), int(cfg.get("d_conv", 4)), int(cfg.get("expand", 2)))

    def forward(self, x: Tensor) -> Tensor:
        t = x.size(1)
        u, z = self.in_proj(x).chunk(2, dim=-1)
        u = F.silu(self.conv(u.transpose(1, 2))[..., :t].transpose(1, 2))
        gate = torch.sigmoid(self.dt_proj(self.x_proj(u)))
        return self.out_proj(u * gate * F.silu(z))


@stage("ttt_linear")
class TTTLinearStage(nn.Module):
    """Test-time-training linear layer: a fast weight updated by one gradient step of a
    self-supervised reconstruction loss per chunk, applied causally."""

    def __init__(self, input_dim: int, output_dim: int, hidden_dim: int = 16) -> None:
        super().__init__()
        self.base = nn.Linear(input_dim, output_dim, bias=False)
        self.k = nn.Linear(input_dim, hidden_dim, bias=False)
        self.v = nn.Linear(input_dim, hidden_dim, bias=False)
        self.q = nn.Linear(input_dim, hidden_dim, bias=False)
        self.o = nn.Linear(hidden_dim, output_dim, bias=False)
        self.lr = nn.Parameter(torch.tensor(0.1))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg["output_dim"]), int(cfg.get("hidden_dim", 16)))

    def forward(self, x: Tensor) -> Tensor:
        k, v, q = self.k(x), self.v(x), self.q(x)
        # fast weight after t tokens: W_t = lr * sum_{s<=t} v_s k_s^T  (one linear-attention step)
        kv = torch.cumsum(torch.einsum("bth,btg->bthg", v, k), dim=1)
        fast = torch.einsum("bthg,btg->bth", kv, q) * self.lr
        return self.base(x) + self.o(fast)


@stage("act_halt_gate")
class ACTHaltGateStage(nn.Module):
    def __init__(self, model_dim: int) -> None:
        super().__init__()
        self.proj = nn.Linear(model_dim, 1)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]))

    def forward(self, x: Tensor) -> Tensor:
        return torch.sigmoid(self.proj(x)).squeeze(-1)


@stage("act_weighted_sum")
class ACTWeightedSumStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, states: Tensor, weights: Tensor) -> Tensor:
        # states [S, B, T, D], weights [S, B, T]
        return (states * weights.unsqueeze(-1)).sum(dim=0)


@stage("universal_transformer")
class UniversalTransformerStage(nn.Module):
    """One shared block applied up to ``max_steps`` times with adaptive-computation-time halting."""

    def __init__(self, model_dim: int, num_heads: int, mlp_mult: float = 4.0, max_steps: int = 4,
                 halt_epsilon: float = 0.01) -> None:
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(model_dim), nn.LayerNorm(model_dim)
        self.attn = nn.MultiheadAttention(model_dim, num_heads, batch_first=True)
        hidden = int(model_dim * mlp_mult)
        self.mlp = nn.Sequential(nn.Linear(model_dim, hidden), nn.GELU(), nn.Linear(hidden, model_dim))
        self.halt = nn.Linear(model_dim, 1)
        self.max_steps, self.halt_epsilon = int(max_steps), float(halt_epsilon)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["num_heads"]), float(cfg.get("mlp_mult", 4.0)),
                   int(cfg.get("max_steps", 4)), float(cfg.get("halt_epsilon", 0.01)))

    def _block(self, x: Tensor) -> Tensor:
        t = x.size(1)
        mask = torch.triu(torch.ones(t, t, dtype=torch.bool, device=x.device), diagonal=1)
        h = self.norm1(x)
        x = x + self.attn(h, h, h, attn_mask=mask, need_weights=False)[0]
        return x + self.mlp(self.norm2(x))

    def forward(self, x: Tensor) -> Tensor:
        halted = torch.zeros(x.shape[:2], device=x.device, dtype=x.dtype)
        out = torch.zeros_like(x)
        for step in range(self.max_steps):
            x = self._block(x)
            p = torch.sigmoid(self.halt(x)).squeeze(-1)
            last = step == self.max_steps - 1
            still = (halted < 1.0 - self.halt_epsilon).to(x.dtype)
            w = torch.where(torch.tensor(last, device=x.device), 1.0 - halted, torch.minimum(p, 1.0 - halted)) * still
            out = out + w.unsqueeze(-1) * x
            halted = halted + w
        return out


# ------------------------------------------------------------------- JEPA / diffusion --
@stage("jepa_mask")
class JEPAMaskStage(nn.Module):
    """tokens -> (context tokens with masked positions replaced, mask [B, T] float)."""

    def __init__(self, mask_ratio=0.5, mask_token_id=0, mask_strategy="random", num_blocks=4,
                 min_block_ratio=0.1, max_block_ratio=0.25) -> None:
        super().__init__()
        self.mask_ratio, self.mask_token_id, self.mask_strategy = float(mask_ratio), int(mask_token_id), str(mask_strategy)
        self.num_blocks, self.min_block_ratio, self.max_block_ratio = int(num_blocks), float(min_block_ratio), float(max_block_ratio)

    @classmethod
    def from_config(cls, cfg):
        return cls(cfg.get("mask_ratio", 0.5), cfg.get("mask_token_id", 0), cfg.get("mask_strategy", "random"),
                   cfg.get("num_blocks", 4), cfg.get("min_block_ratio", 0.1), cfg.get("max_block_ratio", 0.25))

    def forward(self, tokens: Tensor):
        b, t = tokens.shape
        if self.mask_strategy == "block":
            mask = torch.zeros(b, t, dtype=torch.bool, device=tokens.device)
            for i in range(b):
                for _ in range(self.num_blocks):
                    ratio = self.min_block_ratio + (self.max_block_ratio - self.min_block_ratio) * float(torch.rand(()))
                    length = max(1, int(t * ratio))
                    start = int(torch.randint(0, max(t - length, 0) + 1, ()))
                    mask[i, start:start + length] = True
        else:
            mask = torch.rand(b, t, device=tokens.device) < self.mask_ratio
        ctx = torch.where(mask, torch.full_like(tokens, self.mask_token_id), tokens)
        return ctx, mask.float()


@stage("latent_pool")
class LatentPoolStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, hidden: Tensor, mask: Tensor | None = None) -> Tensor:
        if mask is None:
            return hidden.mean(dim=1)
        m = mask.to(hidden.dtype).unsqueeze(-1)
        return (hidden * m).sum(dim=1) / m.sum(dim=1).clamp(min=1.0)


@stage("jepa_projector")
class JEPAProjectorStage(nn.Module):
    def __init__(self, input_dim: int, latent_dim: int) -> None:
        super().__init__()
        self.net = nn.Sequential(nn.Linear(input_dim, latent_dim), nn.GELU(), nn.Linear(latent_dim, latent_dim))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg["latent_dim"]))

    def forward(self, x: Tensor) -> Tensor:
        return self.net(x)


@stage("jepa_predictor")
class JEPAPredictorStage(nn.Module):
    def __init__(self, latent_dim: int) -> None:
        super().__init__()
        self.net = nn.Sequential(nn.Linear(latent_dim, latent_dim), nn.GELU(), nn.Linear(latent_dim, latent_dim))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["latent_dim"]))

    def forward(self, x: Tensor) -> Tensor:
        return self.net(x)


@stage("random_timesteps")
class RandomTimestepsStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, tokens: Tensor) -> Tensor:
        return torch.rand(tokens.size(0), device=tokens.device)


@stage("mask_scheduler")
class MaskSchedulerStage(nn.Module):
    """Masked-diffusion corruption: each token is replaced by the mask id with probability t."""

    def __init__(self, vocab_size: int, mask_token_id: int) -> None:
        super().__init__()
        self.vocab_size, self.mask_token_id = int(vocab_size), int(mask_token_id)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["vocab_size"]), int(cfg["mask_token_id"]))

    def forward(self, tokens: Tensor, timesteps: Tensor):
        drop = torch.rand(tokens.shape, device=tokens.device) < timesteps.view(-1, 1)
        return torch.where(drop, torch.full_like(tokens, self.mask_token_id), tokens), drop.float()


@stage("denoise_head")
class DenoiseHeadStage(nn.Module):
    def __init__(self, model_dim: int, vocab_size: int) -> None:
        super().__init__()
        self.proj = nn.Linear(model_dim, vocab_size, bias=False)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["vocab_size"]))

    def forward(self, x: Tensor) -> Tensor:
        return self.proj(x)


# --------------------------------------------------------------------------- byte patch --
@stage("byte_patch_embed")
class BytePatchEmbedStage(nn.Module):
    """bytes [B, T] -> patches [B, T/stride, D]: byte embeddings summed inside each patch, projected."""

    def __init__(self, model_dim: int, patch_size: int = 4, stride: int = 4, vocab_size: int = 256) -> None:
        super().__init__()
        self.patch_size, self.stride = int(patch_size), int(stride)
        self.embed = nn.Embedding(vocab_size, model_dim)
        self.proj = nn.Linear(model_dim * self.patch_size, model_dim, bias=False)

    @classmethod
    def from_config(cls, cfg):
        p = int(cfg.get("patch_size", 4))
        return cls(int(cfg["model_dim"]), p, int(cfg.get("stride", p)), int(cfg.get("vocab_size", 256)))

    def forward(self, tokens: Tensor) -> Tensor:
        e = self.embed(tokens.long())
        b, t, d = e.shape
        pad = (-(t - self.patch_size)) % self.stride if t >= self.patch_size else self.patch_size - t
        if pad:
            e = F.pad(e, (0, 0, 0, pad))
        patches = e.unfold(1, self.patch_size, self.stride)  # [B, P, D, patch]
        return self.proj(patches.permute(0, 1, 3, 2).reshape(b, patches.size(1), -1))


@stage("byte_patch_merge")
class BytePatchMergeStage(nn.Module):
    """patches [B, P, D] broadcast back to byte resolution [B, T, D]."""

    def __init__(self, patch_size: int = 4, stride: int = 4) -> None:
        super().__init__()
        self.patch_size, self.stride = int(patch_size), int(stride)

    @classmethod
    def from_config(cls, cfg):
        p = int(cfg.get("patch_size", 4))
        return cls(p, int(cfg.get("stride", p)))

    def forward(self, patches: Tensor, like: Tensor) -> Tensor:
        t = like.size(1)
        up = patches.repeat_interleave(self.stride, dim=1)
        if up.size(1) < t:
            up = F.pad(up, (0, 0, 0, t - up.size(1)))
        return up[:, :t]


@stage("running_mean_decoder")
class RunningMeanDecoderStage(nn.Module):
    """Token-mixing-free decoder block: norm -> gated MLP with a causal running mean as context."""

    def __init__(self, model_dim: int, mlp_mult: float = 4.0) -> None:
        super().__init__()
        hidden = int(model_dim * mlp_mult)
        self.norm = nn.LayerNorm(model_dim)
        self.fc = nn.Linear(2 * model_dim, hidden)
        self.proj = nn.Linear(hidden, model_dim)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), float(cfg.get("mlp_mult", 4.0)))

    def forward(self, x: Tensor) -> Tensor:
        h = self.norm(x)
        steps = torch.arange(1, x.size(1) + 1, device=x.device, dtype=x.dtype).view(1, -1, 1)
        ctx = torch.cumsum(h, dim=1) / steps
        return x + self.proj(F.gelu(self.fc(torch.cat([h, ctx], dim=-1))))


@stage("input", "output")
class PassThroughStage(nn.Module):
    """Graph terminals on the tensor runtime: identity."""

    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, x: Tensor) -> Tensor:
        return x
