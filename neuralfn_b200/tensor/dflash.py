"""DFlash block-diffusion speculative drafting: draft model, distillation trainer, acceptance
evaluation.

A frozen target model supplies token embeddings, hidden-state taps of a few layers and the
LM head. The draft predicts a whole block of ``block_size`` tokens at once: its input is the
anchor token followed by mask tokens; every draft layer attends bidirectionally inside the
block and causally (``< anchor``, within ``context_window``) to the projected target taps.
Training samples random valid anchors per sequence and minimises a position-weighted (soft)
cross-entropy against the target's own next-token distribution; position 0 (the anchor,
already known) carries no loss. Weights are either an exponential decay or D-PACE: the
suffix sum of the cumulative product of smoothed target confidences, i.e. how much accepted
continuation depends on getting each position right.

Reference: ``DFlashDistillationTrainer`` and helpers, ``neuralfn/torch_backend.py:7196-8313``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["dpace_position_weights", "exp_decay_position_weights", "sample_anchor_positions", "build_block_inputs",
           "dflash_attention_mask", "DFlashConfig", "DFlashDraftModel", "DFlashDistillationTrainer"]


def dpace_position_weights(confidences: torch.Tensor, alpha: float, valid_mask: torch.Tensor | None = None) -> torch.Tensor:
    """weights[..., i] = sum_{j >= i} prod_{t <= j} (alpha + (1 - alpha) * conf_t); invalid positions
    neither shrink the product nor contribute. Detached."""
    if not 0.0 < alpha <= 1.0:
        raise ValueError("DFlash D-PACE alpha must be in (0, 1]")
    if confidences.ndim < 1 or confidences.size(-1) == 0 or not confidences.is_floating_point():
        raise ValueError("DFlash confidences must be a floating tensor with a non-empty position axis")
    with torch.no_grad():
        c = confidences.float()
        if torch.isnan(c).any() or ((c < 0) | (c > 1)).any():
            raise ValueError("DFlash confidences must be finite probabilities")
        s = alpha + (1.0 - alpha) * c
        if valid_mask is not None:
            if valid_mask.shape != confidences.shape:
                raise ValueError("DFlash D-PACE valid mask must match confidences")
            keep = valid_mask.bool()
            s = torch.where(keep, s, torch.ones_like(s))
        cum = torch.cumprod(s, dim=-1)
        if valid_mask is not None:
            cum = cum * keep.to(cum.dtype)
        w = torch.flip(torch.cumsum(torch.flip(cum, (-1,)), dim=-1), (-1,))
        return w.to(confidences.dtype)


def exp_decay_position_weights(block_size: int, gamma: float, device=None) -> torch.Tensor:
    """exp(-(i - 1) / gamma) for block positions i >= 1, 0 for the anchor position."""
    i = torch.arange(block_size, device=device, dtype=torch.float32)
    w = torch.exp(-(i - 1).clamp(min=0) / max(gamma, 1e-6))
    w[0] = 0.0
    return w


def sample_anchor_positions(loss_mask: torch.Tensor, block_size: int, num_anchors: int, generator: torch.Generator | None = None):
    """Random distinct anchors per row among positions with ``loss_mask > 0.5`` that leave room for a
    full block. Returns (anchors [B, A] sorted, keep [B, A] bool); A <= num_anchors."""
    B, T = loss_mask.shape
    last = max(T - block_size, 0)
    valid = loss_mask[:, :last + 1] > 0.5
    counts = valid.sum(1)
    A = min(int(num_anchors), int(counts.max().item()) - 1) if counts.numel() else 0
    if A <= 0:
        z = torch.zeros(B, 1, dtype=torch.long, device=loss_mask.device)
        return z, torch.zeros_like(z, dtype=torch.bool)
    r = torch.rand(B, last + 1, device=loss_mask.device, generator=generator)
    r = torch.where(valid, r, torch.full_like(r, 2.0))
    order = r.argsort(1)[:, :A]
    keep = torch.arange(A, device=loss_mask.device)[None] < counts.clamp(max=A)[:, None]
    anchors = torch.where(keep, order, torch.full_like(order, T + 1)).sort(1).values
    keep = anchors <= last
    return torch.where(keep, anchors, torch.zeros_like(anchors)), keep


def build_block_inputs(input_ids: torch.Tensor, anchors: torch.Tensor, block_size: int, mask_token_id: int):
    """-> (block_ids [B, A, S]: anchor token then mask tokens, positions [B, A, S], target_index
    [B, A, S] = position in the sequence each block slot predicts)."""
    B, A = anchors.shape
    pos = anchors[..., None] + torch.arange(block_size, device=anchors.device)
    ids = torch.full((B, A, block_size), mask_token_id, dtype=input_ids.dtype, device=input_ids.device)
    ids[..., 0] = input_ids.gather(1, anchors)
    return ids, pos, pos.clamp(max=input_ids.size(1) - 1)


def dflash_attention_mask(seq_len: int, anchors: torch.Tensor, block_size: int, context_window: int) -> torch.Tensor:
    """Boolean [B, A, S, T + S]: block slot -> context position allowed when ``anchor - window <= t <
    anchor``; block slot -> block slot always allowed (bidirectional within the block)."""
    B, A = anchors.shape
    t = torch.arange(seq_len, device=anchors.device)
    ctx = (t[None, None] < anchors[..., None]) & (t[None, None] >= anchors[..., None] - context_window)
    ctx = ctx[:, :, None, :].expand(B, A, block_size, seq_len)
    blk = torch.ones(B, A, block_size, block_size, dtype=torch.bool, device=anchors.device)
    return torch.cat([ctx, blk], dim=-1)


@dataclass
class DFlashConfig:
    d_model: int = 256
    n_layer: int = 2
    n_head: int = 4
    block_size: int = 16
    num_anchors: int = 8
    context_window: int = 512
    tap_layers: tuple[int, ...] = (1, 2)        # target layers whose hidden states feed the draft
    mask_token_id: int = 0
    loss_weighting: str = "dpace"               # "dpace" | "exp"
    dpace_alpha: float = 0.3
    exp_gamma: float = 4.0
    soft_targets: bool = True
    learning_rate: float = 3e-4
    weight_decay: float = 0.0
    seed: int = 0


class _DraftLayer(nn.Module):
    def __init__(self, d: int, h: int) -> None:
        super().__init__()
        self.h = h
        self.n1, self.n2 = nn.RMSNorm(d), nn.RMSNorm(d)
        self.q, self.kv_blk, self.kv_ctx, self.o = nn.Linear(d, d, bias=False), nn.Linear(d, 2 * d, bias=False), nn.Linear(d, 2 * d, bias=False), nn.Linear(d, d, bias=False)
        self.up, self.down = nn.Linear(d, 4 * d, bias=False), nn.Linear(4 * d, d, bias=False)

    def forward(self, x: torch.Tensor, ctx: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        # x [B, A, S, d], ctx [B, T, d], mask [B, A, S, T + S]
        B, A, S, d = x.shape
        hd = d // self.h
        y = self.n1(x)
        q = self.q(y).view(B, A, S, self.h, hd).permute(0, 1, 3, 2, 4)                    # B A h S hd
        kb, vb = self.kv_blk(y).view(B, A, S, 2, self.h, hd).permute(3, 0, 1, 4, 2, 5)    # B A h S hd
        kc, vc = self.kv_ctx(ctx).view(B, -1, 2, self.h, hd).permute(2, 0, 3, 1, 4)       # B h T hd
        k = torch.cat([kc[:, None].expand(B, A, -1, -1, -1), kb], dim=3)
        v = torch.cat([vc[:, None].expand(B, A, -1, -1, -1), vb], dim=3)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask[:, :, None])
        x = x + self.o(a.permute(0, 1, 3, 2, 4).reshape(B, A, S, d))
        return x + self.down(F.silu(self.up(self.n2(x))))


class DFlashDraftModel(nn.Module):
    """Shares the target's embedding and LM head (passed at call time); owns the tap projection,
    a learned block-position embedding and ``n_layer`` draft layers."""

    def __init__(self, cfg: DFlashConfig, target_dim: int) -> None:
        super().__init__()
        self.cfg = cfg
        self.embed_proj = nn.Linear(target_dim, cfg.d_model, bias=False)
        self.tap_proj = nn.Linear(target_dim * len(cfg.tap_layers), cfg.d_model, bias=False)
        self.slot = nn.Parameter(torch.zeros(cfg.block_size, cfg.d_model))
        self.layers = nn.ModuleList([_DraftLayer(cfg.d_model, cfg.n_head) for _ in range(cfg.n_layer)])
        self.norm = nn.RMSNorm(cfg.d_model)
        self.out_proj = nn.Linear(cfg.d_model, target_dim, bias=False)
        nn.init.normal_(self.slot, std=0.02)

    def forward(self, block_embeds: torch.Tensor, taps: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """block_embeds [B, A, S, Ct] (target embeddings of the block ids), taps [B, T, Ct * n_taps]
        -> hidden in the target's width [B, A, S, Ct] (feed to the target LM head)."""
        x = self.embed_proj(block_embeds) + self.slot
        ctx = self.tap_proj(taps)
        for layer in self.layers:
            x = layer(x, ctx, mask)
        return self.out_proj(self.norm(x))


@dataclass
class _TrainState:
    step: int = 0
    losses: list = field(default_factory=list)


class DFlashDistillationTrainer:
    """``target(input_ids) -> {"hidden_states": [L + 1 tensors [B, T, C]], "logits": [B, T, V]}``;
    ``embed(ids) -> [.., C]``; ``lm_head(hidden) -> logits``. All three are frozen."""

    def __init__(self, cfg: DFlashConfig, target: Callable, embed: Callable, lm_head: Callable, target_dim: int, device="cpu") -> None:
        self.cfg, self.target, self.embed, self.lm_head = cfg, target, embed, lm_head
        torch.manual_seed(cfg.seed)
        self.draft = DFlashDraftModel(cfg, target_dim).to(device)
        self.opt = torch.optim.AdamW(self.draft.parameters(), lr=cfg.learning_rate, weight_decay=cfg.weight_decay, betas=(0.9, 0.95))
        self.gen = torch.Generator(device=device).manual_seed(cfg.seed)
        self.state = _TrainState()
        self.device = torch.device(device)

    def _teacher(self, input_ids: torch.Tensor):
        with torch.no_grad():
            out = self.target(input_ids)
            hs = out["hidden_states"]
            taps = torch.cat([hs[l + 1] for l in self.cfg.tap_layers], dim=-1)  # hidden_states[0] is the embedding output
            return taps, out["logits"]

    def _draft_logits(self, input_ids, anchors, taps):
        c = self.cfg
        ids, _pos, tgt_idx = build_block_inputs(input_ids, anchors, c.block_size, c.mask_token_id)
        mask = dflash_attention_mask(input_ids.size(1), anchors, c.block_size, c.context_window)
        with torch.no_grad():
            emb = self.embed(ids)
        return self.lm_head(self.draft(emb, taps, mask)), tgt_idx

    def loss(self, input_ids: torch.Tensor, loss_mask: torch.Tensor | None = None) -> torch.Tensor:
        c = self.cfg
        B, T = input_ids.shape
        loss_mask = torch.ones(B, T, device=input_ids.device) if loss_mask is None else loss_mask
        taps, t_logits = self._teacher(input_ids)
        anchors, keep = sample_anchor_positions(loss_mask, c.block_size, c.num_anchors, self.gen)
        logits, tgt_idx = self._draft_logits(input_ids, anchors, taps)              # [B, A, S, V]
        # slot i predicts the token at anchor + i, whose teacher distribution sits at index anchor + i - 1
        t_at = t_logits.gather(1, (tgt_idx - 1).clamp(min=0).flatten(1)[..., None].expand(-1, -1, t_logits.size(-1))).view_as(logits)
        gold = input_ids.gather(1, tgt_idx.flatten(1)).view(tgt_idx.shape)
        logp = F.log_softmax(logits.float(), -1)
        if c.soft_targets:
            per = -(F.softmax(t_at.float(), -1) * logp).sum(-1)
        else:
            per = -logp.gather(-1, gold[..., None]).squeeze(-1)
        valid = keep[..., None] & (anchors[..., None] + torch.arange(c.block_size, device=anchors.device) < T)
        valid = valid & (loss_mask.gather(1, tgt_idx.flatten(1)).view(tgt_idx.shape) > 0.5)
        valid[..., 0] = False  # the anchor token itself is given
        if c.loss_weighting == "dpace":
            conf = F.softmax(t_at.float(), -1).gather(-1, gold[..., None]).squeeze(-1)
            w = dpace_position_weights(conf[..., 1:], c.dpace_alpha, valid[..., 1:])
            w = torch.cat([torch.zeros_like(w[..., :1]), w], dim=-1)
        else:
            w = exp_decay_position_weights(c.block_size, c.exp_gamma, per.device).expand_as(per)
        w = w * valid
        return (per * w).sum() / w.sum().clamp(min=1e-8)

    def train_step(self, input_ids: torch.Tensor, loss_mask: torch.Tensor | None = None) -> float:
        self.draft.train()
        loss = self.loss(input_ids, loss_mask)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(self.draft.parameters(), 1.0)
        self.opt.step()
        self.state.step += 1
        self.state.losses.append(float(loss.detach()))
        return self.state.losses[-1]

    @torch.no_grad()
    def evaluate_greedy_acceptance(self, input_ids: torch.Tensor, n_anchors: int = 16) -> dict:
        """Mean number of leading block tokens (after the anchor) that equal the target's own greedy
        continuation - the accepted length a speculative step would get."""
        self.draft.eval()
        c = self.cfg
        B, T = input_ids.shape
        taps, t_logits = self._teacher(input_ids)
        anchors, keep = sample_anchor_positions(torch.ones(B, T, device=input_ids.device), c.block_size, n_anchors, self.gen)
        logits, tgt_idx = self._draft_logits(input_ids, anchors, taps)
        greedy_t = t_logits.argmax(-1).gather(1, (tgt_idx - 1).clamp(min=0).flatten(1)).view(tgt_idx.shape)
        match = (logits.argmax(-1) == greedy_t)[..., 1:]
        accepted = torch.cumprod(match.long(), -1).sum(-1).float()
        n = keep.sum().clamp(min=1)
        return {"mean_accepted_tokens": float((accepted * keep).sum() / n), "blocks": int(keep.sum()),
                "position_accuracy": (match.float() * keep[..., None]).sum((0, 1)).div(n).tolist()}

    # ---- persistence -------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"format": "neuralfn_b200.dflash_training.v1", "draft": self.draft.state_dict(), "optimizer": self.opt.state_dict(),
                "step": self.state.step, "losses": self.state.losses, "generator": self.gen.get_state(), "config": self.cfg.__dict__}

    def load_state_dict(self, sd: dict) -> None:
        if sd.get("format") != "neuralfn_b200.dflash_training.v1":
            raise ValueError("not a DFlash training checkpoint")
        self.draft.load_state_dict(sd["draft"])
        self.opt.load_state_dict(sd["optimizer"])
        self.state = _TrainState(sd["step"], list(sd["losses"]))
        self.gen.set_state(sd["generator"])

    def export_native_assistant(self, path) -> str:
        """Draft weights as a named-tensor checkpoint (bf16) for the resident engine's assistant slot."""
        from ..checkpoint.named import write_named_tensors
        tensors = {k: v.detach().to(torch.bfloat16) for k, v in self.draft.state_dict().items()}
        cfg = {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.cfg.__dict__.items()}
        return write_named_tensors(path, tensors, {"kind": "dflash_assistant", "config": cfg, "step": self.state.step})
