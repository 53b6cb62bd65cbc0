"""Online PPO for language policies: sampled rollouts, frozen reference policy, reward model or
reward function, KL-shaped per-token rewards, GAE, clipped policy / value objectives over
minibatches for several epochs per rollout.

``policy(ids) -> (logits [B, T, V], values [B, T])`` is trained; ``reference(ids) -> logits``
and ``reward(ids, prompt_len) -> [B]`` are frozen callables (compiled graphs, nn.Modules or
plain functions). Counterpart of the reference's ``PPOTrainer``
(``neuralfn/torch_backend.py:8316-8663``) and its ``MaskedPPOClippedLossStage``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import torch
import torch.nn.functional as F

__all__ = ["PPOConfig", "PPOTrainer", "gae_advantages", "masked_ppo_clipped_loss", "sample_continuations"]


@dataclass
class PPOConfig:
    max_new_tokens: int = 16
    temperature: float = 1.0
    top_k: int = 0
    kl_coef: float = 0.05
    gamma: float = 1.0
    gae_lambda: float = 0.95
    clip_range: float = 0.2
    value_clip_range: float = 0.2
    value_coef: float = 0.5
    entropy_coef: float = 0.0
    ppo_epochs_per_rollout: int = 4
    minibatch_size: int = 8
    learning_rate: float = 1e-4
    max_grad_norm: float = 1.0
    whiten_advantages: bool = True
    eos_token_id: int | None = None
    pad_token_id: int = 0
    seed: int = 0


def gae_advantages(rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, gamma: float, lam: float):
    """rewards / values / mask: [B, T] over response positions. Returns (advantages, returns)."""
    B, T = rewards.shape
    adv = torch.zeros_like(rewards)
    last = torch.zeros(B, device=rewards.device, dtype=rewards.dtype)
    for t in range(T - 1, -1, -1):
        nxt = values[:, t + 1] * mask[:, t + 1] if t + 1 < T else torch.zeros_like(last)
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = (delta + gamma * lam * last) * mask[:, t]
        adv[:, t] = last
    return adv, adv + values


def masked_ppo_clipped_loss(logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, clip: float):
    """mean over masked tokens of max(-A r, -A clip(r, 1 - c, 1 + c)); also returns the clip fraction."""
    ratio = torch.exp(logp - old_logp)
    l1, l2 = -advantages * ratio, -advantages * ratio.clamp(1.0 - clip, 1.0 + clip)
    n = mask.sum().clamp(min=1.0)
    return (torch.maximum(l1, l2) * mask).sum() / n, ((l2 > l1).float() * mask).sum() / n


@torch.no_grad()
def sample_continuations(policy_logits: Callable, prompts: torch.Tensor, max_new: int, temperature: float, top_k: int,
                         generator: torch.Generator | None, eos: int | None, pad: int):
    """Autoregressive sampling without a KV cache (rollouts are short). Returns (ids [B, P + N],
    response_mask [B, N] = 1 up to and including the first eos)."""
    ids = prompts.clone()
    B = ids.size(0)
    alive = torch.ones(B, dtype=torch.bool, device=ids.device)
    masks = []
    for _ in range(max_new):
        logits = policy_logits(ids)[:, -1].float()
        if temperature <= 0:
            nxt = logits.argmax(-1)
        else:
            logits = logits / temperature
            if top_k > 0:
                kth = logits.topk(min(top_k, logits.size(-1)), -1).values[:, -1:]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            nxt = torch.multinomial(F.softmax(logits, -1), 1, generator=generator).squeeze(1)
        nxt = torch.where(alive, nxt, torch.full_like(nxt, pad))
        masks.append(alive.float())
        ids = torch.cat([ids, nxt[:, None]], dim=1)
        if eos is not None:
            alive = alive & (nxt != eos)
    return ids, torch.stack(masks, 1)


@dataclass
class _Stats:
    rollouts: int = 0
    history: list = field(default_factory=list)


class PPOTrainer:
    def __init__(self, policy: torch.nn.Module, reference: Callable, reward: Callable, config: PPOConfig | None = None) -> None:
        self.policy, self.reference, self.reward = policy, reference, reward
        self.cfg = config or PPOConfig()
        self.opt = torch.optim.AdamW([p for p in policy.parameters() if p.requires_grad], lr=self.cfg.learning_rate)
        dev = next(policy.parameters()).device
        self.gen = torch.Generator(device=dev).manual_seed(self.cfg.seed)
        self.stats = _Stats()

    def _logp(self, logits: torch.Tensor, ids: torch.Tensor, P: int) -> torch.Tensor:
        # log-prob of response token t (at sequence position P + t) comes from logits at P + t - 1
        lp = F.log_softmax(logits[:, P - 1:-1].float(), -1)
        return lp.gather(-1, ids[:, P:, None]).squeeze(-1)

    @torch.no_grad()
    def rollout(self, prompts: torch.Tensor) -> dict:
        c = self.cfg
        P = prompts.size(1)
        self.policy.eval()
        ids, mask = sample_continuations(lambda x: self.policy(x)[0], prompts, c.max_new_tokens, c.temperature, c.top_k, self.gen,
                                         c.eos_token_id, c.pad_token_id)
        logits, values = self.policy(ids)
        old_logp = self._logp(logits, ids, P)
        ref_logp = self._logp(self.reference(ids), ids, P)
        values = values[:, P - 1:-1].float()
        score = self.reward(ids, P).float()
        kl = old_logp - ref_logp
        rewards = -c.kl_coef * kl * mask
        last = (mask.sum(1).long() - 1).clamp(min=0)
        rewards[torch.arange(ids.size(0), device=ids.device), last] += score
        adv, ret = gae_advantages(rewards, values * mask, mask, c.gamma, c.gae_lambda)
        if c.whiten_advantages:
            n = mask.sum().clamp(min=1)
            mean = (adv * mask).sum() / n
            var = (((adv - mean) ** 2) * mask).sum() / n
            adv = (adv - mean) * torch.rsqrt(var + 1e-8) * mask
        return {"ids": ids, "mask": mask, "old_logp": old_logp, "values": values, "advantages": adv, "returns": ret, "prompt_len": P,
                "score": score, "kl": (kl * mask).sum(1)}

    def update(self, batch: dict) -> dict:
        c = self.cfg
        self.policy.train()
        B, P = batch["ids"].size(0), batch["prompt_len"]
        out = {"policy_loss": 0.0, "value_loss": 0.0, "clip_fraction": 0.0, "updates": 0}
        for _ in range(c.ppo_epochs_per_rollout):
            perm = torch.randperm(B, generator=torch.Generator().manual_seed(c.seed + self.stats.rollouts * 131 + out["updates"]))
            for i in range(0, B, c.minibatch_size):
                idx = perm[i:i + c.minibatch_size].to(batch["ids"].device)
                ids, mask = batch["ids"][idx], batch["mask"][idx]
                logits, values = self.policy(ids)
                logp = self._logp(logits, ids, P)
                pl, clipfrac = masked_ppo_clipped_loss(logp, batch["old_logp"][idx], batch["advantages"][idx], mask, c.clip_range)
                v = values[:, P - 1:-1].float()
                v_old, ret = batch["values"][idx], batch["returns"][idx]
                v_clip = v_old + (v - v_old).clamp(-c.value_clip_range, c.value_clip_range)
                n = mask.sum().clamp(min=1)
                vl = 0.5 * (torch.maximum((v - ret) ** 2, (v_clip - ret) ** 2) * mask).sum() / n
                loss = pl + c.value_coef * vl
                if c.entropy_coef:
                    lp = F.log_softmax(logits[:, P - 1:-1].float(), -1)
                    loss = loss - c.entropy_coef * (-(lp.exp() * lp).sum(-1) * mask).sum() / n
                self.opt.zero_grad(set_to_none=True)
                loss.backward()
                torch.nn.utils.clip_grad_norm_(self.policy.parameters(), c.max_grad_norm)
                self.opt.step()
                out["policy_loss"] += float(pl.detach())
                out["value_loss"] += float(vl.detach())
                out["clip_fraction"] += float(clipfrac)
                out["updates"] += 1
        for k in ("policy_loss", "value_loss", "clip_fraction"):
            out[k] /= max(out["updates"], 1)
        return out

    def step(self, prompts: torch.Tensor) -> dict:
        batch = self.rollout(prompts)
        info = self.update(batch)
        info.update(mean_score=float(batch["score"].mean()), mean_kl=float(batch["kl"].mean()),
                    mean_response_len=float(batch["mask"].sum(1).mean()))
        self.stats.rollouts += 1
        self.stats.history.append(info)
        return info
