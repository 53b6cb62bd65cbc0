"""Tensor stages, part 5: losses and post-training heads.

Token CE (+ z-loss), masked CE (SFT), sequence log-prob, token log-prob/entropy, DPO
(sigmoid / hinge / IPO), Bradley-Terry preference BCE, PPO clipped losses, KL-shaped
rewards, GAE, reward / value / policy heads, pair batching, latent MSE and soft-target
distillation. Math follows ``neuralfn/torch_backend.py:762-806,1100-1662,3132,7159``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .stages_core import stage


def _finite_nonneg(mask: Tensor, what: str) -> None:
    if not bool(torch.isfinite(mask).all()) or bool((mask < 0).any()):
        raise ValueError(f"{what} must be finite and non-negative")


def _check_targets(targets: Tensor, vocab: int, ignore_index: int, what: str) -> Tensor:
    valid = targets != ignore_index
    if bool(((targets < 0) & valid).any()) or bool(((targets >= vocab) & valid).any()):
        raise ValueError(f"{what} target ID is outside the vocabulary")
    return valid


@stage("token_cross_entropy")
class TokenCrossEntropyStage(nn.Module):
    """mean(lse - logit_target) + z * mean(lse^2), computed in fp32."""

    def __init__(self, z_loss_coef: float = 0.0) -> None:
        super().__init__()
        self.z_loss_coef = float(z_loss_coef)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("z_loss_coef", 0.0)))

    def forward(self, logits: Tensor, target_ids: Tensor) -> Tensor:
        from .kernel_bridge import token_cross_entropy
        return token_cross_entropy(logits, target_ids, self.z_loss_coef)


@stage("masked_token_cross_entropy")
class MaskedTokenCrossEntropyStage(nn.Module):
    """Cross-entropy averaged over positions with ``loss_mask > 0`` and a valid target."""

    def __init__(self, ignore_index: int = -100) -> None:
        super().__init__()
        self.ignore_index = int(ignore_index)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("ignore_index", -100)))

    def forward(self, logits: Tensor, target_ids: Tensor, loss_mask: Tensor) -> Tensor:
        if logits.ndim < 2 or tuple(logits.shape[:-1]) != tuple(target_ids.shape):
            raise ValueError("masked token cross entropy target shape must match logits without the vocabulary "
                             f"axis: got logits={tuple(logits.shape)}, targets={tuple(target_ids.shape)}")
        if tuple(loss_mask.shape) != tuple(target_ids.shape):
            raise ValueError(f"loss_mask shape {tuple(loss_mask.shape)} must match targets {tuple(target_ids.shape)}")
        if target_ids.is_floating_point():
            raise TypeError("masked token cross entropy targets must use an integer dtype")
        if not bool(torch.isfinite(logits).all()):
            raise ValueError("masked token cross entropy logits contain NaN or infinity")
        fl = logits.reshape(-1, logits.size(-1)).float()
        ft = target_ids.reshape(-1).long()
        fm = loss_mask.reshape(-1).to(fl.dtype)
        _finite_nonneg(fm, "loss_mask")
        valid = _check_targets(ft, fl.size(-1), self.ignore_index, "masked token cross entropy")
        eff = fm * valid.to(fm.dtype)
        denom = eff.sum()
        if not bool(denom > 0):
            raise ValueError("masked token cross entropy requires at least one unmasked valid target")
        per = F.cross_entropy(fl, ft, reduction="none", ignore_index=self.ignore_index)
        return (per * eff).sum() / denom


def _selected_logp(logits: Tensor, targets: Tensor, loss_mask: Tensor, ignore_index: int, what: str):
    if logits.ndim != 3 or targets.shape != logits.shape[:-1] or loss_mask.shape != targets.shape:
        raise ValueError(f"{what} expects logits [batch, sequence, vocab] and matching targets/loss_mask")
    logp = F.log_softmax(logits.float(), dim=-1)
    valid = _check_targets(targets, logits.size(-1), ignore_index, what)
    _finite_nonneg(loss_mask, f"{what} loss_mask")
    eff = loss_mask.to(logp.dtype) * valid.to(logp.dtype)
    if bool((eff.sum(dim=-1) <= 0).any()):
        raise ValueError(f"{what} requires at least one valid selected token per example")
    gathered = logp.gather(-1, targets.masked_fill(~valid, 0).long().unsqueeze(-1)).squeeze(-1)
    return logp, gathered, eff


@stage("sequence_logp")
class SequenceLogpStage(nn.Module):
    def __init__(self, ignore_index: int = -100) -> None:
        super().__init__()
        self.ignore_index = int(ignore_index)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("ignore_index", -100)))

    def forward(self, logits: Tensor, targets: Tensor, loss_mask: Tensor) -> Tensor:
        _, g, eff = _selected_logp(logits, targets, loss_mask, self.ignore_index, "sequence_logp")
        return (g * eff).sum(dim=-1)


@stage("token_logp_entropy")
class TokenLogpEntropyStage(nn.Module):
    def __init__(self, ignore_index: int = -100) -> None:
        super().__init__()
        self.ignore_index = int(ignore_index)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("ignore_index", -100)))

    def forward(self, logits: Tensor, targets: Tensor, loss_mask: Tensor):
        logp, g, eff = _selected_logp(logits, targets, loss_mask, self.ignore_index, "token_logp_entropy")
        entropy = -(logp.exp() * logp).sum(dim=-1)
        return g * eff, entropy * eff


@stage("dpo_pairwise_loss")
class DPOPairwiseLossStage(nn.Module):
    def __init__(self, beta: float = 0.1, label_smoothing: float = 0.0, loss_type: str = "sigmoid") -> None:
        super().__init__()
        self.beta, self.label_smoothing, self.loss_type = float(beta), float(label_smoothing), str(loss_type)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("beta", 0.1)), float(cfg.get("label_smoothing", 0.0)), str(cfg.get("loss_type", "sigmoid")))

    def forward(self, policy_logp_chosen, policy_logp_rejected, ref_logp_chosen, ref_logp_rejected):
        chosen = policy_logp_chosen - ref_logp_chosen
        rejected = policy_logp_rejected - ref_logp_rejected
        z = self.beta * (chosen - rejected)
        if self.loss_type == "hinge":
            per = F.relu(1.0 - z)
        elif self.loss_type == "ipo":
            per = (z - 1.0 / (2.0 * max(self.beta, 1e-8))) ** 2
        elif self.label_smoothing > 0.0:
            per = -F.logsigmoid(z) * (1.0 - self.label_smoothing) - F.logsigmoid(-z) * self.label_smoothing
        else:
            per = -F.logsigmoid(z)
        return per.mean(), self.beta * chosen.detach(), self.beta * rejected.detach()


@stage("preference_bce_loss")
class PreferenceBCELossStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, reward_chosen: Tensor, reward_rejected: Tensor) -> Tensor:
        return -F.logsigmoid(reward_chosen - reward_rejected).mean()


def _ppo_terms(logp_new, logp_old, adv, value_new, value_old, returns, clip):
    ratio = (logp_new - logp_old).exp()
    policy = -torch.minimum(ratio * adv, ratio.clamp(1.0 - clip, 1.0 + clip) * adv)
    v_clip = value_old + (value_new - value_old).clamp(-clip, clip)
    value = 0.5 * torch.maximum((value_new - returns) ** 2, (v_clip - returns) ** 2)
    return policy, value


@stage("ppo_clipped_loss")
class PPOClippedLossStage(nn.Module):
    def __init__(self, clip_range: float = 0.2, vf_coef: float = 0.5, ent_coef: float = 0.0) -> None:
        super().__init__()
        self.clip_range, self.vf_coef, self.ent_coef = float(clip_range), float(vf_coef), float(ent_coef)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("clip_range", 0.2)), float(cfg.get("vf_coef", 0.5)), float(cfg.get("ent_coef", 0.0)))

    def forward(self, logp_new, logp_old, advantages, value_new, value_old, returns):
        pol, val = _ppo_terms(logp_new, logp_old, advantages, value_new, value_old, returns, self.clip_range)
        policy_loss, value_loss = pol.mean(), val.mean()
        return policy_loss, value_loss, policy_loss + self.vf_coef * value_loss


@stage("masked_ppo_clipped_loss")
class MaskedPPOClippedLossStage(nn.Module):
    def __init__(self, clip_range: float = 0.2, vf_coef: float = 0.5, ent_coef: float = 0.0,
                 normalize_advantages: bool = True) -> None:
        super().__init__()
        self.clip_range, self.vf_coef, self.ent_coef = float(clip_range), float(vf_coef), float(ent_coef)
        self.normalize_advantages = bool(normalize_advantages)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("clip_range", 0.2)), float(cfg.get("vf_coef", 0.5)), float(cfg.get("ent_coef", 0.0)),
                   bool(cfg.get("normalize_advantages", True)))

    def forward(self, logp_new, logp_old, advantages, value_new, value_old, returns, loss_mask, entropy):
        others = (logp_old, advantages, value_new, value_old, returns, loss_mask, entropy)
        if any(t.shape != logp_new.shape for t in others):
            raise ValueError("masked PPO loss tensors must all share one shape")
        mask = loss_mask.to(logp_new.dtype)
        _finite_nonneg(mask, "masked PPO loss_mask")
        denom = mask.sum()
        if not bool(denom > 0):
            raise ValueError("masked PPO loss requires at least one selected token")
        adv = advantages.to(logp_new.dtype)
        if self.normalize_advantages:
            mean = (adv * mask).sum() / denom
            var = (((adv - mean) ** 2) * mask).sum() / denom
            adv = (adv - mean) / torch.sqrt(var + 1e-8)
        pol, val = _ppo_terms(logp_new, logp_old, adv, value_new, value_old, returns, self.clip_range)
        policy_loss = (pol * mask).sum() / denom
        value_loss = (val * mask).sum() / denom
        ent = (entropy * mask).sum() / denom
        return policy_loss, value_loss, ent, policy_loss + self.vf_coef * value_loss - self.ent_coef * ent


@stage("kl_penalty")
class KLPenaltyStage(nn.Module):
    def __init__(self, kl_coef: float = 0.1) -> None:
        super().__init__()
        self.kl_coef = float(kl_coef)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("kl_coef", 0.1)))

    def forward(self, logp_policy: Tensor, logp_ref: Tensor, rewards: Tensor) -> Tensor:
        return rewards - self.kl_coef * (logp_policy - logp_ref)


@stage("gae_compute")
class GAEComputeStage(nn.Module):
    """Generalised advantage estimation over [batch, T] rewards/values (bootstrap value 0)."""

    def __init__(self, gamma: float = 1.0, lambda_: float = 0.95) -> None:
        super().__init__()
        self.gamma, self.lam = float(gamma), float(lambda_)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("gamma", 1.0)), float(cfg.get("lambda_", cfg.get("lambda", 0.95))))

    def forward(self, rewards: Tensor, values: Tensor):
        b, t = rewards.shape
        adv = torch.zeros_like(rewards)
        nxt_adv = torch.zeros(b, device=rewards.device, dtype=rewards.dtype)
        nxt_val = torch.zeros(b, device=rewards.device, dtype=rewards.dtype)
        for i in range(t - 1, -1, -1):
            delta = rewards[:, i] + self.gamma * nxt_val - values[:, i]
            nxt_adv = delta + self.gamma * self.lam * nxt_adv
            adv[:, i] = nxt_adv
            nxt_val = values[:, i]
        return adv, adv + values


# ----------------------------------------------------------------------------- heads --
@stage("reward_head")
class RewardHeadStage(nn.Module):
    def __init__(self, model_dim: int = 128, pool: str = "last") -> None:
        super().__init__()
        self.pool = str(pool)
        self.proj = nn.Linear(int(model_dim), 1, bias=False)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("model_dim", 128)), str(cfg.get("pool", "last")))

    def forward(self, hidden: Tensor) -> Tensor:
        pooled = hidden.mean(dim=1) if self.pool == "mean" else hidden[:, -1, :]
        return self.proj(pooled).squeeze(-1)


@stage("masked_reward_head")
class MaskedRewardHeadStage(nn.Module):
    """Scalar reward read at the last selected position of each sequence."""

    def __init__(self, model_dim: int = 128) -> None:
        super().__init__()
        self.model_dim = int(model_dim)
        self.proj = nn.Linear(self.model_dim, 1, bias=False)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("model_dim", 128)))

    def forward(self, hidden: Tensor, sequence_mask: Tensor) -> Tensor:
        if hidden.ndim != 3 or hidden.size(-1) != self.model_dim or sequence_mask.shape != hidden.shape[:2]:
            raise ValueError("masked_reward_head expects hidden [batch, seq, dim] and mask [batch, seq]")
        _finite_nonneg(sequence_mask, "masked_reward_head mask")
        sel = sequence_mask > 0
        if bool((sel.sum(dim=-1) <= 0).any()):
            raise ValueError("masked_reward_head requires at least one selected token per example")
        pos = torch.arange(hidden.size(1), device=hidden.device).view(1, -1)
        last = pos.masked_fill(~sel, -1).amax(dim=-1)
        return self.proj(hidden[torch.arange(hidden.size(0), device=hidden.device), last]).squeeze(-1)


@stage("value_head")
class ValueHeadStage(nn.Module):
    def __init__(self, model_dim: int = 128) -> None:
        super().__init__()
        self.proj = nn.Linear(int(model_dim), 1, bias=False)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("model_dim", 128)))

    def forward(self, hidden: Tensor) -> Tensor:
        return self.proj(hidden).squeeze(-1)


@stage("policy_logits_value")
class PolicyLogitsValueStage(nn.Module):
    def __init__(self, model_dim: int = 128, vocab_size: int = 256, output_multiplier: float = 1.0,
                 logit_softcap: float = 0.0) -> None:
        super().__init__()
        self.model_dim = int(model_dim)
        self.output_multiplier, self.logit_softcap = float(output_multiplier), float(logit_softcap)
        self.lm_head = nn.Linear(self.model_dim, int(vocab_size), bias=False)
        self.value_head = nn.Linear(self.model_dim, 1, bias=False)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("model_dim", 128)), int(cfg.get("vocab_size", 256)),
                   float(cfg.get("output_multiplier", 1.0)), float(cfg.get("logit_softcap", 0.0)))

    def forward(self, hidden: Tensor):
        logits = self.lm_head(hidden) * self.output_multiplier
        if self.logit_softcap > 0.0:
            logits = self.logit_softcap * torch.tanh(logits / self.logit_softcap)
        return logits, self.value_head(hidden).squeeze(-1)


@stage("pair_batch_concat")
class PairBatchConcatStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, chosen: Tensor, rejected: Tensor) -> Tensor:
        if chosen.shape != rejected.shape or chosen.dtype != rejected.dtype or chosen.size(0) <= 0:
            raise ValueError("pair_batch_concat expects two non-empty tensors of identical shape and dtype")
        return torch.cat((chosen, rejected), dim=0)


@stage("pair_batch_split")
class PairBatchSplitStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, paired: Tensor):
        if paired.ndim < 1 or paired.size(0) <= 0 or paired.size(0) % 2:
            raise ValueError("pair_batch_split expects an even, non-empty leading dimension")
        return paired.chunk(2, dim=0)


@stage("latent_mse_loss")
class LatentMSELossStage(nn.Module):
    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, predicted: Tensor, target: Tensor) -> Tensor:
        return F.mse_loss(predicted.float(), target.detach().float())


@stage("softmax_distillation_loss")
class SoftmaxDistillationLossStage(nn.Module):
    """Soft-target cross-entropy against teacher logits at a temperature."""

    def __init__(self, temperature: float = 1.0) -> None:
        super().__init__()
        self.temperature = float(temperature)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("temperature", 1.0)))

    def forward(self, student_logits: Tensor, teacher_logits: Tensor) -> Tensor:
        t = self.temperature
        p = F.softmax(teacher_logits.detach().float() / t, dim=-1)
        return -(p * F.log_softmax(student_logits.float() / t, dim=-1)).sum(-1).mean() * (t * t)
