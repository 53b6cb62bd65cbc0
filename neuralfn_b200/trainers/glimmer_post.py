"""Post-training of the native Glimmer engine: response-only SFT, pairwise DPO, the Bradley-Terry reward model and PPO
(rollouts sampled with the engine's own forward pass, clipped-surrogate updates on the native step), from prepared record shards, on the dense trainer's step (sharded AdamW over peer memory, CUDA-graph replay).

SFT feeds each batch's loss mask to the engine; the step is otherwise the pre-training step. DPO stacks
every batch as (chosen rows, rejected rows), so one forward / backward covers the pair. The frozen
reference model of DPO is the policy at the start of the run, so its sequence log-probabilities are
computed ONCE for the batches the run will visit, before the first optimizer step, with the same engine
and buffers: no second copy of the weights or activations lives on the device.

Reference: ``neuralfn/csrc/native_train/muse_glimmer_native_train.cpp:187`` (``--objective``), ``:452-478``
(reference-policy and DPO options); record shards are the ones ``data.shards.RecordReader`` reads.
"""
from __future__ import annotations

import time

import torch

from ..models.glimmer import GlimmerConfig
from ..parallel.dp import AdamWConfig
from .dense_gpt import DenseGPTTrainer

__all__ = ["GlimmerPostTrainer"]


class GlimmerPostTrainer:
    def __init__(self, cfg: GlimmerConfig, batch: int, seq: int, objective: str, optim: AdamWConfig | None = None, *, seed: int = 1337,
                 use_cuda_graph: bool = True, group=None) -> None:
        if objective not in ("sft", "dpo", "reward_model", "ppo"):
            raise ValueError("objective must be 'sft', 'dpo', 'reward_model' or 'ppo' (pre-training uses DenseGPTTrainer directly)")
        from dataclasses import replace
        if objective == "reward_model" and not cfg.reward_head:
            cfg = replace(cfg, reward_head=True)
        if objective == "ppo" and not cfg.value_head:
            cfg = replace(cfg, value_head=True)
        self.objective, self.pairs = objective, batch
        rows = batch if objective in ("sft", "ppo") else 2 * batch
        self.trainer = DenseGPTTrainer(cfg, rows, seq, optim, seed=seed, use_cuda_graph=use_cuda_graph, group=group)
        self.engine = self.trainer.engine
        self.engine.set_objective(objective)
        self._h_stats = torch.zeros(3, dtype=torch.float32).pin_memory()

    # ------------------------------------------------------------------------------ batches --
    @staticmethod
    def stack_preference(rec: dict) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(ids, targets, mask) with the chosen rows first and the rejected rows second."""
        cat = lambda k: torch.cat([rec["chosen_" + k], rec["rejected_" + k]], 0)  # noqa: E731
        return cat("input_ids"), cat("targets"), cat("loss_mask")

    def sft_step(self, rec: dict) -> float:
        self.engine.set_loss_mask(rec["loss_mask"])
        return self.trainer.train_step(rec["input_ids"], rec["targets"])

    @torch.no_grad()
    def reference_logps(self, rec: dict) -> torch.Tensor:
        ids, tg, mask = self.stack_preference(rec)
        return self.engine.sequence_logps(ids.to(self.trainer.device), tg.to(self.trainer.device), mask).cpu()

    def dpo_step(self, rec: dict, ref_logps: torch.Tensor | None = None) -> dict:
        """One preference step: DPO against ``ref_logps``, or the reward-model loss when the objective is ``reward_model``."""
        ids, tg, mask = self.stack_preference(rec)
        self.engine.set_loss_mask(mask)
        if ref_logps is not None:
            self.engine.set_reference_logps(ref_logps)
        self.trainer.train_step(ids, tg, return_loss=False)
        self._h_stats.copy_(self.engine.dpo_stats, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return {"loss": float(self._h_stats[0]), "reward_accuracy": float(self._h_stats[1]), "reward_margin": float(self._h_stats[2])}

    # ---------------------------------------------------------------------------------- PPO --
    @torch.no_grad()
    def _policy_logits(self, ids: torch.Tensor) -> torch.Tensor:
        """Logits [B, L, V] of a batch of equal-length prefixes (right-padded to the engine's sequence length; causal
        attention makes the padding invisible to the positions that are read)."""
        eng, L = self.engine, ids.shape[1]
        tok = torch.zeros(eng.B, eng.T, dtype=torch.int32, device=ids.device)
        tok[:, :L] = ids
        eng.tokens.copy_(tok.reshape(-1))
        keep, eng.objective = eng.objective, "ar"
        eng.forward(compute_grad_logits=False)
        eng.objective = keep
        return eng.logits_view()[:, :L].float()

    @torch.no_grad()
    def ppo_rollout(self, prompts: torch.Tensor, reward, *, max_new_tokens: int = 16, temperature: float = 1.0, top_k: int = 0,
                    gamma: float = 1.0, gae_lambda: float = 0.95, eos_token_id: int | None = None, pad_token_id: int = 0,
                    generator: torch.Generator | None = None, kl_coef: float = 0.0) -> dict:
        """Samples continuations of ``prompts`` [B, P] with the current policy, scores them with ``reward(ids, P) -> [B]``
        (added at the last response token) and returns the per-row rollout the ``ppo`` objective consumes. ``kl_coef > 0``
        shapes the per-token rewards with ``-kl_coef * (log p_policy - log p_reference)`` against the parameters kept by
        ``freeze_reference`` (called here on first use: the reference is then the policy before its first update)."""
        from ..tensor.ppo import gae_advantages, sample_continuations
        eng = self.engine
        dev = self.trainer.device
        prompts = prompts.to(dev)
        B, P = prompts.shape
        if B != eng.B or P + max_new_tokens > eng.T + 1:
            raise ValueError("prompts must fill the trainer's batch and leave room for the rollout inside its sequence length")
        ids, mask = sample_continuations(self._policy_logits, prompts, max_new_tokens, temperature, top_k, generator, eos_token_id, pad_token_id)
        L = ids.shape[1] - 1                                            # rows: position j predicts token j + 1
        tok = torch.zeros(B, eng.T, dtype=torch.int32, device=dev)
        tgt = torch.zeros_like(tok)
        tok[:, :L], tgt[:, :L] = ids[:, :-1], ids[:, 1:]
        row_mask = torch.zeros(B, eng.T, device=dev)
        row_mask[:, P - 1:L] = mask
        eng.set_batch(tok, tgt)
        eng.set_loss_mask(row_mask)
        eng.set_ppo_batch(*(torch.zeros(B, eng.T, device=dev) for _ in range(4)))
        eng.forward(compute_grad_logits=False)                           # the ppo objective fills row losses and values
        logp_old, values = (-eng.row_loss).view(B, eng.T).clone(), eng.values.view(B, eng.T).clone()
        rewards = torch.zeros(B, max_new_tokens, device=dev)
        kl = torch.zeros(B, device=dev)
        if kl_coef > 0.0:
            per_token = (logp_old - self._reference_logp())[:, P - 1:L] * mask
            rewards -= kl_coef * per_token
            kl = per_token.sum(1)
        last = (mask.sum(1).long() - 1).clamp(min=0)
        score = reward(ids, P).float().to(dev)
        rewards[torch.arange(B, device=dev), last] += score
        adv, ret = gae_advantages(rewards, values[:, P - 1:L] * mask, mask, gamma, gae_lambda)
        full = lambda t: torch.nn.functional.pad(t, (P - 1, eng.T - L))  # noqa: E731
        return {"tokens": tok, "targets": tgt, "mask": row_mask, "logp_old": logp_old, "value_old": values, "advantages": full(adv),
                "returns": full(ret), "score": score, "ids": ids, "kl": kl}

    def freeze_reference(self) -> None:
        """Keeps a copy of the current trainable parameters (the whole model, or just the adapters under LoRA) as the frozen
        reference policy of the KL penalty."""
        self._ref_params = self.engine.params.clone()

    @torch.no_grad()
    def _reference_logp(self) -> torch.Tensor:
        """[B, T] log-probabilities of the resident batch's targets under the frozen reference: its parameters are swapped into
        the engine's buffer for one forward pass (no second engine, no second set of activations)."""
        eng = self.engine
        if getattr(self, "_ref_params", None) is None:
            self.freeze_reference()
        live = eng.params.clone()
        eng.params.copy_(self._ref_params)
        eng.forward(compute_grad_logits=False)
        out = (-eng.row_loss).view(eng.B, eng.T).clone()
        eng.params.copy_(live)
        return out

    def ppo_update(self, rollout: dict) -> dict:
        """One optimizer step of the clipped surrogate on a stored rollout."""
        eng = self.engine
        eng.set_loss_mask(rollout["mask"])
        eng.set_ppo_batch(rollout["logp_old"], rollout["advantages"], rollout["returns"], rollout["value_old"])
        self.trainer.train_step(rollout["tokens"], rollout["targets"], return_loss=False)
        stats = eng.ppo_stats.tolist()
        return {"policy_loss": stats[0], "value_loss": stats[1], "clip_fraction": stats[2], "approx_kl": stats[3]}

    def ppo_step(self, prompts: torch.Tensor, reward, *, epochs: int = 2, **rollout_kw) -> dict:
        roll = self.ppo_rollout(prompts, reward, **rollout_kw)
        out = {}
        for _ in range(max(1, epochs)):
            out = self.ppo_update(roll)
        return {**out, "mean_score": float(roll["score"].mean()), "mean_kl": float(roll["kl"].mean())}

    # ---------------------------------------------------------------------------------- run --
    def fit(self, records: str, steps: int, *, split: str = "train", allow_train_as_val: bool = True, log_every: int = 0) -> dict:
        """``steps`` optimizer steps over the record shards at ``records`` (wrapping around at the end)."""
        from ..data.shards import RecordReader
        tr = self.trainer
        reader = RecordReader(records, "sft" if self.objective == "sft" else "preference", split, self.pairs,
                              allow_train_as_val=allow_train_as_val, rank=tr.rank, world=tr.world)
        if reader.seq_len != tr.seq:
            raise ValueError(f"records hold sequences of {reader.seq_len} tokens, the trainer was built for {tr.seq}")

        def batches(n):
            got = 0
            while got < n:
                rec = reader.next()
                if rec is None:
                    reader.reset()
                    rec = reader.next()
                    if rec is None:
                        raise ValueError("record shards hold no complete batch")
                got += 1
                yield rec

        history, refs = [], []
        t0 = time.perf_counter()
        if self.objective == "dpo":
            visit = min(steps, max(1, reader.total_batches))
            refs = [self.reference_logps(rec) for rec in batches(visit)]
            reader.reset()
        ref_ms = (time.perf_counter() - t0) * 1e3
        t0 = time.perf_counter()
        for i, rec in enumerate(batches(steps)):
            if self.objective == "sft":
                out = {"loss": self.sft_step(rec)}
            else:
                out = self.dpo_step(rec, refs[i % len(refs)] if refs else None)
            history.append(out)
            if log_every and (i + 1) % log_every == 0 and tr.rank == 0:
                import sys
                print(f"step {i + 1}/{steps} " + " ".join(f"{k} {v:.4f}" for k, v in out.items()), file=sys.stderr, flush=True)
        torch.cuda.synchronize()
        tr.check_status()
        reader.close()
        loop_ms = (time.perf_counter() - t0) * 1e3
        return {"objective": self.objective, "steps": steps, "history": history, "reference_pass_wall_ms": ref_ms,
                "train_loop_wall_ms": loop_ms, "rows_per_step": tr.batch * tr.world,
                "tokens_per_second": steps * tr.tokens_per_step / (loop_ms / 1e3)}
