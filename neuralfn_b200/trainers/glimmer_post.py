"""Post-training of the native Glimmer engine: response-only SFT, pairwise DPO and the Bradley-Terry reward model
from prepared record shards, on the dense trainer's step (sharded AdamW over peer memory, CUDA-graph replay).

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
        if objective not in ("sft", "dpo", "reward_model"):
            raise ValueError("objective must be 'sft', 'dpo' or 'reward_model' (pre-training uses DenseGPTTrainer directly)")
        if objective == "reward_model" and not cfg.reward_head:
            from dataclasses import replace
            cfg = replace(cfg, reward_head=True)
        self.objective, self.pairs = objective, batch
        rows = batch if objective == "sft" else 2 * batch
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
