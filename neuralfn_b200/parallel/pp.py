"""Pipeline parallelism for the native Llama-family engine: contiguous layer stages, one
process per GPU, activations and their gradients exchanged with NCCL point-to-point
send/recv between neighbouring stages.

Stage ``r`` of ``W`` owns layers ``[L*r/W, L*(r+1)/W)``; the first stage also owns the
embedding, the last one the final norm, the head and the loss - the partition rule of the
reference's pipeline mode (``muse_glimmer_native_train.cpp:914-960``). A step is synchronous
over ``micro_batches`` micro-batches: every micro-batch runs forward through all stages and
backward through all stages before the next one starts (gradients accumulate in fp32), then
every stage applies its own optimizer to the parameters it owns. Each stage keeps its own
optimizer state, so checkpoints are naturally rank-sharded (``stage-%05d/`` directories).

Gradient clipping uses the norm of the stage's own parameters (no cross-stage reduction).
"""
from __future__ import annotations

import ctypes
from dataclasses import replace
from pathlib import Path

import torch
import torch.distributed as dist

from ..trainers.dense_gpt import DenseGPTTrainer

__all__ = ["stage_layer_range", "PipelineParallelTrainer"]


def stage_layer_range(n_layer: int, rank: int, world: int) -> tuple[int, int]:
    return n_layer * rank // world, n_layer * (rank + 1) // world


class PipelineParallelTrainer:
    def __init__(self, cfg, batch: int, seq: int, optim=None, *, micro_batches: int = 1, seed: int = 1337, device=None) -> None:
        if not dist.is_initialized():
            raise RuntimeError("PipelineParallelTrainer needs an initialised process group (one rank per stage)")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        if cfg.n_layer < self.world:
            raise ValueError("more pipeline stages than layers")
        lo, hi = stage_layer_range(cfg.n_layer, self.rank, self.world)
        self.first, self.last = self.rank == 0, self.rank == self.world - 1
        self.stage_cfg = replace(cfg, pp_layer_begin=lo, pp_layer_end=hi, pp_first=self.first, pp_last=self.last)
        # a single-rank group per stage: the stage's optimizer shards over nobody
        solo = None
        for r in range(self.world):
            g = dist.new_group([r])
            if r == self.rank:
                solo = g
        self.micro_batches = max(1, micro_batches)
        self.inner = DenseGPTTrainer(self.stage_cfg, batch, seq, optim, device=device, seed=seed + self.rank, use_cuda_graph=False, group=solo)
        self.engine = self.inner.engine
        self.device = self.inner.device
        self._acc = (torch.zeros(self.inner.layout.n_total, dtype=torch.float32, device=self.device)
                     if self.micro_batches > 1 else None)
        self._loss = torch.zeros(1, dtype=torch.float32, device=self.device)

    @property
    def layout(self):
        return self.inner.layout

    def _accumulate(self, i: int) -> None:
        from ..ops import _lib
        k = self.micro_batches
        mode = 0 if i == 0 else (2 if i == k - 1 else 1)
        rc = _lib.load().nfn_grad_accumulate(ctypes.c_void_p(self._acc.data_ptr()), ctypes.c_void_p(self.inner.bufs.grads.data_ptr()),
                                             ctypes.c_longlong(self.layout.n_total), ctypes.c_int(mode), ctypes.c_float(1.0 / k),
                                             ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "nfn_grad_accumulate")

    def train_step(self, tokens: list[torch.Tensor] | torch.Tensor, targets: list[torch.Tensor] | torch.Tensor) -> float:
        """One optimizer step. ``tokens`` / ``targets``: one tensor per micro-batch (or a single
        tensor). The first stage reads tokens, the last one targets; other stages ignore both.
        Returns the mean loss over the micro-batches (identical on every rank)."""
        toks = tokens if isinstance(tokens, (list, tuple)) else [tokens]
        tgts = targets if isinstance(targets, (list, tuple)) else [targets]
        if len(toks) != self.micro_batches or len(tgts) != self.micro_batches:
            raise ValueError(f"expected {self.micro_batches} micro-batches")
        eng = self.engine
        total = torch.zeros(1, dtype=torch.float32, device=self.device)
        for i in range(self.micro_batches):
            self.inner.upload(toks[i], tgts[i])
            if not self.first:
                dist.recv(eng.x0, src=self.rank - 1)
            out = eng.forward()
            if not self.last:
                dist.send(out, dst=self.rank + 1)
                dist.recv(eng.d_a, src=self.rank + 1)
            else:
                total += eng.loss
            eng.backward()
            if not self.first:
                dist.send(eng.d_input, dst=self.rank - 1)
            if self.micro_batches > 1:
                self._accumulate(i)
        self.inner.opt.stage_hyper()
        self.inner.opt.launch_step()
        self.inner.opt.step_count += 1
        total /= self.micro_batches
        dist.broadcast(total, src=self.world - 1)
        return float(total.item())

    def save(self, out_dir, step: int | None = None) -> dict:
        from ..checkpoint.named import save_named_checkpoint
        return save_named_checkpoint(self.inner, Path(out_dir) / f"stage-{self.rank:05d}", step)

    def load(self, out_dir, step: int | None = None) -> dict:
        from ..checkpoint.named import load_named_checkpoint
        return load_named_checkpoint(self.inner, Path(out_dir) / f"stage-{self.rank:05d}", step)
