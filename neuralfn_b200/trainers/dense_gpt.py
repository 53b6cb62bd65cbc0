"""Dense GPT trainer: engine + sharded optimizer + CUDA-graph step.

Public call a user makes::

    trainer = DenseGPTTrainer(GPT2Config.variant("gpt2_qknorm_softcap_zloss"), batch=16, seq=1024)
    loss = trainer.train_step(tokens, targets)      # host (pinned) or device int tensors

One optimizer step = forward + backward + (data-parallel reduce) + AdamW, captured
once into a CUDA graph and replayed; per step the host only uploads the batch and
the 16-float hyper-parameter block. Under ``torch.distributed`` (one process per
GPU) every rank trains on its own micro-batch and the gradient reduction, sharded
update and parameter all-gather run inside the peer-memory kernels of
``neuralfn_b200.parallel.dp`` - the step makes no NCCL call.

Mirrors the contract of the reference's native dense trainer loop
(``nfn_gpt2_native_train.cpp:28362-28470``: zero/accumulate grads, clip on device,
scheduled lr, one AdamW launch) for the no-accumulation case.
"""
from __future__ import annotations

import ctypes
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.gpt2 import FlatLayout, GPT2Config
from ..parallel.dp import AdamWConfig, ShardedAdamW, SymmetricBuffers

__all__ = ["DenseGPTTrainer", "TrainReport"]


@dataclass
class TrainReport:
    steps: int
    tokens_processed: int
    train_loop_wall_ms: float
    train_compute_tokens_per_second: float
    train_losses: list[float]


class DenseGPTTrainer:
    def __init__(self, cfg, batch: int, seq: int, optim: AdamWConfig | None = None, *,
                 device: torch.device | str | None = None, seed: int = 1337, use_cuda_graph: bool = True,
                 group=None, grad_accum_steps: int = 1) -> None:
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("DenseGPTTrainer runs on CUDA (sm_100a); use models.gpt2.reference_forward on CPU")
        self.cfg, self.batch, self.seq = cfg, batch, seq
        self.optim_cfg = optim or AdamWConfig()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.layout = FlatLayout(cfg.param_specs(), world=self.world)
        self.bufs = SymmetricBuffers(self.layout.n_total, self.device, group)
        # identical initial weights on every rank (same seed), fp32 master -> bf16 params
        master = torch.empty(self.layout.n_total, dtype=torch.float32, device=self.device)
        cfg.init_params_(self.layout, master, seed)
        self.opt = ShardedAdamW(self.layout, self.bufs, self.optim_cfg, master_init=master)
        self.bufs.params.copy_(master.to(torch.bfloat16))
        del master
        self.bufs.grads.zero_()
        self.engine = cfg.make_engine(self.layout, self.bufs.params, self.bufs.grads, batch, seq)
        from ..utils.stage_timing import StageTimer
        self.timer = StageTimer()  # NFN_NATIVE_GPT_STAGE_TIMING=1: per-stage CUDA events (+ NVTX with NFN_NVTX=1)
        self.engine.timer = self.timer
        if getattr(self.opt, "overlap", False) and max(1, int(grad_accum_steps)) == 1 and hasattr(self.engine, "grad_ready_hook"):
            # the gradient reduction of each group of layers runs under the rest of the backward pass
            self.engine.grad_ready_hook = self.opt.reduce_range
        # a captured graph cannot be timed stage by stage: the diagnostic mode runs eagerly
        self.use_cuda_graph = use_cuda_graph and not self.timer.enabled
        # gradient accumulation: `grad_accum_steps` micro-batches per optimizer step, summed in
        # an fp32 side buffer; each phase of the cycle is its own captured graph
        self.grad_accum = max(1, int(grad_accum_steps))
        self._micro = 0
        self._acc = (torch.zeros(self.layout.n_total, dtype=torch.float32, device=self.device)
                     if self.grad_accum > 1 else None)
        self._graphs: dict[str, torch.cuda.CUDAGraph] = {}
        self._warm: set[str] = set()
        self.launches_per_step = 0
        from ..utils.pinned import PinnedRing
        self._h_tokens = PinnedRing(batch * seq, torch.int32, slots=3)
        self._h_targets = PinnedRing(batch * seq, torch.int32, slots=3)
        self._h_loss = torch.zeros(1, dtype=torch.float32).pin_memory()
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group)

    # ------------------------------------------------------------------ step --
    def _launch_phase(self, phase: str) -> None:
        from ..ops import _lib
        self.engine.forward()
        if phase == "single" and getattr(self.engine, "grad_ready_hook", None) is not None:
            self.opt.begin_overlap()
        self.engine.backward()
        if phase != "single":
            mode = {"first": 0, "mid": 1, "last": 2}[phase]
            rc = _lib.load().nfn_grad_accumulate(ctypes.c_void_p(self._acc.data_ptr()), ctypes.c_void_p(self.bufs.grads.data_ptr()),
                                                 ctypes.c_longlong(self.layout.n_total), ctypes.c_int(mode),
                                                 ctypes.c_float(1.0 / self.grad_accum), ctypes.c_void_p(_lib.stream_ptr()))
            _lib.check(rc, "nfn_grad_accumulate")
        if phase in ("single", "last"):
            with self.timer.stage("adamw_update"):  # gradient reduction, clip factor and the sharded update
                self.opt.launch_step()

    def _run_step(self) -> None:
        """forward + backward (+ accumulate) (+ optimizer) on the batch already in the engine
        buffers. The optimizer runs on the last micro-batch of each accumulation cycle."""
        from ..ops import _lib
        k, i = self.grad_accum, self._micro
        phase = "single" if k == 1 else ("first" if i == 0 else ("last" if i == k - 1 else "mid"))
        final = phase in ("single", "last")
        if final:
            self.opt.stage_hyper()
        if getattr(self.engine, "graph_key", ""):
            phase_key = f"{phase}:{self.engine.graph_key}"   # e.g. the MLP activation a mixture-of-activations run selected
        else:
            phase_key = phase
        if not self.use_cuda_graph or phase_key not in self._warm:
            # the first run of a phase is eager: it sets kernel attributes and fills the
            # tensor-map cache, neither of which may happen during stream capture
            before = _lib.launch_count()
            self._launch_phase(phase)
            if final:
                self.launches_per_step = _lib.launch_count() - before
            self._warm.add(phase_key)
        elif phase_key not in self._graphs:
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch_phase(phase)
            self._graphs[phase_key] = g
            g.replay()
        else:
            self._graphs[phase_key].replay()
        if final:
            self.opt.step_count += 1
            self._micro = 0
            self.timer.next_step()
        else:
            self._micro += 1

    def upload(self, tokens: torch.Tensor, targets: torch.Tensor) -> int:
        """Copy a batch into the device input buffers; returns the bytes moved host->device."""
        moved = 0
        with self.timer.stage("token_upload"):
            moved = self._upload(tokens, targets)
        return moved

    def _upload(self, tokens: torch.Tensor, targets: torch.Tensor) -> int:
        moved = 0
        for src, stage, dst in ((tokens, self._h_tokens, self.engine.tokens),
                                (targets, self._h_targets, self.engine.targets)):
            src = src.reshape(-1)
            if src.device.type == "cpu":
                if src.dtype == torch.int32 and src.is_pinned():
                    dst.copy_(src, non_blocking=True)
                else:
                    stage.upload(dst, src.to(torch.int32))
                moved += dst.numel() * dst.element_size()
            else:
                dst.copy_(src)
        return moved

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor, *, return_loss: bool = True):
        """One micro-batch: forward, backward and - on the last micro-batch of an accumulation
        cycle (every call when ``grad_accum_steps == 1``) - the optimizer step. Returns the mean
        token loss of this rank's micro-batch (python float, read back from the device) when
        ``return_loss``."""
        self.upload(tokens, targets)
        if self._micro == 0 and hasattr(self.engine, "moa_probe_due") and self.engine.moa_probe_due(self.opt.step_count + 1):
            self.engine.moa_select(self.opt.step_count + 1)
        self._run_step()
        if return_loss:
            self._h_loss.copy_(self.engine.loss, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return float(self._h_loss[0])
        return None

    def step_on_device_batch(self) -> None:
        """Step on whatever batch is already resident (used by kernel-only timing)."""
        self._run_step()

    @property
    def tokens_per_step(self) -> int:
        """Tokens consumed by one ``train_step`` call (one micro-batch on every rank)."""
        return self.batch * self.seq * self.world

    # --------------------------------------------------------------- training --
    def train(self, batches, max_steps: int, log_every: int = 0) -> TrainReport:
        losses = []
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        n = 0
        for tokens, targets in batches:
            loss = self.train_step(tokens, targets)
            losses.append(loss)
            n += 1
            if log_every and n % log_every == 0:
                self.check_status()  # a timed-out device wait must stop the run, not poison later steps
            if log_every and n % log_every == 0 and self.rank == 0:
                print(f"step {n:6d} loss {loss:.4f} lr {self.opt.hyper_host[0].item():.3e} "
                      f"gnorm {self.opt.grad_norm:.3f}", flush=True)
            if n >= max_steps:
                break
        torch.cuda.synchronize(self.device)
        wall = (time.perf_counter() - t0) * 1e3
        self.check_status()
        toks = n * self.tokens_per_step
        return TrainReport(n, toks, wall, toks / (wall / 1e3) if wall > 0 else 0.0, losses)

    def check_status(self) -> None:
        from ..ops import _lib
        _lib.assert_status_ok("dense gpt step")

    # ------------------------------------------------------------ checkpoints --
    def full_master(self) -> torch.Tensor:
        """fp32 master weights of the whole model on this rank (gathers shards)."""
        if self.world == 1:
            return self.opt.master.clone()
        parts = [torch.empty_like(self.opt.master) for _ in range(self.world)]
        dist.all_gather(parts, self.opt.master)
        return torch.cat(parts)
