"""Data parallelism with a sharded AdamW whose collectives are fused into the kernels.

One process per GPU. Parameters and gradients live in flat bf16 buffers allocated
from NVLink symmetric memory, so every rank holds the device addresses of all peers'
buffers. After the backward pass each rank

1. signals "gradients ready" to all peers and waits for theirs (bounded),
2. reduces its 1/W shard of the gradient by *loading the peers' bf16 gradients
   directly* (fp32 accumulation, shard squared-norm on the side),
3. exchanges shard norms through peer stores (this doubles as the "all reads of my
   gradients are finished" barrier) and derives the global clip factor,
4. runs AdamW on its fp32 master/m/v shard and *stores the bf16 parameters of the
   shard into every peer's parameter buffer* (the all-gather),
5. signals/waits "parameters ready".

No NCCL call is made in a training step. On CPU (gloo) and when symmetric memory is
unavailable the same maths runs through ``torch.distributed`` reduce-scatter /
all-gather, which is what the multi-process CPU tests exercise.

The reference has no data parallelism (its only distributed mode is pipeline
stages); its single-GPU counterpart is the descriptor-table AdamW
``adamw_step_many_with_device_scale_*`` (``neuralfn/csrc/tile_cuda/kernels.cu:11852-12137``).
"""
from __future__ import annotations

import contextlib
import math
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

__all__ = ["AdamWConfig", "SymmetricBuffers", "ShardedAdamW", "lr_at_step"]


@dataclass
class AdamWConfig:
    lr: float = 6e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    warmup_steps: int = 60
    total_steps: int = 20000
    final_lr_fraction: float = 0.0
    schedule: str = "cosine"  # "cosine" | "constant"


def lr_at_step(cfg: AdamWConfig, step: int) -> float:
    """1-based ``step``. Linear warm-up ``lr*max(1,step)/warmup`` then constant or cosine
    from lr to ``lr*final_lr_fraction`` over ``max(1, horizon - warmup)`` steps
    (same schedule as ``nfn_gpt2_native_train.cpp:5643-5676``)."""
    if cfg.warmup_steps > 0 and step <= cfg.warmup_steps:
        return cfg.lr * max(1, step) / cfg.warmup_steps
    if cfg.schedule == "constant":
        return cfg.lr
    span = max(1, cfg.total_steps - cfg.warmup_steps)
    t = min(1.0, max(0.0, (step - cfg.warmup_steps) / span))
    lo = cfg.lr * cfg.final_lr_fraction
    return lo + 0.5 * (cfg.lr - lo) * (1.0 + math.cos(math.pi * t))


class SymmetricBuffers:
    """Flat parameter / gradient / control buffers visible to every rank of a group.

    ``world == 1`` (or CPU): ordinary tensors. Otherwise tensors come from
    ``torch.distributed._symmetric_memory`` and ``*_ptrs`` list each rank's device
    address of the same buffer (index = rank)."""

    CTRL_INT64 = 64  # [0,16): norm slots (8 B each); [16,64): flags as int32 pairs

    def __init__(self, n_total: int, device: torch.device, group=None) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device
        self.symmetric = False
        if self.world > 1 and device.type == "cuda":
            import torch.distributed._symmetric_memory as symm
            gname = (group or dist.group.WORLD).group_name
            self.params = symm.empty(n_total, dtype=torch.bfloat16, device=device)
            self.grads = symm.empty(n_total, dtype=torch.bfloat16, device=device)
            self.ctrl = symm.empty(self.CTRL_INT64, dtype=torch.int64, device=device)
            self.ctrl.zero_()
            # fp32 reduced-gradient shard, peer-writable: the bucketed reduce stores into its owner's shard
            self.gshard = symm.empty(n_total // self.world, dtype=torch.float32, device=device)
            self._handles = [symm.rendezvous(t, gname) for t in (self.params, self.grads, self.ctrl, self.gshard)]
            self.gshard_ptrs = list(self._handles[3].buffer_ptrs)
            self.param_ptrs = list(self._handles[0].buffer_ptrs)
            self.grad_ptrs = list(self._handles[1].buffer_ptrs)
            ctrl_ptrs = list(self._handles[2].buffer_ptrs)
            self.slot_ptrs = ctrl_ptrs
            self.flag_ptrs = [p + 16 * 8 for p in ctrl_ptrs]
            self.multicast_grad_ptr = int(getattr(self._handles[1], "multicast_ptr", 0) or 0)
            self.symmetric = True
            torch.cuda.synchronize(device)
            dist.barrier(group)
        else:
            self.params = torch.empty(n_total, dtype=torch.bfloat16, device=device)
            self.grads = torch.zeros(n_total, dtype=torch.bfloat16, device=device)
            self.ctrl = torch.zeros(self.CTRL_INT64, dtype=torch.int64, device=device)
            self.param_ptrs = [self.params.data_ptr()]
            self.grad_ptrs = [self.grads.data_ptr()]
            self.slot_ptrs = [self.ctrl.data_ptr()]
            self.flag_ptrs = [self.ctrl.data_ptr() + 16 * 8]
            self.multicast_grad_ptr = 0


class ShardedAdamW:
    """AdamW over a flat parameter space, optimizer state sharded 1/W per rank."""

    def __init__(self, layout, bufs: SymmetricBuffers, cfg: AdamWConfig, master_init: torch.Tensor | None = None,
                 peer_timeout_s: float = 5.0) -> None:
        self.layout, self.bufs, self.cfg = layout, bufs, cfg
        self.world, self.rank = bufs.world, bufs.rank
        if layout.n_total % (8 * self.world):
            raise ValueError("flat layout is not divisible into 8-aligned shards")
        self.shard = layout.n_total // self.world
        self.lo = self.rank * self.shard
        dev = bufs.device
        self.master = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        if master_init is not None:
            self.master.copy_(master_init[self.lo:self.lo + self.shard])
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.step_count = 0
        self.epoch = 0
        self.peer_timeout_s = peer_timeout_s
        self.on_cuda = dev.type == "cuda"
        if self.on_cuda:
            from ..ops import kernels as K
            self.K = K
            self.hyper = torch.zeros(K.HYPER_SIZE, dtype=torch.float32, device=dev)
            from ..utils.pinned import PinnedRing
            self._hyper_ring = PinnedRing(K.HYPER_SIZE, torch.float32, slots=8)
            self.partial = torch.empty(K.optim_max_partials(), dtype=torch.float32, device=dev)
            self.clip = torch.ones(2, dtype=torch.float32, device=dev)
            self.gshard = getattr(bufs, "gshard", None) if self.world > 1 else None
            if self.world > 1 and self.gshard is None:
                self.gshard = torch.empty(self.shard, dtype=torch.float32, device=dev)
            self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)
            # Bucketed reduction of the gradients under the backward pass (multi-GPU only). Opt-in: the
            # persistent GEMM CTAs of the backward pass own their SMs with a static tile schedule, and a
            # block of any other kernel that lands on an SM first keeps that GEMM CTA - and with it the
            # whole GEMM - waiting until the block exits. Measured on two B200s the bucketed path costs
            # 0.3 - 0.45 ms per step more than reducing after the backward pass, so the default stays off.
            self.overlap = (self.world > 1 and getattr(bufs, "symmetric", False)
                            and os.environ.get("NFN_DP_OVERLAP", "0") == "1")
            self._side = torch.cuda.Stream(device=dev) if self.overlap else None
            self._relay_partial = (torch.zeros(K.dp_relay_blocks(), dtype=torch.float32, device=dev) if self.overlap else None)
            self._covered: list[tuple[int, int]] = []
            self._in_overlap = False
        else:
            self.clip = torch.ones(2, dtype=torch.float32)

    # ----------------------------------------------------------------- helpers --
    def publish_params(self) -> None:
        """Write bf16(master shard) into every rank's parameter buffer (initial sync)."""
        if self.world == 1:
            self.bufs.params.copy_(self.master.to(torch.bfloat16))
            return
        mine = self.master.to(torch.bfloat16)
        if dist.get_backend(self.bufs.group) == "gloo" or not self.on_cuda:
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.bufs.group)
            self.bufs.params.copy_(torch.cat(parts))
        else:
            dist.all_gather_into_tensor(self.bufs.params, mine, group=self.bufs.group)

    def _hyper_values(self, step: int, grad_scale: float) -> list[float]:
        c = self.cfg
        return [lr_at_step(c, step), c.beta1, c.beta2, c.eps, c.weight_decay,
                1.0 - c.beta1 ** step, 1.0 - c.beta2 ** step, grad_scale, c.max_grad_norm]

    def stage_hyper(self, step: int | None = None, grad_scale: float | None = None) -> None:
        """Upload the hyper-parameter block of the coming step (outside a captured graph)."""
        step = self.step_count + 1 if step is None else step
        gs = 1.0 / self.world if grad_scale is None else grad_scale
        # each step's values go through their own pinned slot (guarded by an event): the host may
        # be several steps ahead of the GPU, and a single reused buffer would hand a queued copy
        # the values of a later step
        self._hyper_ring.upload(self.hyper, self._hyper_values(step, gs))

    @property
    def hyper_host(self) -> torch.Tensor:
        """Pinned copy of the hyper-parameter block staged most recently (lr first)."""
        ring = getattr(self, "_hyper_ring", None)
        if ring is not None:
            return ring.last
        return torch.tensor(self._hyper_values(max(1, self.step_count), 1.0 / self.world), dtype=torch.float32)

    # -------------------------------------------------------------------- step --
    def step(self, *, stage: bool = True) -> None:
        """One optimizer step over the current contents of the gradient buffer."""
        if not self.on_cuda:
            return self._step_torch()
        if stage:
            self.stage_hyper()
        self.launch_step()
        self.step_count += 1

    # ------------------------------------------------ reduction under the backward --
    MAX_BUCKETS = 10      # flag slots 2..11 of the control block

    def begin_overlap(self) -> None:
        """Call on the main stream before the backward pass of a step whose gradients will be reduced
        bucket by bucket (``reduce_range``) while later layers are still being differentiated."""
        if not self.overlap:
            return
        self.K.counter_add(self.epoch_dev, 1)
        self._relay_partial.zero_()
        self._covered = []
        self._slots_used = 0
        self._in_overlap = True

    def reduce_range(self, lo: int, hi: int) -> None:
        """Gradients of flat elements [lo, hi) are final on this rank (everything launched so far on
        the current stream produces them): reduce that bucket across ranks on the side stream. All
        ranks must call this with the same ranges in the same order."""
        if not self._in_overlap or hi <= lo:
            return
        if self._slots_used >= self.MAX_BUCKETS - 1:
            return                                  # the rest is reduced at the step
        self._relay(lo, hi, stream=self._side)

    def _relay(self, lo: int, hi: int, stream=None, sync: bool = True) -> None:
        """``sync``: first wait until every rank's gradients of the range are final (one flag slot)."""
        K, b = self.K, self.bufs
        W, r, ed = self.world, self.rank, self.epoch_dev
        main = torch.cuda.current_stream()
        if stream is not None:
            stream.wait_stream(main)
        with torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext():
            if sync:
                slot = 2 + self._slots_used
                self._slots_used += 1
                K.peer_arrive(b.flag_ptrs, r, W, slot, 0, ed)
                K.peer_wait(b.flag_ptrs[r], W, slot, 0, self.peer_timeout_s, ed)
            K.dp_reduce_relay(b.grad_ptrs, b.gshard_ptrs, r, W, lo, hi - lo, self.shard, self._relay_partial,
                              accumulate=True, background=stream is not None)
        self._covered.append((lo, hi))

    def _uncovered(self) -> list[tuple[int, int]]:
        out, cur = [], 0
        for lo, hi in sorted(self._covered):
            if lo > cur:
                out.append((cur, lo))
            cur = max(cur, hi)
        if cur < self.layout.n_total:
            out.append((cur, self.layout.n_total))
        return out

    def launch_step(self) -> None:
        """Kernel launches only (capturable); uses ``self.epoch`` as the signal epoch base."""
        K, b = self.K, self.bufs
        if self.world == 1:
            K.grad_clip_scale(b.grads, self.partial, self.hyper, self.clip)
            K.adamw_flat(self.master, self.m, self.v, b.grads, b.params, self.layout.n_decay, self.hyper, self.clip)
            return
        if not b.symmetric:
            raise RuntimeError("multi-GPU ShardedAdamW needs symmetric-memory buffers")
        W, r, ed = self.world, self.rank, self.epoch_dev
        if self._in_overlap:
            # what the backward pass did not hand over (embeddings, the small non-decayed tail) is
            # reduced here, after one wait for all of it
            for i, (lo, hi) in enumerate(self._uncovered()):
                self._relay(lo, hi, stream=None, sync=i == 0)
            torch.cuda.current_stream().wait_stream(self._side)
            self._in_overlap = False
            # a rank publishes its squared norm after its last bucket, so collecting every rank's norm
            # also tells this rank that all stores into its reduced-gradient shard have landed
            K.dp_norm_publish_n(self._relay_partial, self._relay_partial.numel(), b.slot_ptrs, r, W, 0, ed)
            K.dp_norm_collect(b.slot_ptrs[r], W, 0, self.hyper, self.clip, self.peer_timeout_s, ed)
            K.dp_adamw(self.master, self.m, self.v, self.gshard, b.param_ptrs, r, W, self.lo, self.shard,
                       self.layout.n_decay, self.hyper, self.clip)
            K.peer_arrive(b.flag_ptrs, r, W, 1, 0, ed)
            K.peer_wait(b.flag_ptrs[r], W, 1, 0, self.peer_timeout_s, ed)
            return
        # the signal epoch lives on the device and advances once per launch of this
        # sequence, so replaying a captured graph produces fresh epochs every time
        K.counter_add(ed, 1)
        K.peer_arrive(b.flag_ptrs, r, W, 0, 0, ed)
        K.peer_wait(b.flag_ptrs[r], W, 0, 0, self.peer_timeout_s, ed)
        K.dp_reduce(b.grad_ptrs, r, W, self.lo, self.shard, self.gshard, self.partial)
        K.dp_norm_publish(self.partial, self.shard, b.slot_ptrs, r, W, 0, ed)
        K.dp_norm_collect(b.slot_ptrs[r], W, 0, self.hyper, self.clip, self.peer_timeout_s, ed)
        K.dp_adamw(self.master, self.m, self.v, self.gshard, b.param_ptrs, r, W, self.lo, self.shard,
                   self.layout.n_decay, self.hyper, self.clip)
        K.peer_arrive(b.flag_ptrs, r, W, 1, 0, ed)
        K.peer_wait(b.flag_ptrs[r], W, 1, 0, self.peer_timeout_s, ed)

    # fallback used on CPU ranks (gloo) - same maths through torch.distributed
    def _step_torch(self) -> None:
        c, b = self.cfg, self.bufs
        self.step_count += 1
        step = self.step_count
        g_full = b.grads.float()
        if self.world > 1:
            chunks = list(g_full.view(self.world, self.shard).unbind(0))
            g = torch.empty(self.shard, dtype=torch.float32)
            dist.reduce_scatter(g, [ch.contiguous() for ch in chunks], group=b.group)
            g /= self.world
            sq = (g * g).sum()
            dist.all_reduce(sq, group=b.group)
        else:
            g = g_full
            sq = (g * g).sum()
        norm = sq.sqrt()
        clip = 1.0
        if c.max_grad_norm > 0 and norm.item() > c.max_grad_norm:
            clip = c.max_grad_norm / (norm.item() + 1e-6)
        self.clip[0], self.clip[1] = clip, norm
        g = g * clip
        lr = lr_at_step(c, step)
        self.m.mul_(c.beta1).add_(g, alpha=1 - c.beta1)
        self.v.mul_(c.beta2).addcmul_(g, g, value=1 - c.beta2)
        mh = self.m / (1 - c.beta1 ** step)
        vh = self.v / (1 - c.beta2 ** step)
        idx = torch.arange(self.lo, self.lo + self.shard)
        wd = torch.where(idx < self.layout.n_decay, c.weight_decay, 0.0).float()
        self.master -= lr * (mh / (vh.sqrt() + c.eps) + wd * self.master)
        self.publish_params()

    @property
    def grad_norm(self) -> float:
        return float(self.clip[1].item())

    # ------------------------------------------------------------- checkpoints --
    def state_dict(self) -> dict:
        return {"master": self.master.detach().cpu(), "m": self.m.detach().cpu(), "v": self.v.detach().cpu(),
                "step": self.step_count, "rank": self.rank, "world": self.world, "lo": self.lo,
                "shard": self.shard}

    def load_state_dict(self, sd: dict) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank or sd["shard"] != self.shard:
            raise ValueError("optimizer shard does not match this rank/world size")
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])
