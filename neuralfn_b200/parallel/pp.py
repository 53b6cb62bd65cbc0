"""Pipeline parallelism for the native Llama-family engine: contiguous layer stages, one process per
GPU, a one-forward-one-backward (1F1B) schedule over the micro-batches of a step, activations and
their gradients exchanged with NCCL point-to-point operations between neighbouring stages.

Stage ``r`` of ``W`` owns layers ``[L*r/W, L*(r+1)/W)``; the first stage also owns the embedding, the
last one the final norm, the head and the loss - the partition rule of the reference's pipeline mode
(``muse_glimmer_native_train.cpp:914-960``). Within a step stage ``r`` runs ``min(W - r - 1, M)``
warm-up forwards, then alternates one forward with one backward, then drains the remaining
backwards, so at most ``W - r`` micro-batches are in flight on it and the pipeline bubble is
``(W - 1) / (M + W - 1)`` of the step instead of ``(W - 1) / W``. Each in-flight micro-batch needs its own
activations: the stage keeps that many engines over ONE parameter and gradient buffer. A send and the
receive that follows it on the same neighbour link are issued as one batched group (the neighbour issues
the mirror-image group at the same point of its schedule), which keeps the schedule deadlock-free
without relying on eager buffering; ``simulate_schedule`` checks that property on the CPU.

Gradients of the micro-batches accumulate in fp32; every stage then applies its own optimizer to the
parameters it owns (optimizer state is naturally stage-sharded: ``stage-%05d/`` checkpoint
directories). Gradient clipping uses the norm of the stage's own parameters.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import replace
from pathlib import Path

import torch
import torch.distributed as dist

from ..trainers.dense_gpt import DenseGPTTrainer

__all__ = ["stage_layer_range", "one_f_one_b_schedule", "simulate_schedule", "PipelineParallelTrainer", "main"]


def stage_layer_range(n_layer: int, rank: int, world: int) -> tuple[int, int]:
    return n_layer * rank // world, n_layer * (rank + 1) // world


# ------------------------------------------------------------------------------ schedule --
# An action is a tuple: ("F", i) / ("B", i) compute on micro-batch i; ("comm", [ops]) one batched group of
# point-to-point operations, each op = (kind, peer, what, i) with kind "send" | "recv", what "act" | "grad".
def one_f_one_b_schedule(rank: int, world: int, micro_batches: int) -> list[tuple]:
    M, first, last = micro_batches, rank == 0, rank == world - 1
    prev, nxt = rank - 1, rank + 1
    warm = min(world - rank - 1, M)
    steady = M - warm
    acts: list[tuple] = []

    def comm(*ops):
        ops = [o for o in ops if o is not None]
        if ops:
            acts.append(("comm", ops))

    recv_f = lambda i: None if first else ("recv", prev, "act", i)     # noqa: E731
    send_f = lambda i: None if last else ("send", nxt, "act", i)       # noqa: E731
    recv_b = lambda i: None if last else ("recv", nxt, "grad", i)      # noqa: E731
    send_b = lambda i: None if first else ("send", prev, "grad", i)    # noqa: E731
    for i in range(warm):
        comm(recv_f(i))
        acts.append(("F", i))
        comm(send_f(i))
    if steady > 0:
        comm(recv_f(warm))
    for j in range(steady):
        k = warm + j
        acts.append(("F", k))
        comm(send_f(k), recv_b(j))                      # one group: the next stage mirrors it
        acts.append(("B", j))
        if j < steady - 1:
            comm(send_b(j), recv_f(k + 1))              # one group: the previous stage mirrors it
        else:
            comm(send_b(j))
    for j in range(steady, M):
        comm(recv_b(j))
        acts.append(("B", j))
        comm(send_b(j))
    return acts


def simulate_schedule(world: int, micro_batches: int) -> dict:
    """Runs every stage's schedule against the others with rendezvous semantics (a group completes only
    when every operation in it has met its mirror operation on the peer, itself inside a posted group).
    Raises on a deadlock or a data hazard; returns the peak number of in-flight micro-batches per stage
    and the number of time slots the step took (forward = 1 slot, backward = 2)."""
    sched = [one_f_one_b_schedule(r, world, micro_batches) for r in range(world)]
    pc = [0] * world
    clock = [0.0] * world
    done_f = [set() for _ in range(world)]
    done_b = [set() for _ in range(world)]
    have_act = [set(range(micro_batches)) if r == 0 else set() for r in range(world)]
    have_grad = [set(range(micro_batches)) if r == world - 1 else set() for r in range(world)]
    inflight, peak = [0] * world, [0] * world

    def group_at(r):
        return sched[r][pc[r]][1] if pc[r] < len(sched[r]) and sched[r][pc[r]][0] == "comm" else None

    progressed = True
    while progressed:
        progressed = False
        for r in range(world):
            while pc[r] < len(sched[r]) and sched[r][pc[r]][0] in ("F", "B"):
                kind, i = sched[r][pc[r]]
                if kind == "F":
                    if i not in have_act[r]:
                        raise RuntimeError(f"stage {r} runs forward {i} without its input")
                    done_f[r].add(i)
                    inflight[r] += 1
                    peak[r] = max(peak[r], inflight[r])
                    clock[r] += 1
                else:
                    if i not in done_f[r] or i not in have_grad[r]:
                        raise RuntimeError(f"stage {r} runs backward {i} too early")
                    done_b[r].add(i)
                    inflight[r] -= 1
                    clock[r] += 2
                pc[r] += 1
                progressed = True
        for r in range(world):
            g = group_at(r)
            if g is None:
                continue
            peers = {op[1] for op in g}
            if len(peers) != 1:
                raise RuntimeError(f"stage {r}: a group talks to {len(peers)} neighbours; the schedule uses one per group")
            p = next(iter(peers))
            gp = group_at(p)
            mirror = sorted(("recv" if k == "send" else "send", r, w, i) for k, _q, w, i in g)
            if gp is None or sorted(gp) != mirror:
                continue                                  # the neighbour has not reached the matching group yet
            t = max(clock[r], clock[p])
            for q in (r, p):
                for kind, _peer, what, i in group_at(q):
                    if kind == "recv":
                        (have_act if what == "act" else have_grad)[q].add(i)
                    elif what == "act" and i not in done_f[q]:
                        raise RuntimeError(f"stage {q} sends activation {i} before computing it")
                    elif what == "grad" and i not in done_b[q]:
                        raise RuntimeError(f"stage {q} sends gradient {i} before computing it")
            for q in (r, p):
                clock[q] = t
                pc[q] += 1
            progressed = True
    stuck = [r for r in range(world) if pc[r] < len(sched[r])]
    if stuck:
        raise RuntimeError(f"pipeline schedule deadlocks: stages {stuck} at {[sched[r][pc[r]] for r in stuck]}")
    return {"peak_in_flight": peak, "slots": max(clock), "ideal_slots": 3.0 * micro_batches}


# ------------------------------------------------------------------------------- trainer --
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
        self.device = self.inner.device
        # one engine (= one set of activation buffers) per micro-batch that can be in flight on this stage
        slots = min(self.micro_batches, self.world - self.rank)
        self.engines = [self.inner.engine] + [self.stage_cfg.make_engine(self.inner.layout, self.inner.bufs.params, self.inner.bufs.grads, batch, seq)
                                              for _ in range(slots - 1)]
        self.engine = self.inner.engine
        self.schedule = one_f_one_b_schedule(self.rank, self.world, self.micro_batches)
        self._acc = (torch.zeros(self.inner.layout.n_total, dtype=torch.float32, device=self.device)
                     if self.micro_batches > 1 else None)

    @property
    def layout(self):
        return self.inner.layout

    def _accumulate(self, index: int) -> None:
        """index = how many micro-batches of this step have already been accumulated."""
        from ..ops import _lib
        k = self.micro_batches
        mode = 0 if index == 0 else (2 if index == k - 1 else 1)
        rc = _lib.load().nfn_grad_accumulate(ctypes.c_void_p(self._acc.data_ptr()), ctypes.c_void_p(self.inner.bufs.grads.data_ptr()),
                                             ctypes.c_longlong(self.layout.n_total), ctypes.c_int(mode), ctypes.c_float(1.0 / k),
                                             ctypes.c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "nfn_grad_accumulate")

    def _slot(self, i: int):
        return self.engines[i % len(self.engines)]

    def _comm(self, ops: list[tuple]) -> None:
        p2p = []
        for kind, peer, what, i in ops:
            eng = self._slot(i)
            if kind == "recv":
                buf = eng.x0 if what == "act" else eng.d_a
                p2p.append(dist.P2POp(dist.irecv, buf, peer))
            else:
                buf = eng.stage_output if what == "act" else eng.d_input
                p2p.append(dist.P2POp(dist.isend, buf, peer))
        for req in dist.batch_isend_irecv(p2p):
            req.wait()

    def train_step(self, tokens: list[torch.Tensor] | torch.Tensor, targets: list[torch.Tensor] | torch.Tensor) -> float:
        """One optimizer step. ``tokens`` / ``targets``: one tensor per micro-batch (or a single
        tensor). The first stage reads tokens, the last one targets; other stages ignore both.
        Returns the mean loss over the micro-batches (identical on every rank)."""
        toks = tokens if isinstance(tokens, (list, tuple)) else [tokens]
        tgts = targets if isinstance(targets, (list, tuple)) else [targets]
        if len(toks) != self.micro_batches or len(tgts) != self.micro_batches:
            raise ValueError(f"expected {self.micro_batches} micro-batches")
        total = torch.zeros(1, dtype=torch.float32, device=self.device)
        accumulated = 0
        for act in self.schedule:
            if act[0] == "comm":
                self._comm(act[1])
                continue
            kind, i = act
            eng = self._slot(i)
            if kind == "F":
                eng.set_batch(toks[i], tgts[i])
                eng.stage_output = eng.forward()
                if self.last:
                    total += eng.loss
            else:
                eng.backward()
                if self.micro_batches > 1:
                    self._accumulate(accumulated)
                    accumulated += 1
        opt = self.inner.opt
        opt.stage_hyper()
        # clip by the norm of the WHOLE model's gradient: every stage contributes its squared norm (one scalar all-reduce),
        # as the reference's pipeline step does (``muse_glimmer_native_train.cpp:2739-2808``: local norm^2 -> all-reduce -> clip)
        K = opt.K
        K.grad_clip_scale(opt.bufs.grads, opt.partial, opt.hyper, opt.clip)
        sq = opt.clip[1:2].double() ** 2
        dist.all_reduce(sq)
        norm = sq.sqrt().float()
        mx = opt.cfg.max_grad_norm
        opt.clip[1:2] = norm
        opt.clip[0:1] = torch.where(norm > mx, mx / (norm + 1e-6), torch.ones_like(norm)) if mx > 0 else torch.ones_like(norm)
        K.adamw_flat(opt.master, opt.m, opt.v, opt.bufs.grads, opt.bufs.params, opt.layout.n_decay, opt.hyper, opt.clip)
        opt.step_count += 1
        total /= self.micro_batches
        dist.broadcast(total, src=self.world - 1)
        return float(total.item())

    def save(self, out_dir, step: int | None = None) -> dict:
        from ..checkpoint.named import save_named_checkpoint
        return save_named_checkpoint(self.inner, Path(out_dir) / f"stage-{self.rank:05d}", step)

    def load(self, out_dir, step: int | None = None) -> dict:
        from ..checkpoint.named import load_named_checkpoint
        return load_named_checkpoint(self.inner, Path(out_dir) / f"stage-{self.rank:05d}", step)


# ----------------------------------------------------------------------------------- CLI --
def main(argv=None) -> int:
    """``python -m torch.distributed.run --nproc-per-node STAGES -m neuralfn_b200.parallel.pp --stages STAGES ...``
    (what ``nfn train --pipeline-parallel-size STAGES`` launches): Llama-family pipeline training on
    synthetic tokens or a token dataset; rank 0 prints one JSON report."""
    import argparse
    import os
    import time
    ap = argparse.ArgumentParser(prog="neuralfn_b200.parallel.pp")
    ap.add_argument("--stages", type=int, default=0)
    ap.add_argument("--base-model", default="llama", help="llama | muse-glimmer (engines with pipeline stage views)")
    ap.add_argument("--head-dim", type=int, default=0, help="muse-glimmer: attention head width (0: d_model / n_head)")
    ap.add_argument("--micro-batches", type=int, default=0, help="micro-batches per step (default: 2 x stages)")
    ap.add_argument("--dataset", default="")
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--max-steps", type=int, default=20)
    ap.add_argument("--learning-rate", type=float, default=3e-4)
    ap.add_argument("--n-layer", type=int, default=8)
    ap.add_argument("--n-head", type=int, default=8)
    ap.add_argument("--n-kv-head", type=int, default=0)
    ap.add_argument("--d-model", type=int, default=512)
    ap.add_argument("--d-ff", type=int, default=0)
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--seed", type=int, default=1337)
    ap.add_argument("--output-dir", default="")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if a.stages and a.stages != world:
        raise SystemExit(f"--stages {a.stages} needs exactly that many ranks (got {world})")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    from ..models.llama import LlamaConfig
    from .dp import AdamWConfig
    if a.base_model.lower().replace("_", "-") in ("muse-glimmer", "glimmer"):
        from ..models.glimmer import GlimmerConfig
        cfg = GlimmerConfig(n_layer=a.n_layer, n_head=a.n_head, n_kv_head=a.n_kv_head or a.n_head, head_dim=a.head_dim or a.d_model // a.n_head,
                            d_model=a.d_model, d_ff=a.d_ff or 3 * a.d_model, vocab_size=a.vocab_size, max_seq_len=a.seq_len,
                            window=min(2048, a.seq_len))
    else:
        cfg = LlamaConfig(n_layer=a.n_layer, n_head=a.n_head, n_kv_head=a.n_kv_head or a.n_head, d_model=a.d_model,
                          d_ff=a.d_ff or 4 * a.d_model, vocab_size=a.vocab_size, max_seq_len=a.seq_len)
    M = a.micro_batches or 2 * world
    tr = PipelineParallelTrainer(cfg, a.batch_size, a.seq_len, AdamWConfig(lr=a.learning_rate, warmup_steps=min(10, a.max_steps), total_steps=a.max_steps),
                                 micro_batches=M, seed=a.seed, device=dev)
    gen = torch.Generator().manual_seed(a.seed)
    sampler = None
    if a.dataset:
        from ..data.shards import TokenDataset
        sampler = TokenDataset(a.dataset, allow_train_as_val=True, require_validation=False).sampler("train", a.seq_len, a.batch_size)
    losses = []
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _step in range(a.max_steps):
        if sampler is not None:
            pairs = [sampler.next(wrap=True) for _ in range(M)]
            toks, tgts = [p[0] for p in pairs], [p[1] for p in pairs]
        else:
            toks = [torch.randint(0, a.vocab_size, (a.batch_size, a.seq_len), generator=gen, dtype=torch.int32) for _ in range(M)]
            tgts = [torch.roll(t, -1, 1) for t in toks]
        losses.append(tr.train_step(toks, tgts))
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    tr.inner.check_status()
    if a.output_dir:
        tr.save(a.output_dir, a.max_steps)
    if rank == 0:
        sim = simulate_schedule(world, M)
        print(json.dumps({"status": "ok", "model_family": a.base_model, "parallelism": f"pp{world}", "micro_batches": M, "steps": a.max_steps, "first_loss": losses[0],
                          "final_loss": losses[-1], "tokens_per_second": a.max_steps * M * a.batch_size * a.seq_len / wall,
                          "schedule": "1f1b", "bubble_fraction": round(1.0 - sim["ideal_slots"] / sim["slots"], 4),
                          "peak_in_flight": sim["peak_in_flight"]}))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
