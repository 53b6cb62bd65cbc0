"""``TorchTrainer``: trains a graph of tensor stages (any preset, any objective).

Flow: compile graph -> fine-tune pre-hook (load base weights, freeze everything but
adapters) -> optimizers by profile (``adamw`` | ``split_muon``/``parameter_golf``) ->
optional resume (``neuralfn.torch_training.v1``) -> step loop with gradient accumulation
derived from ``train_batch_tokens``, bf16 autocast on CUDA, warm-up + cosine / warm-down
schedules, global-norm clipping, EMA targets for JEPA objectives, ``on_step`` telemetry
(loss, learning rates, routing stats) -> ``sync_state_back`` into the graph.
Reference: ``neuralfn/torch_backend.py:4323-4444,5250-5360,5717-6373``.

On a CUDA device the stages route to the sm_100a kernels through ``kernel_bridge``;
data parallelism wraps the same loop with the peer-memory gradient reduction of
``neuralfn_b200.parallel.dp`` when ``torch.distributed`` is initialised.
"""
from __future__ import annotations

import hashlib
import json
import math
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch
import torch.nn as nn
from torch import Tensor

from ..graph import NeuronGraph
from .compiler import CompiledTorchGraph

__all__ = ["TorchTrainConfig", "TorchTrainer", "Muon", "resolve_amp_settings", "graph_topology_sha256"]

TRAINING_CKPT_FORMAT = "neuralfn.torch_training.v1"


@dataclass
class TorchTrainConfig:
    learning_rate: float = 3e-4
    epochs: int = 50
    batch_size: int = 8
    weight_decay: float = 0.01
    beta1: float = 0.9
    beta2: float = 0.95
    adam_eps: float = 1e-8
    device: str = "cuda"
    amp_dtype: str = "float32"
    compile: bool = False
    activation_checkpointing: bool = False
    fsdp2_enabled: bool = False
    max_steps: int | None = None
    grad_clip_norm: float = 0.0
    optimizer_profile: str = "adamw"
    train_batch_tokens: int | None = None
    warmup_steps: int = 0
    warmdown_fraction: float = 0.75
    lr_decay_iters: int | None = None
    min_lr: float | None = None
    max_wallclock_seconds: float = 0.0
    embed_lr: float | None = None
    head_lr: float | None = None
    tied_embed_lr: float | None = None
    matrix_lr: float | None = None
    scalar_lr: float | None = None
    muon_momentum: float = 0.95
    muon_backend_steps: int = 5
    muon_momentum_warmup_start: float = 0.85
    muon_momentum_warmup_steps: int = 500
    drop_last: bool | None = None
    respect_epoch_boundaries: bool = False
    kernel_backend: str = "auto"
    tile_cuda_strict: bool = False
    tile_cuda_report_path: str | None = None
    evolutionary: bool = False
    evo_population_size: int = 50
    evo_mutation_rate: float = 0.1
    evo_mutation_scale: float = 0.3
    evo_crossover_rate: float = 0.5
    evo_tournament_size: int = 3
    evo_elite_count: int = 2
    evo_seed: int | None = None
    seed: int | None = None
    data_parallel: bool = True   # use torch.distributed (when initialised) to average gradients


def resolve_amp_settings(name: str | None) -> tuple[torch.dtype, str, bool]:
    n = str(name or "float32").strip().lower()
    if n in {"float16", "fp16", "half"}:
        return torch.float16, "float16", True
    if n in {"bfloat16", "bf16"}:
        return torch.bfloat16, "bfloat16", True
    if n in {"float32", "fp32", "full", "none"}:
        return torch.float32, "float32", False
    raise ValueError(f"Unsupported amp dtype: {name!r}")


def graph_topology_sha256(graph: NeuronGraph) -> str:
    """Digest of the graph structure (nodes, module types/configs, edges) without weights."""
    def strip(g: dict) -> dict:
        out = {"nodes": {}, "edges": sorted((e["src_node"], e["src_port"], e["dst_node"], e["dst_port"])
                                            for e in g.get("edges", {}).values()),
               "inputs": g.get("input_node_ids", []), "outputs": g.get("output_node_ids", [])}
        for nid, n in g.get("nodes", {}).items():
            nd = n["neuron_def"]
            out["nodes"][nid] = {"kind": nd.get("kind"), "name": nd.get("name"),
                                 "module_type": nd.get("module_type"), "module_config": nd.get("module_config"),
                                 "subgraph": strip(nd["subgraph"]) if nd.get("subgraph") else None}
        return out
    blob = json.dumps(strip(graph.to_dict()), sort_keys=True, separators=(",", ":")).encode()
    return hashlib.sha256(blob).hexdigest()


def _newton_schulz5(g: Tensor, steps: int = 5, eps: float = 1e-7) -> Tensor:
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.bfloat16()
    x = x / (x.norm() + eps)
    transposed = g.size(0) > g.size(1)
    if transposed:
        x = x.T
    for _ in range(steps):
        s = x @ x.T
        x = a * x + (b * s + c * s @ s) @ x
    return x.T if transposed else x


class Muon(torch.optim.Optimizer):
    """Momentum + Newton-Schulz orthogonalised updates for 2-D matrices."""

    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, backend_steps: int = 5,
                 nesterov: bool = True, weight_decay: float = 0.0) -> None:
        super().__init__(params, dict(lr=lr, momentum=momentum, backend_steps=backend_steps, nesterov=nesterov,
                                      weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                buf = self.state[p].setdefault("momentum_buffer", torch.zeros_like(g))
                buf.mul_(group["momentum"]).add_(g)
                upd = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                upd = _newton_schulz5(upd.reshape(upd.size(0), -1), group["backend_steps"]).reshape(p.shape)
                scale = max(1.0, p.size(0) / max(p[0].numel(), 1)) ** 0.5
                if group["weight_decay"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                p.add_(upd.to(p.dtype), alpha=-group["lr"] * scale)


class TorchTrainer:
    def __init__(self, graph: NeuronGraph, config: TorchTrainConfig | None = None) -> None:
        self.graph = graph
        self.config = config or TorchTrainConfig()
        self.loss_history: list[float] = []
        self.compiled: CompiledTorchGraph | None = None
        self.global_step = 0
        self._stop = False
        self._resume_state: dict | None = None

    def stop(self) -> None:
        self._stop = True

    # ------------------------------------------------------------------- helpers --
    def _device(self) -> torch.device:
        name = str(self.graph.torch_config.get("device", self.config.device or "cuda")).lower()
        if name.startswith("cuda") and not torch.cuda.is_available():
            raise RuntimeError("Torch training is configured for CUDA, but no CUDA device is available")
        return torch.device(name)

    @staticmethod
    def _extract_scalar_loss(outputs, graph_name: str) -> Tensor:
        out = outputs[0] if isinstance(outputs, (tuple, list)) else outputs
        if out.ndim != 0:
            out = out.mean()
        return out

    def _apply_finetune_prehook(self, compiled: CompiledTorchGraph) -> None:
        raw = self.graph.torch_config.get("finetune_spec") or {}
        base = str(raw.get("base_checkpoint", "") or "")
        if base:
            from ..inference import load_pt_checkpoint
            digest = str(raw.get("base_checkpoint_sha256", "") or "")
            if digest:
                got = hashlib.sha256(Path(base).read_bytes()).hexdigest()
                if got != digest:
                    raise ValueError("base checkpoint SHA-256 does not match the pinned digest")
            state, _meta = load_pt_checkpoint(base, map_location="cpu")
            own = compiled.state_dict()
            # adapter-wrapped projections keep the base weight under ".base.weight" / NF4 buffers
            remapped = {}
            for k, v in state.items():
                if k in own:
                    remapped[k] = v
                else:
                    alt = k.replace(".proj.weight", ".base.weight").replace(".proj.bias", ".base.bias")
                    if alt in own:
                        remapped[alt] = v
            compiled.load_state_dict(remapped, strict=False)
            for name, mod in compiled.named_modules():
                if hasattr(mod, "load_base_weight"):
                    key = f"{name}.proj.weight"
                    if key in state:
                        mod.load_base_weight(state[key])
        adapters = [m for m in compiled.modules() if hasattr(m, "lora_A")]
        if adapters:
            for p in compiled.parameters():
                p.requires_grad = False
            for m in adapters:
                m.lora_A.requires_grad = True
                m.lora_B.requires_grad = True
            for name, p in compiled.named_parameters():
                if "reward_head" in name or "value_head" in name or ".up" == name[-3:]:
                    p.requires_grad = True

    def _build_optimizers(self, module: nn.Module) -> list[torch.optim.Optimizer]:
        c = self.config
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("graph has no trainable parameters")
        if c.optimizer_profile in ("parameter_golf", "split_muon"):
            embed, head, matrix, scalar = [], [], [], []
            for name, p in module.named_parameters():
                if not p.requires_grad:
                    continue
                if "embedding" in name:
                    embed.append(p)
                elif "lm_head" in name or name.endswith("head.proj.weight"):
                    head.append(p)
                elif p.ndim == 2:
                    matrix.append(p)
                else:
                    scalar.append(p)
            lr = c.learning_rate
            opts: list[torch.optim.Optimizer] = []
            adam = dict(betas=(c.beta1, c.beta2), eps=c.adam_eps)
            if embed:
                opts.append(torch.optim.Adam(embed, lr=c.tied_embed_lr or c.embed_lr or lr, **adam))
            if head:
                opts.append(torch.optim.Adam(head, lr=c.head_lr or lr, **adam))
            if matrix:
                opts.append(Muon(matrix, lr=c.matrix_lr or lr, momentum=c.muon_momentum,
                                 backend_steps=c.muon_backend_steps))
            if scalar:
                opts.append(torch.optim.AdamW(scalar, lr=c.scalar_lr or lr, weight_decay=c.weight_decay, **adam))
            return opts
        return [torch.optim.AdamW(params, lr=c.learning_rate, betas=(c.beta1, c.beta2), eps=c.adam_eps,
                                  weight_decay=c.weight_decay)]

    def _lr_scale(self, step: int, total_steps: int) -> float:
        c = self.config
        if c.warmup_steps > 0 and step < c.warmup_steps:
            return (step + 1) / c.warmup_steps
        if c.lr_decay_iters:
            if step >= c.lr_decay_iters:
                return (c.min_lr or 0.0) / c.learning_rate
            t = (step - c.warmup_steps) / max(1, c.lr_decay_iters - c.warmup_steps)
            floor = (c.min_lr or 0.0) / c.learning_rate
            return floor + 0.5 * (1.0 - floor) * (1.0 + math.cos(math.pi * t))
        if c.max_steps and 0.0 < c.warmdown_fraction < 1.0 and total_steps > 0:
            start = int(total_steps * (1.0 - c.warmdown_fraction))
            if step >= start:
                return max(0.0, (total_steps - step) / max(1, total_steps - start))
        return 1.0

    # ---------------------------------------------------------------- checkpoints --
    def save_training_checkpoint(self, path: str | Path, optimizers: list[torch.optim.Optimizer] | None = None) -> None:
        if self.compiled is None:
            raise RuntimeError("nothing to save: train() has not compiled the graph yet")
        payload = {
            "format": TRAINING_CKPT_FORMAT, "graph_topology_sha256": graph_topology_sha256(self.graph),
            "state_dict": {k: v.detach().cpu() for k, v in self.compiled.state_dict().items()},
            "optimizer_states": [o.state_dict() for o in (optimizers or getattr(self, "_optimizers", []))],
            "global_step": self.global_step, "torch_rng_state": torch.get_rng_state(),
            "cuda_rng_state_all": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else [],
            "loss_history": list(self.loss_history)}
        tmp = Path(str(path) + ".tmp")
        torch.save(payload, tmp)
        tmp.replace(path)

    def load_training_checkpoint(self, path: str | Path) -> None:
        payload = torch.load(path, map_location="cpu", weights_only=False)
        if payload.get("format") != TRAINING_CKPT_FORMAT:
            raise ValueError(f"not a {TRAINING_CKPT_FORMAT} checkpoint")
        if payload.get("graph_topology_sha256") != graph_topology_sha256(self.graph):
            raise ValueError("training checkpoint was written for a different graph topology")
        self._resume_state = payload

    # ---------------------------------------------------------------------- train --
    def _as_batches(self, inputs, targets):
        if isinstance(inputs, dict):
            tensors = [torch.as_tensor(v) for v in inputs.values()]
        else:
            tensors = [torch.as_tensor(inputs)]
            if targets is not None:
                tensors.append(torch.as_tensor(targets))
        n = tensors[0].size(0)
        if any(t.size(0) != n for t in tensors):
            raise ValueError("all training tensors must share the leading (example) dimension")
        return tensors, n

    def train(self, train_inputs, train_targets=None, *, on_epoch: Callable[[int, float], None] | None = None,
              on_step: Callable[[dict[str, Any]], None] | None = None) -> list[float]:
        c = self.config
        if c.seed is not None:
            torch.manual_seed(c.seed)
        resume_path = str((self.graph.torch_config.get("finetune_spec") or {}).get("resume_checkpoint", "") or "")
        if resume_path and self._resume_state is None:
            self.load_training_checkpoint(resume_path)
        tensors, n_rows = self._as_batches(train_inputs, train_targets)
        compiled = CompiledTorchGraph(self.graph, kernel_backend=c.kernel_backend)
        self.compiled = compiled
        self._apply_finetune_prehook(compiled)
        device = self._device()
        amp_dtype, amp_name, use_amp = resolve_amp_settings(self.graph.torch_config.get("amp_dtype", c.amp_dtype)
                                                            if c.amp_dtype == "float32" else c.amp_dtype)
        use_amp = use_amp and device.type == "cuda"
        compiled.to(device)
        run: nn.Module = torch.compile(compiled) if c.compile else compiled
        optimizers = self._build_optimizers(compiled)
        self._optimizers = optimizers
        base_lrs = [[g["lr"] for g in o.param_groups] for o in optimizers]
        if self._resume_state is not None:
            compiled.load_state_dict(self._resume_state["state_dict"])
            for o, s in zip(optimizers, self._resume_state["optimizer_states"]):
                o.load_state_dict(s)
            self.global_step = int(self._resume_state["global_step"])
            self.loss_history = list(self._resume_state.get("loss_history", []))
            torch.set_rng_state(self._resume_state["torch_rng_state"])
        import torch.distributed as dist
        world = dist.get_world_size() if (c.data_parallel and dist.is_initialized()) else 1
        seq = tensors[0].size(1) if tensors[0].ndim > 1 else 1
        accum = 1
        if c.train_batch_tokens:
            accum = max(1, c.train_batch_tokens // max(1, c.batch_size * seq * world))
        drop_last = c.drop_last if c.drop_last is not None else n_rows >= c.batch_size
        micro_per_epoch = (n_rows // c.batch_size) if drop_last else math.ceil(n_rows / c.batch_size)
        micro_per_epoch = max(1, micro_per_epoch)
        steps_per_epoch = max(1, micro_per_epoch // accum)
        total_steps = c.max_steps or steps_per_epoch * c.epochs
        routing = compiled.routing_modules()
        params = [p for p in compiled.parameters() if p.requires_grad]
        start = time.perf_counter()
        gen = torch.Generator().manual_seed(int(c.seed if c.seed is not None else 0) + self.global_step)
        self._stop = False
        for epoch in range(c.epochs):
            if self._stop:
                break
            perm = torch.randperm(n_rows, generator=gen)
            cursor, total_loss, total_rows = 0, 0.0, 0
            for _ in range(steps_per_epoch):
                if self._stop or (c.max_steps is not None and self.global_step >= c.max_steps):
                    self._stop = True
                    break
                for o in optimizers:
                    o.zero_grad(set_to_none=True)
                for m in routing:
                    m.reset_routing_accum()
                step_loss, step_rows = torch.zeros((), device=device), 0
                for _a in range(accum):
                    idx = perm[cursor:cursor + c.batch_size]
                    if idx.numel() == 0 or (drop_last and idx.numel() < c.batch_size):
                        cursor = 0
                        idx = perm[:c.batch_size]
                    cursor += c.batch_size
                    batch = tuple(t[idx].to(device, non_blocking=True) for t in tensors)
                    with torch.autocast(device_type=device.type, dtype=amp_dtype, enabled=use_amp):
                        loss = self._extract_scalar_loss(run(*batch), self.graph.name)
                    (loss / accum).backward()
                    for m in routing:
                        m.add_to_routing_accum()
                    rows = int(batch[0].size(0))
                    step_rows += rows
                    step_loss += loss.detach().float() * rows
                if world > 1:
                    for p in params:
                        if p.grad is not None:
                            dist.all_reduce(p.grad)
                            p.grad.div_(world)
                scale = self._lr_scale(self.global_step, total_steps)
                for o, lrs in zip(optimizers, base_lrs):
                    for g, lr in zip(o.param_groups, lrs):
                        g["lr"] = lr * scale
                    if isinstance(o, Muon):
                        frac = min(1.0, self.global_step / max(1, c.muon_momentum_warmup_steps))
                        for g in o.param_groups:
                            g["momentum"] = (1 - frac) * c.muon_momentum_warmup_start + frac * c.muon_momentum
                if c.grad_clip_norm > 0:
                    torch.nn.utils.clip_grad_norm_(params, c.grad_clip_norm)
                for o in optimizers:
                    o.step()
                self._ema_update(compiled)
                loss_total = float(step_loss.item())
                total_loss += loss_total
                total_rows += step_rows
                self.global_step += 1
                if on_step is not None:
                    info = {"phase": "train", "optimization_method": "gradient", "step": self.global_step,
                            "max_steps": int(total_steps), "epoch": epoch + 1, "max_epochs": c.epochs,
                            "steps_per_epoch": steps_per_epoch, "loss": loss_total / max(step_rows, 1),
                            "elapsed_seconds": time.perf_counter() - start, "grad_accum_steps": accum,
                            "learning_rates": [g["lr"] for o in optimizers for g in o.param_groups]}
                    stats = [m.merged_routing_stats() for m in routing]
                    if any(stats):
                        info["routing_stats"] = [s for s in stats if s]
                    on_step(info)
                if c.max_wallclock_seconds > 0 and time.perf_counter() - start >= c.max_wallclock_seconds:
                    self._stop = True
                    break
            avg = total_loss / max(total_rows, 1)
            if total_rows:
                self.loss_history.append(avg)
                if on_epoch is not None:
                    on_epoch(epoch, avg)
        compiled.sync_state_back()
        return self.loss_history

    def _ema_update(self, compiled: nn.Module) -> None:
        spec = (self.graph.torch_config.get("template_spec") or {})
        objective = str((spec.get("template") or {}).get("objective", "ar"))
        if "jepa" not in objective:
            return
        decay = float(spec.get("ema_decay", 0.99))
        targets = getattr(compiled, "_ema_pairs", None)
        if not targets:
            return
        with torch.no_grad():
            for tgt, src in targets:
                tgt.mul_(decay).add_(src.detach(), alpha=1 - decay)
