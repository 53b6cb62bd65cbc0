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
        template_spec = dict(self.graph.torch_config.get("template_spec") or {})
        tensors = self._complete_semantic_inputs(tensors, compiled, template_spec)
        self._prepare_ema_targets(compiled)
        if c.activation_checkpointing and not c.evolutionary:
            compiled.enable_activation_checkpointing()
        device = self._device()
        amp_dtype, amp_name, use_amp = resolve_amp_settings(self.graph.torch_config.get("amp_dtype", c.amp_dtype)
                                                            if c.amp_dtype == "float32" else c.amp_dtype)
        use_amp = use_amp and device.type == "cuda"
        compiled.to(device)
        run: nn.Module = torch.compile(compiled) if (c.compile and not c.evolutionary) else compiled
        from . import evolution as evo
        layer_cfg = None if c.evolutionary else evo.layer_evo_config(template_spec)
        layer_params: list[Tensor] = []
        if layer_cfg is not None:
            layer_params = evo.layer_evo_parameters(compiled, layer_cfg["layer_index"])
            if not layer_params:
                raise ValueError(f"layer_evo_index={layer_cfg['layer_index']} matched no parameters; expected a transformer "
                                 f"block index in [0, {int(template_spec.get('num_layers', 0)) - 1}]")
            for p in layer_params:      # this block is trained by evolution only
                p.requires_grad_(False)
        route_cfg = None if c.evolutionary else evo.route_evo_config(template_spec)
        route_params = evo.route_evo_parameters(compiled) if route_cfg is not None else []
        optimizers = [] if c.evolutionary else self._build_optimizers(compiled)
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
        owner_of = self._shard_optimizer_state(optimizers, params, world) if (c.fsdp2_enabled and world > 1) else None
        start = time.perf_counter()
        autocast = lambda: torch.autocast(device_type=device.type, dtype=amp_dtype, enabled=use_amp)  # noqa: E731
        extract = lambda out: self._extract_scalar_loss(out, self.graph.name)  # noqa: E731
        population = None
        if c.evolutionary:
            if not params:
                raise ValueError("Evolutionary torch training requires at least one trainable parameter")
            population = evo.Population(torch.nn.utils.parameters_to_vector(params), evo.EvolutionSettings.from_train_config(c))
            self.graph.torch_config["evolutionary"] = population.s.as_dict()
        else:
            self.graph.torch_config.pop("evolutionary", None)
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
                macro: list[tuple[Tensor, ...]] = []
                for _a in range(accum):
                    idx = perm[cursor:cursor + c.batch_size]
                    if idx.numel() == 0 or (drop_last and idx.numel() < c.batch_size):
                        cursor = 0
                        idx = perm[:c.batch_size]
                    cursor += c.batch_size
                    macro.append(tuple(t[idx].to(device, non_blocking=True) for t in tensors))
                extra_info: dict[str, Any] = {}
                if population is not None:
                    # one generation: score every member on this step's batches, keep the best in the model
                    scored = [evo.evaluate_candidate(run, row, params, macro, extract=extract, autocast=autocast, routing=routing)
                              for row in population.members]
                    scores = torch.stack([sc[0] for sc in scored])
                    best = int(scores.argmin())
                    with torch.no_grad():
                        torch.nn.utils.vector_to_parameters(population.members[best].to(params[0].dtype), params)
                    step_rows = scored[best][1]
                    step_loss = scores[best] * step_rows
                    if scored[best][2]:
                        extra_info["routing_stats"] = scored[best][2]
                    population.next_generation(scores)
                    self._ema_update(compiled)
                    loss_total = float(step_loss.item())
                    total_loss += loss_total
                    total_rows += step_rows
                    self.global_step += 1
                    if on_step is not None:
                        on_step({"phase": "train", "optimization_method": "evolutionary", "step": self.global_step,
                                 "max_steps": int(total_steps), "epoch": epoch + 1, "max_epochs": c.epochs,
                                 "steps_per_epoch": steps_per_epoch, "loss": loss_total / max(step_rows, 1),
                                 "elapsed_seconds": time.perf_counter() - start, "grad_accum_steps": accum,
                                 "learning_rates": [], "population_size": population.s.population_size, **extra_info})
                    if c.max_wallclock_seconds > 0 and time.perf_counter() - start >= c.max_wallclock_seconds:
                        self._stop = True
                        break
                    continue
                for batch in macro:
                    with autocast():
                        loss = extract(run(*batch))
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
                if owner_of is not None:
                    self._broadcast_owned_params(params, owner_of, world)
                self._ema_update(compiled)
                stats_before_evo = [m.merged_routing_stats() for m in routing]
                if evo.evolution_interval_due(route_cfg, self.global_step) and route_params:
                    info_r = evo.partial_evolution_step(run, route_params, macro, extract=extract, autocast=autocast, routing=routing,
                                                        population=route_cfg["population"], mutation_scale=route_cfg["mutation_scale"],
                                                        seed=route_cfg["seed"], step=self.global_step)
                    if info_r is not None:
                        extra_info["route_evo"] = info_r
                if evo.evolution_interval_due(layer_cfg, self.global_step) and layer_params:
                    info_l = evo.partial_evolution_step(run, layer_params, macro, extract=extract, autocast=autocast, routing=routing,
                                                        population=layer_cfg["population"], mutation_scale=layer_cfg["mutation_scale"],
                                                        seed=layer_cfg["seed"], step=self.global_step)
                    if info_l is not None:
                        extra_info["layer_evo"] = {**info_l, "layer_index": int(layer_cfg["layer_index"])}
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
                    if any(stats_before_evo):
                        info["routing_stats"] = [s for s in stats_before_evo if s]
                    info.update(extra_info)
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

    # -------------------------------------------------------- EMA target encoders --
    @staticmethod
    def _ema_groups(compiled: nn.Module) -> list[tuple[list[Tensor], list[Tensor], list[tuple[Tensor, Tensor]], nn.Module]]:
        """For every ``target_encoder`` node: (target params, matching online params, buffer pairs).
        The online side is the sibling ``online_encoder`` when there is one; otherwise (the trunk is
        the online network) the sibling nodes that carry the same names as the target encoder's
        backbone nodes, and ``online_projector`` for its projector."""
        groups = []

        def visit(g: nn.Module) -> None:
            mods = getattr(g, "node_modules", None)
            if mods is None:
                return
            for child in mods.values():
                if isinstance(child, CompiledTorchGraph):
                    visit(child)
            if "target_encoder" not in mods:
                return
            target = mods["target_encoder"]
            if "online_encoder" in mods:
                online_p = dict(mods["online_encoder"].named_parameters())
                online_b = dict(mods["online_encoder"].named_buffers())
            else:
                online_p, online_b = {}, {}
                for name, mod in mods.items():
                    if name == "target_encoder":
                        continue
                    alias = {"online_projector": "node_modules.projector"}.get(name, f"node_modules.backbone.node_modules.{name}")
                    for k, v in mod.named_parameters():
                        online_p[f"{alias}.{k}"] = v
                    for k, v in mod.named_buffers():
                        online_b[f"{alias}.{k}"] = v
            tp, op, bufs = [], [], []
            for k, v in target.named_parameters():
                src = online_p.get(k)
                if src is not None and src.shape == v.shape:
                    tp.append(v)
                    op.append(src)
            for k, v in target.named_buffers():
                src = online_b.get(k)
                if src is not None and src.shape == v.shape:
                    bufs.append((v, src))
            groups.append((tp, op, bufs, target))

        visit(compiled)
        return groups

    def _prepare_ema_targets(self, compiled: nn.Module) -> None:
        """Target encoders start as copies of their online networks and never receive gradients."""
        self._ema = self._ema_groups(compiled)
        with torch.no_grad():
            for tp, op, bufs, target in self._ema:
                for t, o in zip(tp, op):
                    t.copy_(o)
                for t, o in bufs:
                    t.copy_(o)
                for p in target.parameters():
                    p.requires_grad_(False)

    def _ema_update(self, compiled: nn.Module) -> None:
        """target <- decay * target + (1 - decay) * online, as one multi-tensor lerp per encoder."""
        groups = getattr(self, "_ema", None)
        if not groups:
            return
        decay = float((self.graph.torch_config.get("template_spec") or {}).get("ema_decay", 0.99))
        with torch.no_grad():
            for tp, op, bufs, _target in groups:
                if tp:
                    torch._foreach_lerp_(tp, [o.detach() for o in op], 1.0 - decay)
                for t, o in bufs:
                    t.copy_(o)

    # ------------------------------------------------- semantic targets / sharding --
    @staticmethod
    def _complete_semantic_inputs(tensors: list[Tensor], compiled: CompiledTorchGraph, template_spec: dict) -> list[Tensor]:
        """Semantic objectives take a third input (one target topic per vocabulary dimension). When the
        caller passes only tokens and targets, derive it from the tokens through the token -> topic
        table (``semantic_table_path``; a deterministic synthetic table without one)."""
        names = [compiled.graph.nodes[n].neuron_def.output_ports[0].name for n in compiled.graph.input_node_ids]
        if len(tensors) + 1 == len(names) and names[-1] == "sem_targets":
            from .stages_semantic import SemanticTargetsFromTokensStage
            stage = SemanticTargetsFromTokensStage(int(template_spec.get("vocab_size", 0) or int(tensors[0].max()) + 1),
                                                   str(template_spec.get("semantic_vocab_ref", "")),
                                                   str(template_spec.get("semantic_table_path", "")),
                                                   2 ** min(int(template_spec.get("semantic_n_lsh_planes", 12)), 12))
            return list(tensors) + [stage(tensors[0])]
        return tensors

    @staticmethod
    def _shard_optimizer_state(optimizers: list[torch.optim.Optimizer], params: list[Tensor], world: int) -> dict[int, int]:
        """Optimizer-state sharding over the data-parallel group: every parameter tensor gets one
        owner rank (greedy by size); a rank keeps only its own parameters in its optimizers, so moment
        buffers exist once per group instead of once per rank. Returns ``id(param) -> owner``."""
        import torch.distributed as dist
        rank = dist.get_rank()
        load = [0] * world
        owner: dict[int, int] = {}
        for p in sorted(params, key=lambda t: -t.numel()):
            r = min(range(world), key=load.__getitem__)
            owner[id(p)] = r
            load[r] += p.numel()
        for o in optimizers:
            for g in o.param_groups:
                g["params"] = [p for p in g["params"] if owner.get(id(p), rank) == rank]
        return owner

    @staticmethod
    def _broadcast_owned_params(params: list[Tensor], owner: dict[int, int], world: int) -> None:
        import torch.distributed as dist
        for r in range(world):
            mine = [p for p in params if owner[id(p)] == r]
            if not mine:
                continue
            flat = torch.cat([p.detach().reshape(-1) for p in mine])
            dist.broadcast(flat, src=r)
            for p, chunk in zip(mine, flat.split([p.numel() for p in mine])):
                p.detach().copy_(chunk.view_as(p))
