"""Gradient-free optimisation of graph parameters: whole-model evolutionary training and the partial
"route evolution" / "layer evolution" steps that interleave with gradient training.

Behaviour follows the reference trainer (``neuralfn/torch_backend.py:5435-5720`` operators and
partial evolution, ``:5995-6140`` the generation loop): a population of flat parameter vectors whose
first member is the current model; each generation every member is scored by the graph's loss on the
step's batches, the best one is written into the model, ``elite_count`` best survive unchanged and the
rest are bred by tournament selection, uniform crossover and sparse Gaussian mutation.

The layout differs. The population is one ``[P, N]`` tensor on the training device, and selection,
crossover and mutation of a whole generation are a handful of batched tensor operations driven by a
device ``torch.Generator``: no per-candidate host round trip, no numpy, and the only synchronisation
per generation is reading the ``P`` losses.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Sequence

import torch
from torch import Tensor
from torch.nn.utils import parameters_to_vector, vector_to_parameters

__all__ = ["EvolutionSettings", "Population", "evaluate_candidate", "partial_evolution_step", "route_evo_config",
           "layer_evo_config", "layer_evo_parameters", "route_evo_parameters", "validate_evolution_settings"]


@dataclass
class EvolutionSettings:
    population_size: int = 50
    mutation_rate: float = 0.1
    mutation_scale: float = 0.3
    crossover_rate: float = 0.5
    tournament_size: int = 3
    elite_count: int = 2
    seed: int | None = None

    @classmethod
    def from_train_config(cls, c: Any) -> "EvolutionSettings":
        return cls(int(c.evo_population_size), float(c.evo_mutation_rate), float(c.evo_mutation_scale),
                   float(c.evo_crossover_rate), int(c.evo_tournament_size), int(c.evo_elite_count), c.evo_seed)

    def as_dict(self) -> dict[str, Any]:
        return {"population_size": self.population_size, "mutation_rate": self.mutation_rate,
                "mutation_scale": self.mutation_scale, "crossover_rate": self.crossover_rate,
                "tournament_size": self.tournament_size, "elite_count": self.elite_count, "seed": self.seed}


def validate_evolution_settings(s: EvolutionSettings) -> None:
    if s.population_size <= 0:
        raise ValueError("Evolutionary torch training requires evo_population_size >= 1")
    if s.tournament_size <= 0:
        raise ValueError("Evolutionary torch training requires evo_tournament_size >= 1")
    if s.elite_count < 0:
        raise ValueError("Evolutionary torch training requires evo_elite_count >= 0")
    if s.elite_count > s.population_size:
        raise ValueError("Evolutionary torch training requires evo_elite_count <= evo_population_size")
    if s.mutation_rate < 0.0:
        raise ValueError("Evolutionary torch training requires evo_mutation_rate >= 0")
    if s.mutation_scale < 0.0:
        raise ValueError("Evolutionary torch training requires evo_mutation_scale >= 0")
    if not 0.0 <= s.crossover_rate <= 1.0:
        raise ValueError("Evolutionary torch training requires 0 <= evo_crossover_rate <= 1")


class Population:
    """``members[0]`` starts as the base vector; the others are forced mutations of it."""

    def __init__(self, base: Tensor, settings: EvolutionSettings) -> None:
        validate_evolution_settings(settings)
        self.s = settings
        self.gen = torch.Generator(device=base.device)
        self.gen.manual_seed(int(settings.seed) if settings.seed is not None else int(torch.seed() % (2 ** 31)))
        base = base.detach().clone()
        p, n = settings.population_size, base.numel()
        self.members = base.unsqueeze(0).repeat(p, 1)
        if p > 1:
            self.members[1:] = self._mutate(self.members[1:], force=True)

    # -- operators on a block of rows -------------------------------------------------
    def _mutate(self, rows: Tensor, force: bool = False) -> Tensor:
        s = self.s
        n = rows.size(1)
        if n == 0 or s.mutation_scale == 0.0:
            return rows
        rate = s.mutation_rate
        if force and rate <= 0.0:
            rate = 1.0 / max(n, 1)
        if rate <= 0.0:
            return rows
        mask = torch.rand(rows.shape, generator=self.gen, device=rows.device) < rate
        if force:
            # every forced mutant changes in at least one coordinate
            empty = ~mask.any(dim=1)
            pick = torch.randint(0, n, (rows.size(0),), generator=self.gen, device=rows.device)
            mask[torch.arange(rows.size(0), device=rows.device)[empty], pick[empty]] = True
        noise = torch.randn(rows.shape, generator=self.gen, device=rows.device, dtype=rows.dtype) * s.mutation_scale
        return torch.where(mask, rows + noise, rows)

    def _tournament(self, scores: Tensor, count: int) -> Tensor:
        p = scores.numel()
        size = min(max(self.s.tournament_size, 1), p)
        # `size` distinct entrants per tournament: the first columns of a random permutation
        entrants = torch.rand(count, p, generator=self.gen, device=scores.device).argsort(dim=1)[:, :size]
        best = scores[entrants].argmin(dim=1)
        return entrants.gather(1, best.unsqueeze(1)).squeeze(1)

    def next_generation(self, scores: Sequence[float] | Tensor) -> None:
        s = self.s
        sc = torch.as_tensor(scores, dtype=torch.float32, device=self.members.device)
        sc = torch.where(torch.isfinite(sc), sc, torch.full_like(sc, float("inf")))
        order = sc.argsort()
        elites = self.members[order[:min(s.elite_count, s.population_size)]].clone()
        n_children = s.population_size - elites.size(0)
        if n_children <= 0:
            self.members = elites
            return
        pa = self.members[self._tournament(sc, n_children)]
        pb = self.members[self._tournament(sc, n_children)]
        if s.crossover_rate > 0.0:
            take_b = torch.rand(pa.shape, generator=self.gen, device=pa.device) < s.crossover_rate
            pa = torch.where(take_b, pb, pa)
        self.members = torch.cat([elites, self._mutate(pa)], dim=0)


@torch.no_grad()
def evaluate_candidate(run: Callable[..., tuple[Tensor, ...]], vector: Tensor, params: list[Tensor],
                       batches: list[tuple[Tensor, ...]], *, extract: Callable[[tuple[Tensor, ...]], Tensor],
                       autocast: Callable[[], Any], routing: Sequence[Any] = ()) -> tuple[Tensor, int, list[dict]]:
    """Loads ``vector`` into ``params`` and returns (row-weighted mean loss as a 0-d device tensor,
    rows, routing stats). Non-finite losses score as +inf."""
    if not params:
        raise ValueError("Evolutionary torch training requires at least one trainable parameter")
    vector_to_parameters(vector.to(device=params[0].device, dtype=params[0].dtype), params)
    total = torch.zeros((), device=params[0].device)
    rows = 0
    for m in routing:
        m.reset_routing_accum()
    for flat in batches:
        with autocast():
            loss = extract(run(*flat))
        n = int(flat[0].size(0))
        total += loss.float() * n
        rows += n
        for m in routing:
            m.add_to_routing_accum()
    mean = total / max(rows, 1)
    mean = torch.where(torch.isfinite(mean), mean, torch.full_like(mean, float("inf")))
    return mean, rows, [s for s in (m.merged_routing_stats() for m in routing) if s]


def partial_evolution_step(run, params: list[Tensor], batches, *, extract, autocast, routing=(), population: int = 8,
                           mutation_scale: float = 0.05, seed: int | None = None, step: int = 0) -> dict[str, Any] | None:
    """One (1 + lambda) step over a parameter subset: the current values and ``population - 1`` dense
    Gaussian perturbations are scored on ``batches``; the best is kept."""
    if not params or not batches:
        return None
    base = parameters_to_vector(params).detach()
    gen = torch.Generator(device=base.device)
    gen.manual_seed((int(seed) + int(step)) if seed is not None else int(torch.seed() % (2 ** 31)))
    noise = torch.randn(max(population - 1, 0), base.numel(), generator=gen, device=base.device, dtype=base.dtype)
    candidates = torch.cat([base.unsqueeze(0), base.unsqueeze(0) + noise * mutation_scale], dim=0)
    losses, stats = [], []
    for row in candidates:
        loss, _rows, st = evaluate_candidate(run, row, params, batches, extract=extract, autocast=autocast, routing=routing)
        losses.append(loss)
        stats.append(st)
    scores = torch.stack(losses)
    best = int(scores.argmin())
    with torch.no_grad():
        vector_to_parameters(candidates[best], params)
    return {"candidate_count": int(candidates.size(0)), "best_loss": float(scores[best]), "best_index": best,
            "mutation_scale": float(mutation_scale), "routing_stats": stats[best] or None}


def _interval_config(enabled: bool, fraction: float, population: int, scale: float, seed: Any) -> dict[str, Any] | None:
    if not enabled or fraction <= 0.0:
        return None
    fraction = min(float(fraction), 1.0)
    return {"fraction": fraction, "interval": max(1, int(round(1.0 / fraction))), "population": max(1, int(population)),
            "mutation_scale": max(0.0, float(scale)), "seed": None if seed in (None, "") else int(seed)}


def route_evo_config(template_spec: dict[str, Any]) -> dict[str, Any] | None:
    """Settings of route evolution: only the ``semantic_moe_jepa_evo`` objective has it; every
    ``1 / fraction``-th optimizer step is followed by one evolution step over the router parameters."""
    if str((template_spec.get("template") or {}).get("objective", "ar")) != "semantic_moe_jepa_evo":
        return None
    return _interval_config(bool(template_spec.get("route_evo_enabled", True)), float(template_spec.get("route_evo_fraction", 0.10)),
                            int(template_spec.get("route_evo_population", 8)), float(template_spec.get("route_evo_mutation_scale", 0.05)),
                            template_spec.get("route_evo_seed"))


def layer_evo_config(template_spec: dict[str, Any]) -> dict[str, Any] | None:
    cfg = _interval_config(bool(template_spec.get("layer_evo_enabled", False)), float(template_spec.get("layer_evo_fraction", 0.10)),
                           int(template_spec.get("layer_evo_population", 8)), float(template_spec.get("layer_evo_mutation_scale", 0.02)),
                           template_spec.get("layer_evo_seed"))
    if cfg is None:
        return None
    index = template_spec.get("layer_evo_index")
    cfg["layer_index"] = int(template_spec.get("num_layers", 0)) // 2 if index in (None, "") else int(index)
    return cfg


def layer_evo_parameters(compiled: torch.nn.Module, layer_index: int) -> list[Tensor]:
    """Parameters of decoder block ``layer_index`` of the main trunk (node id ``block_<i>``)."""
    needle = f"node_modules.block_{int(layer_index)}."
    out, seen = [], set()
    for name, p in compiled.named_parameters():
        if needle in name and id(p) not in seen:
            seen.add(id(p))
            out.append(p)
    return out


def route_evo_parameters(compiled: torch.nn.Module) -> list[Tensor]:
    out, seen = [], set()
    for m in compiled.modules():
        fn = getattr(m, "route_evo_parameters", None)
        if fn is None:
            continue
        for p in fn():
            if id(p) not in seen:
                seen.add(id(p))
                out.append(p)
    return out


def evolution_interval_due(cfg: dict[str, Any] | None, global_step: int) -> bool:
    return cfg is not None and (global_step + 1) % int(cfg["interval"]) == 0
