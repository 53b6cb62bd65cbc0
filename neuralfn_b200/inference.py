"""Weight export/import for graph models, adapter checkpoints, int8 export and cached
generation over a compiled graph. Reference: ``neuralfn/inference.py:43-673``."""
from __future__ import annotations

from pathlib import Path
from typing import Any

import torch
from torch import Tensor

from .graph import NeuronGraph
from .tensor.compiler import CompiledTorchGraph
from .tensor.trainer import graph_topology_sha256

__all__ = ["export_to_pt", "import_from_pt", "load_pt_checkpoint", "save_adapter_checkpoint",
           "load_adapter_checkpoint", "merge_adapter_into_base", "export_quantized_pt",
           "load_quantized_pt", "InferenceCache", "graph_topology_sha256"]

PT_FORMAT = "neuralfn.graph_weights.v1"
ADAPTER_FORMAT = "neuralfn.adapter_weights.v1"
QUANT_FORMAT = "neuralfn.graph_weights_int8.v1"


def _compiled(model: NeuronGraph | CompiledTorchGraph) -> CompiledTorchGraph:
    return model if isinstance(model, CompiledTorchGraph) else CompiledTorchGraph(model)


def export_to_pt(model: NeuronGraph | CompiledTorchGraph, path: str | Path, metadata: dict[str, Any] | None = None) -> None:
    """``torch.save`` of {format, state_dict, metadata(graph_topology_sha256, ...)}."""
    cm = _compiled(model)
    meta = {"graph_topology_sha256": graph_topology_sha256(cm.graph), "graph_name": cm.graph.name}
    meta.update(metadata or {})
    torch.save({"format": PT_FORMAT, "state_dict": {k: v.detach().cpu() for k, v in cm.state_dict().items()},
                "metadata": meta}, path)


def load_pt_checkpoint(path: str | Path, map_location: Any = "cpu") -> tuple[dict[str, Tensor], dict[str, Any]]:
    payload = torch.load(path, map_location=map_location, weights_only=False)
    if isinstance(payload, dict) and "state_dict" in payload:
        return payload["state_dict"], dict(payload.get("metadata") or {})
    if isinstance(payload, dict):
        return payload, {}
    raise ValueError(f"{path} is not a weights checkpoint")


def import_from_pt(graph: NeuronGraph, path: str | Path, *, strict: bool = True) -> CompiledTorchGraph:
    """Compile ``graph`` and load weights; refuses weights saved for another topology."""
    state, meta = load_pt_checkpoint(path)
    digest = str(meta.get("graph_topology_sha256", ""))
    if digest and digest != graph_topology_sha256(graph):
        raise ValueError("checkpoint was saved for a different graph topology")
    cm = CompiledTorchGraph(graph)
    cm.load_state_dict(state, strict=strict)
    cm.sync_state_back()
    return cm


def _adapter_keys(cm: CompiledTorchGraph) -> list[str]:
    return [k for k in cm.state_dict() if ".lora_A" in k or ".lora_B" in k or k.endswith(".up")
            or "reward_head" in k or "value_head" in k]


def save_adapter_checkpoint(model: NeuronGraph | CompiledTorchGraph, path: str | Path,
                            metadata: dict[str, Any] | None = None) -> None:
    cm = _compiled(model)
    sd = cm.state_dict()
    keys = _adapter_keys(cm)
    if not keys:
        raise ValueError("graph has no adapter parameters")
    meta = {"graph_topology_sha256": graph_topology_sha256(cm.graph)}
    meta.update(metadata or {})
    torch.save({"format": ADAPTER_FORMAT, "state_dict": {k: sd[k].detach().cpu() for k in keys}, "metadata": meta}, path)


def load_adapter_checkpoint(model: CompiledTorchGraph, path: str | Path) -> list[str]:
    payload = torch.load(path, map_location="cpu", weights_only=False)
    if payload.get("format") != ADAPTER_FORMAT:
        raise ValueError("not an adapter checkpoint")
    digest = str((payload.get("metadata") or {}).get("graph_topology_sha256", ""))
    if digest and digest != graph_topology_sha256(model.graph):
        raise ValueError("adapter checkpoint was saved for a different graph topology")
    missing, unexpected = model.load_state_dict(payload["state_dict"], strict=False)
    if unexpected:
        raise ValueError(f"adapter checkpoint has unknown keys: {unexpected[:4]}")
    return sorted(payload["state_dict"])


def merge_adapter_into_base(model: CompiledTorchGraph) -> int:
    """Fold every LoRA update into its base weight and zero the adapter; returns layers merged."""
    n = 0
    with torch.no_grad():
        for mod in model.modules():
            if hasattr(mod, "lora_A") and hasattr(mod, "base"):
                mod.base.weight.add_(mod.scaling * (mod.lora_B @ mod.lora_A).to(mod.base.weight.dtype))
                mod.lora_B.zero_()
                n += 1
    return n


def export_quantized_pt(model: NeuronGraph | CompiledTorchGraph, path: str | Path) -> None:
    """int8 per-output-row symmetric quantisation of every 2-D weight; other tensors stay fp."""
    cm = _compiled(model)
    out: dict[str, Any] = {}
    for k, v in cm.state_dict().items():
        v = v.detach().cpu()
        if v.ndim == 2 and v.is_floating_point():
            scale = v.abs().amax(dim=1, keepdim=True).clamp(min=1e-8) / 127.0
            out[k] = {"q": torch.round(v / scale).clamp(-127, 127).to(torch.int8), "scale": scale.float()}
        else:
            out[k] = v
    torch.save({"format": QUANT_FORMAT, "state_dict": out,
                "metadata": {"graph_topology_sha256": graph_topology_sha256(cm.graph)}}, path)


def load_quantized_pt(graph: NeuronGraph, path: str | Path) -> CompiledTorchGraph:
    payload = torch.load(path, map_location="cpu", weights_only=False)
    if payload.get("format") != QUANT_FORMAT:
        raise ValueError("not an int8 graph-weights checkpoint")
    state = {k: (v["q"].float() * v["scale"] if isinstance(v, dict) else v) for k, v in payload["state_dict"].items()}
    cm = CompiledTorchGraph(graph)
    cm.load_state_dict(state)
    return cm


class InferenceCache:
    """Greedy / sampled generation over a compiled ``tokens -> logits`` graph. The graph is
    re-run on the growing window (graphs are opaque, so the cache keeps the token prefix and
    the last logits; resident engines in ``neuralfn_b200.inference_engine`` keep real KV)."""

    def __init__(self, model: CompiledTorchGraph, max_context: int = 1024) -> None:
        self.model, self.max_context = model, int(max_context)
        self.tokens: list[int] = []
        self.last_logits: Tensor | None = None

    def reset(self) -> None:
        self.tokens, self.last_logits = [], None

    @torch.no_grad()
    def prefill(self, tokens: list[int]) -> Tensor:
        self.tokens.extend(int(t) for t in tokens)
        window = self.tokens[-self.max_context:]
        dev = next(self.model.parameters()).device
        out = self.model(torch.tensor([window], device=dev))[0]
        self.last_logits = out[0, -1].float()
        return self.last_logits

    @torch.no_grad()
    def decode_one(self, temperature: float = 0.0, top_k: int = 0, generator: torch.Generator | None = None) -> int:
        if self.last_logits is None:
            raise RuntimeError("prefill first")
        logits = self.last_logits
        if temperature <= 0:
            tok = int(logits.argmax())
        else:
            logits = logits / temperature
            if top_k > 0:
                kth = torch.topk(logits, min(top_k, logits.numel())).values[-1]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            tok = int(torch.multinomial(torch.softmax(logits, -1).cpu(), 1, generator=generator))
        self.prefill([tok])
        return tok

    def generate(self, prompt: list[int], max_new_tokens: int, **kw) -> list[int]:
        self.reset()
        self.prefill(prompt)
        return [self.decode_one(**kw) for _ in range(max_new_tokens)]
