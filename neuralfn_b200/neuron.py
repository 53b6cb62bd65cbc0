"""Neuron definitions: function, module and subgraph kinds.

A ``NeuronDef`` is a reusable node type. ``function`` neurons wrap a Python
callable whose source text travels with the graph JSON and is rebuilt on load;
``module`` neurons name a tensor stage (``module_type`` + ``module_config`` +
optional base64 ``module_state``) that only the tensor runtime can execute;
``subgraph`` neurons embed a whole ``NeuronGraph`` behind aliased ports.

Behavioural counterpart of the reference's ``neuralfn/neuron.py:20-294`` (same
JSON keys and 12-hex ids).
"""
from __future__ import annotations

import base64
import inspect
import io
import math
import textwrap
import uuid
from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Any, Callable, Optional, Sequence

from .port import Port

if TYPE_CHECKING:  # pragma: no cover
    from .graph import NeuronGraph

__all__ = [
    "NeuronDef", "neuron", "neuron_from_source", "module_neuron", "subgraph_neuron",
    "encode_module_state_dict", "decode_module_state_dict", "new_id",
]


def new_id() -> str:
    return uuid.uuid4().hex[:12]


def _compile_source(source: str, wanted: str, *, strict: bool) -> Callable[..., Any]:
    """Execute neuron source text and pick the callable named ``wanted``.

    The namespace offers ``math``, ``Port`` and a no-op ``neuron`` decorator so
    that decorated source round-trips. Graph files are code: load only trusted ones.
    """
    scope: dict[str, Any] = {"math": math, "Port": Port}
    scope["neuron"] = lambda *a, **k: (lambda fn: fn)
    before = set(scope)
    exec(source, scope)  # noqa: S102 - graph JSON carries executable neuron source by contract
    found = scope.get(wanted)
    if callable(found):
        return found
    fresh = [scope[k] for k in scope if k not in before and k != "__builtins__"
             and callable(scope[k]) and not isinstance(scope[k], type)]
    if fresh:
        return fresh[0]
    if strict:
        raise ValueError(f"No callable named '{wanted}' found in source")
    return lambda *args: 0.0


@dataclass
class NeuronDef:
    name: str
    fn: Optional[Callable[..., Any]]
    input_ports: list[Port]
    output_ports: list[Port]
    source_code: str = ""
    kind: str = "function"
    subgraph: Optional["NeuronGraph"] = None
    module_type: str = ""
    module_config: dict[str, Any] = field(default_factory=dict)
    module_state: str = ""
    input_aliases: list[str] = field(default_factory=list)
    output_aliases: list[str] = field(default_factory=list)
    variant_ref: Optional[dict[str, str]] = None
    id: str = field(default_factory=new_id)

    # -- evaluation -----------------------------------------------------------
    def raw_call(self, *args: float):
        """Evaluate without output conditioning (used by the gradient trainer)."""
        if self.kind == "subgraph":
            if self.subgraph is None:
                raise ValueError(f"Subgraph neuron '{self.name}' is missing a nested graph")
            return self.subgraph.execute_flat(tuple(float(a) for a in args))
        if self.kind == "module":
            raise TypeError(
                f"Module neuron '{self.name}' requires the torch runtime and cannot be called "
                "through scalar graph execution")
        if self.fn is None:
            raise ValueError(f"Function neuron '{self.name}' is missing a callable")
        return self.fn(*args)

    def __call__(self, *args: float) -> tuple[float, ...]:
        result = self.raw_call(*args)
        if not isinstance(result, (tuple, list)):
            result = (result,)
        return tuple(port.condition(float(v)) for v, port in zip(result, self.output_ports))

    def refresh_interface_ports(self) -> None:
        if self.kind != "subgraph" or self.subgraph is None:
            return
        self.input_ports = self.subgraph.flattened_input_ports(self.input_aliases or None)
        self.output_ports = self.subgraph.flattened_output_ports(self.output_aliases or None)
        self.input_aliases = [p.name for p in self.input_ports]
        self.output_aliases = [p.name for p in self.output_ports]

    @property
    def n_inputs(self) -> int:
        return len(self.input_ports)

    @property
    def n_outputs(self) -> int:
        return len(self.output_ports)

    # -- JSON -------------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        if self.kind == "subgraph":
            self.refresh_interface_ports()
        return {
            "id": self.id,
            "name": self.name,
            "kind": self.kind,
            "input_ports": [p.to_dict() for p in self.input_ports],
            "output_ports": [p.to_dict() for p in self.output_ports],
            "source_code": self.source_code,
            "subgraph": None if self.subgraph is None else self.subgraph.to_dict(),
            "module_type": self.module_type,
            "module_config": self.module_config,
            "module_state": self.module_state,
            "input_aliases": self.input_aliases,
            "output_aliases": self.output_aliases,
            "variant_ref": self.variant_ref,
        }

    @classmethod
    def from_dict(cls, payload: dict[str, Any]) -> "NeuronDef":
        kind = payload.get("kind", "function")
        if kind == "subgraph":
            ndef = cls.from_dict_raw(payload)
            if ndef.subgraph is not None:
                ndef.subgraph.validate(as_subgraph=True)
                ndef.refresh_interface_ports()
            return ndef
        ins = [Port.from_dict(p) for p in payload["input_ports"]]
        outs = [Port.from_dict(p) for p in payload["output_ports"]]
        if kind == "module":
            return module_neuron(
                name=payload["name"],
                module_type=payload.get("module_type", payload["name"]),
                input_ports=ins,
                output_ports=outs,
                module_config=payload.get("module_config") or {},
                module_state=payload.get("module_state", ""),
                neuron_id=payload.get("id"),
            )
        fn = _compile_source(payload["source_code"], payload["name"], strict=False)
        return cls(id=payload["id"], name=payload["name"], fn=fn, input_ports=ins,
                   output_ports=outs, source_code=payload["source_code"], kind=kind)

    @classmethod
    def from_dict_raw(cls, payload: dict[str, Any]) -> "NeuronDef":
        """Like ``from_dict`` but nested graphs are neither validated nor variant-resolved."""
        if payload.get("kind", "function") != "subgraph":
            return cls.from_dict(payload)
        from .graph import NeuronGraph

        sub_payload = payload.get("subgraph")
        sub = None if sub_payload is None else NeuronGraph.from_dict_raw(sub_payload)
        ins = [Port.from_dict(p) for p in payload.get("input_ports", [])]
        outs = [Port.from_dict(p) for p in payload.get("output_ports", [])]
        if sub is not None:
            if not ins:
                ins = sub.flattened_input_ports(payload.get("input_aliases") or None)
            if not outs:
                outs = sub.flattened_output_ports(payload.get("output_aliases") or None)
        ref = payload.get("variant_ref")
        return cls(
            id=payload.get("id") or new_id(), name=payload["name"], fn=None,
            input_ports=ins, output_ports=outs, source_code="", kind="subgraph", subgraph=sub,
            input_aliases=list(payload.get("input_aliases", [])),
            output_aliases=list(payload.get("output_aliases", [])),
            variant_ref=dict(ref) if ref else None,
        )


def neuron(inputs: Sequence[Port], outputs: Sequence[Port], *, name: str | None = None):
    """Decorator: turn a plain function into a ``function`` neuron definition."""

    def wrap(fn: Callable[..., Any]) -> NeuronDef:
        try:
            src = textwrap.dedent(inspect.getsource(fn))
        except (OSError, TypeError):
            src = ""
        return NeuronDef(name=name or fn.__name__, fn=fn, input_ports=list(inputs),
                         output_ports=list(outputs), source_code=src, kind="function")

    return wrap


def neuron_from_source(source_code: str, fn_name: str, input_ports: list[Port],
                       output_ports: list[Port], *, neuron_id: str | None = None) -> NeuronDef:
    fn = _compile_source(source_code, fn_name, strict=True)
    return NeuronDef(id=neuron_id or new_id(), name=fn_name, fn=fn, input_ports=input_ports,
                     output_ports=output_ports, source_code=source_code, kind="function")


def module_neuron(*, name: str, module_type: str, input_ports: list[Port],
                  output_ports: list[Port], module_config: dict[str, Any] | None = None,
                  module_state: str = "", neuron_id: str | None = None) -> NeuronDef:
    return NeuronDef(id=neuron_id or new_id(), name=name, fn=None, input_ports=input_ports,
                     output_ports=output_ports, source_code="", kind="module",
                     module_type=module_type, module_config=dict(module_config or {}),
                     module_state=module_state)


def subgraph_neuron(graph: "NeuronGraph", *, name: str, input_aliases: list[str] | None = None,
                    output_aliases: list[str] | None = None,
                    variant_ref: dict[str, str] | None = None,
                    neuron_id: str | None = None) -> NeuronDef:
    graph.validate(as_subgraph=True)
    ins = graph.flattened_input_ports(input_aliases)
    outs = graph.flattened_output_ports(output_aliases)
    return NeuronDef(id=neuron_id or new_id(), name=name, fn=None, input_ports=ins,
                     output_ports=outs, source_code="", kind="subgraph", subgraph=graph,
                     input_aliases=[p.name for p in ins], output_aliases=[p.name for p in outs],
                     variant_ref=dict(variant_ref) if variant_ref else None)


def encode_module_state_dict(state_dict: dict[str, Any]) -> str:
    """base64(torch.save(state_dict)) - the ``module_state`` wire format."""
    import torch

    buf = io.BytesIO()
    torch.save(state_dict, buf)
    return base64.b64encode(buf.getvalue()).decode("ascii")


def decode_module_state_dict(blob: str) -> dict[str, Any]:
    import torch

    if not blob:
        return {}
    return torch.load(io.BytesIO(base64.b64decode(blob.encode("ascii"))), map_location="cpu")
