"""Catalog of built-in scalar neurons with analytic partial derivatives.

Each entry is declared once as (name, input names, output names, source text,
partial-derivative function). The source text is what travels in graph JSON; the
derivative is used by the exact-gradient edge trainer (``neuralfn_b200.sgd``).
Function names and formulas follow the reference catalog
(``neuralfn/builtins.py:175-440``); ports are unbounded unless the dtype is a
token/bool type (``:159-172``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Sequence

from .neuron import NeuronDef, neuron_from_source
from .port import Port

SELU_ALPHA = 1.6732632423543772
SELU_LAMBDA = 1.0507009873554805


@dataclass(frozen=True)
class ScalarSpec:
    name: str              # neuron name in graphs
    fn_name: str           # python function name inside ``source``
    inputs: tuple[str, ...]
    outputs: tuple[str, ...]
    source: str
    # jacobian(inputs) -> rows of d out_i / d in_j
    jacobian: Callable[..., Sequence[Sequence[float]]]
    out_port: Port | None = None


def _sig(x: float) -> float:
    if x >= 0:
        return 1.0 / (1.0 + math.exp(-x))
    e = math.exp(x)
    return e / (1.0 + e)


def _unary(name, body, deriv, *, fn_name=None, out_port=None, prelude=""):
    fn_name = fn_name or name
    src = f"{prelude}def {fn_name}(x):\n{body}\n"
    return ScalarSpec(name, fn_name, ("x",), ("y",), src, lambda x: ((deriv(x),),), out_port)


def _softplus_d(x):
    return _sig(x)


def _mish_d(x):
    sp = math.log1p(math.exp(x)) if x < 30 else x
    t = math.tanh(sp)
    return t + x * (1 - t * t) * _sig(x)


def _gelu_d(x):
    cdf = 0.5 * (1.0 + math.erf(x / math.sqrt(2.0)))
    pdf = math.exp(-0.5 * x * x) / math.sqrt(2.0 * math.pi)
    return cdf + x * pdf


def _softmax2_jac(a, b):
    m = max(a, b)
    ea, eb = math.exp(a - m), math.exp(b - m)
    pa, pb = ea / (ea + eb), eb / (ea + eb)
    return ((pa * (1 - pa), -pa * pb), (-pa * pb, pb * (1 - pb)))


def _logsoftmax2_jac(a, b):
    m = max(a, b)
    ea, eb = math.exp(a - m), math.exp(b - m)
    pa, pb = ea / (ea + eb), eb / (ea + eb)
    return ((1 - pa, -pb), (-pa, 1 - pb))


SPECS: tuple[ScalarSpec, ...] = (
    _unary("sigmoid", "    return 1.0 / (1.0 + math.exp(-x))", lambda x: _sig(x) * (1 - _sig(x))),
    _unary("relu", "    return max(0.0, x)", lambda x: 1.0 if x > 0 else 0.0),
    _unary("tanh_neuron", "    return math.tanh(x)", lambda x: 1 - math.tanh(x) ** 2),
    _unary("threshold", "    return 1.0 if x >= 0.0 else 0.0", lambda x: 0.0,
           out_port=Port("y", range=(0, 1), precision=1.0, dtype="bool")),
    _unary("identity", "    return x", lambda x: 1.0),
    _unary("negate", "    return -x", lambda x: -1.0),
    ScalarSpec("add", "add", ("a", "b"), ("sum",), "def add(a, b):\n    return a + b\n",
               lambda a, b: ((1.0, 1.0),)),
    ScalarSpec("multiply", "multiply", ("a", "b"), ("product",),
               "def multiply(a, b):\n    return a * b\n", lambda a, b: ((b, a),)),
    _unary("gaussian", "    return math.exp(-x * x)", lambda x: -2 * x * math.exp(-x * x)),
    _unary("log", "    return math.log(max(x, 1e-7))", lambda x: 1.0 / x if x > 1e-7 else 0.0,
           fn_name="log_neuron"),
    _unary("leaky_relu", "    return x if x >= 0.0 else 0.01 * x", lambda x: 1.0 if x >= 0 else 0.01),
    _unary("prelu", "    return x if x >= 0.0 else 0.25 * x", lambda x: 1.0 if x >= 0 else 0.25),
    _unary("relu6", "    return min(max(0.0, x), 6.0)", lambda x: 1.0 if 0 < x < 6 else 0.0),
    _unary("elu", "    return x if x >= 0.0 else math.exp(x) - 1.0",
           lambda x: 1.0 if x >= 0 else math.exp(x)),
    _unary("selu",
           "    return _SELU_LAMBDA * (x if x >= 0.0 else _SELU_ALPHA * (math.exp(x) - 1.0))",
           lambda x: SELU_LAMBDA * (1.0 if x >= 0 else SELU_ALPHA * math.exp(x)),
           prelude=f"_SELU_ALPHA = {SELU_ALPHA!r}\n_SELU_LAMBDA = {SELU_LAMBDA!r}\n\n\n"),
    _unary("gelu", "    return x * 0.5 * (1.0 + math.erf(x / math.sqrt(2.0)))", _gelu_d),
    _unary("silu", "    return x / (1.0 + math.exp(-x))",
           lambda x: _sig(x) * (1 + x * (1 - _sig(x)))),
    _unary("mish", "    sp = math.log(1.0 + math.exp(x))\n    return x * math.tanh(sp)", _mish_d),
    _unary("softplus", "    return math.log(1.0 + math.exp(x))", _softplus_d),
    _unary("softsign", "    return x / (1.0 + abs(x))", lambda x: 1.0 / (1.0 + abs(x)) ** 2),
    _unary("hard_sigmoid", "    return max(0.0, min(1.0, x / 6.0 + 0.5))",
           lambda x: 1.0 / 6.0 if -3 < x < 3 else 0.0),
    _unary("hard_tanh", "    return max(-1.0, min(1.0, x))", lambda x: 1.0 if -1 < x < 1 else 0.0),
    _unary("hard_swish", "    return x * max(0.0, min(1.0, x / 6.0 + 0.5))",
           lambda x: 0.0 if x <= -3 else (1.0 if x >= 3 else x / 3.0 + 0.5)),
    ScalarSpec("softmax_2", "softmax_2", ("a", "b"), ("pa", "pb"),
               "def softmax_2(a, b):\n    m = max(a, b)\n    ea = math.exp(a - m)\n"
               "    eb = math.exp(b - m)\n    s = ea + eb\n    return ea / s, eb / s\n",
               _softmax2_jac),
    ScalarSpec("logsoftmax_2", "logsoftmax_2", ("a", "b"), ("la", "lb"),
               "def logsoftmax_2(a, b):\n    m = max(a, b)\n"
               "    lse = m + math.log(math.exp(a - m) + math.exp(b - m))\n"
               "    return a - lse, b - lse\n", _logsoftmax2_jac),
    _unary("input", "    return x", lambda x: 1.0, fn_name="input_node"),
    _unary("output", "    return x", lambda x: 1.0, fn_name="output_node"),
)

SPEC_BY_NAME: dict[str, ScalarSpec] = {s.name: s for s in SPECS}
# a function neuron loaded from JSON carries the python function name for some entries
SPEC_BY_FN: dict[str, ScalarSpec] = {s.fn_name: s for s in SPECS}


def _port(name: str, spec_port: Port | None = None) -> Port:
    if spec_port is not None and spec_port.dtype in {"tokens", "bool"}:
        return Port(name=spec_port.name, range=spec_port.range, precision=spec_port.precision,
                    dtype=spec_port.dtype)
    return Port(name)


def make_builtin(name: str) -> NeuronDef:
    """A fresh ``NeuronDef`` (new id) of the named built-in scalar function."""
    spec = SPEC_BY_NAME[name]
    ins = [_port(n) for n in spec.inputs]
    if spec.out_port is not None:
        outs = [_port(spec.out_port.name, spec.out_port)]
    else:
        outs = [_port(n) for n in spec.outputs]
    nd = neuron_from_source(spec.source, spec.fn_name, ins, outs)
    nd.name = spec.name
    return nd


def jacobian_for(ndef: NeuronDef) -> Callable[..., Sequence[Sequence[float]]] | None:
    """Analytic Jacobian for a function neuron if it is a known built-in whose stored
    source matches the catalog; ``None`` otherwise (callers fall back to central
    differences)."""
    spec = SPEC_BY_NAME.get(ndef.name) or SPEC_BY_FN.get(ndef.name)
    if spec is None or ndef.kind != "function":
        return None
    body = lambda s: [ln.strip() for ln in s.strip().splitlines()  # noqa: E731
                      if ln.strip() and not ln.strip().startswith(("@", "inputs=", "outputs=", "name=", ")", "#"))]
    have = body(ndef.source_code)
    want = body(spec.source)
    # tolerate a decorator header in stored source: compare the trailing function text
    if have[-len(want):] != want and have:
        tail = [ln for ln in have if not ln.startswith("_SELU")]
        ref_tail = [ln for ln in want if not ln.startswith("_SELU")]
        if tail[-len(ref_tail):] != ref_tail:
            return None
    return spec.jacobian
