"""Scalar graph runtime: execution semantics, JSON round trip, XOR by exact-gradient SGD."""
import json
import math
import random

import pytest

from neuralfn_b200.graph import Edge, NeuronGraph, NeuronInstance
from neuralfn_b200.neuron import neuron, subgraph_neuron
from neuralfn_b200.port import Port
from neuralfn_b200.scalar_builtins import SPECS, make_builtin
from neuralfn_b200.serialization import graph_from_json, graph_to_json, load_graph, save_graph
from neuralfn_b200.sgd import GraphSGDTrainer, SGDConfig, init_edge_params_normal

XOR_X = [(0.0, 0.0), (0.0, 1.0), (1.0, 0.0), (1.0, 1.0)]
XOR_Y = [(0.0,), (1.0,), (1.0,), (0.0,)]


def build_xor(hidden: int = 4) -> NeuronGraph:
    g = NeuronGraph(name="xor")
    ins = [NeuronInstance(make_builtin("input"), instance_id=f"in{i}") for i in range(2)]
    hid = [NeuronInstance(make_builtin("sigmoid"), instance_id=f"h{i}") for i in range(hidden)]
    out = NeuronInstance(make_builtin("sigmoid"), instance_id="out")
    for n in (*ins, *hid, out):
        g.add_node(n)
    k = 0
    for i in ins:
        for h in hid:
            g.add_edge(Edge(id=f"e{k:03d}", src_node=i.instance_id, dst_node=h.instance_id))
            k += 1
    for h in hid:
        g.add_edge(Edge(id=f"e{k:03d}", src_node=h.instance_id, dst_node="out"))
        k += 1
    g.input_node_ids = [n.instance_id for n in ins]
    g.output_node_ids = ["out"]
    return g


def test_port_condition():
    p = Port("x", range=(-1.0, 1.0), precision=0.25)
    assert p.condition(3.0) == 1.0
    assert p.condition(0.3) == 0.25
    assert Port("y").condition(1.2345) == 1.2345
    with pytest.raises(ValueError):
        Port("bad", range=(1.0, 1.0))
    assert Port.from_dict(p.to_dict()) == p


def test_builtin_catalog_matches_formulas():
    assert len(SPECS) == 27
    for spec in SPECS:
        nd = make_builtin(spec.name)
        args = [0.3 * (i + 1) for i in range(len(spec.inputs))]
        out = nd(*args)
        assert len(out) == len(nd.output_ports)
        # analytic jacobian vs central differences
        jac = spec.jacobian(*args)
        if spec.name == "threshold":
            continue
        for j in range(len(args)):
            hi, lo = list(args), list(args)
            hi[j] += 1e-6
            lo[j] -= 1e-6
            yh, yl = nd.raw_call(*hi), nd.raw_call(*lo)
            if not isinstance(yh, tuple):
                yh, yl = (yh,), (yl,)
            for i in range(len(yh)):
                assert abs((yh[i] - yl[i]) / 2e-6 - jac[i][j]) < 1e-5, spec.name


def test_dag_execution_and_edge_transform():
    g = build_xor()
    init_edge_params_normal(g, seed=3)
    out = g.execute({"in0": (1.0,), "in1": (0.0,)})
    # manual evaluation
    sig = lambda v: 1 / (1 + math.exp(-v))  # noqa: E731
    hs = []
    for h in range(4):
        acc = 0.0
        for e in g.edges.values():
            if e.dst_node == f"h{h}":
                acc += (1.0 if e.src_node == "in0" else 0.0) * e.weight + e.bias
        hs.append(sig(acc))
    acc = sum(hs[int(e.src_node[1:])] * e.weight + e.bias for e in g.edges.values() if e.dst_node == "out")
    assert out["out"][0] == pytest.approx(sig(acc), abs=1e-15)
    trace = g.execute_trace({"in0": (1.0,), "in1": (0.0,)})
    assert set(trace) == set(g.nodes)


def test_cyclic_settling():
    g = NeuronGraph(name="loop")
    a = NeuronInstance(make_builtin("input"), instance_id="a")
    b = NeuronInstance(make_builtin("tanh_neuron"), instance_id="b")
    c = NeuronInstance(make_builtin("tanh_neuron"), instance_id="c")
    for n in (a, b, c):
        g.add_node(n)
    g.add_edge(Edge(id="1", src_node="a", dst_node="b"))
    g.add_edge(Edge(id="2", src_node="b", dst_node="c", weight=0.5))
    g.add_edge(Edge(id="3", src_node="c", dst_node="b", weight=0.5))
    g.input_node_ids, g.output_node_ids = ["a"], ["c"]
    assert g.has_cycles()
    y = g.execute({"a": (0.7,)}, max_iters=200, tolerance=1e-10)["c"][0]
    # fixed point: b = tanh(0.7 + 0.5 c), c = tanh(0.5 b)
    bb = cc = 0.0
    for _ in range(500):
        bb, cc = math.tanh(0.7 + 0.5 * cc), math.tanh(0.5 * bb)
    assert y == pytest.approx(cc, abs=1e-6)


def test_json_round_trip_bit_exact(tmp_path):
    g = build_xor()
    init_edge_params_normal(g, seed=0)
    text = graph_to_json(g)
    g2 = graph_from_json(text)
    assert g2.get_edge_params() == g.get_edge_params()  # exact float equality
    assert graph_to_json(g2) == text
    save_graph(g, tmp_path / "g.json")
    g3 = load_graph(tmp_path / "g.json")
    for row in XOR_X:
        feed = {"in0": (row[0],), "in1": (row[1],)}
        assert g3.execute(feed) == g.execute(feed)


def test_reference_example_json_loads():
    """The on-disk exemplar of the reference format (terminals with range +-100, precision 1e-3)."""
    import os
    import pathlib
    root = os.environ.get("NFN_REFERENCE_CHECKOUT", "")
    path = pathlib.Path(root) / "examples" / "xor_trained.json"
    if not root or not path.exists():
        pytest.skip("set NFN_REFERENCE_CHECKOUT to a checkout of the reference project to run this")
    g = load_graph(path)
    assert g.input_node_ids and g.output_node_ids
    feeds = {nid: (1.0,) for nid in g.input_node_ids}
    out = g.execute(feeds)
    assert all(len(v) >= 1 for v in out.values())
    assert json.loads(graph_to_json(g))["edges"].keys() == json.loads(path.read_text())["edges"].keys()


def test_nested_subgraph_and_variant_fallback():
    inner = build_xor(hidden=2)
    init_edge_params_normal(inner, seed=1)
    outer = NeuronGraph(name="outer")
    a = NeuronInstance(make_builtin("input"), instance_id="a")
    b = NeuronInstance(make_builtin("input"), instance_id="b")
    sub = NeuronInstance(subgraph_neuron(inner, name="xor_block", input_aliases=["p", "q"],
                                         output_aliases=["r"], variant_ref={"family": "gpt2", "version": "v1"}),
                         instance_id="s")
    o = NeuronInstance(make_builtin("output"), instance_id="o")
    for n in (a, b, sub, o):
        outer.add_node(n)
    outer.add_edge(Edge(id="1", src_node="a", dst_node="s", dst_port=0))
    outer.add_edge(Edge(id="2", src_node="b", dst_node="s", dst_port=1))
    outer.add_edge(Edge(id="3", src_node="s", dst_node="o"))
    outer.input_node_ids, outer.output_node_ids = ["a", "b"], ["o"]
    # library entry stored under the allied family name resolves through the alias table
    outer.variant_library = {"transformer_block": {"v1": NeuronGraph.from_dict_raw(inner.to_dict())}}
    want = inner.execute_flat((1.0, 0.0))
    rt = graph_from_json(graph_to_json(outer))
    assert rt.execute({"a": (1.0,), "b": (0.0,)})["o"] == want
    # a library entry with a different interface is ignored: the inline subgraph stays
    three = build_xor(hidden=3)
    three.input_node_ids = three.input_node_ids[:1]
    outer.variant_library = {"gpt2": {"v1": three}}
    rt2 = graph_from_json(graph_to_json(outer))
    assert rt2.execute({"a": (1.0,), "b": (0.0,)})["o"] == want
    with pytest.raises(ValueError):
        outer.variant_library = {}
        graph_from_json(graph_to_json(outer))


def test_gradient_matches_finite_differences():
    g = build_xor()
    init_edge_params_normal(g, seed=5)
    tr = GraphSGDTrainer(g, SGDConfig())
    grad = tr.gradient(XOR_X, XOR_Y)
    p0 = g.get_edge_params()
    for i in range(0, len(p0), 5):
        hi, lo = list(p0), list(p0)
        hi[i] += 1e-6
        lo[i] -= 1e-6
        g.set_edge_params(hi)
        lh = tr.loss(XOR_X, XOR_Y)
        g.set_edge_params(lo)
        ll = tr.loss(XOR_X, XOR_Y)
        assert (lh - ll) / 2e-6 == pytest.approx(grad[i], abs=1e-7)
    g.set_edge_params(p0)


def test_xor_sgd_converges_and_round_trips(tmp_path):
    """2 inputs -> 4 sigmoid -> 1 sigmoid, fp64 N(0,1) init from seed 0, MSE, SGD lr 0.5, 2000 steps."""
    g = build_xor()
    init_edge_params_normal(g, seed=0)
    tr = GraphSGDTrainer(g, SGDConfig(learning_rate=0.5, steps=2000))
    hist = tr.train(XOR_X, XOR_Y)
    assert hist[-1] < 0.01, hist[-1]
    save_graph(g, tmp_path / "xor.json")
    g2 = load_graph(tmp_path / "xor.json")
    assert g2.get_edge_params() == g.get_edge_params()
    for x, y in zip(XOR_X, XOR_Y):
        out = g2.execute({"in0": (x[0],), "in1": (x[1],)})["out"][0]
        assert round(out) == y[0]
