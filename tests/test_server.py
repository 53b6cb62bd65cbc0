"""Platform state store, MCP tool server (JSON-RPC) and REST app routes, all in-process."""
import json

import pytest

from neuralfn_b200.server import LiveStateStore
from neuralfn_b200.server.mcp_server import McpToolServer

XOR_X = [[0, 0], [0, 1], [1, 0], [1, 1]]
XOR_Y = [[0], [1], [1], [0]]


def _xor_session(call):
    sid = call("create_session", {"name": "xor"})["session_id"]
    ins = [call("add_node", {"session_id": sid, "builtin": "input", "role": "input"})["node_id"] for _ in range(2)]
    hid = [call("add_node", {"session_id": sid, "builtin": "sigmoid"})["node_id"] for _ in range(4)]
    out = call("add_node", {"session_id": sid, "builtin": "sigmoid", "role": "output"})["node_id"]
    k = 0
    for i in ins:
        for h in hid:
            k += 1
            call("add_edge", {"session_id": sid, "src_node": i, "dst_node": h, "weight": 0.5 * ((-1) ** k) * (1 + k % 3), "bias": 0.1 * (k % 4)})
    for j, h in enumerate(hid):
        call("add_edge", {"session_id": sid, "src_node": h, "dst_node": out, "weight": 0.7 * ((-1) ** j), "bias": 0.0})
    return sid


def test_mcp_tools_build_execute_and_train(tmp_path):
    server = McpToolServer(LiveStateStore(tmp_path / "snap"))
    names = {t["name"] for t in server.list_tools()}
    assert {"get_graph", "replace_graph", "execute", "train_start", "train_status", "list_presets", "semantic_match", "native_info"} <= names
    call = server.call
    sid = _xor_session(call)
    before = call("execute", {"session_id": sid, "inputs": [0, 1]})["outputs"]
    assert len(before) == 1 and 0 < before[0] < 1
    rid = call("train_start", {"session_id": sid, "inputs": XOR_X, "targets": XOR_Y, "method": "sgd", "steps": 1500, "learning_rate": 0.5})["run_id"]
    status = server.store.wait(rid, timeout=120)
    assert status["status"] == "finished" and status["steps"] == 1500 and status["last_loss"] < 0.1, status
    # snapshots survive a restart
    again = LiveStateStore(tmp_path / "snap")
    assert again.execute(sid, [0, 1]) == call("execute", {"session_id": sid, "inputs": [0, 1]})["outputs"]
    assert "gpt2" in call("list_presets") and call("trace_torch", {"name": "gpt2"})["parameters"] > 0
    assert call("semantic_match", {"text": "repair the software"})["action"] == "repair"
    assert call("training_plan", {"config": {"batch_size": 16}})["grad_accum_steps"] == 32


def test_json_rpc_protocol():
    server = McpToolServer()
    init = server.handle({"jsonrpc": "2.0", "id": 1, "method": "initialize", "params": {}})
    assert init["result"]["serverInfo"]["name"] == "neuralfn_b200"
    tools = server.handle({"jsonrpc": "2.0", "id": 2, "method": "tools/list"})["result"]["tools"]
    assert all("inputSchema" in t for t in tools)
    ok = server.handle({"jsonrpc": "2.0", "id": 3, "method": "tools/call", "params": {"name": "create_session", "arguments": {"name": "a"}}})
    assert not ok["result"]["isError"] and "session_id" in json.loads(ok["result"]["content"][0]["text"])
    bad = server.handle({"jsonrpc": "2.0", "id": 4, "method": "tools/call", "params": {"name": "get_graph", "arguments": {"session_id": "nope"}}})
    assert bad["result"]["isError"]
    assert server.handle({"jsonrpc": "2.0", "id": 5, "method": "bogus"})["error"]["code"] == -32601
    assert server.handle({"jsonrpc": "2.0", "method": "notifications/initialized"}) is None


def test_rest_routes_share_the_store(monkeypatch):
    pytest.importorskip("fastapi")
    from neuralfn_b200.server.app import InferenceConcurrencyGate, create_app
    monkeypatch.setenv("NEURALFN_API_TOKEN", "s3cret")
    store = LiveStateStore()
    app = create_app(store)
    routes = {r.path: r for r in app.routes if hasattr(r, "endpoint")}
    assert {"/api/bootstrap", "/api/sessions", "/api/sessions/{sid}/execute", "/api/runs/{rid}", "/v1/generate"} <= set(routes)
    sid = routes["/api/sessions"].endpoint.__globals__ and store.create_session("rest")
    n1 = store.add_builtin_node(sid, "input", role="input")
    n2 = store.add_builtin_node(sid, "identity", role="output")
    store.add_edge(sid, n1, n2, weight=2.0, bias=1.0)
    execute = next(r.endpoint for r in app.routes if getattr(r, "path", "") == "/api/sessions/{sid}/execute")
    assert execute(sid, {"inputs": [3.0]}) == {"outputs": [7.0]}
    from fastapi import HTTPException
    with pytest.raises(HTTPException) as e:
        execute("missing", {"inputs": [1.0]})
    assert e.value.status_code == 404
    gen = next(r.endpoint for r in app.routes if getattr(r, "path", "") == "/v1/generate")
    with pytest.raises(HTTPException) as e:
        gen({"prompts": [[1]]})
    assert e.value.status_code == 503
    with InferenceConcurrencyGate(max_waiting=1) as g:
        with pytest.raises(RuntimeError):
            g.__class__.__enter__(g)


def test_mcp_edit_tools_nodes_edges_variants_settings():
    from neuralfn_b200.server.mcp_server import McpToolServer
    srv = McpToolServer()
    call = srv.call
    assert len(srv.list_tools()) >= 37
    sid = call("create_session", {"name": "edit"})["session_id"]
    a = call("add_node", {"session_id": sid, "builtin": "input", "role": "input"})["node_id"]
    src = "def double_plus(x):\n    return (2.0 * x + 1.0,)\n"
    c = call("add_custom_node", {"session_id": sid, "source_code": src, "fn_name": "double_plus", "inputs": [{"name": "x", "range": [-2.0, 2.0]}],
                                 "outputs": [{"name": "y"}]})["node_id"]
    e = call("add_edge", {"session_id": sid, "src_node": a, "dst_node": c})["edge_id"]
    call("set_io", {"session_id": sid, "input_ids": [a], "output_ids": [c]})
    assert call("execute", {"session_id": sid, "inputs": [1.5]})["outputs"] == [4.0]
    assert call("update_edge", {"session_id": sid, "edge_id": e, "weight": 2.0, "bias": -1.0})["weight"] == 2.0
    assert call("execute", {"session_id": sid, "inputs": [1.5]})["outputs"] == [5.0]  # 2 * (2 * 1.5 - 1) + 1
    node = call("update_node", {"session_id": sid, "node_id": c, "name": "triple", "position": [3, 4],
                                "source_code": "def triple(x):\n    return (3.0 * x,)\n"})
    assert node["position"] == [3.0, 4.0] or tuple(node["position"]) == (3.0, 4.0)
    assert call("execute", {"session_id": sid, "inputs": [1.5]})["outputs"] == [6.0]
    assert call("get_node", {"session_id": sid, "node_id": c})["incoming"] == [e]
    assert call("update_node_positions", {"session_id": sid, "positions": {a: [1, 1], c: [2, 2]}})["moved"] == 2
    probe = call("probe_node", {"session_id": sid, "node_id": c, "n_samples": 200})
    assert probe["samples"] == 200 and -6.0 <= probe["outputs"][0]["min"] < probe["outputs"][0]["max"] <= 6.0
    with pytest.raises(ValueError):
        call("update_node", {"session_id": sid, "node_id": c, "source_code": "x = 1\n"})  # no callable in the source
    st = call("update_graph_settings", {"session_id": sid, "training_method": "sgd", "evo_config": {"population": 8}})
    assert st["training_method"] == "sgd" and st["evo_config"]["population"] == 8
    with pytest.raises(ValueError):
        call("update_graph_settings", {"session_id": sid, "training_method": "magic"})

    # subgraph nodes and the variant library
    inner = call("get_graph", {"session_id": sid})
    outer = call("create_session", {"name": "outer"})["session_id"]
    n = call("add_subgraph_node", {"session_id": outer, "name": "inner", "subgraph": inner})["node_id"]
    lib = call("save_node_as_variant", {"session_id": outer, "node_id": n, "family": "blocks", "version": "v1"})
    assert lib == {"blocks": ["v1"]}
    m = call("add_variant_node", {"session_id": outer, "family": "blocks", "version": "v1"})["node_id"]
    assert call("get_node", {"session_id": outer, "node_id": m})["neuron_def"]["variant_ref"] == {"family": "blocks", "version": "v1"}
    assert call("swap_node_variant", {"session_id": outer, "node_id": n, "family": "blocks", "version": "v1"})["id" if False else "instance_id"] == n
    with pytest.raises(KeyError):
        call("swap_node_variant", {"session_id": outer, "node_id": n, "family": "blocks", "version": "v9"})
    tpl = call("load_gpt_template", {"session_id": outer, "preset": "nanogpt", "config": {"vocab_size": 64, "num_layers": 1, "model_dim": 32, "num_heads": 2}})
    assert tpl["runtime"] == "torch" and tpl["nodes"] > 3


def test_editor_page_and_the_routes_it_uses():
    pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient

    from neuralfn_b200.server.app import create_app
    c = TestClient(create_app())
    page = c.get("/")
    assert page.status_code == 200 and "text/html" in page.headers["content-type"] and 'id="canvas"' in page.text and "/api/sessions" in page.text
    names = c.get("/api/builtins").json()
    assert "sigmoid" in names and "input" in names
    sid = c.post("/api/sessions", json={"name": "ui"}).json()["session_id"]
    a = c.post(f"/api/sessions/{sid}/nodes", json={"builtin": "input", "role": "input"}).json()["node_id"]
    b = c.post(f"/api/sessions/{sid}/nodes", json={"builtin": "sigmoid", "role": "output"}).json()["node_id"]
    c.post(f"/api/sessions/{sid}/edges", json={"src_node": a, "dst_node": b})
    g = c.get(f"/api/sessions/{sid}/graph").json()
    assert set(g["nodes"]) == {a, b} and len(g["edges"]) == 1 and g["input_node_ids"] == [a]
    assert c.delete(f"/api/sessions/{sid}/nodes/{b}").status_code == 200
    assert set(c.get(f"/api/sessions/{sid}/graph").json()["nodes"]) == {a}
    assert c.delete(f"/api/sessions/{sid}/nodes/nope").status_code == 404
