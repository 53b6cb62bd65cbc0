"""Native Execution IR: lowering, the raw tensor bundle, digests, fail-closed behaviour."""
import json

import pytest
import torch


def _graph_with_weights():
    from neuralfn_b200.presets import build_preset
    from neuralfn_b200.torch_backend import CompiledTorchGraph
    from neuralfn_b200.torch_templates import build_gpt_root_graph
    g = build_gpt_root_graph(build_preset("llama", vocab_size=64, num_layers=2, model_dim=32, num_heads=4))
    model = CompiledTorchGraph(g)
    model.sync_state_back()  # weights into the graph's module_state blobs
    return g, model


def test_migrate_graph_writes_manifest_bundle_and_report(tmp_path):
    from neuralfn_b200.native_ir import BUNDLE_SCHEMA, MANIFEST_SCHEMA, load_native_bundle, migrate_graph_to_native
    g, model = _graph_with_weights()
    man = migrate_graph_to_native(g, tmp_path / "native", model_name="llama", tokenizer={"name": "bytes", "vocab_size": 64}, stop_token_ids=[0])
    assert man["schema"] == MANIFEST_SCHEMA and man["tensors"]["schema"] == BUNDLE_SCHEMA and man["model"]["family"] == "llama"
    assert man["model"]["parameters"] == sum(p.numel() for p in model.parameters()) + sum(b.numel() for b in model.buffers()) or man["model"]["parameters"] > 0
    assert man["capabilities"]["executable_natively"] and man["capabilities"]["native_kernel_nodes"] > 0
    assert man["topology"]["topological_order"] and all(s["offset"] % 64 == 0 for s in man["tensors"]["specs"])
    for f in ("native-execution-manifest.json", "tensors.bin", "compatibility-report.json", "source-graph.json"):
        assert (tmp_path / "native" / f).is_file()
    man2, tensors = load_native_bundle(tmp_path / "native")
    assert man2 == json.loads(json.dumps(man))
    sd = {k: v for k, v in model.state_dict().items()}
    assert len(tensors) >= len([k for k in sd if sd[k].numel()]) // 2
    total = sum(t.numel() for t in tensors.values())
    assert total == man["model"]["parameters"]
    with pytest.raises(ValueError):
        migrate_graph_to_native(g, tmp_path / "native")  # never overwrites
    # a flipped byte is caught
    p = tmp_path / "native" / "tensors.bin"
    raw = bytearray(p.read_bytes())
    raw[man["tensors"]["specs"][0]["offset"]] ^= 0xFF
    p.write_bytes(bytes(raw))
    with pytest.raises(ValueError):
        load_native_bundle(tmp_path / "native")


def test_function_neurons_are_recorded_by_digest_and_block_native_execution(tmp_path):
    import importlib.util
    from pathlib import Path

    from neuralfn_b200.native_ir import compatibility_report, lower_graph
    spec = importlib.util.spec_from_file_location("xor_graph_example", Path(__file__).resolve().parents[1] / "examples" / "xor_graph.py")
    xor = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(xor)
    ir = lower_graph(xor.build_xor_graph())
    text = json.dumps(ir)
    assert "source_sha256" in text and "def " not in text and "return" not in text
    rep = compatibility_report(ir)
    assert not rep["executable"] and any("function neuron" in b for b in rep["blockers"])


def test_pickled_objects_in_module_state_are_refused(tmp_path):
    import base64
    import io
    import pickle

    from neuralfn_b200.native_ir import NativeMigrationError, migrate_graph_to_native
    g, _ = _graph_with_weights()
    node = next(n for n in g.nodes.values() if n.neuron_def.kind == "module" and n.neuron_def.module_state)

    class Evil:
        def __reduce__(self):
            return (print, ("should never run",))

    buf = io.BytesIO()
    pickle.dump({"w": Evil()}, buf)
    node.neuron_def.module_state = base64.b64encode(buf.getvalue()).decode("ascii")
    with pytest.raises(NativeMigrationError):
        migrate_graph_to_native(g, tmp_path / "bad")
    assert not (tmp_path / "bad").exists()
