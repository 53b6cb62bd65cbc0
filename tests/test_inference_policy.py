"""Strict (temperature 0) inference policy: validation, the readers / writer gate, switch save / restore."""
import threading
import time

import pytest
import torch

import neuralfn_b200.inference_policy as P


def test_temperature_validation_and_trigger():
    assert P.temperature_uses_strict_inference(0) and P.temperature_uses_strict_inference(-0.0) and not P.temperature_uses_strict_inference(0.7)
    for bad in (-1, float("nan"), float("inf"), "hot", None, True):
        with pytest.raises(ValueError):
            P.validate_inference_temperature(bad)
    pay = P.compute_policy_payload(P.STRICT_INFERENCE_POLICY, backend="tensor")
    assert pay["mode"] == "strict" and pay["trigger"] == "temperature_zero" and pay["tf32_disabled"] and pay["version"] == 1


def test_gate_orders_strict_after_running_standard_and_blocks_new_standard():
    gate, log = P.InferenceConcurrencyGate(), []
    release = threading.Event()

    def reader(name, hold):
        with gate.shared():
            log.append(("in", name))
            if hold:
                release.wait(5)
        log.append(("out", name))

    def writer():
        with gate.exclusive():
            log.append(("in", "strict"))
        log.append(("out", "strict"))

    r1 = threading.Thread(target=reader, args=("r1", True)); r1.start()
    time.sleep(0.05)
    w = threading.Thread(target=writer); w.start()
    time.sleep(0.05)
    r2 = threading.Thread(target=reader, args=("r2", False)); r2.start()   # must wait behind the waiting writer
    time.sleep(0.05)
    assert log == [("in", "r1")]
    release.set()
    for t in (r1, w, r2):
        t.join(5)
    assert log.index(("in", "strict")) < log.index(("in", "r2")) and log.index(("out", "r1")) < log.index(("in", "strict"))


def test_strict_execution_flips_and_restores_switches(monkeypatch):
    monkeypatch.setenv("CUBLAS_WORKSPACE_CONFIG", P.DETERMINISTIC_CUBLAS_WORKSPACE_CONFIG)
    before = (torch.are_deterministic_algorithms_enabled(), torch.backends.cuda.matmul.allow_tf32, torch.get_float32_matmul_precision())
    with P.inference_execution(0.0, torch_module=torch) as pol:
        assert pol.strict and torch.are_deterministic_algorithms_enabled() and not torch.backends.cuda.matmul.allow_tf32
        assert torch.get_float32_matmul_precision() == "highest" and not torch.is_autocast_enabled()
    assert (torch.are_deterministic_algorithms_enabled(), torch.backends.cuda.matmul.allow_tf32, torch.get_float32_matmul_precision()) == before
    with P.inference_execution(0.8) as pol:
        assert not pol.strict
    with P.inference_execution(0.0, native_engine=True) as pol:
        assert pol.strict and not torch.are_deterministic_algorithms_enabled() or before[0]
    with pytest.raises(RuntimeError):
        with P.inference_execution(0.0):
            pass


def test_strict_graph_support_fails_closed_on_lossy_graphs():
    from neuralfn_b200.presets import build_preset
    from neuralfn_b200.torch_templates import build_gpt_root_graph
    kw = dict(vocab_size=64, num_layers=1, model_dim=32, num_heads=2)
    P.validate_strict_graph_support(build_gpt_root_graph(build_preset("llama", **kw)))
    with pytest.raises(RuntimeError):
        P.validate_strict_graph_support(build_gpt_root_graph(build_preset("fp8_llama", **kw)))
    g = build_gpt_root_graph(build_preset("llama", **kw))
    g.torch_config["tile_cuda_activation_dtype"] = "bf16"
    with pytest.raises(RuntimeError):
        P.validate_strict_graph_support(g)
