"""Family registry (capability proofs) and the Llama family checkpoint directory format (CPU)."""
import json

import pytest
import torch

from neuralfn_b200.checkpoint.family import (FamilyCheckpointError, expected_llama_layout, inspect_family_llama_checkpoint,
                                             load_family_llama_checkpoint, save_family_llama_checkpoint)
from neuralfn_b200.models.llama import LlamaConfig
from neuralfn_b200.native_registry import NATIVE_FAMILIES, capability_proof_for, classify_native_model, native_families_report, resolve_family


def test_registry_resolution_and_proofs():
    assert resolve_family("GPT2").family == "gpt" and resolve_family("glimmer").family == "muse-glimmer"
    assert classify_native_model("gpt2_qknorm")[1] == "gpt2_qknorm" and classify_native_model("deepseek_v3")[0].family == "mixllama"
    with pytest.raises(KeyError):
        classify_native_model("not-a-model")
    p = capability_proof_for("gpt2_qknorm")
    assert p.native_training and p.route == "native-gpt" and "dp" in p.parallel and p.native_inference
    q = capability_proof_for("gpt2_moa")
    assert not q.native_training and q.route == "tensor-runtime" and q.reasons
    with pytest.raises(ValueError):
        q.require("native_training")
    assert capability_proof_for("jamba").route == "tensor-runtime"
    assert len(native_families_report()) == len(NATIVE_FAMILIES) == 16
    assert all(s.reference_binary.startswith("nfn_") and s.reference_binary.endswith("_native_train") for s in NATIVE_FAMILIES.values())


def _tiny():
    cfg = LlamaConfig(n_layer=2, n_head=4, n_kv_head=2, d_model=64, d_ff=96, vocab_size=250, max_seq_len=32, vocab_pad_to=8, norm_eps=1e-6)
    g = torch.Generator().manual_seed(0)
    tensors = {s.name: torch.randn(*s.shape, generator=g).bfloat16() for s in cfg.param_specs()}
    return cfg, tensors


def test_family_checkpoint_round_trip_and_fail_closed(tmp_path):
    cfg, tensors = _tiny()
    out = tmp_path / "ckpt"
    doc = save_family_llama_checkpoint(out, cfg, tensors, steps=7)
    assert (out / "DONE").read_text().strip() == "done" and doc["inference_contract"]["artifact"]["nbytes"] == (out / "model.f32").stat().st_size
    info = inspect_family_llama_checkpoint(out)
    assert [t["name"] for t in info["tensors"]] == [n for n, _ in expected_llama_layout(info["geometry"])]
    cfg2, back, doc2 = load_family_llama_checkpoint(out)
    assert (cfg2.n_layer, cfg2.d_ff, cfg2.padded_vocab, doc2["steps"]) == (2, 96, cfg.padded_vocab, 7)
    for k, v in tensors.items():
        assert torch.equal(back[k].reshape(v.shape), v), k
    with pytest.raises(FamilyCheckpointError):
        save_family_llama_checkpoint(out, cfg, tensors)  # never overwrites
    # one flipped byte in the parameter file
    raw = bytearray((out / "model.f32").read_bytes())
    raw[100] ^= 1
    (out / "model.f32").write_bytes(bytes(raw))
    with pytest.raises(FamilyCheckpointError):
        inspect_family_llama_checkpoint(out)
    raw[100] ^= 1
    (out / "model.f32").write_bytes(bytes(raw))
    inspect_family_llama_checkpoint(out)
    # missing marker, foreign semantics, path escape
    (out / "DONE").unlink()
    with pytest.raises(FamilyCheckpointError):
        inspect_family_llama_checkpoint(out)
    (out / "DONE").write_text("done\n")
    d = json.loads((out / "checkpoint.json").read_text())
    d["inference_contract"]["semantics"]["linear_bias"] = True
    (out / "checkpoint.json").write_text(json.dumps(d))
    with pytest.raises(FamilyCheckpointError):
        inspect_family_llama_checkpoint(out)
    d["inference_contract"]["semantics"]["linear_bias"] = False
    d["inference_contract"]["artifact"]["path"] = "../model.f32"
    (out / "checkpoint.json").write_text(json.dumps(d))
    with pytest.raises(FamilyCheckpointError):
        inspect_family_llama_checkpoint(out)


def test_shipped_preset_header_matches_generator_and_runtime():
    from pathlib import Path

    import neuralfn_b200
    from neuralfn_b200.data import _rt
    from neuralfn_b200.native_registry import shipped_preset_header
    from neuralfn_b200.presets import SHIPPED_GPT_TEMPLATE_PRESETS
    header = Path(neuralfn_b200.__file__).parent / "csrc" / "runtime" / "shipped_presets.h"
    assert header.read_text() == shipped_preset_header(), "regenerate csrc/runtime/shipped_presets.h"
    compiled = _rt.shipped_presets()
    assert list(compiled) == list(SHIPPED_GPT_TEMPLATE_PRESETS) and compiled["gpt2"] == "gpt" and compiled["llama"] == "llama"
    assert _rt.lib().nfn_rt_preset_family(b"no_such_preset") is None
