"""Muse-Glimmer weight ingestion: safetensors directories and GGUF files of a tiny geometry against the strict
tensor contract, the converted named checkpoint, and the `nfn migrate` front end."""
import json

import numpy as np
import pytest
import torch

from neuralfn_b200.checkpoint import glimmer_weights as gw
from neuralfn_b200.checkpoint.safetensors_io import SafetensorsError, write_safetensors

G = gw.GlimmerGeometry(n_layer=2, d_model=64, n_head=4, n_kv_head=2, head_dim=16, d_ff=96, vocab_size=120, vocab_pad_to=64)


def _source_tensors(contracts, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {c.source: (torch.randn(*c.shape, generator=g) * 0.1).to(torch.bfloat16) for c in contracts}


def _write_sharded(root, tensors, n_shards=2):
    root.mkdir()
    names = sorted(tensors)
    wmap = {}
    for i in range(n_shards):
        part = {n: tensors[n] for n in names[i::n_shards]}
        fname = f"model-{i + 1:05d}-of-{n_shards:05d}.safetensors"
        write_safetensors(root / fname, part)
        wmap.update({n: fname for n in part})
    (root / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wmap}))


def test_safetensors_directory_round_trip(tmp_path):
    src = _source_tensors(gw.safetensors_contracts(G))
    _write_sharded(tmp_path / "hf", src)
    report = gw.inspect_glimmer_safetensors(tmp_path / "hf", G)
    assert report["status"] == "ok" and report["tensors"] == len(src) and len(report["shards"]) == 2
    p = gw.load_glimmer_safetensors(tmp_path / "hf", G)
    pre = "model.language_model.layers.1."
    want = torch.cat([src[pre + f"self_attn.{k}_proj.weight"] for k in ("q", "k", "v", "gate")], 0)
    assert torch.equal(p["layers.1.wqkvg"], want)
    assert torch.equal(p["layers.1.w_gate_up"], torch.cat([src[pre + "mlp.gate_proj.weight"], src[pre + "mlp.up_proj.weight"]], 0))
    assert torch.equal(p["layers.0.post_mlp_norm"], src["model.language_model.layers.0.post_feedforward_layernorm.weight"])
    assert p["tok_embeddings"].shape == (128, 64) and float(p["tok_embeddings"][120:].abs().max()) == 0.0
    # the engine's own parameter list and the converted dictionary agree name by name and shape by shape
    from neuralfn_b200.models.glimmer import GlimmerConfig
    cfg = GlimmerConfig(n_layer=2, d_model=64, n_head=4, n_kv_head=2, head_dim=16, d_ff=96, vocab_size=120, vocab_pad_to=64)
    assert {s.name: tuple(s.shape) for s in cfg.param_specs()} == {k: tuple(v.shape) for k, v in p.items()}
    # and the serving decoder's names produce the same logits as the training oracle
    from neuralfn_b200.models.glimmer import glimmer_reference_loss
    from neuralfn_b200.serving.tp_glimmer import GlimmerTPConfig, glimmer_reference_logits
    scfg = GlimmerTPConfig(n_layer=2, d_model=64, n_head=4, n_kv_head=2, head_dim=16, d_ff=96, vocab_size=120, window=cfg.window,
                           global_every=cfg.global_every, rope_theta=cfg.rope_theta, q_scale=cfg.q_scale, norm_eps=cfg.norm_eps,
                           post_norm_eps=cfg.post_norm_eps, qk_norm_eps=cfg.qk_norm_eps, logit_softcap=cfg.logit_softcap,
                           output_multiplier=cfg.output_multiplier, vocab_pad_to=64)
    tok = torch.randint(0, 120, (2, 12), generator=torch.Generator().manual_seed(1))
    pf = {k: v.float() for k, v in p.items()}
    _, logits, _ = glimmer_reference_loss(cfg, pf, tok, tok)
    assert (glimmer_reference_logits(scfg, gw.to_serving_names(pf, G), tok) - logits).abs().max() < 1e-4


def test_contract_violations_are_refused(tmp_path):
    src = _source_tensors(gw.safetensors_contracts(G))
    bad = dict(src)
    bad.pop("model.language_model.layers.0.self_attn.gate_proj.weight")
    _write_sharded(tmp_path / "missing", bad)
    with pytest.raises(SafetensorsError, match="missing"):
        gw.inspect_glimmer_safetensors(tmp_path / "missing", G)
    bad = dict(src)
    bad["model.language_model.layers.0.mlp.up_proj.weight"] = torch.zeros(95, 64, dtype=torch.bfloat16)
    _write_sharded(tmp_path / "shape", bad)
    with pytest.raises(SafetensorsError, match="shape"):
        gw.inspect_glimmer_safetensors(tmp_path / "shape", G)
    extra = dict(src)
    extra["model.vision_tower.patch_embed.weight"] = torch.zeros(4, 4, dtype=torch.bfloat16)
    _write_sharded(tmp_path / "extra", extra)
    with pytest.raises(SafetensorsError, match="outside the text contract"):
        gw.inspect_glimmer_safetensors(tmp_path / "extra", G)
    assert gw.inspect_glimmer_safetensors(tmp_path / "extra", G, allow_extra_prefixes=("model.vision_tower.",))["status"] == "ok"


def test_gguf_files_and_converted_checkpoint(tmp_path, capsys):
    from neuralfn_b200.checkpoint.gguf import write_gguf
    from neuralfn_b200.checkpoint.named import read_named_tensors
    src = _source_tensors(gw.gguf_contracts(G), seed=3)
    enc = {}
    for name, t in src.items():
        if t.ndim == 1:
            enc[name] = (0, tuple(t.shape), t.float().numpy().astype("<f4").tobytes())                     # F32 norms
        else:
            enc[name] = (30, tuple(t.shape), (t.view(torch.int16).numpy().astype("<u2")).tobytes())         # BF16 matrices
    enc["blk.0.attn_q_norm.weight"] = (0, (16,), np.ones(16, "<f4").tobytes())                             # ignored: weightless norm
    names = sorted(enc)
    write_gguf(tmp_path / "a.gguf", {"general.architecture": "muse-glimmer"}, {n: enc[n] for n in names[::2]})
    write_gguf(tmp_path / "b.gguf", {"general.architecture": "muse-glimmer"}, {n: enc[n] for n in names[1::2]})
    p = gw.load_glimmer_gguf([tmp_path / "a.gguf", tmp_path / "b.gguf"], G)
    assert torch.equal(p["layers.0.wo"], src["blk.0.attn_output.weight"])
    assert torch.equal(p["norm"], src["output_norm.weight"])
    with pytest.raises(ValueError, match="missing"):
        gw.load_glimmer_gguf([tmp_path / "a.gguf"], G)
    # command line: dry run, conversion, refusal to overwrite
    from neuralfn_b200.cli.nfn import main
    geom = json.dumps({k: getattr(G, k) for k in G.__dataclass_fields__})
    argv = ["migrate", "muse-glimmer-gguf-to-native", "--gguf", str(tmp_path / "a.gguf"), "--gguf", str(tmp_path / "b.gguf"), "--geometry", geom]
    assert main(argv + ["--dry-run"]) == 0
    assert main(argv + ["--output-dir", str(tmp_path / "out")]) == 0
    capsys.readouterr()
    tensors, meta, _sha = read_named_tensors(tmp_path / "out" / "weights_00000000.nfnw")
    assert meta["model_family"] == "muse-glimmer" and torch.equal(tensors["layers.1.wqkvg"], p["layers.1.wqkvg"])
    assert json.loads((tmp_path / "out" / "DONE_00000000").read_text()).keys() == {"weights_00000000.nfnw"}
    assert main(argv + ["--output-dir", str(tmp_path / "out")]) != 0          # never overwritten
    assert "FileExistsError" in capsys.readouterr().out
