"""Strict safetensors reading, sharded checkpoints, Hugging Face Llama ingestion (CPU)."""
import json
import struct

import pytest
import torch

from neuralfn_b200.checkpoint.safetensors_io import (SafetensorsError, load_hf_llama_directory, read_safetensors, read_sharded_checkpoint,
                                                     write_safetensors)


def test_round_trip_and_strictness(tmp_path):
    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32), "c": torch.zeros(0, 4)}
    p = tmp_path / "x.safetensors"
    write_safetensors(p, t, {"format": "pt"})
    got, meta = read_safetensors(p)
    assert meta == {"format": "pt"} and all(torch.equal(got[k], v) for k, v in t.items())
    assert set(read_safetensors(p, names={"b"})[0]) == {"b"}
    raw = p.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])

    def rewrite(h, tail=raw[8 + hlen:], name="bad.safetensors"):
        hj = json.dumps(h).encode()
        q = tmp_path / name
        q.write_bytes(struct.pack("<Q", len(hj)) + hj + tail)
        return q

    bad = json.loads(json.dumps(header))
    bad["a"]["data_offsets"][1] += 2  # overlaps the next tensor
    with pytest.raises(SafetensorsError):
        read_safetensors(rewrite(bad))
    bad = json.loads(json.dumps(header))
    bad["a"]["dtype"] = "F8_E4M3"
    with pytest.raises(SafetensorsError):
        read_safetensors(rewrite(bad))
    with pytest.raises(SafetensorsError):
        read_safetensors(rewrite(header, raw[8 + hlen:] + b"\0\0"))  # trailing bytes
    dup = raw[8:8 + hlen].decode().rstrip()[:-1] + ',"b":{"dtype":"I32","shape":[7],"data_offsets":[30,58]}}'
    q = tmp_path / "dup.safetensors"
    q.write_bytes(struct.pack("<Q", len(dup)) + dup.encode() + raw[8 + hlen:])
    with pytest.raises(SafetensorsError):
        read_safetensors(q)
    (tmp_path / "short.safetensors").write_bytes(b"\x01\x00")
    with pytest.raises(SafetensorsError):
        read_safetensors(tmp_path / "short.safetensors")


def _hf_llama(tmp_path, shards=True, tie=False):
    d, L, H, Hkv, F, V = 32, 2, 4, 2, 48, 50
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g).bfloat16()  # noqa: E731
    sd = {"model.embed_tokens.weight": r(V, d), "model.norm.weight": r(d)}
    if not tie:
        sd["lm_head.weight"] = r(V, d)
    for l in range(L):
        p = f"model.layers.{l}."
        sd.update({p + "input_layernorm.weight": r(d), p + "self_attn.q_proj.weight": r(d, d), p + "self_attn.k_proj.weight": r(Hkv * 8, d),
                   p + "self_attn.v_proj.weight": r(Hkv * 8, d), p + "self_attn.o_proj.weight": r(d, d),
                   p + "post_attention_layernorm.weight": r(d), p + "mlp.gate_proj.weight": r(F, d), p + "mlp.up_proj.weight": r(F, d),
                   p + "mlp.down_proj.weight": r(d, F)})
    root = tmp_path / "hf"
    root.mkdir()
    (root / "config.json").write_text(json.dumps({"hidden_size": d, "num_hidden_layers": L, "num_attention_heads": H, "num_key_value_heads": Hkv,
                                                  "vocab_size": V, "intermediate_size": F, "max_position_embeddings": 64, "rope_theta": 10000.0,
                                                  "rms_norm_eps": 1e-5, "tie_word_embeddings": tie}))
    if shards:
        names = sorted(sd)
        parts = [names[:len(names) // 2], names[len(names) // 2:]]
        wmap = {}
        for i, part in enumerate(parts):
            fn = f"model-{i + 1:05d}-of-00002.safetensors"
            write_safetensors(root / fn, {k: sd[k] for k in part})
            wmap.update({k: fn for k in part})
        (root / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wmap}))
    else:
        write_safetensors(root / "model.safetensors", sd)
    return root, sd


@pytest.mark.parametrize("shards,tie", [(True, False), (False, True)])
def test_hf_llama_ingestion(tmp_path, shards, tie):
    root, sd = _hf_llama(tmp_path, shards, tie)
    assert set(read_sharded_checkpoint(root)) == set(sd)
    cfg, t = load_hf_llama_directory(root, max_batch=2)
    assert (cfg.n_layer, cfg.n_kv_head, cfg.head_dim, cfg.padded_vocab, cfg.tie_embeddings) == (2, 2, 8, 56, int(tie))
    assert t["tok_embeddings"].shape == (56, 32) and torch.equal(t["tok_embeddings"][:50], sd["model.embed_tokens.weight"])
    assert torch.equal(t["layers.1.wqkv"][32:48], sd["model.layers.1.self_attn.k_proj.weight"])
    assert torch.equal(t["layers.0.w_gate_up"][48:], sd["model.layers.0.mlp.up_proj.weight"]) and ("lm_head" in t) == (not tie)


def test_sharded_index_must_agree(tmp_path):
    root, sd = _hf_llama(tmp_path, True)
    idx = json.loads((root / "model.safetensors.index.json").read_text())
    first = sorted(idx["weight_map"])[0]
    idx["weight_map"].pop(first)
    (root / "model.safetensors.index.json").write_text(json.dumps(idx))
    with pytest.raises(SafetensorsError):
        read_sharded_checkpoint(root)
    idx["weight_map"][first] = "../evil.safetensors"
    (root / "model.safetensors.index.json").write_text(json.dumps(idx))
    with pytest.raises(SafetensorsError):
        read_sharded_checkpoint(root)
