"""Dense GPT checkpoint files: byte layout against the documented reference format,
exclusive writes, exact-size reads, single-file and rank-sharded optimizer round trips."""
import json
import struct
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from neuralfn_b200.checkpoint import (consolidate_sharded_optimizer, inspect_dense_model, load_dense_checkpoint,
                                      read_dense_model, save_dense_checkpoint, write_container)
from neuralfn_b200.data._rt import NativeRuntimeError
from neuralfn_b200.models.gpt2 import FlatLayout, GPT2Config, gpt2_param_specs, init_gpt2_params_
from neuralfn_b200.parallel.dp import AdamWConfig, ShardedAdamW, SymmetricBuffers


def _cpu_trainer(seed=3):
    cfg = GPT2Config.variant("gpt2_qknorm_softcap_zloss", n_layer=2, n_head=2, d_model=32, vocab_size=100, max_seq_len=16)
    layout = FlatLayout(gpt2_param_specs(cfg), world=1)
    bufs = SymmetricBuffers(layout.n_total, torch.device("cpu"))
    master = torch.empty(layout.n_total)
    init_gpt2_params_(cfg, layout, master, seed)
    opt = ShardedAdamW(layout, bufs, AdamWConfig(), master_init=master)
    bufs.params.copy_(master.bfloat16())
    opt.m.normal_(generator=torch.Generator().manual_seed(seed))
    opt.v.uniform_(generator=torch.Generator().manual_seed(seed + 1))
    opt.step_count = 7
    return SimpleNamespace(cfg=cfg, layout=layout, bufs=bufs, opt=opt, device=torch.device("cpu"))


def test_model_file_layout_and_roundtrip(tmp_path):
    tr = _cpu_trainer()
    digests = save_dense_checkpoint(tr, tmp_path, sharded_optimizer=False)
    raw = (tmp_path / "model_00000007.bin").read_bytes()
    head = struct.unpack("<256i", raw[:1024])
    assert head[:8] == (20240326, 5, 16, 100, 2, 2, 32, 128) and not any(head[8:])
    specs = gpt2_param_specs(tr.cfg)
    assert len(raw) == 1024 + 2 * sum(s.numel for s in specs)
    # first tensor is wte[Vp, C] in bf16, directly after the header
    wte = torch.frombuffer(bytearray(raw[1024:1024 + 2 * 128 * 32]), dtype=torch.bfloat16).view(128, 32)
    assert torch.equal(wte, tr.layout.view(tr.bufs.params, "wte"))
    info = inspect_dense_model(tmp_path / "model_00000007.bin")
    assert info["parameter_count"] == sum(s.numel for s in specs)
    cfg, tensors, sha = read_dense_model(tmp_path / "model_00000007.bin")
    assert cfg.qk_norm and cfg.logit_softcap == 30.0 and sha == digests["model_00000007.bin"]
    assert torch.equal(tensors["h.1.mlp.c_proj.weight"], tr.layout.view(tr.bufs.params, "h.1.mlp.c_proj.weight"))
    phead = struct.unpack("<32q", (tmp_path / "parameters_00000007.bin").read_bytes()[:256])
    assert phead[:3] == (20260711, 1, 7) and phead[9] == len(specs)
    ohead = struct.unpack("<32q", (tmp_path / "optimizer_00000007.bin").read_bytes()[:256])
    assert ohead[0] == 20260710 and ohead[10] == 2 * phead[10]
    assert json.loads((tmp_path / "DONE_00000007").read_text()) == digests


def test_resume_restores_master_and_moments(tmp_path):
    a = _cpu_trainer(seed=3)
    save_dense_checkpoint(a, tmp_path, sharded_optimizer=False)
    b = _cpu_trainer(seed=9)
    got = load_dense_checkpoint(b, tmp_path)
    assert got == {"step": 7, "model": True, "master": True, "moments": True} and b.opt.step_count == 7
    used = a.layout.n_used
    for name in ("master", "m", "v"):
        x, y = getattr(a.opt, name), getattr(b.opt, name)
        for s in gpt2_param_specs(a.cfg):
            assert torch.equal(a.layout.view(x, s.name), b.layout.view(y, s.name)), (name, s.name)
    assert torch.equal(a.bufs.params[:used], b.bufs.params[:used])


def test_sharded_optimizer_manifest_and_consolidation(tmp_path):
    a = _cpu_trainer()
    digests = save_dense_checkpoint(a, tmp_path, sharded_optimizer=True)
    man = json.loads((tmp_path / "optimizer_00000007.manifest.json").read_text())
    assert man["world_size"] == 1 and man["shards"][0]["sha256"] == digests["optimizer_00000007.rank00000.bin"]
    master, m, v = consolidate_sharded_optimizer(tmp_path, 7, a.cfg)
    assert torch.equal(m, a.opt.m) and torch.equal(v, a.opt.v) and torch.equal(master, a.opt.master)
    b = _cpu_trainer(seed=11)
    assert load_dense_checkpoint(b, tmp_path)["moments"]
    assert torch.equal(b.opt.v, a.opt.v)
    blob = bytearray((tmp_path / "optimizer_00000007.rank00000.bin").read_bytes())
    blob[-1] ^= 1
    (tmp_path / "optimizer_00000007.rank00000.bin").write_bytes(bytes(blob))
    with pytest.raises(ValueError, match="checksum"):
        load_dense_checkpoint(_cpu_trainer(), tmp_path)


def test_model_only_is_a_warm_start(tmp_path):
    a = _cpu_trainer()
    save_dense_checkpoint(a, tmp_path, sharded_optimizer=False)
    for f in ("parameters_00000007.bin", "optimizer_00000007.bin"):
        (tmp_path / f).unlink()
    b = _cpu_trainer(seed=5)
    got = load_dense_checkpoint(b, tmp_path)
    assert got["model"] and not got["moments"] and b.opt.step_count == 0
    assert float(b.opt.m.abs().sum()) == 0.0
    assert torch.equal(b.opt.master[:a.layout.n_used], a.bufs.params[:a.layout.n_used].float())


def test_container_refuses_overwrite_symlink_and_wrong_size(tmp_path):
    p = tmp_path / "x.bin"
    write_container(p, b"head", [np.arange(4, dtype=np.int32)])
    with pytest.raises(NativeRuntimeError, match="overwrite"):
        write_container(p, b"head", [np.arange(4, dtype=np.int32)])
    link = tmp_path / "link.bin"
    link.symlink_to(tmp_path / "target.bin")
    with pytest.raises(NativeRuntimeError):
        write_container(link, b"head", [])
    from neuralfn_b200.checkpoint import read_container
    with pytest.raises(NativeRuntimeError, match="size"):
        read_container(p, 4, [torch.empty(5, dtype=torch.int32)])
    hdr, _ = read_container(p, 4, [torch.empty(4, dtype=torch.int32)])
    assert hdr == b"head"


def _write_sharded_by_hand(tmp_path, cfg, world, step, fulls, params):
    """What ``save_dense_checkpoint`` writes for ``world`` ranks, produced in one process."""
    from neuralfn_b200.checkpoint import dense as D
    layout = FlatLayout(gpt2_param_specs(cfg), world=world)
    digests = {f"model_{step:08d}.bin": D.write_dense_model(tmp_path / f"model_{step:08d}.bin", cfg, layout, params[:layout.n_total])}
    entries = []
    for r in range(world):
        lo = r * layout.shard
        name = f"optimizer_{step:08d}.rank{r:05d}.bin"
        hdr = D._state_header(D.SHARD_MAGIC, step, cfg, r, world, lo, layout.shard, layout.n_total)
        sha = write_container(tmp_path / name, hdr, [t[lo:lo + layout.shard].contiguous() for t in fulls])
        entries.append({"rank": r, "file": name, "sha256": sha, "lo": lo, "shard": layout.shard})
        digests[name] = sha
    (tmp_path / f"optimizer_{step:08d}.manifest.json").write_text(json.dumps(
        {"schema": "neuralfn_b200.dense_sharded_optimizer.v1", "step": step, "world_size": world, "n_total": layout.n_total,
         "geometry": D._geometry(cfg), "shards": entries}))
    (tmp_path / f"DONE_{step:08d}").write_text(json.dumps(digests, sort_keys=True))
    return layout


def test_resharding_between_world_sizes_whose_padding_differs(tmp_path):
    """Saved by 2 ranks, loaded by rank 2 of 3: the flat buffer is padded to a multiple of 8 * world, so
    the two layouts have different lengths and the last rank's slice reaches into the padding."""
    cfg = GPT2Config.variant("gpt2", n_layer=1, n_head=1, d_model=8, vocab_size=11, max_seq_len=5, vocab_pad_to=1)
    specs = gpt2_param_specs(cfg)
    l2, l3 = FlatLayout(specs, world=2), FlatLayout(specs, world=3)
    assert l2.n_used % 24 != 0 and l2.n_total != l3.n_total
    g = torch.Generator().manual_seed(0)
    fulls = [torch.randn(l2.n_total, generator=g) for _ in range(3)]
    for t in fulls:
        t[l2.n_used:] = 0  # padding carries nothing
    params = torch.zeros(max(l2.n_total, l3.n_total), dtype=torch.bfloat16)
    params[:l2.n_used] = fulls[0][:l2.n_used].bfloat16()
    _write_sharded_by_hand(tmp_path, cfg, 2, 5, fulls, params)
    for rank in range(3):
        lo = rank * l3.shard
        opt = SimpleNamespace(world=3, rank=rank, lo=lo, shard=l3.shard, step_count=0,
                              master=torch.empty(l3.shard), m=torch.empty(l3.shard), v=torch.empty(l3.shard))
        bufs = SimpleNamespace(params=torch.zeros(l3.n_total, dtype=torch.bfloat16))
        tr = SimpleNamespace(cfg=cfg, layout=l3, bufs=bufs, opt=opt, device=torch.device("cpu"))
        got = load_dense_checkpoint(tr, tmp_path)
        assert got["master"] and got["moments"]
        for dst, full in zip((opt.master, opt.m, opt.v), fulls):
            want = torch.zeros(l3.n_total)
            want[:l2.n_used] = full[:l2.n_used]
            assert torch.equal(dst, want[lo:lo + l3.shard]), rank


def test_same_world_load_checks_the_shard_header(tmp_path):
    """A manifest entry that points at a shard written for another step must be refused even when the
    digest in the manifest matches that file."""
    cfg = GPT2Config.variant("gpt2", n_layer=1, n_head=1, d_model=8, vocab_size=11, max_seq_len=5, vocab_pad_to=1)
    specs = gpt2_param_specs(cfg)
    layout = FlatLayout(specs, world=1)
    fulls = [torch.randn(layout.n_total, generator=torch.Generator().manual_seed(i)) for i in range(3)]
    params = fulls[0].bfloat16()
    _write_sharded_by_hand(tmp_path, cfg, 1, 5, fulls, params)
    other = tmp_path / "other"
    other.mkdir()
    _write_sharded_by_hand(other, cfg, 1, 9, fulls, params)
    # swap in the step-9 shard under the step-5 name and make the manifest agree with its digest
    blob = (other / "optimizer_00000009.rank00000.bin").read_bytes()
    (tmp_path / "optimizer_00000005.rank00000.bin").write_bytes(blob)
    import hashlib
    man = json.loads((tmp_path / "optimizer_00000005.manifest.json").read_text())
    man["shards"][0]["sha256"] = json.loads((other / "optimizer_00000009.manifest.json").read_text())["shards"][0]["sha256"]
    (tmp_path / "optimizer_00000005.manifest.json").write_text(json.dumps(man))
    opt = SimpleNamespace(world=1, rank=0, lo=0, shard=layout.shard, step_count=0,
                          master=torch.empty(layout.shard), m=torch.empty(layout.shard), v=torch.empty(layout.shard))
    tr = SimpleNamespace(cfg=cfg, layout=layout, bufs=SimpleNamespace(params=torch.zeros(layout.n_total, dtype=torch.bfloat16)),
                         opt=opt, device=torch.device("cpu"))
    with pytest.raises(ValueError, match="header or checksum"):
        load_dense_checkpoint(tr, tmp_path)


def test_model_file_is_accepted_by_the_reference_reader(tmp_path):
    """The dense-v5 model file is a byte-for-byte contract: the reference's own pure-Python inspector
    (``neuralfn/native_dense_checkpoint.py``, importable from the ``baseline/_ref`` install) must accept
    our file and report the same geometry, tensor order, offsets, per-tensor digests and file digest."""
    import hashlib
    import importlib.util
    import sys
    from pathlib import Path
    ref_file = Path(__file__).resolve().parent.parent / "baseline" / "_ref" / "neuralfn" / "native_dense_checkpoint.py"
    if not ref_file.exists():
        pytest.skip("the reference package is not installed under baseline/_ref")
    spec = importlib.util.spec_from_file_location("_ref_native_dense_checkpoint", ref_file)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod   # dataclasses resolve their module through sys.modules
    try:
        spec.loader.exec_module(mod)
    finally:
        sys.modules.pop(spec.name, None)
    tr = _cpu_trainer()
    digests = save_dense_checkpoint(tr, tmp_path, sharded_optimizer=False)
    info = mod.inspect_native_dense_checkpoint(tmp_path / "model_00000007.bin")
    assert (info.max_seq_len, info.vocab_size, info.num_layers, info.num_heads, info.channels, info.padded_vocab_size) == (16, 100, 2, 2, 32, 128)
    assert info.sha256 == digests["model_00000007.bin"]
    ours = gpt2_param_specs(tr.cfg)
    assert info.parameter_count == sum(s.numel for s in ours) and len(info.tensors) == len(ours)
    raw = (tmp_path / "model_00000007.bin").read_bytes()
    for t, s in zip(info.tensors, ours):
        assert tuple(t.shape) == tuple(s.shape), (t.name, s.name)
        want = tr.layout.view(tr.bufs.params, s.name).contiguous().view(torch.uint8).numpy().tobytes()
        assert raw[t.offset:t.offset + t.nbytes] == want, s.name          # same tensor at the reference's offset
        assert t.sha256 == hashlib.sha256(want).hexdigest()


def _cpu_diff_trainer(seed=3):
    cfg = GPT2Config.variant("gpt2_diff", n_layer=3, n_head=2, d_model=128, vocab_size=100, max_seq_len=16)
    layout = FlatLayout(cfg.param_specs(), world=1)
    bufs = SymmetricBuffers(layout.n_total, torch.device("cpu"))
    master = torch.empty(layout.n_total)
    init_gpt2_params_(cfg, layout, master, seed)
    for l in range(cfg.n_layer):                       # distinct trained values
        layout.view(master, f"h.{l}.attn.diff_lambda")[0] = 0.8 - 0.1 * (l + 1) - 0.01 * seed
    opt = ShardedAdamW(layout, bufs, AdamWConfig(), master_init=master)
    bufs.params.copy_(master.bfloat16())
    opt.m.normal_(generator=torch.Generator().manual_seed(seed))
    opt.v.uniform_(generator=torch.Generator().manual_seed(seed + 1))
    opt.step_count = 5
    return SimpleNamespace(cfg=cfg, layout=layout, bufs=bufs, opt=opt, device=torch.device("cpu"))


def test_differential_variant_sidecars_roundtrip_and_are_required(tmp_path):
    a = _cpu_diff_trainer(seed=3)
    digests = save_dense_checkpoint(a, tmp_path, sharded_optimizer=False)
    # the dense model file holds exactly the ordinary tensors: lambdas live in the sidecars
    raw = (tmp_path / "model_00000005.bin").read_bytes()
    assert len(raw) == 1024 + 2 * sum(s.numel for s in gpt2_param_specs(a.cfg))
    lam = np.frombuffer((tmp_path / "diff_parameters_00000005.bin").read_bytes(), dtype="<f4")
    assert lam.shape == (3,) and np.allclose(lam, [0.67, 0.57, 0.47], atol=1e-6)
    assert len((tmp_path / "diff_optimizer_00000005.bin").read_bytes()) == 4 * 2 * 3
    meta = json.loads((tmp_path / "model_00000005.diff.json").read_text())
    assert meta["layers"] == 3 and meta["lambda_init"] == 0.8 and set(meta["sha256"]) <= set(digests)
    b = _cpu_diff_trainer(seed=9)
    got = load_dense_checkpoint(b, tmp_path)
    assert got["diff_sidecars"] and got["moments"]
    for l in range(3):
        name = f"h.{l}.attn.diff_lambda"
        for buf in ("master", "m", "v"):
            assert a.layout.view(getattr(a.opt, buf), name)[0] == b.layout.view(getattr(b.opt, buf), name)[0], (buf, l)
        assert a.layout.view(a.bufs.params, name)[0] == b.layout.view(b.bufs.params, name)[0]
    cfg, tensors, _sha = read_dense_model(tmp_path / "model_00000005.bin")
    assert cfg.differential and float(tensors["h.2.attn.diff_lambda"][0]) == pytest.approx(0.47, abs=4e-3)
    # a tampered or missing sidecar is refused
    (tmp_path / "diff_parameters_00000005.bin").write_bytes(b"\0" * 12)
    with pytest.raises(ValueError):
        load_dense_checkpoint(_cpu_diff_trainer(seed=1), tmp_path)
    (tmp_path / "model_00000005.diff.json").unlink()
    with pytest.raises(FileNotFoundError):
        load_dense_checkpoint(_cpu_diff_trainer(seed=1), tmp_path)
