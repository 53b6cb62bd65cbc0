"""Tensor runtime on CPU: every preset builds, compiles and trains a step; stage math;
post-training graphs; save/resume strictness; adapters."""
import math

import pytest
import torch
import torch.nn.functional as F

from neuralfn_b200 import presets
from neuralfn_b200.config import FineTuneSpec, spec_from_dict
from neuralfn_b200.serialization import graph_from_json, graph_to_json
from neuralfn_b200.torch_backend import CompiledTorchGraph, TorchTrainConfig, TorchTrainer, build_module
from neuralfn_b200.torch_templates import build_gpt_root_graph

SMALL = dict(vocab_size=64, num_layers=2, model_dim=32, num_heads=4)


@pytest.mark.parametrize("name", presets.preset_names())
def test_preset_builds_compiles_and_runs(name):
    kw = dict(SMALL)
    if name.startswith("muse"):
        kw["num_layers"] = 4
    spec = presets.build_preset(name, **kw)
    assert spec_from_dict(spec.to_dict()).to_dict() == spec.to_dict()
    graph = build_gpt_root_graph(spec)
    rt = graph_from_json(graph_to_json(graph))          # JSON round trip incl. variant library
    model = CompiledTorchGraph(rt)
    names = [rt.nodes[n].neuron_def.output_ports[0].name for n in rt.input_node_ids]
    expected = {"seq2seq": ["enc_tokens", "dec_tokens", "target_ids"], "diffusion": ["tokens"], "jepa": ["tokens"]}
    objective = spec.template.objective
    if "semantic" in objective:
        assert names == ["tokens", "target_ids", "sem_targets"]
    else:
        assert names == expected.get(objective, ["tokens", "target_ids"])
    inputs = []
    for n in names:
        if n == "sem_targets":
            sem = torch.full((2, 9), -100)
            sem[:, 0], sem[0, 3] = 1, 2
            inputs.append(sem)
        else:
            inputs.append(torch.randint(0, 64, (2, 16)))
    loss = model(*inputs)[0]
    assert loss.ndim == 0 and torch.isfinite(loss)
    loss.backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in model.parameters())


def test_compiler_rejects_fan_in_and_cycles():
    from neuralfn_b200.graph import Edge
    spec = presets.build_preset("gpt2", **SMALL)
    g = build_gpt_root_graph(spec)
    e = next(iter(g.edges.values()))
    g.add_edge(Edge(id="dup", src_node=e.src_node, src_port=e.src_port, dst_node=e.dst_node, dst_port=e.dst_port))
    with pytest.raises(ValueError, match="multiple incoming edges"):
        CompiledTorchGraph(g)


def test_trace_has_nested_keys():
    spec = presets.build_preset("llama", **SMALL)
    model = CompiledTorchGraph(build_gpt_root_graph(spec))
    out, trace = model.trace(torch.randint(0, 64, (1, 8)), torch.randint(0, 64, (1, 8)))
    assert "block_0" in trace and any(k.startswith("block_0/attention/") for k in trace)


def test_trainer_learns_and_resumes(tmp_path):
    torch.manual_seed(0)
    spec = presets.build_preset("gpt2_stable", **SMALL)
    graph = build_gpt_root_graph(spec)
    data = torch.randint(0, 64, (32, 17))
    x, y = data[:, :-1], data[:, 1:]
    cfg = TorchTrainConfig(learning_rate=3e-3, epochs=6, batch_size=8, device="cpu", seed=1, grad_clip_norm=1.0)
    tr = TorchTrainer(graph, cfg)
    steps = []
    hist = tr.train(x, y, on_step=steps.append)
    assert hist[-1] < hist[0]
    assert steps[-1]["step"] == tr.global_step and "learning_rates" in steps[-1]
    ckpt = tmp_path / "train.pt"
    tr.save_training_checkpoint(ckpt)
    # resume into a fresh trainer on the same topology
    tr2 = TorchTrainer(graph_from_json(graph_to_json(graph)), cfg)
    tr2.load_training_checkpoint(ckpt)
    tr2.train(x, y)
    assert tr2.global_step > tr.global_step
    # a different topology is refused
    other = build_gpt_root_graph(presets.build_preset("gpt2", **{**SMALL, "num_layers": 3}))
    with pytest.raises(ValueError, match="different graph topology"):
        TorchTrainer(other, cfg).load_training_checkpoint(ckpt)


def test_sft_dpo_reward_ppo_graphs(tmp_path):
    from neuralfn_b200.inference import export_to_pt
    from neuralfn_b200.serialization import save_graph
    from neuralfn_b200.torch_templates import build_model_stage_graph
    base = presets.build_preset("llama", **SMALL)
    B, T = 2, 12
    tok = torch.randint(0, 64, (B, T))
    tgt = torch.randint(0, 64, (B, T))
    mask = torch.ones(B, T)
    mask[:, :4] = 0
    # SFT
    sft = presets.build_preset("llama", finetune=FineTuneSpec(objective="sft"), **SMALL)
    loss = CompiledTorchGraph(build_gpt_root_graph(sft))(tok, tgt, mask)[0]
    assert torch.isfinite(loss)
    # frozen reference for DPO
    ref_graph = build_model_stage_graph(base, with_loss=False)
    save_graph(ref_graph, tmp_path / "ref.json", include_module_state=False)
    export_to_pt(ref_graph, tmp_path / "ref.pt")
    dpo = presets.build_preset("llama", finetune=FineTuneSpec(objective="dpo", ref_graph_path=str(tmp_path / "ref.json"),
                                                              ref_checkpoint=str(tmp_path / "ref.pt")), **SMALL)
    m = CompiledTorchGraph(build_gpt_root_graph(dpo))
    loss = m(tok, tgt, mask, tok.flip(0), tgt.flip(0), mask)[0]
    assert torch.isfinite(loss)
    loss.backward()
    # reward model
    rm = presets.build_preset("llama", finetune=FineTuneSpec(objective="reward_model"), **SMALL)
    loss = CompiledTorchGraph(build_gpt_root_graph(rm))(tok, mask, tok.flip(1), mask)[0]
    assert torch.isfinite(loss)
    # PPO update graph
    ppo = presets.build_preset("llama", finetune=FineTuneSpec(objective="ppo"), **SMALL)
    z = torch.zeros(B, T)
    loss = CompiledTorchGraph(build_gpt_root_graph(ppo))(tok, tgt, mask, z - 3.0, z, torch.randn(B, T), z)[0]
    assert torch.isfinite(loss)


def test_lora_and_nf4_freeze_base_and_merge():
    from neuralfn_b200.inference import merge_adapter_into_base
    from neuralfn_b200.tensor.stages_linear import nf4_dequantize, nf4_quantize
    w = torch.randn(16, 128) * 0.1
    packed, absmax = nf4_quantize(w, 64)
    deq = nf4_dequantize(packed, absmax, 64)
    assert (deq - w).abs().max() < 0.15 * w.abs().max()   # widest NF4 code gap is 0.277 of absmax
    assert packed.dtype == torch.uint8 and packed.shape == (16, 64) and absmax.shape == (16, 2)
    spec = presets.build_preset("llama", adapter_type="lora", lora_targets=("q_proj", "v_proj"), **SMALL)
    graph = build_gpt_root_graph(spec)
    data = torch.randint(0, 64, (16, 9))
    tr = TorchTrainer(graph, TorchTrainConfig(learning_rate=1e-2, epochs=2, batch_size=8, device="cpu", seed=0))
    tr.train(data[:, :-1], data[:, 1:])
    trainable = [n for n, p in tr.compiled.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    x = torch.randint(0, 64, (1, 8))
    before = tr.compiled(x, x)[0]
    assert merge_adapter_into_base(tr.compiled) == 4
    assert torch.allclose(tr.compiled(x, x)[0], before, atol=1e-4)


def test_stage_math_spot_checks():
    ce = build_module("token_cross_entropy", {"z_loss_coef": 1e-2})
    logits, tgt = torch.randn(2, 5, 11), torch.randint(0, 11, (2, 5))
    lse = torch.logsumexp(logits.reshape(-1, 11), -1)
    want = F.cross_entropy(logits.reshape(-1, 11), tgt.reshape(-1)) + 1e-2 * lse.pow(2).mean()
    assert torch.allclose(ce(logits, tgt), want, atol=1e-6)
    lb = build_module("load_balance_loss", {"experts": 4})
    rl = torch.randn(2, 3, 4)
    dens = F.softmax(rl, -1).mean((0, 1))
    assert torch.allclose(lb(rl, None, None)[0], 4 * (dens * dens).sum())
    route = build_module("topk_route", {"top_k": 2, "experts": 4})
    w, idx = route(rl)
    assert torch.allclose(w.sum(-1), torch.ones(2, 3)) and idx.shape == (2, 3, 2)
    sel = torch.softmax(torch.gather(rl, -1, idx), -1)   # top-k of softmax renormalised == softmax over selected
    assert torch.allclose(w, sel, atol=1e-6)
    rope = build_module("rotary_embedding", {"head_dim": 8, "rope_base": 10000.0, "convention": "legacy"})
    hf = build_module("rotary_embedding", {"head_dim": 8, "rope_base": 10000.0, "convention": "hf"})
    q = torch.randn(1, 2, 5, 8)
    ql, _ = rope(q, q)
    qh, _ = hf(q, q)
    assert torch.allclose(ql.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    assert torch.allclose(ql[:, :, 0], q[:, :, 0]) and not torch.allclose(ql[:, :, 3], qh[:, :, 3])
    gae = build_module("gae_compute", {"gamma": 1.0, "lambda_": 1.0})
    adv, ret = gae(torch.tensor([[1.0, 1.0, 1.0]]), torch.zeros(1, 3))
    assert adv.tolist() == [[3.0, 2.0, 1.0]] and ret.tolist() == [[3.0, 2.0, 1.0]]
    mhc = build_module("manifold_hyper_connection", {"dim": 4, "beta_init": 0.6})
    x, d = torch.ones(1, 4), torch.zeros(1, 4)
    assert torch.allclose(mhc(x, d), math.sqrt(1 - 0.36) * x, atol=1e-5)
    moe = build_module("expert_dispatch", {"model_dim": 8, "experts": 4, "mlp_mult": 2.0})
    xx = torch.randn(2, 3, 8)
    ww, ii = torch.full((2, 3, 2), 0.5), torch.randint(0, 4, (2, 3, 2))
    got = moe(xx, ww, ii)
    want = torch.zeros_like(xx)
    for b in range(2):
        for t in range(3):
            for k in range(2):
                e = ii[b, t, k]
                h = F.silu(xx[b, t] @ moe.w1[e]) * (xx[b, t] @ moe.w3[e])
                want[b, t] += 0.5 * (h @ moe.w2[e])
    assert torch.allclose(got, want, atol=1e-5)
