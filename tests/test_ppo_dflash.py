"""PPO trainer and DFlash distillation on toy models (CPU)."""
import torch
import torch.nn as nn

from neuralfn_b200.tensor.dflash import (DFlashConfig, DFlashDistillationTrainer, build_block_inputs, dflash_attention_mask,
                                         dpace_position_weights, sample_anchor_positions)
from neuralfn_b200.tensor.ppo import PPOConfig, PPOTrainer, gae_advantages, masked_ppo_clipped_loss


class TinyPolicy(nn.Module):
    def __init__(self, V=12, d=32):
        super().__init__()
        self.emb = nn.Embedding(V, d)
        self.rnn = nn.GRU(d, d, batch_first=True)
        self.head, self.vhead = nn.Linear(d, V), nn.Linear(d, 1)

    def forward(self, ids):
        h, _ = self.rnn(self.emb(ids))
        return self.head(h), self.vhead(h).squeeze(-1)


def test_gae_and_clipped_loss_reference_values():
    r = torch.tensor([[0.0, 0.0, 1.0]])
    v = torch.tensor([[0.5, 0.4, 0.3]])
    adv, ret = gae_advantages(r, v, torch.ones(1, 3), gamma=1.0, lam=1.0)
    assert torch.allclose(adv, torch.tensor([[0.5, 0.6, 0.7]]), atol=1e-6) and torch.allclose(ret, torch.ones(1, 3), atol=1e-6)
    lp, old = torch.log(torch.tensor([[0.5, 0.2]])), torch.log(torch.tensor([[0.25, 0.4]]))
    loss, frac = masked_ppo_clipped_loss(lp, old, torch.tensor([[1.0, -1.0]]), torch.ones(1, 2), 0.2)
    # ratios 2.0 (clipped to 1.2 for A > 0) and 0.5 (clipped to 0.8 for A < 0)
    assert abs(float(loss) - (-1.2 + 0.8) / 2) < 1e-6 and float(frac) == 1.0


def test_ppo_raises_reward_on_a_toy_task():
    torch.manual_seed(0)
    pol, ref = TinyPolicy(), TinyPolicy()
    ref.load_state_dict(pol.state_dict())
    for p in ref.parameters():
        p.requires_grad_(False)
    reward = lambda ids, P: (ids[:, P:] == 7).float().mean(1)  # noqa: E731 - likes token 7
    tr = PPOTrainer(pol, lambda x: ref(x)[0], reward, PPOConfig(max_new_tokens=6, kl_coef=0.01, learning_rate=3e-3, minibatch_size=16,
                                                              ppo_epochs_per_rollout=2, seed=1))
    prompts = torch.randint(0, 12, (32, 3))
    first = tr.step(prompts)["mean_score"]
    for _ in range(25):
        info = tr.step(prompts)
    assert info["mean_score"] > first + 0.25, (first, info)
    assert info["updates"] == 4 and 0 <= info["clip_fraction"] <= 1


def test_dpace_weights_and_block_construction():
    conf = torch.tensor([[1.0, 0.5, 0.0]])
    w = dpace_position_weights(conf, alpha=0.5)
    # smoothed = [1, .75, .5]; cumprod = [1, .75, .375]; suffix sums = [2.125, 1.125, .375]
    assert torch.allclose(w, torch.tensor([[2.125, 1.125, 0.375]]))
    wv = dpace_position_weights(conf, 0.5, torch.tensor([[True, False, True]]))
    assert torch.allclose(wv, torch.tensor([[1.5, 0.5, 0.5]]))  # the skipped slot neither shrinks nor counts
    mask = torch.ones(2, 20)
    mask[1, :5] = 0
    g = torch.Generator().manual_seed(0)
    anchors, keep = sample_anchor_positions(mask, block_size=4, num_anchors=3, generator=g)
    assert anchors.shape == (2, 3) and keep.all() and (anchors[1] >= 5).all() and (anchors <= 16).all()
    assert (anchors[:, 1:] > anchors[:, :-1]).all()
    ids = torch.arange(40).view(2, 20)
    blk, pos, tgt = build_block_inputs(ids, anchors, 4, mask_token_id=99)
    assert (blk[..., 0] == ids.gather(1, anchors)).all() and (blk[..., 1:] == 99).all() and (pos[..., 1] == anchors + 1).all()
    m = dflash_attention_mask(20, anchors, 4, context_window=6)
    a = int(anchors[0, 0])
    assert m.shape == (2, 3, 4, 24) and m[0, 0, 0, max(0, a - 6):a].all() and not m[0, 0, 0, a:20].any() and m[0, 0, :, 20:].all()


def test_dflash_distillation_learns_a_deterministic_teacher():
    torch.manual_seed(0)
    V, C, T = 16, 24, 32
    emb = nn.Embedding(V, C)
    # teacher: next token = (token + 1) % V, expressed through hidden taps that carry the current token
    def target(ids):
        h0 = emb(ids)
        logits = torch.full((*ids.shape, V), -8.0)
        logits.scatter_(-1, ((ids + 1) % V)[..., None], 8.0)
        return {"hidden_states": [h0, h0 * 1.0, h0 * 0.5], "logits": logits}
    head = nn.Linear(C, V, bias=False)
    cfg = DFlashConfig(d_model=48, n_layer=2, n_head=4, block_size=4, num_anchors=4, context_window=8, tap_layers=(0, 1), mask_token_id=0,
                       learning_rate=5e-3, dpace_alpha=0.5)
    tr = DFlashDistillationTrainer(cfg, target, lambda i: emb(i).detach(), lambda h: head(h), C)
    # the shared LM head is frozen in real use; here it is random, so let the draft learn through it
    start = torch.randint(0, V, (16, 1))
    ids = (start + torch.arange(T)[None]) % V
    losses = [tr.train_step(ids) for _ in range(150)]
    assert losses[-1] < 0.5 * losses[0], (losses[0], losses[-1])
    acc = tr.evaluate_greedy_acceptance(ids)
    assert acc["mean_accepted_tokens"] > 1.5 and acc["blocks"] > 0
    sd = tr.state_dict()
    tr2 = DFlashDistillationTrainer(cfg, target, lambda i: emb(i).detach(), lambda h: head(h), C)
    tr2.load_state_dict(sd)
    assert tr2.state.step == 150 and torch.equal(tr2.draft.slot, tr.draft.slot)
