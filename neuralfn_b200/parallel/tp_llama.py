"""Tensor-parallel Llama training: sequence-parallel residual stream, column / row parallel
projections whose all-gather and reduce-scatter run inside the GEMM kernels.

Layout for a TP group of W ranks over M = batch x seq token rows:
  * the residual stream, the norms, the embedding lookup and the LM head work on this rank's
    M / W rows (sequence parallel); embedding, head and norm weights are replicated and their
    gradients summed over the group after the backward pass;
  * ``wqkv`` and ``w_gate_up`` are column-parallel (rows of the weight split by head / by hidden
    unit): all-gather(rows) -> GEMM gives [M, N / W]; attention runs on H / W query heads and
    Hkv / W key-value heads over the full sequence;
  * ``wo`` and ``w_down`` are row-parallel (the contraction dimension split): GEMM ->
    reduce-scatter (+ residual) gives this rank's [M / W, d] rows again.
The backward pass uses the transposed pairing: d(column-parallel input) is GEMM ->
reduce-scatter with the transposed weight shard, d(row-parallel input) is all-gather -> GEMM,
and both weight gradients are local GEMMs against the gathered operand, accumulated straight
into the flat gradient buffer.

``TPLlama`` holds the shards in one flat bf16 parameter buffer (sharded tensors first) with a
flat gradient buffer of the same layout; ``TPLlamaTrainer`` adds fp32 master weights and the
fused flat AdamW with a group-wide clipping norm. On CPU (gloo) every collective GEMM falls
back to ``torch.distributed`` + matmul, which is what the parity tests run.

The reference trains dense models on one GPU only; tensor parallelism is on its to-do list
(``todo-kernels.md:133-145``). The model is the Llama block of ``neuralfn/torch_templates.py``
(RMSNorm, rotary GQA attention, SwiGLU), the same as ``models/llama.py`` here.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..models.gpt2 import FlatLayout, ParamSpec
from ..models.llama import LlamaConfig
from ..tensor import kernel_bridge as KB
from .dp import AdamWConfig, lr_at_step
from .tp import TensorParallelContext

__all__ = ["tp_dp_mesh", "TPLlama", "TPLlamaTrainer", "shard_llama_params", "tp_llama_param_specs"]


# ------------------------------------------------------------------ parameter sharding --
def tp_vocab_rows(cfg: LlamaConfig, world: int) -> int:
    """Rows of the embedding / head shard of one rank: the vocabulary padded so that every shard is a
    whole number of 128-row GEMM tiles."""
    q = 128 * world
    return (cfg.vocab_size + q - 1) // q * 128


def tp_llama_param_specs(cfg: LlamaConfig, world: int) -> list[ParamSpec]:
    C, hd, Vl = cfg.d_model, cfg.head_dim, tp_vocab_rows(cfg, world)
    if cfg.n_head % world or cfg.n_kv_head % world or cfg.d_ff % world:
        raise ValueError(f"heads ({cfg.n_head}/{cfg.n_kv_head}) and d_ff ({cfg.d_ff}) must divide by the TP size {world}")
    if cfg.tie_embeddings or cfg.qk_norm or cfg.logit_softcap > 0:
        raise ValueError("the tensor-parallel Llama supports untied embeddings without qk-norm or logit soft-capping")
    Hq, Hkv, Fl = cfg.n_head // world, cfg.n_kv_head // world, cfg.d_ff // world
    specs = []
    for l in range(cfg.n_layer):
        p = f"layers.{l}."
        specs += [ParamSpec(p + "wqkv", ((Hq + 2 * Hkv) * hd, C), True, "normal"), ParamSpec(p + "wo", (C, Hq * hd), True, "resid"),
                  ParamSpec(p + "w_gate_up", (2 * Fl, C), True, "normal"), ParamSpec(p + "w_down", (C, Fl), True, "resid")]
    # vocabulary-parallel: every rank keeps Vl consecutive rows of the embedding and of the head
    specs += [ParamSpec("tok_embeddings", (Vl, C), True, "normal"), ParamSpec("lm_head", (Vl, C), True, "normal")]
    for l in range(cfg.n_layer):
        specs += [ParamSpec(f"layers.{l}.attn_norm", (C,), False, "ones"), ParamSpec(f"layers.{l}.ffn_norm", (C,), False, "ones")]
    specs.append(ParamSpec("norm", (C,), False, "ones"))
    return specs


def is_sharded(name: str) -> bool:
    return name.endswith((".wqkv", ".wo", ".w_gate_up", ".w_down")) or name in ("tok_embeddings", "lm_head")


def shard_llama_params(cfg: LlamaConfig, full: dict[str, torch.Tensor], rank: int, world: int) -> dict[str, torch.Tensor]:
    """This rank's tensors cut out of an unsharded parameter dictionary (names of ``models/llama.py``)."""
    hd, F_ = cfg.head_dim, cfg.d_ff
    Hq, Hkv, Fl = cfg.n_head // world, cfg.n_kv_head // world, cfg.d_ff // world
    q0, k0, v0 = 0, cfg.n_head * hd, (cfg.n_head + cfg.n_kv_head) * hd
    out = {}
    for name, t in full.items():
        if name.endswith(".wqkv"):
            out[name] = torch.cat([t[q0 + rank * Hq * hd:q0 + (rank + 1) * Hq * hd], t[k0 + rank * Hkv * hd:k0 + (rank + 1) * Hkv * hd],
                                   t[v0 + rank * Hkv * hd:v0 + (rank + 1) * Hkv * hd]], 0)
        elif name.endswith(".wo"):
            out[name] = t[:, rank * Hq * hd:(rank + 1) * Hq * hd]
        elif name.endswith(".w_gate_up"):
            out[name] = torch.cat([t[rank * Fl:(rank + 1) * Fl], t[F_ + rank * Fl:F_ + (rank + 1) * Fl]], 0)
        elif name.endswith(".w_down"):
            out[name] = t[:, rank * Fl:(rank + 1) * Fl]
        elif name in ("tok_embeddings", "lm_head"):
            Vl = tp_vocab_rows(cfg, world)
            rows = t[rank * Vl:(rank + 1) * Vl]          # rows past the end of the table are zero padding
            out[name] = torch.cat([rows, torch.zeros(Vl - rows.shape[0], t.shape[1], dtype=t.dtype)], 0) if rows.shape[0] < Vl else rows
        else:
            out[name] = t
    return {k: v.contiguous() for k, v in out.items()}


# ------------------------------------------------------------------- autograd functions --
def _matmul_tn(dy: torch.Tensor, x: torch.Tensor, into: torch.Tensor) -> None:
    """into += dy^T x  (dy [M, N], x [M, K], into [N, K])."""
    if dy.is_cuda and dy.dtype == torch.bfloat16:
        from ..ops.gemm import gemm
        gemm(dy, x, a_mn=True, b_mn=True, out=into, accum=True)
    else:
        into += (dy.float().T @ x.float()).to(into.dtype)


class _ColumnParallel(torch.autograd.Function):
    """x_local [M / W, K], weight [N / W, K] -> [M, N / W]."""

    @staticmethod
    def forward(ctx, x_local, weight, tp: TensorParallelContext):
        y, x_full = tp.column_linear(x_local, weight, return_gathered=True)
        ctx.save_for_backward(x_full.clone() if tp.impl == "fused" else x_full)
        ctx.tp, ctx.weight = tp, weight
        return y

    @staticmethod
    def backward(ctx, dy):
        (x_full,), weight = ctx.saved_tensors, ctx.weight
        dy = dy.contiguous()
        dx_local = ctx.tp.row_linear(dy, weight.t().contiguous())
        _matmul_tn(dy, x_full, weight.main_grad)
        return dx_local, None, None


class _RowParallel(torch.autograd.Function):
    """x [M, K / W], weight [N, K / W], resid [M / W, N] -> [M / W, N] (+ resid)."""

    @staticmethod
    def forward(ctx, x, weight, resid, tp: TensorParallelContext):
        ctx.save_for_backward(x)
        ctx.tp, ctx.weight = tp, weight
        return tp.row_linear(x, weight, resid=resid)

    @staticmethod
    def backward(ctx, dy_local):
        (x,), weight = ctx.saved_tensors, ctx.weight
        dy_local = dy_local.contiguous()
        dx, dy_full = ctx.tp.column_linear(dy_local, weight.t().contiguous(), return_gathered=True)
        _matmul_tn(dy_full, x, weight.main_grad)  # dy_full is consumed before the next collective GEMM
        return dx, None, dy_local, None


def _group_reduce_scatter(full: torch.Tensor, tp: TensorParallelContext) -> torch.Tensor:
    """[M, C] partial sums on every rank -> this rank's [M / W, C] rows of the total."""
    W = tp.world
    if W == 1:
        return full
    rows = full.shape[0] // W
    out = torch.empty(rows, full.shape[1], dtype=full.dtype, device=full.device)
    if full.is_cuda:
        dist.reduce_scatter_tensor(out, full.contiguous(), group=tp.group)
    else:
        dist.reduce_scatter(out, [c.contiguous() for c in full.chunk(W, 0)], group=tp.group)
    return out


def _group_all_gather(local: torch.Tensor, tp: TensorParallelContext) -> torch.Tensor:
    W = tp.world
    if W == 1:
        return local
    full = torch.empty(W * local.shape[0], *local.shape[1:], dtype=local.dtype, device=local.device)
    if local.is_cuda:
        dist.all_gather_into_tensor(full, local.contiguous(), group=tp.group)
    else:
        parts = [torch.empty_like(local) for _ in range(W)]
        dist.all_gather(parts, local.contiguous(), group=tp.group)
        full.copy_(torch.cat(parts, 0))
    return full


class _VocabParallelEmbedding(torch.autograd.Function):
    """tokens [M] (all of them, on every rank), weight [Vl, C] (rows v0 ... v0 + Vl of the table) -> this
    rank's [M / W, C] rows of the embedded sequence. Every rank looks up the tokens that fall into its
    rows (zero elsewhere); a reduce-scatter adds the shards and hands each rank its sequence slice."""

    @staticmethod
    def forward(ctx, tokens, weight, tp: TensorParallelContext):
        Vl = weight.shape[0]
        v0 = tp.rank * Vl
        idx = tokens.long() - v0
        mine = (idx >= 0) & (idx < Vl)
        part = F.embedding(idx.clamp(0, Vl - 1), weight) * mine.unsqueeze(-1).to(weight.dtype)
        ctx.save_for_backward(idx.clamp(0, Vl - 1), mine)
        ctx.tp, ctx.weight = tp, weight
        return _group_reduce_scatter(part, tp)

    @staticmethod
    def backward(ctx, dy_local):
        idx, mine = ctx.saved_tensors
        dy = _group_all_gather(dy_local.contiguous(), ctx.tp)                 # [M, C]
        ctx.weight.main_grad.index_add_(0, idx[mine], dy[mine].to(ctx.weight.main_grad.dtype))
        return None, None, None


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """logits_local [M, Vl] (this rank's vocabulary columns of every row), targets [M] -> mean over rows of
    lse - logit[target] + z * lse^2. Three small exchanges per step - row maxima, row sums of exponentials
    and the target logits, [M] floats each - replace the gather of the logits; the full-vocabulary logits
    never exist on one rank. The backward pass turns the logits into their gradient in place."""

    @staticmethod
    def forward(ctx, logits, targets, z_coef: float, vocab_size: int, tp: TensorParallelContext):
        M, Vl = logits.shape
        v0 = tp.rank * Vl
        live = min(max(vocab_size - v0, 0), Vl)                                  # columns of real vocabulary entries
        lf = logits.float()
        if live < Vl:
            lf[:, live:] = float("-inf")
        mx = lf.max(dim=-1).values if live > 0 else torch.full((M,), float("-inf"), device=logits.device)
        if tp.world > 1:
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=tp.group)
        ex = torch.exp(lf - mx.unsqueeze(-1))
        stats = torch.stack([ex.sum(-1), torch.zeros_like(mx)], 0)
        idx = targets.long() - v0
        mine = (idx >= 0) & (idx < live)
        stats[1] = torch.where(mine, lf.gather(1, idx.clamp(0, Vl - 1).unsqueeze(1)).squeeze(1), torch.zeros_like(mx))
        if tp.world > 1:
            dist.all_reduce(stats, group=tp.group)
        lse = mx + torch.log(stats[0])
        loss = (lse - stats[1] + z_coef * lse * lse).mean()
        ctx.save_for_backward(ex, stats[0], lse, idx.clamp(0, Vl - 1), mine)
        ctx.z, ctx.dtype = z_coef, logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        ex, denom, lse, idx, mine = ctx.saved_tensors
        M = ex.shape[0]
        d = ex * ((1.0 + 2.0 * ctx.z * lse) / denom).unsqueeze(-1)            # softmax * d(loss_row)/d(lse)
        d[mine, idx[mine]] -= 1.0
        return (d * (g / M)).to(ctx.dtype), None, None, None, None


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, sign: float) -> torch.Tensor:
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    return torch.cat((a * cos - sign * b * sin, b * cos + sign * a * sin), dim=-1)


# ------------------------------------------------------------------------------- model --
def tp_dp_mesh(tp_size: int):
    """Splits the default process group into a TP x DP mesh: consecutive ranks form a tensor-parallel group (they
    share NVLink peer memory for the fused collective GEMMs), ranks with the same position in their groups form a
    data-parallel group. Collective: every rank creates every group. Returns (tp_group, dp_group, tp_index, dp_index)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if tp_size < 1 or world % tp_size:
        raise ValueError(f"world size {world} is not a multiple of the tensor-parallel size {tp_size}")
    n_dp = world // tp_size
    tp_group = dp_group = None
    for d in range(n_dp):
        g = dist.new_group(list(range(d * tp_size, (d + 1) * tp_size)))
        if rank // tp_size == d:
            tp_group = g
    for t in range(tp_size):
        g = dist.new_group([d * tp_size + t for d in range(n_dp)])
        if rank % tp_size == t:
            dp_group = g
    return tp_group, dp_group, rank % tp_size, rank // tp_size


class TPLlama:
    def __init__(self, cfg: LlamaConfig, tp: TensorParallelContext, *, dtype=None, seed: int = 1337,
                 full_params: dict[str, torch.Tensor] | None = None, dp_group=None) -> None:
        """``dp_group``: the ranks that hold the SAME shard in other tensor-parallel groups (a TP x DP mesh, see
        ``tp_dp_mesh``); every replica trains on its own batch and gradients are averaged over that group."""
        self.cfg, self.tp = cfg, tp
        self.dp_group = dp_group
        self.dp_world = dist.get_world_size(dp_group) if dp_group is not None else 1
        dev = tp.device
        self.dtype = dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        self.layout = FlatLayout(tp_llama_param_specs(cfg, tp.world))
        self.n_sharded = self.layout.offsets["layers.0.attn_norm"]  # the sharded tensors (incl. embedding and head rows) come first
        self.params = torch.zeros(self.layout.n_total, dtype=self.dtype, device=dev)
        self.grads = torch.zeros_like(self.params)
        self.p = {}
        gviews = self.layout.views(self.grads)
        for name, view in self.layout.views(self.params).items():
            view.requires_grad_(True)
            view.main_grad = gviews[name]
            self.p[name] = view
        if full_params is not None:
            self.load_full(full_params)
        else:
            self.init_(seed)

    @torch.no_grad()
    def init_(self, seed: int) -> None:
        """N(0, 0.02) (residual projections scaled by 1 / sqrt(2 L)); shards draw from streams
        keyed by (seed, rank), replicated tensors from (seed) alone so every rank agrees."""
        dev = self.params.device
        g_rep = torch.Generator(device=dev).manual_seed(seed)
        g_shard = torch.Generator(device=dev).manual_seed(seed * 1000003 + 17 + self.tp.rank)
        for s in self.layout.order:
            v = self.p[s.name]
            gen = g_shard if is_sharded(s.name) else g_rep
            if s.init == "ones":
                v.fill_(1.0)
            else:
                std = 0.02 / math.sqrt(2 * self.cfg.n_layer) if s.init == "resid" else 0.02
                v.copy_(torch.empty(v.shape, dtype=torch.float32, device=dev).normal_(0.0, std, generator=gen))
        Vl = tp_vocab_rows(self.cfg, self.tp.world)
        live = min(max(self.cfg.vocab_size - self.tp.rank * Vl, 0), Vl)
        for name in ("tok_embeddings", "lm_head"):
            self.p[name][live:].zero_()                       # rows of the vocabulary padding

    @torch.no_grad()
    def load_full(self, full: dict[str, torch.Tensor]) -> None:
        for name, t in shard_llama_params(self.cfg, full, self.tp.rank, self.tp.world).items():
            self.p[name].copy_(t)

    @torch.no_grad()
    def full_state(self) -> dict[str, torch.Tensor]:
        """Unsharded fp32 parameters on the host under the names of ``models/llama.py`` (shards
        gathered over the group and put back in head / hidden-unit order): the inverse of
        ``shard_llama_params``, so a tensor-parallel run exports what the single-GPU engines load."""
        cfg, W = self.cfg, self.tp.world
        hd, Hq, Hkv, Fl = cfg.head_dim, cfg.n_head // W, cfg.n_kv_head // W, cfg.d_ff // W
        out = {}
        for name, v in self.p.items():
            t = v.detach().float().contiguous()
            if is_sharded(name) and W > 1:
                parts = [torch.empty_like(t) for _ in range(W)]
                dist.all_gather(parts, t, group=self.tp.group)
            else:
                parts = [t]
            if not is_sharded(name):
                full = t
            elif name.endswith(".wqkv"):
                full = torch.cat([q[:Hq * hd] for q in parts] + [q[Hq * hd:(Hq + Hkv) * hd] for q in parts] + [q[(Hq + Hkv) * hd:] for q in parts], 0)
            elif name.endswith(".w_gate_up"):
                full = torch.cat([q[:Fl] for q in parts] + [q[Fl:] for q in parts], 0)
            elif name in ("tok_embeddings", "lm_head"):
                full = torch.cat(parts, 0)[:cfg.padded_vocab]
                if full.shape[0] < cfg.padded_vocab:
                    full = torch.cat([full, torch.zeros(cfg.padded_vocab - full.shape[0], full.shape[1])], 0)
            else:  # wo / w_down: column shards
                full = torch.cat(parts, 1)
            out[name] = full.cpu()
        return out

    def _tables(self, T: int, device):
        hd = self.cfg.head_dim
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
        ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
        return ang.cos().to(device, self.dtype)[None, :, None], ang.sin().to(device, self.dtype)[None, :, None]

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """tokens, targets [B, T] (the same on every rank of the group). Returns this rank's share
        of the mean token loss: summing it over the group gives the batch mean."""
        cfg, tp, p = self.cfg, self.tp, self.p
        B, T = tokens.shape
        M, W = B * T, tp.world
        if M % W:
            raise ValueError(f"batch x seq = {M} must divide by the TP size {W}")
        rows = M // W
        if tp.impl == "fused" and rows % 128:
            raise ValueError(f"the fused collective GEMMs work on 128-row tiles: batch x seq / TP size = {rows} must be a multiple of 128 "
                             "(or build the context with impl='nccl')")
        lo = tp.rank * rows
        hd, Hq, Hkv, Fl = cfg.head_dim, cfg.n_head // W, cfg.n_kv_head // W, cfg.d_ff // W
        if getattr(self, "_rope_T", None) != (T, tokens.device):
            hd_ = cfg.head_dim
            inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd_, 2, dtype=torch.float64) / hd_))
            ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
            self._rope_f32 = (ang.cos().float().to(tokens.device).contiguous(), ang.sin().float().to(tokens.device).contiguous())
            self._rope_T = (T, tokens.device)
        x = _VocabParallelEmbedding.apply(tokens.reshape(-1), p["tok_embeddings"], tp)
        for l in range(cfg.n_layer):
            q_ = f"layers.{l}."
            h = KB.rms_norm(x, p[q_ + "attn_norm"], cfg.norm_eps)
            qkv = _ColumnParallel.apply(h, p[q_ + "wqkv"], tp)
            qkv = KB.rope_packed_qkv(qkv, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=self._rope_f32[0], sin=self._rope_f32[1],
                                     convention=cfg.rope_convention)
            a = KB.attention_packed_qkv(qkv, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, causal=True, window=cfg.window)
            x = _RowParallel.apply(a, p[q_ + "wo"], x, tp)
            h = KB.rms_norm(x, p[q_ + "ffn_norm"], cfg.norm_eps)
            gu = _ColumnParallel.apply(h, p[q_ + "w_gate_up"], tp)
            x = _RowParallel.apply(KB.swiglu(gu, Fl), p[q_ + "w_down"], x, tp)
        x = KB.rms_norm(x, p["norm"], cfg.norm_eps)
        # vocabulary-parallel head: all-gather -> GEMM like every other column-parallel product, then a
        # cross-entropy that exchanges three [M] vectors instead of the logits
        logits = _ColumnParallel.apply(x, p["lm_head"], tp)                      # [M, Vl]
        full = _VocabParallelCrossEntropy.apply(logits, targets.reshape(-1), float(cfg.z_loss), cfg.vocab_size, tp)
        # every rank holds the whole batch mean; callers sum the returned shares over the group, so hand
        # back 1 / W of the value while the gradient stays that of the full loss
        return full - full.detach() * (1.0 - 1.0 / W)

    def backward(self, loss: torch.Tensor) -> None:
        """Fills the flat gradient buffer: sharded weights are accumulated by the parallel
        linears themselves, replicated ones come from autograd and are summed over the group."""
        self.grads.zero_()
        rep = [v for n, v in self.p.items() if not is_sharded(n)]
        for v in rep:
            v.grad = None
        loss.backward()
        with torch.no_grad():
            for v in rep:
                if v.grad is not None:
                    v.main_grad.copy_(v.grad)
                    v.grad = None
            if self.tp.world > 1:
                dist.all_reduce(self.grads[self.n_sharded:], group=self.tp.group)
            if self.dp_world > 1:
                # replicas of this shard saw different batches: one flat all-reduce averages the whole buffer
                dist.all_reduce(self.grads, group=self.dp_group)
                self.grads.mul_(1.0 / self.dp_world)

    def reduce_loss(self, share: torch.Tensor) -> torch.Tensor:
        """Batch-mean loss from this rank's share (``loss`` returns mean-over-local-rows / W), averaged over the replicas."""
        if self.tp.world > 1:
            dist.all_reduce(share, group=self.tp.group)
        if self.dp_world > 1:
            dist.all_reduce(share, group=self.dp_group)
            share /= self.dp_world
        return share

    def grad_norm(self) -> torch.Tensor:
        """Norm of the whole (unsharded) gradient, without a host synchronisation."""
        s = torch.linalg.vector_norm(self.grads[:self.n_sharded], dtype=torch.float32) ** 2
        if self.tp.world > 1:
            dist.all_reduce(s, group=self.tp.group)
        return torch.sqrt(s + torch.linalg.vector_norm(self.grads[self.n_sharded:], dtype=torch.float32) ** 2)


class TPLlamaTrainer:
    """fp32 master weights + AdamW over the flat shard (fused kernel on CUDA), clipping by the
    group-wide gradient norm. ``step(tokens, targets)`` returns the batch-mean loss as a tensor."""

    def __init__(self, model: TPLlama, optim: AdamWConfig | None = None) -> None:
        self.model, self.cfg = model, optim or AdamWConfig()
        self.master = model.params.detach().float().clone()
        self.m, self.v = torch.zeros_like(self.master), torch.zeros_like(self.master)
        self.step_count = 0
        self.on_cuda = model.params.is_cuda and model.dtype == torch.bfloat16
        dev = model.params.device
        self.clip = torch.ones(2, dtype=torch.float32, device=dev)
        if self.on_cuda:
            from ..ops import kernels as K
            self.K = K
            self.hyper = torch.zeros(K.HYPER_SIZE, dtype=torch.float32, device=dev)
            from ..utils.pinned import PinnedRing
            self._hyper_ring = PinnedRing(K.HYPER_SIZE, torch.float32, slots=8)

    def _clip_scale(self) -> None:
        norm = self.model.grad_norm()
        mx = self.cfg.max_grad_norm
        self.clip[1] = norm
        self.clip[0] = torch.where(norm > mx, mx / (norm + 1e-6), torch.ones_like(norm)) if mx > 0 else 1.0

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        mdl, c = self.model, self.cfg
        loss = mdl.loss(tokens, targets)
        mdl.backward(loss)
        self.step_count += 1
        t = self.step_count
        self._clip_scale()
        lr = lr_at_step(c, t)
        if self.on_cuda:
            vals = [lr, c.beta1, c.beta2, c.eps, c.weight_decay, 1.0 - c.beta1 ** t, 1.0 - c.beta2 ** t, 1.0, c.max_grad_norm]
            self._hyper_ring.upload(self.hyper, vals)  # one pinned slot per step in flight
            self.K.adamw_flat(self.master, self.m, self.v, mdl.grads, mdl.params.detach(), mdl.layout.n_decay, self.hyper, self.clip)
        else:
            with torch.no_grad():
                g = mdl.grads.float() * self.clip[0]
                self.m.mul_(c.beta1).add_(g, alpha=1 - c.beta1)
                self.v.mul_(c.beta2).addcmul_(g, g, value=1 - c.beta2)
                upd = (self.m / (1 - c.beta1 ** t)) / ((self.v / (1 - c.beta2 ** t)).sqrt() + c.eps)
                upd[:mdl.layout.n_decay] += c.weight_decay * self.master[:mdl.layout.n_decay]
                self.master -= lr * upd
                mdl.params.detach().copy_(self.master.to(mdl.dtype))
        return mdl.reduce_loss(loss.detach().clone())
