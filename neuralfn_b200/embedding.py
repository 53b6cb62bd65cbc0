"""Text-embedding models: a bidirectional transformer encoder trained with masked-token prediction
plus an in-batch contrastive objective, and the ``nfn embed`` inference path.

Model: token + learned position embeddings -> ``num_layers`` pre-LayerNorm blocks (bidirectional
multi-head attention with a key-padding mask, GELU(tanh) MLP) -> final LayerNorm -> masked mean (or
first-token) pooling -> linear projection to ``output_dim`` -> L2 normalisation. The hot operations
go through the kernel bridge, so bf16 CUDA runs use the sm_100a GEMM kernels; padded batches keep
the PyTorch attention path (the flash kernel has no key-padding mask).

Training (``EmbeddingTrainer``), per step on a batch of texts:
  * masked-token loss: ``mlm_probability`` of the tokens become ``mask_token_id``, the encoder's
    hidden states are scored against the (tied) token table;
  * contrastive loss: two independently masked views of every text are pooled; InfoNCE with
    temperature ``temperature`` pulls the two views of a text together against the rest of the
    batch (both directions).
Checkpoints are a directory: ``config.json`` + ``model.safetensors`` (+ ``optimizer.pt`` for
resume). ``load_embedding_model(dir).embed(texts)`` returns unit vectors.

Behavioural counterpart: ``csrc/native_embedding/embedding_transformer.h`` and
``nfn_embedding_native_train.cpp`` (``bert`` architecture, ``pretrain`` stage, mean pooling,
gelu-tanh, MLM + contrastive weights, temperature 0.05), ``nfn embed`` (``cli/nfn.py:480-492``).
"""
from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Iterable, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .tensor import kernel_bridge as KB

__all__ = ["EmbeddingConfig", "EmbeddingEncoder", "EmbeddingTrainer", "save_embedding_model", "load_embedding_model"]


@dataclass
class EmbeddingConfig:
    vocab_size: int = 260            # byte tokenizer: 256 bytes + pad, mask, bos, eos
    hidden_dim: int = 128
    output_dim: int = 128
    num_layers: int = 2
    num_heads: int = 4
    intermediate_dim: int = 0        # 0 = 4 x hidden
    max_tokens: int = 128
    pooling: str = "mean"            # "mean" | "cls"
    pad_token_id: int = 256
    mask_token_id: int = 257
    bos_token_id: int = 258
    mlm_probability: float = 0.15
    mlm_weight: float = 1.0
    contrastive_weight: float = 1.0
    temperature: float = 0.05
    norm_eps: float = 1e-5
    tokenizer: str = "bytes"

    def __post_init__(self) -> None:
        if self.hidden_dim % self.num_heads:
            raise ValueError("hidden_dim must divide by num_heads")
        if self.pooling not in ("mean", "cls"):
            raise ValueError("pooling is 'mean' or 'cls'")
        if not 0.0 <= self.mlm_probability < 1.0 or self.temperature <= 0:
            raise ValueError("mlm_probability must be in [0, 1) and temperature positive")
        if max(self.pad_token_id, self.mask_token_id, self.bos_token_id) >= self.vocab_size:
            raise ValueError("special token ids must lie inside the vocabulary")


class _Block(nn.Module):
    def __init__(self, c: EmbeddingConfig) -> None:
        super().__init__()
        d, f = c.hidden_dim, c.intermediate_dim or 4 * c.hidden_dim
        self.norm1, self.norm2 = nn.LayerNorm(d, eps=c.norm_eps), nn.LayerNorm(d, eps=c.norm_eps)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc1, self.fc2 = nn.Linear(d, f), nn.Linear(f, d)
        self.heads = c.num_heads

    def forward(self, x: torch.Tensor, key_mask: torch.Tensor | None) -> torch.Tensor:
        B, T, d = x.shape
        h = self.heads
        qkv = KB.linear(self.norm1(x), self.qkv.weight, self.qkv.bias).view(B, T, 3, h, d // h)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        if key_mask is None:
            a = KB.attention(q, k, v, causal=False)
        else:
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=key_mask[:, None, None, :])
        x = x + KB.linear(a.transpose(1, 2).reshape(B, T, d), self.proj.weight, self.proj.bias)
        return x + KB.linear(F.gelu(KB.linear(self.norm2(x), self.fc1.weight, self.fc1.bias), approximate="tanh"), self.fc2.weight, self.fc2.bias)


class EmbeddingEncoder(nn.Module):
    def __init__(self, config: EmbeddingConfig) -> None:
        super().__init__()
        c = self.config = config
        self.tok = nn.Embedding(c.vocab_size, c.hidden_dim)
        self.pos = nn.Embedding(c.max_tokens, c.hidden_dim)
        self.blocks = nn.ModuleList(_Block(c) for _ in range(c.num_layers))
        self.norm = nn.LayerNorm(c.hidden_dim, eps=c.norm_eps)
        self.out = nn.Linear(c.hidden_dim, c.output_dim, bias=False)
        self.mlm_bias = nn.Parameter(torch.zeros(c.vocab_size))
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    # -- tokenisation ---------------------------------------------------------------------------
    def tokenize(self, texts: Sequence[str]) -> tuple[torch.Tensor, torch.Tensor]:
        """Byte tokenizer with a leading BOS; returns (ids [B, T], attention mask [B, T] bool)."""
        c = self.config
        rows = [[c.bos_token_id] + list(t.encode("utf-8"))[:c.max_tokens - 1] for t in texts]
        T = max(len(r) for r in rows)
        ids = torch.full((len(rows), T), c.pad_token_id, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, :len(r)] = torch.tensor(r)
        return ids, ids != c.pad_token_id

    # -- forward --------------------------------------------------------------------------------
    def hidden(self, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        T = ids.shape[1]
        x = self.tok(ids) + self.pos(torch.arange(T, device=ids.device))[None]
        key_mask = None if bool(mask.all()) else mask
        for blk in self.blocks:
            x = blk(x, key_mask)
        return self.norm(x)

    def pool(self, hidden: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        if self.config.pooling == "cls":
            pooled = hidden[:, 0]
        else:
            m = mask.unsqueeze(-1).to(hidden.dtype)
            pooled = (hidden * m).sum(1) / m.sum(1).clamp_min(1.0)
        return F.normalize(self.out(pooled).float(), dim=-1)

    def forward(self, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        return self.pool(self.hidden(ids, mask), mask)

    @torch.no_grad()
    def embed(self, texts: Sequence[str], batch_size: int = 64) -> torch.Tensor:
        """Unit vectors [len(texts), output_dim] (fp32, on the host)."""
        was, dev = self.training, next(self.parameters()).device
        self.eval()
        out = []
        for i in range(0, len(texts), batch_size):
            ids, mask = self.tokenize(texts[i:i + batch_size])
            out.append(self(ids.to(dev), mask.to(dev)).cpu())
        self.train(was)
        return torch.cat(out) if out else torch.zeros(0, self.config.output_dim)


class EmbeddingTrainer:
    def __init__(self, model: EmbeddingEncoder, *, learning_rate: float = 1e-3, weight_decay: float = 0.01, warmup_steps: int = 50,
                 max_steps: int = 1000, grad_clip: float = 1.0, seed: int = 1337) -> None:
        self.model, self.max_steps, self.warmup, self.lr, self.clip = model, max_steps, warmup_steps, learning_rate, grad_clip
        decay = [p for n, p in model.named_parameters() if p.dim() >= 2]
        rest = [p for n, p in model.named_parameters() if p.dim() < 2]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": weight_decay}, {"params": rest, "weight_decay": 0.0}], lr=learning_rate,
                                     betas=(0.9, 0.999), eps=1e-8)
        self.step_count = 0
        self.gen = torch.Generator().manual_seed(seed)

    def _lr(self, step: int) -> float:
        if step <= self.warmup:
            return self.lr * step / max(1, self.warmup)
        t = min(1.0, (step - self.warmup) / max(1, self.max_steps - self.warmup))
        return self.lr * 0.5 * (1.0 + math.cos(math.pi * t))

    def _masked(self, ids: torch.Tensor, mask: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        c = self.model.config
        pick = (torch.rand(ids.shape, generator=self.gen) < c.mlm_probability) & mask & (ids != c.bos_token_id)
        return torch.where(pick, torch.full_like(ids, c.mask_token_id), ids), pick

    def losses(self, texts: Sequence[str]) -> dict[str, torch.Tensor]:
        m, c = self.model, self.model.config
        dev = next(m.parameters()).device
        ids, mask = m.tokenize(texts)
        views, mlm = [], ids.new_zeros((), dtype=torch.float32).to(dev)
        for _ in range(2):
            masked, pick = self._masked(ids, mask)
            h = m.hidden(masked.to(dev), mask.to(dev))
            views.append(m.pool(h, mask.to(dev)))
            if pick.any() and c.mlm_weight > 0:
                rows = h[pick.to(dev)]
                logits = rows.float() @ m.tok.weight.float().T + m.mlm_bias.float()
                mlm = mlm + 0.5 * F.cross_entropy(logits, ids[pick].to(dev))
        sim = views[0] @ views[1].T / c.temperature
        target = torch.arange(len(texts), device=dev)
        contrastive = 0.5 * (F.cross_entropy(sim, target) + F.cross_entropy(sim.T, target))
        return {"mlm": mlm, "contrastive": contrastive, "total": c.mlm_weight * mlm + c.contrastive_weight * contrastive}

    def step(self, texts: Sequence[str]) -> dict[str, float]:
        self.model.train()
        self.step_count += 1
        for g in self.opt.param_groups:
            g["lr"] = self._lr(self.step_count)
        self.opt.zero_grad(set_to_none=True)
        out = self.losses(texts)
        out["total"].backward()
        norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.clip)
        self.opt.step()
        return {k: float(v.detach()) for k, v in out.items()} | {"grad_norm": float(norm), "lr": self.opt.param_groups[0]["lr"]}

    def train(self, corpus: Sequence[str], batch_size: int = 32, on_step=None) -> list[dict]:
        """Runs to ``max_steps`` over shuffled batches of ``corpus`` (texts)."""
        if len(corpus) < 2:
            raise ValueError("the contrastive objective needs at least two texts")
        hist = []
        while self.step_count < self.max_steps:
            order = torch.randperm(len(corpus), generator=self.gen).tolist()
            for i in range(0, len(order) - 1, batch_size):
                batch = [corpus[j] for j in order[i:i + batch_size]]
                if len(batch) < 2:
                    continue
                hist.append(self.step(batch))
                if on_step:
                    on_step(self.step_count, hist[-1])
                if self.step_count >= self.max_steps:
                    break
        return hist


def save_embedding_model(model: EmbeddingEncoder, directory, trainer: EmbeddingTrainer | None = None) -> None:
    from .checkpoint.safetensors_io import write_safetensors
    root = Path(directory)
    root.mkdir(parents=True, exist_ok=True)
    (root / "config.json").write_text(json.dumps({"schema": "neuralfn_b200.embedding_model.v1", **asdict(model.config)}, indent=2))
    target = root / "model.safetensors"
    if target.exists():
        target.unlink()
    write_safetensors(target, {k: v.detach().float().cpu() for k, v in model.state_dict().items()}, {"kind": "embedding"})
    if trainer is not None:
        torch.save({"optimizer": trainer.opt.state_dict(), "step": trainer.step_count}, root / "optimizer.pt")


def load_embedding_model(directory, device="cpu") -> EmbeddingEncoder:
    from .checkpoint.safetensors_io import read_safetensors
    root = Path(directory)
    cfg = json.loads((root / "config.json").read_text())
    if cfg.pop("schema", None) != "neuralfn_b200.embedding_model.v1":
        raise ValueError(f"{root} is not an embedding model directory")
    model = EmbeddingEncoder(EmbeddingConfig(**cfg))
    tensors, _ = read_safetensors(root / "model.safetensors")
    model.load_state_dict(tensors, strict=True)
    return model.to(device)


def read_corpus(paths: Iterable[str | Path]) -> list[str]:
    """One text per non-empty line of every file."""
    out: list[str] = []
    for p in paths:
        out += [ln.strip() for ln in Path(p).read_text(encoding="utf-8").splitlines() if ln.strip()]
    return out
