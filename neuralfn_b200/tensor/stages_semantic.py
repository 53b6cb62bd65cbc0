"""Semantic-routing stages of the tensor runtime: vocabulary-topic projectors, LSH hashers, the
semantic / hash / chunk routers, chunk-state pooling, route broadcast, routed attention experts,
the attention-less decoder and the route / alignment losses.

Behavioural counterparts of the reference's experimental semantic stages
(``neuralfn/torch_backend.py:6409-7157``): same inputs, outputs, parameter names and arithmetic, so
that checkpoints and graphs interchange. The topic vocabulary comes from
``neuralfn_b200.semantic.ConversationalVocabulary`` (a small built-in vocabulary unless
``semantic_vocab_ref`` / ``NFN_SEMANTIC_VOCAB_DIR`` names the reference's ``vocab_86d_*.json`` files).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .stages_core import stage
from .stages_moe import RoutingStatsMixin

IGNORE = -100


_warned_refs: set[str] = set()


def _vocab(ref: str = "", semantic_dim: int | None = None):
    """The vocabulary a reference names; the built-in one when the reference cannot be resolved (no
    vocabulary directory configured), with one warning per reference."""
    from ..semantic import ConversationalVocabulary
    try:
        return ConversationalVocabulary(ref or None)
    except FileNotFoundError:
        if ref not in _warned_refs:
            _warned_refs.add(ref)
            import warnings
            warnings.warn(f"semantic vocabulary {ref!r} not found; using the built-in vocabulary "
                          "(set NFN_SEMANTIC_VOCAB_DIR to the directory holding it)", stacklevel=3)
        return ConversationalVocabulary(None)


def semantic_geometry(ref: str = "") -> tuple[int, int]:
    """(vocabulary dimensions, semantic vector width = dimensions + the signature slot)."""
    v = _vocab(ref)
    return v.num_vocab_dims, v.vector_dim


def _term_counts(vocab) -> list[int]:
    return [len(vocab.terms(n)) for n in vocab.dim_names]


def _topic_confidence(topic_logits: Tensor, term_counts: list[int]) -> Tensor:
    """max softmax probability per vocabulary dimension: [..., dims, terms] -> [..., dims] (fp32)."""
    cols = []
    for i, n in enumerate(term_counts):
        cols.append(F.softmax(topic_logits[..., i, :n].float(), dim=-1).amax(dim=-1))
    return torch.stack(cols, dim=-1)


class _TopicProjector(nn.Module):
    """Shared body of the pooled and the chunk-wise projector: per-dimension topic heads, a
    signature-bucket head whose expectation becomes the last semantic coordinate, and a residual MLP."""

    def __init__(self, input_dim: int, semantic_dim: int, residual_dim: int, n_sig_buckets: int, semantic_vocab_ref: str) -> None:
        super().__init__()
        vocab = _vocab(semantic_vocab_ref, semantic_dim)
        self.semantic_dim = int(semantic_dim)
        self.num_vocab_dims = vocab.num_vocab_dims
        self.term_counts = _term_counts(vocab)
        self.max_terms = max(self.term_counts, default=0)
        self.topic_heads = nn.ModuleList(nn.Linear(input_dim, max(c, 1), bias=False) for c in self.term_counts)
        self.sig_head = nn.Linear(input_dim, n_sig_buckets, bias=False)
        self.residual_head = nn.Sequential(nn.Linear(input_dim, residual_dim, bias=False), nn.GELU(),
                                           nn.Linear(residual_dim, residual_dim, bias=False))

    def _project_rows(self, rows: Tensor) -> tuple[Tensor, Tensor]:
        """rows [n, d] -> (semantic vector [n, dims + 1], topic logits [n, dims, max_terms])."""
        n = rows.size(0)
        dt = rows.dtype
        topic = rows.new_zeros((n, self.num_vocab_dims, self.max_terms))
        coords = []
        for i, head in enumerate(self.topic_heads):
            c = self.term_counts[i]
            lg = head(rows)
            topic[:, i, :c] = lg
            idx = lg.float().argmax(dim=-1)
            coords.append(2.0 * idx.to(dt) / float(c - 1) - 1.0 if c > 1 else torch.zeros(n, device=rows.device, dtype=dt))
        sig = F.softmax(self.sig_head(rows).float(), dim=-1)
        axis = torch.linspace(0.0, 1.0, sig.size(-1), device=sig.device)
        coords.append((sig * axis).sum(dim=-1).to(dt))
        return torch.stack(coords, dim=-1), topic


@stage("semantic_projector")
class SemanticProjectorStage(_TopicProjector):
    """hidden [b, s, d] (or [b, d]) -> (semantic vector of the mean-pooled sequence, residual state per
    position, topic logits)."""

    def __init__(self, input_dim: int, semantic_dim: int = 86, residual_dim: int = 64, n_sig_buckets: int = 4096,
                 semantic_vocab_ref: str = "") -> None:
        super().__init__(input_dim, semantic_dim, residual_dim, n_sig_buckets, semantic_vocab_ref)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg.get("semantic_dim", 86)), int(cfg.get("residual_dim", 64)),
                   int(cfg.get("n_sig_buckets", 4096)), str(cfg.get("semantic_vocab_ref", "")))

    def forward(self, x: Tensor):
        if x.ndim == 2:
            x = x.unsqueeze(1)
        sem, topic = self._project_rows(x.mean(dim=1))
        return sem, self.residual_head(x).to(x.dtype), topic


@stage("semantic_chunk_projector")
class SemanticChunkProjectorStage(_TopicProjector):
    """chunk states [b, chunks, d] -> the same three outputs with the chunk axis kept."""

    def __init__(self, input_dim: int, semantic_dim: int = 86, residual_dim: int = 64, n_sig_buckets: int = 4096,
                 semantic_vocab_ref: str = "") -> None:
        super().__init__(input_dim, semantic_dim, residual_dim, n_sig_buckets, semantic_vocab_ref)

    from_config = classmethod(SemanticProjectorStage.from_config.__func__)  # type: ignore[attr-defined]

    def forward(self, x: Tensor):
        if x.ndim == 2:
            x = x.unsqueeze(1)
        if x.ndim != 3:
            raise ValueError("semantic_chunk_projector expects [batch, chunks, dim]")
        b, c, d = x.shape
        flat = x.reshape(b * c, d)
        sem, topic = self._project_rows(flat)
        res = self.residual_head(flat).to(flat.dtype)
        return sem.reshape(b, c, -1), res.reshape(b, c, -1), topic.reshape(b, c, self.num_vocab_dims, self.max_terms)


class _LshPlanes(nn.Module):
    def __init__(self, dim: int, tables: int, planes: int, seed: int) -> None:
        super().__init__()
        rng = np.random.RandomState(seed)
        self.register_buffer("proj", torch.from_numpy(rng.randn(tables, planes, dim).astype("float32")))

    def _buckets(self, rows: Tensor) -> Tensor:
        bits = torch.einsum("tpd,bd->btp", self.proj.to(rows.dtype), rows) > 0
        weights = (2 ** torch.arange(bits.shape[-1], device=bits.device, dtype=torch.long)).view(1, 1, -1)
        return (bits.long() * weights).sum(dim=-1)


@stage("semantic_hasher")
class SemanticHasherStage(_LshPlanes):
    """Random-hyperplane LSH of semantic vectors: [b, dim] -> bucket ids [b, tables]."""

    def __init__(self, dim: int = 86, tables: int = 8, planes: int = 12, seed: int = 42) -> None:
        super().__init__(dim, tables, planes, seed)
        self.n_tables = tables

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("dim", 86)), int(cfg.get("tables", 8)), int(cfg.get("planes", 12)), int(cfg.get("seed", 42)))

    def forward(self, sem_vec: Tensor) -> Tensor:
        return self._buckets(sem_vec)


@stage("semantic_chunk_hasher")
class SemanticChunkHasherStage(_LshPlanes):
    """[b, chunks, dim] -> bucket ids [b, chunks, tables]."""

    def __init__(self, dim: int = 86, tables: int = 8, planes: int = 12, seed: int = 42) -> None:
        super().__init__(dim, tables, planes, seed)

    from_config = classmethod(SemanticHasherStage.from_config.__func__)  # type: ignore[attr-defined]

    def forward(self, sem_vec: Tensor) -> Tensor:
        if sem_vec.ndim == 2:
            sem_vec = sem_vec.unsqueeze(1)
        if sem_vec.ndim != 3:
            raise ValueError("semantic_chunk_hasher expects [batch, chunks, semantic_dim]")
        b, c, d = sem_vec.shape
        return self._buckets(sem_vec.reshape(b * c, d)).reshape(b, c, -1)


@stage("semantic_moe_router")
class SemanticMoERouterStage(RoutingStatsMixin, nn.Module):
    """Cosine similarity of the (pooled) semantic vector to learned expert centroids, top-k, softmax."""

    def __init__(self, n_experts: int, semantic_dim: int = 86, top_k: int = 2) -> None:
        super().__init__()
        self.centroids = nn.Parameter(torch.randn(n_experts, semantic_dim))
        self.top_k = int(top_k)
        self._init_routing_stats(num_experts=n_experts, top_k=self.top_k)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["n_experts"]), int(cfg.get("semantic_dim", 86)), int(cfg.get("top_k", 2)))

    def forward(self, sem_vec: Tensor):
        dt = sem_vec.dtype if sem_vec.is_floating_point() else self.centroids.dtype
        s = sem_vec.mean(dim=1) if sem_vec.ndim == 3 else sem_vec
        sim = F.normalize(s.float(), dim=-1).to(dt) @ F.normalize(self.centroids.float(), dim=-1).to(dt).T
        w, idx = torch.topk(sim, self.top_k, dim=-1)
        w = F.softmax(w.float(), dim=-1).to(dt)
        self._update_routing_stats(scores=F.softmax(sim.float(), dim=-1), routing_weights=w, routing_indices=idx)
        return w.unsqueeze(1), idx.unsqueeze(1)


def _pad_targets(targets: Tensor, width: int) -> Tensor:
    t = targets.long()
    if t.ndim == 1:
        t = t.unsqueeze(0)
    if t.size(1) < width:
        t = torch.cat([t, t.new_full((t.size(0), width - t.size(1)), IGNORE)], dim=1)
    return t


@stage("semantic_hash_router")
class SemanticHashRouterStage(RoutingStatsMixin, nn.Module):
    """One expert per vocabulary dimension. Scores are the topic confidences (or the semantic vector
    itself) plus a learned per-bucket bias; dimensions named by the semantic targets are forced."""

    def __init__(self, n_experts: int, semantic_dim: int = 86, top_k: int = 2, tables: int = 8, n_buckets: int = 4096,
                 ignore_index: int = IGNORE, semantic_vocab_ref: str = "", routing_source: str = "topic_logits") -> None:
        super().__init__()
        vocab = _vocab(semantic_vocab_ref, semantic_dim)
        self.num_vocab_dims = vocab.num_vocab_dims
        if int(n_experts) != self.num_vocab_dims:
            raise ValueError(f"semantic_hash_router requires exactly {self.num_vocab_dims} experts, got {n_experts}")
        self.semantic_dim = semantic_dim
        self.top_k = max(1, min(int(top_k), self.num_vocab_dims))
        self.n_buckets = max(int(n_buckets), 1)
        self.ignore_index = int(ignore_index)
        self.routing_source = str(routing_source)
        self.term_counts = _term_counts(vocab)
        self.hash_embed = nn.Embedding(self.n_buckets, self.num_vocab_dims)
        self.table_gate = nn.Parameter(torch.zeros(int(tables)))
        self.dimension_bias = nn.Parameter(torch.zeros(self.num_vocab_dims))
        self.register_buffer("expert_map", torch.arange(self.num_vocab_dims, dtype=torch.long))
        nn.init.zeros_(self.hash_embed.weight)
        self._init_routing_stats(num_experts=self.num_vocab_dims, top_k=self.top_k)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["n_experts"]), int(cfg.get("semantic_dim", 86)), int(cfg.get("top_k", 2)), int(cfg.get("tables", 8)),
                   int(cfg.get("n_buckets", 4096)), int(cfg.get("ignore_index", IGNORE)), str(cfg.get("semantic_vocab_ref", "")),
                   str(cfg.get("routing_source", "topic_logits")))

    def _scores(self, sem_vec: Tensor, topic_logits: Tensor, buckets: Tensor) -> Tensor:
        if self.routing_source == "semantic_vec":
            v = sem_vec.float()
            v = v.mean(dim=1) if v.ndim == 3 else v
            if v.size(-1) < self.num_vocab_dims:
                raise ValueError(f"semantic_hash_router expected semantic_vec width >= {self.num_vocab_dims}, got {v.size(-1)}")
            return v[:, :self.num_vocab_dims] + self.dimension_bias
        conf = _topic_confidence(topic_logits, self.term_counts)
        if buckets.ndim == 1:
            buckets = buckets.unsqueeze(-1)
        feat = self.hash_embed(buckets.long() % self.n_buckets).float()
        gate = F.softmax(self.table_gate[:feat.size(1)], dim=0)
        return conf + (feat * gate.view(1, -1, 1)).sum(dim=1) + self.dimension_bias

    def forward(self, sem_vec: Tensor, bucket_indices: Tensor, topic_logits: Tensor, sem_targets: Tensor):
        dt = topic_logits.dtype if topic_logits.is_floating_point() else torch.float32
        scores = self._scores(sem_vec, topic_logits, bucket_indices)
        n = len(self.term_counts)
        forced = _pad_targets(sem_targets, n)[:, :n] != self.ignore_index
        any_forced = forced.any(dim=-1)
        neg = scores.new_full((), float("-inf"))
        order = torch.where(any_forced.unsqueeze(-1), torch.argsort(torch.where(forced, scores, neg), dim=-1, descending=True),
                            torch.argsort(scores, dim=-1, descending=True))
        k_row = torch.where(any_forced, forced.sum(dim=-1).clamp(min=1, max=self.top_k), torch.full_like(any_forced, self.top_k, dtype=torch.long))
        dims = order[:, :self.top_k]
        experts = self.expert_map[dims]
        live = torch.arange(self.top_k, device=scores.device).unsqueeze(0) < k_row.unsqueeze(-1)
        w = F.softmax(torch.where(live, torch.gather(scores, 1, dims), neg), dim=-1).to(dt)
        w = torch.where(live, w, torch.zeros_like(w))
        idx = torch.where(live, experts, experts[:, :1].expand(-1, self.top_k))
        self._update_routing_stats(scores=F.softmax(scores.float(), dim=-1), routing_weights=w, routing_indices=idx)
        return w, idx


@stage("causal_chunk_state")
class CausalChunkStateStage(nn.Module):
    """Chunk states from token states. ``prefix``: state of chunk c = mean of all tokens before the
    chunk's first position (so it is safe to route that chunk's tokens with it); ``mean``: plain
    mean of the chunk's own tokens."""

    def __init__(self, chunk_size: int = 32, mode: str = "prefix") -> None:
        super().__init__()
        self.chunk_size, self.mode = max(int(chunk_size), 1), str(mode)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("chunk_size", 32)), str(cfg.get("mode", "prefix")))

    def forward(self, hidden: Tensor) -> Tensor:
        if hidden.ndim != 3:
            raise ValueError("causal_chunk_state expects hidden shaped [batch, seq, dim]")
        b, s, d = hidden.shape
        cs = self.chunk_size
        chunks = max(math.ceil(s / cs), 1)
        if self.mode == "mean":
            pad = chunks * cs - s
            work = F.pad(hidden, (0, 0, 0, pad)) if pad else hidden
            counts = torch.full((chunks,), cs, device=hidden.device, dtype=hidden.dtype)
            if pad:
                counts[-1] = cs - pad
            return work.reshape(b, chunks, cs, d).sum(dim=2) / counts.view(1, chunks, 1)
        edge = (torch.arange(chunks, device=hidden.device) * cs - 1).clamp(min=0, max=s - 1)
        return hidden.cumsum(dim=1)[:, edge, :] / (edge + 1).to(hidden.dtype).view(1, chunks, 1)


@stage("semantic_moe_jepa_evo_router")
class SemanticMoeJepaEvoRouterStage(RoutingStatsMixin, nn.Module):
    """Chunk-level router over [shared | one expert per vocabulary dimension | free] experts. The
    shared experts are always on; ``top_k`` more are chosen among the semantic and free experts
    (semantic ones forced by the targets when any are given). Returns weights and indices of width
    shared + top_k and the full route logits for the route losses."""

    def __init__(self, semantic_dim: int = 86, top_k: int = 2, shared_experts: int = 2, free_experts: int = 8, tables: int = 8,
                 n_buckets: int = 4096, ignore_index: int = IGNORE, semantic_vocab_ref: str = "") -> None:
        super().__init__()
        vocab = _vocab(semantic_vocab_ref, semantic_dim)
        self.num_vocab_dims = vocab.num_vocab_dims
        self.semantic_dim = int(semantic_dim)
        self.shared_experts, self.free_experts = max(int(shared_experts), 0), max(int(free_experts), 0)
        self.total_experts = self.shared_experts + self.num_vocab_dims + self.free_experts
        self.top_k = max(1, min(int(top_k), self.num_vocab_dims + self.free_experts))
        self.route_width = self.shared_experts + self.top_k
        self.n_buckets = max(int(n_buckets), 1)
        self.ignore_index = int(ignore_index)
        self.term_counts = _term_counts(vocab)
        self.hash_embed = nn.Embedding(self.n_buckets, self.num_vocab_dims + self.free_experts)
        self.table_gate = nn.Parameter(torch.zeros(int(tables)))
        self.dimension_bias = nn.Parameter(torch.zeros(self.num_vocab_dims))
        self.shared_logits = nn.Parameter(torch.zeros(self.shared_experts))
        self.free_head = nn.Linear(self.semantic_dim, self.free_experts, bias=True) if self.free_experts > 0 else None
        nn.init.zeros_(self.hash_embed.weight)
        if self.free_head is not None:
            nn.init.zeros_(self.free_head.weight)
            nn.init.zeros_(self.free_head.bias)
        self._init_routing_stats(num_experts=self.total_experts, top_k=max(self.route_width, 1))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("semantic_dim", 86)), int(cfg.get("top_k", 2)), int(cfg.get("shared_experts", 2)), int(cfg.get("free_experts", 8)),
                   int(cfg.get("tables", 8)), int(cfg.get("n_buckets", 4096)), int(cfg.get("ignore_index", IGNORE)),
                   str(cfg.get("semantic_vocab_ref", "")))

    def route_evo_parameters(self) -> list[Tensor]:
        ps = [self.hash_embed.weight, self.table_gate, self.dimension_bias, self.shared_logits]
        if self.free_head is not None:
            ps += [self.free_head.weight, self.free_head.bias]
        return [p for p in ps if p.requires_grad]

    def forward(self, sem_vec: Tensor, bucket_indices: Tensor, topic_logits: Tensor, sem_targets: Tensor):
        if sem_vec.ndim == 2:
            sem_vec = sem_vec.unsqueeze(1)
        if topic_logits.ndim == 3:
            topic_logits = topic_logits.unsqueeze(1)
        if bucket_indices.ndim == 2:
            bucket_indices = bucket_indices.unsqueeze(1)
        if sem_vec.ndim != 3 or topic_logits.ndim != 4:
            raise ValueError("semantic_moe_jepa_evo_router expects chunked semantic inputs")
        b, c, _ = sem_vec.shape
        dt = topic_logits.dtype if topic_logits.is_floating_point() else torch.float32
        V, S, Fr = self.num_vocab_dims, self.shared_experts, self.free_experts
        feat = self.hash_embed(bucket_indices.long() % self.n_buckets).float()
        hash_bias = (feat * F.softmax(self.table_gate[:feat.size(2)], dim=0).view(1, 1, -1, 1)).sum(dim=2)
        sem_scores = _topic_confidence(topic_logits, self.term_counts) + hash_bias[..., :V] + self.dimension_bias
        cand = sem_scores
        if Fr > 0 and self.free_head is not None:
            cand = torch.cat([sem_scores, self.free_head(sem_vec.float()) + hash_bias[..., V:]], dim=-1)
        route_logits = torch.cat([self.shared_logits.float().view(1, 1, -1).expand(b, c, -1), cand], dim=-1)

        forced = _pad_targets(sem_targets, V)[:, :V] != self.ignore_index
        any_forced = forced.any(dim=-1)
        neg = cand.new_full((), float("-inf"))
        forced_scores = torch.full_like(cand, float("-inf"))
        forced_scores[..., :V] = torch.where(forced.unsqueeze(1), sem_scores, neg)
        order = torch.where(any_forced.view(b, 1, 1), torch.argsort(forced_scores, dim=-1, descending=True),
                            torch.argsort(cand, dim=-1, descending=True))
        k_row = torch.where(any_forced, forced.sum(dim=-1).clamp(min=1, max=self.top_k), torch.full_like(any_forced, self.top_k, dtype=torch.long))
        chosen = order[..., :self.top_k]
        live = torch.arange(self.top_k, device=sem_vec.device).view(1, 1, -1) < k_row.view(b, 1, 1)
        scores = torch.where(live, torch.gather(cand, -1, chosen), neg)
        experts = chosen + S   # candidate j is expert S + j (semantic block first, then the free experts)
        experts = torch.where(live, experts, experts[..., :1].expand(-1, -1, self.top_k))
        if S > 0:
            scores = torch.cat([self.shared_logits.to(scores.dtype).view(1, 1, -1).expand(b, c, -1), scores], dim=-1)
            experts = torch.cat([torch.arange(S, device=sem_vec.device).view(1, 1, -1).expand(b, c, -1), experts], dim=-1)
        w = F.softmax(scores.float(), dim=-1).to(dt)
        self._update_routing_stats(scores=F.softmax(route_logits.float(), dim=-1), routing_weights=w, routing_indices=experts)
        return w, experts, route_logits.to(dt)


@stage("broadcast_chunk_routes")
class BroadcastChunkRoutesStage(nn.Module):
    """Chunk-level routes [b, chunks, width] -> per-token routes [b, seq, width] for the MoE dispatch."""

    def __init__(self, chunk_size: int = 32) -> None:
        super().__init__()
        self.chunk_size = max(int(chunk_size), 1)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("chunk_size", 32)))

    def forward(self, hidden: Tensor, expert_weights: Tensor, expert_indices: Tensor):
        if hidden.ndim != 3 or expert_weights.ndim != 3 or expert_indices.ndim != 3:
            raise ValueError("broadcast_chunk_routes expects hidden [batch, seq, dim] and routes [batch, chunks, width]")
        if expert_weights.size(0) != hidden.size(0) or expert_indices.size(0) != hidden.size(0):
            raise ValueError("broadcast_chunk_routes batch size must match hidden batch size")
        which = (torch.arange(hidden.size(1), device=hidden.device) // self.chunk_size).clamp_max(expert_weights.size(1) - 1)
        return expert_weights[:, which, :].to(hidden.dtype).contiguous(), expert_indices.long()[:, which, :].contiguous()


@stage("semantic_unforced_targets")
class SemanticUnforcedTargetsStage(nn.Module):
    """hidden [b, ...] -> int64 [b, dims] filled with the ignore index: routing with no dimension
    forced, for graphs whose semantic targets are not wired into the block."""

    def __init__(self, dims: int, ignore_index: int = IGNORE) -> None:
        super().__init__()
        self.dims, self.ignore_index = int(dims), int(ignore_index)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["dims"]), int(cfg.get("ignore_index", IGNORE)))

    def forward(self, hidden: Tensor) -> Tensor:
        return torch.full((hidden.size(0), self.dims), self.ignore_index, device=hidden.device, dtype=torch.long)


@stage("semantic_targets_from_tokens")
class SemanticTargetsFromTokensStage(nn.Module):
    """tokens [b, s] -> semantic targets [b, dims + 1] through a token -> topic table: per vocabulary
    dimension the most frequent non-ignored topic among the sequence's tokens, last column the
    signature bucket. The table is loaded from ``table_path`` (int64 ``[vocab, dims + 1]`` in an
    ``.npy``) or, without one, derived deterministically from the token id (every ``period``-th token
    names a topic of dimension ``token % dims``), which is what synthetic runs use."""

    def __init__(self, vocab_size: int, semantic_vocab_ref: str = "", table_path: str = "", n_sig_buckets: int = 4096,
                 period: int = 3, ignore_index: int = IGNORE) -> None:
        super().__init__()
        vocab = _vocab(semantic_vocab_ref)
        counts = _term_counts(vocab)
        dims = len(counts)
        self.ignore_index = int(ignore_index)
        if table_path:
            table = torch.from_numpy(np.load(table_path).astype("int64"))
            if table.shape != (vocab_size, dims + 1):
                raise ValueError(f"semantic table must be [{vocab_size}, {dims + 1}], got {tuple(table.shape)}")
        else:
            ids = torch.arange(vocab_size)
            table = torch.full((vocab_size, dims + 1), self.ignore_index, dtype=torch.long)
            named = ids % max(int(period), 1) == 0
            dim_of = ids % max(dims, 1)
            term_of = (ids // max(dims, 1)) % torch.tensor(counts, dtype=torch.long).clamp(min=1)[dim_of]
            table[ids[named], dim_of[named]] = term_of[named]
            table[:, dims] = (ids * 2654435761 % n_sig_buckets)
        self.register_buffer("table", table)
        self.register_buffer("term_counts", torch.tensor(counts + [int(n_sig_buckets)], dtype=torch.long))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["vocab_size"]), str(cfg.get("semantic_vocab_ref", "")), str(cfg.get("table_path", "")),
                   int(cfg.get("n_sig_buckets", 4096)), int(cfg.get("period", 3)), int(cfg.get("ignore_index", IGNORE)))

    def forward(self, tokens: Tensor) -> Tensor:
        rows = self.table[tokens.long().clamp(0, self.table.size(0) - 1)]          # [b, s, dims + 1]
        b, s, w = rows.shape
        out = torch.full((b, w), self.ignore_index, device=tokens.device, dtype=torch.long)
        for j in range(w):
            col = rows[:, :, j]
            n = int(self.term_counts[j])
            valid = (col >= 0) & (col < n)
            hist = torch.zeros(b, n, device=tokens.device, dtype=torch.long)
            hist.scatter_add_(1, col.clamp(0, n - 1), valid.long())
            top = hist.argmax(dim=1)
            out[:, j] = torch.where(hist.sum(dim=1) > 0, top, out[:, j])
        return out


@stage("routed_attention_experts")
class RoutedAttentionExpertsStage(nn.Module):
    """Sequence-level mixture of attention experts: each sequence's top-k experts run a full rotary
    GQA attention (weightless QK RMS norm, per-head query gain) over the whole sequence."""

    def __init__(self, model_dim: int, num_heads: int, num_kv_heads: int, rope_base: float, qk_gain_init: float, experts: int,
                 top_k: int = 2, is_causal: bool = True) -> None:
        super().__init__()
        if model_dim % num_heads or num_heads % num_kv_heads or (model_dim // num_heads) % 2:
            raise ValueError("model_dim / num_heads / num_kv_heads do not give an even head_dim that divides evenly")
        hd = model_dim // num_heads
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, hd
        self.experts, self.top_k, self.is_causal, self.rope_base = experts, top_k, is_causal, float(rope_base)
        kv = num_kv_heads * hd
        self.q_proj = nn.Parameter(torch.empty(experts, model_dim, model_dim))
        self.k_proj = nn.Parameter(torch.empty(experts, model_dim, kv))
        self.v_proj = nn.Parameter(torch.empty(experts, model_dim, kv))
        self.out_proj = nn.Parameter(torch.empty(experts, model_dim, model_dim))
        self.q_gain = nn.Parameter(torch.full((experts, num_heads), float(qk_gain_init)))
        for p in (self.q_proj, self.k_proj, self.v_proj, self.out_proj):
            nn.init.normal_(p, std=0.02)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["num_heads"]), int(cfg.get("num_kv_heads", cfg["num_heads"])), float(cfg.get("rope_base", 10000.0)),
                   float(cfg.get("qk_gain_init", 1.0)), int(cfg["experts"]), int(cfg.get("top_k", 2)), bool(cfg.get("is_causal", True)))

    def _rope(self, t: Tensor) -> Tensor:
        # "legacy" convention of the runtime: half-split pairs rotated by the negative angle
        s, hd = t.size(-2), t.size(-1)
        inv = 1.0 / (self.rope_base ** (torch.arange(0, hd, 2, device=t.device, dtype=torch.float32) / hd))
        ang = torch.outer(torch.arange(s, device=t.device, dtype=torch.float32), inv)
        cos, sin = ang.cos().to(t.dtype), ang.sin().to(t.dtype)
        a, b_ = t[..., :hd // 2], t[..., hd // 2:]
        return torch.cat([a * cos + b_ * sin, -a * sin + b_ * cos], dim=-1)

    def _expert(self, x: Tensor, e: int) -> Tensor:
        n, s, d = x.shape
        q = (x @ self.q_proj[e]).reshape(n, s, self.num_heads, self.head_dim).transpose(1, 2)
        k = (x @ self.k_proj[e]).reshape(n, s, self.num_kv_heads, self.head_dim).transpose(1, 2)
        v = (x @ self.v_proj[e]).reshape(n, s, self.num_kv_heads, self.head_dim).transpose(1, 2)
        q, k = F.rms_norm(q, (self.head_dim,)), F.rms_norm(k, (self.head_dim,))
        q, k = self._rope(q), self._rope(k)
        q = q * self.q_gain[e].to(q.dtype)[None, :, None, None]
        g = self.num_heads // self.num_kv_heads
        if g > 1:
            k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=self.is_causal)
        return y.transpose(1, 2).reshape(n, s, d) @ self.out_proj[e]

    def forward(self, x: Tensor, routing_weights: Tensor, routing_indices: Tensor) -> Tensor:
        if routing_weights.ndim == 3:
            routing_weights, routing_indices = routing_weights.squeeze(1), routing_indices.squeeze(1)
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows, slot = torch.where(routing_indices == e)
            if rows.numel() == 0:
                continue
            out.index_add_(0, rows, self._expert(x[rows], e) * routing_weights[rows, slot].to(x.dtype).view(-1, 1, 1))
        return out


@stage("attentionless_decoder")
class AttentionlessDecoderStage(nn.Module):
    """(bucket ids, expert output) -> logits [b, 1, vocab]: the expert state plus an embedding of the
    first LSH bucket, projected onto the vocabulary."""

    def __init__(self, semantic_dim: int = 86, residual_dim: int = 64, vocab_size: int = 256, n_buckets: int = 256) -> None:
        super().__init__()
        self.bucket_embed = nn.Embedding(n_buckets, residual_dim)
        self.out_proj = nn.Linear(residual_dim, vocab_size, bias=False)
        self.n_buckets = n_buckets

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("semantic_dim", 86)), int(cfg.get("residual_dim", 64)), int(cfg.get("vocab_size", 256)), int(cfg.get("n_buckets", 256)))

    def forward(self, bucket_indices: Tensor, expert_output: Tensor) -> Tensor:
        first = (bucket_indices[:, 0] if bucket_indices.ndim == 2 else bucket_indices) % self.n_buckets
        if expert_output.ndim == 3:
            expert_output = expert_output.squeeze(1)
        return self.out_proj(expert_output + self.bucket_embed(first).to(expert_output.dtype)).unsqueeze(1)


# ------------------------------------------------------------------------------- losses --
@stage("semantic_alignment_loss")
class SemanticAlignmentLossStage(nn.Module):
    """Mean over vocabulary dimensions of the cross-entropy between topic logits and the target topic
    of that dimension (targets equal to the ignore index, or out of range, do not count)."""

    def __init__(self, ignore_index: int = IGNORE, semantic_vocab_ref: str = "") -> None:
        super().__init__()
        self.ignore_index = int(ignore_index)
        self.semantic_vocab_ref = str(semantic_vocab_ref)
        self.term_counts: list[int] = []

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg.get("ignore_index", IGNORE)), str(cfg.get("semantic_vocab_ref", "")))

    def forward(self, pred: Tensor, target: Tensor) -> Tensor:
        if not self.term_counts:
            self.term_counts = _term_counts(_vocab(self.semantic_vocab_ref))
        logits, t = pred.float(), target.detach().long()
        if t.ndim == 1:
            t = t.unsqueeze(0)
        if logits.ndim == 4:
            b, c, dims, terms = logits.shape
            logits = logits.reshape(b * c, dims, terms)
            t = t.unsqueeze(1).expand(b, c, t.size(-1)).reshape(b * c, t.size(-1))
        per_dim = []
        for i in range(min(len(self.term_counts), logits.size(1), t.size(1))):
            n = min(self.term_counts[i], logits.size(-1))
            if n <= 0:
                continue
            ti = t[:, i]
            ok = (ti != self.ignore_index) & (ti >= 0) & (ti < n)
            total = F.cross_entropy(logits[:, i, :n], torch.where(ok, ti, torch.full_like(ti, self.ignore_index)),
                                    ignore_index=self.ignore_index, reduction="sum")
            cnt = ok.sum().to(total.dtype)
            per_dim.append(torch.where(cnt > 0, total / cnt.clamp(min=1), total * 0.0))
        return torch.stack(per_dim).mean() if per_dim else logits.sum() * 0.0


@stage("route_balance_loss")
class RouteBalanceLossStage(nn.Module):
    """experts * sum_e mean(softmax(route logits))_e ^ 2 (density form, as ``load_balance_loss``)."""

    @classmethod
    def from_config(cls, cfg):
        return cls()

    def forward(self, route_logits: Tensor) -> Tensor:
        density = F.softmax(route_logits.float().reshape(-1, route_logits.size(-1)), dim=-1).mean(dim=0)
        return route_logits.size(-1) * (density * density).sum()


class _RouteLossBase(nn.Module):
    def __init__(self, semantic_vocab_ref: str, shared_experts: int, free_experts: int) -> None:
        super().__init__()
        vocab = _vocab(semantic_vocab_ref)
        self.num_vocab_dims = vocab.num_vocab_dims
        self.term_counts = _term_counts(vocab)
        self.shared_experts, self.free_experts = max(int(shared_experts), 0), max(int(free_experts), 0)
        self.total_experts = self.shared_experts + self.num_vocab_dims + self.free_experts


@stage("route_selection_loss")
class RouteSelectionLossStage(_RouteLossBase):
    """Binary cross-entropy pushing the semantic experts named by the targets on (only those
    dimensions count)."""

    def __init__(self, semantic_vocab_ref: str = "", shared_experts: int = 2, free_experts: int = 8, ignore_index: int = IGNORE) -> None:
        super().__init__(semantic_vocab_ref, shared_experts, free_experts)
        self.ignore_index = int(ignore_index)

    @classmethod
    def from_config(cls, cfg):
        return cls(str(cfg.get("semantic_vocab_ref", "")), int(cfg.get("shared_experts", 2)), int(cfg.get("free_experts", 8)),
                   int(cfg.get("ignore_index", IGNORE)))

    def forward(self, route_logits: Tensor, sem_targets: Tensor) -> Tensor:
        lg = route_logits.float()
        if lg.ndim == 2:
            lg = lg.unsqueeze(1)
        V = self.num_vocab_dims
        active = _pad_targets(sem_targets, V)[:, :V] != self.ignore_index
        if not bool(active.any()):
            return lg.sum() * 0.0
        sem = lg[..., self.shared_experts:self.shared_experts + V]
        mask = active.unsqueeze(1).expand_as(sem)
        return F.binary_cross_entropy_with_logits(sem, mask.to(sem.dtype), reduction="none")[mask].mean()


@stage("route_distillation_loss")
class RouteDistillationLossStage(_RouteLossBase):
    """KL(teacher || student) where the teacher puts the target topic confidences on the semantic
    experts, zero logits on the shared ones and -10 on the free ones."""

    def __init__(self, semantic_vocab_ref: str = "", shared_experts: int = 2, free_experts: int = 8) -> None:
        super().__init__(semantic_vocab_ref, shared_experts, free_experts)

    @classmethod
    def from_config(cls, cfg):
        return cls(str(cfg.get("semantic_vocab_ref", "")), int(cfg.get("shared_experts", 2)), int(cfg.get("free_experts", 8)))

    def forward(self, student_route_logits: Tensor, target_topic_logits: Tensor) -> Tensor:
        st = student_route_logits.float()
        if st.ndim == 2:
            st = st.unsqueeze(1)
        tl = target_topic_logits.float()
        if tl.ndim == 3:
            tl = tl.unsqueeze(1)
        teacher = st.new_full(st.shape, -10.0)
        S, V = self.shared_experts, self.num_vocab_dims
        teacher[..., :S] = 0.0
        teacher[..., S:S + V] = _topic_confidence(tl, self.term_counts)
        p = F.softmax(teacher.detach().reshape(-1, teacher.size(-1)), dim=-1)
        return F.kl_div(F.log_softmax(st.reshape(-1, st.size(-1)), dim=-1), p, reduction="batchmean")
