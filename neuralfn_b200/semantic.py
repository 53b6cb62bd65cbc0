"""Vocabulary-grounded semantic space: every dimension of a routing vocabulary (entity type,
action, domain, ...) is one coordinate whose value encodes which term of that dimension is
active, plus one trailing coordinate carrying a hashed "signature" of the row.

* ``ConversationalVocabulary`` loads a vocabulary file (``{"vocabulary": {dimension:
  [terms...]}}`` - the schema of the reference's ``vocab_86d_*.json`` files, which load
  unchanged when their directory is named by ``NFN_SEMANTIC_VOCAB_DIR`` or passed as a path),
  resolves terms, finds the longest contiguous phrase match per dimension in free text and
  encodes / decodes rows: coordinate ``i`` = ``2 * index / (n_terms - 1) - 1``.
* Categorical targets (term index per dimension, ``-100`` = unset, last slot = signature
  bucket) convert to float vectors for regression heads and to 0..1 router vectors.
* ``SemanticHasher`` is multi-table random-hyperplane LSH with exact re-ranking;
  ``SemanticMatrix`` wraps an ``.npz`` of ``ids`` / ``vectors``.

A small built-in vocabulary keeps everything usable without external files.
Reference: ``neuralfn/semantic.py:50-779``.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
from collections import defaultdict
from pathlib import Path
from typing import Any, NamedTuple

import numpy as np

__all__ = ["SemanticDim", "ConversationalVocabulary", "SemanticHasher", "SemanticMatrix", "SEMANTIC_IGNORE_INDEX",
           "TAXONOMY_HASH_NAME", "signature_to_bucket", "signature_to_float", "normalize_semantic_term", "semantic_text_words",
           "build_semantic_signature", "resolve_semantic_topics", "extract_semantic_topics_from_text",
           "build_semantic_targets_from_topics", "semantic_targets_to_vectors", "semantic_targets_to_router_vectors",
           "load_training_targets", "load_training_data", "generate_synthetic_semantic_data", "resolve_semantic_vocab_path"]

SEMANTIC_IGNORE_INDEX = -100
TAXONOMY_HASH_NAME = "taxonomy_hash"
_SIGNATURE_DIMS = ("entity_type", "action", "domain")

_BUILTIN_VOCAB = {
    "entity_type": ["person", "group", "organization", "product", "document", "place", "event", "animal", "software", "concept"],
    "action": ["move", "create", "change", "analyze", "communicate", "trade", "learn", "repair", "protect", "decide"],
    "property": ["large", "small", "fast", "slow", "new", "old", "safe", "risky", "simple", "complex"],
    "emotion_sentiment": ["joy", "trust", "fear", "surprise", "sadness", "anger", "neutral", "curiosity"],
    "domain": ["science", "technology", "health", "finance", "law", "education", "arts", "sports", "politics", "daily_life"],
    "temporal": ["past", "present", "future", "recurring", "deadline", "duration"],
    "causality": ["cause", "effect", "condition", "purpose", "prevention", "correlation"],
    "social_register": ["formal", "casual", "technical", "playful", "polite", "urgent"],
}


class SemanticDim(NamedTuple):
    name: str
    index: int
    n_terms: int


def semantic_text_words(text: str | None) -> tuple[str, ...]:
    """Lower-cased word tokens (letters, digits, apostrophes folded away)."""
    if not text:
        return ()
    return tuple(re.findall(r"[a-z0-9]+", text.lower().replace("'", "")))


def normalize_semantic_term(term: str | None) -> str:
    return "_".join(semantic_text_words((term or "").replace("_", " ")))


def resolve_semantic_vocab_path(path_or_ref: str | Path | None = None) -> Path | None:
    """A path, a bare reference such as ``vocab_86d_gpt2`` looked up under
    ``NFN_SEMANTIC_VOCAB_DIR``, or ``None`` for the built-in vocabulary."""
    if path_or_ref is None or str(path_or_ref) in ("", "builtin"):
        return None
    p = Path(path_or_ref)
    if p.is_file():
        return p
    base = os.environ.get("NFN_SEMANTIC_VOCAB_DIR", "")
    for cand in (Path(base) / p.name, Path(base) / f"{p.name}.json"):
        if base and cand.is_file():
            return cand
    raise FileNotFoundError(f"semantic vocabulary {path_or_ref!r} not found (set NFN_SEMANTIC_VOCAB_DIR or pass a file path)")


def signature_to_bucket(sig: str, n_buckets: int = 4096, *, n_sig_buckets: int | None = None) -> int:
    """md5-based bucket of a signature string (stable across runs and platforms)."""
    n = n_sig_buckets if n_sig_buckets is not None else n_buckets
    if n <= 0:
        raise ValueError("n_buckets must be positive")
    return int(hashlib.md5(sig.encode("utf-8")).hexdigest()[:8], 16) % n


def signature_to_float(sig: str, n_buckets: int = 4096, *, n_sig_buckets: int | None = None) -> float:
    n = n_sig_buckets if n_sig_buckets is not None else n_buckets
    return signature_to_bucket(sig, n) / n


class ConversationalVocabulary:
    def __init__(self, path: str | Path | None = None) -> None:
        resolved = resolve_semantic_vocab_path(path)
        raw = _BUILTIN_VOCAB if resolved is None else json.loads(Path(resolved).read_text())["vocabulary"]
        self.path = resolved
        self._vocab: dict[str, list[str]] = {}
        self._index: dict[str, dict[str, int]] = {}
        self._phrases: dict[str, dict[tuple[str, ...], str]] = {}
        for dim, terms in raw.items():
            if not isinstance(terms, list) or any(not isinstance(t, str) for t in terms):
                raise ValueError(f"semantic vocabulary dimension {dim!r} must be a list of strings")
            self._vocab[dim] = list(terms)
            idx, phrases = {}, {}
            for i, t in enumerate(terms):
                key = normalize_semantic_term(t)
                idx.setdefault(key, i)
                words = tuple(key.split("_")) if key else ()
                if words:
                    phrases.setdefault(words, t)
            self._index[dim], self._phrases[dim] = idx, phrases
        self.dim_names = list(self._vocab)
        self.dimension_to_expert = {n: i for i, n in enumerate(self.dim_names)}
        self.expert_to_dimension = {i: n for n, i in self.dimension_to_expert.items()}

    # sizes
    @property
    def num_vocab_dims(self) -> int:
        return len(self.dim_names)

    @property
    def vector_dim(self) -> int:
        return self.num_vocab_dims + 1  # + signature slot

    @property
    def semantic_dims(self) -> list[SemanticDim]:
        return [SemanticDim(n, i, len(self._vocab[n])) for i, n in enumerate(self.dim_names)]

    @property
    def semantic_dim_names(self) -> list[str]:
        return self.dim_names + [TAXONOMY_HASH_NAME]

    @property
    def term_counts(self) -> dict[str, int]:
        return {n: len(t) for n, t in self._vocab.items()}

    @property
    def max_terms(self) -> int:
        return max(self.term_counts.values(), default=0)

    def terms(self, dim_name: str) -> list[str]:
        return self._vocab.get(dim_name, [])

    def term_to_index(self, dim_name: str, term: str) -> int:
        return self._index.get(dim_name, {}).get(normalize_semantic_term(term), -1)

    def resolve_term(self, dim_name: str, term: str) -> str | None:
        i = self.term_to_index(dim_name, term)
        return self._vocab[dim_name][i] if i >= 0 else None

    def match_topics_in_text(self, text: str) -> dict[str, str]:
        """Per dimension, the longest contiguous phrase of the text that is a term
        (earliest occurrence wins among equally long matches)."""
        words = semantic_text_words(text)
        out: dict[str, str] = {}
        for dim in self.dim_names:
            phrases = self._phrases[dim]
            if not phrases:
                continue
            longest = max(len(p) for p in phrases)
            best: tuple[int, int, str] | None = None  # (-length, start, term)
            for start in range(len(words)):
                for n in range(min(longest, len(words) - start), 0, -1):
                    term = phrases.get(words[start:start + n])
                    if term is not None:
                        cand = (-n, start, term)
                        if best is None or cand < best:
                            best = cand
                        break
            if best is not None:
                out[dim] = best[2]
        return out

    def encode_row(self, row: dict[str, str], n_sig_buckets: int = 4096) -> np.ndarray:
        vec = np.zeros(self.vector_dim, dtype=np.float32)
        for i, dim in enumerate(self.dim_names):
            idx, n = self.term_to_index(dim, row.get(dim, "")), len(self._vocab[dim])
            if idx >= 0 and n > 1:
                vec[i] = 2.0 * idx / (n - 1) - 1.0
        sig = row.get("semantic_signature", "")
        if sig:
            vec[self.num_vocab_dims] = signature_to_float(sig, n_sig_buckets)
        return vec

    def decode_vector(self, vec: np.ndarray) -> dict[str, str | float]:
        vec = np.asarray(vec, dtype=np.float32).ravel()
        out: dict[str, str | float] = {}
        for i, dim in enumerate(self.dim_names):
            terms = self._vocab[dim]
            if not terms:
                out[dim] = ""
                continue
            idx = int(round((float(vec[i]) + 1.0) / 2.0 * (len(terms) - 1)))
            out[dim] = terms[max(0, min(idx, len(terms) - 1))]
        if len(vec) > self.num_vocab_dims:
            out[TAXONOMY_HASH_NAME] = float(vec[self.num_vocab_dims])
        return out


def _vocab(v: ConversationalVocabulary | None) -> ConversationalVocabulary:
    return v if v is not None else ConversationalVocabulary()


def build_semantic_signature(target: np.ndarray, *, vocab: ConversationalVocabulary | None = None) -> str:
    """``ent_act_dom``: first three letters of the entity / action / domain terms (``non`` if unset)."""
    vocab = _vocab(vocab)
    target = np.asarray(target, dtype=np.int64).ravel()
    parts = []
    for dim in _SIGNATURE_DIMS:
        di = vocab.dimension_to_expert.get(dim)
        terms = vocab.terms(dim)
        ti = int(target[di]) if di is not None and di < target.shape[0] else SEMANTIC_IGNORE_INDEX
        parts.append(terms[ti][:3].lower() if 0 <= ti < len(terms) else "non")
    return "_".join(parts)


def resolve_semantic_topics(topics: dict[str, str], *, vocab: ConversationalVocabulary | None = None) -> dict[str, str]:
    vocab = _vocab(vocab)
    out = {}
    for dim, topic in topics.items():
        if dim not in vocab.dimension_to_expert:
            raise ValueError(f"Unknown semantic dimension {dim!r}")
        term = vocab.resolve_term(dim, topic)
        if term is None:
            raise ValueError(f"Unknown topic {topic!r} for dimension {dim!r}")
        out[dim] = term
    return out


def extract_semantic_topics_from_text(text: str, *, vocab: ConversationalVocabulary | None = None) -> dict[str, str]:
    return _vocab(vocab).match_topics_in_text(text)


def build_semantic_targets_from_topics(topics: dict[str, str], *, vocab: ConversationalVocabulary | None = None,
                                       n_sig_buckets: int = 4096) -> np.ndarray:
    vocab = _vocab(vocab)
    target = np.full(vocab.vector_dim, SEMANTIC_IGNORE_INDEX, dtype=np.int64)
    for dim, term in resolve_semantic_topics(topics, vocab=vocab).items():
        target[vocab.dimension_to_expert[dim]] = vocab.term_to_index(dim, term)
    target[vocab.num_vocab_dims] = signature_to_bucket(build_semantic_signature(target, vocab=vocab), n_sig_buckets)
    return target


def semantic_targets_to_vectors(targets: np.ndarray, *, vocab: ConversationalVocabulary | None = None,
                                n_sig_buckets: int = 4096) -> np.ndarray:
    vocab = _vocab(vocab)
    arr = np.atleast_2d(np.asarray(targets, dtype=np.int64))
    vecs = np.zeros((arr.shape[0], vocab.vector_dim), dtype=np.float32)
    for di, dim in enumerate(vocab.dim_names):
        n, idx = len(vocab.terms(dim)), arr[:, di]
        ok = idx >= 0
        if n > 1:
            vecs[ok, di] = 2.0 * idx[ok].astype(np.float32) / float(n - 1) - 1.0
    if arr.shape[1] > vocab.num_vocab_dims and n_sig_buckets > 1:
        h = arr[:, vocab.num_vocab_dims]
        ok = h >= 0
        vecs[ok, vocab.num_vocab_dims] = h[ok].astype(np.float32) / float(n_sig_buckets - 1)
    return vecs


def semantic_targets_to_router_vectors(targets: np.ndarray, *, vocab: ConversationalVocabulary | None = None) -> np.ndarray:
    vocab = _vocab(vocab)
    arr = np.atleast_2d(np.asarray(targets, dtype=np.int64))
    vecs = np.zeros((arr.shape[0], vocab.num_vocab_dims), dtype=np.float32)
    for di, dim in enumerate(vocab.dim_names):
        n, idx = len(vocab.terms(dim)), arr[:, di]
        ok = idx >= 0
        if n > 1:
            vecs[ok, di] = idx[ok].astype(np.float32) / float(n - 1)
        elif n == 1:
            vecs[ok, di] = 1.0
    return vecs


def load_training_targets(n: int = 100_000, *, vocab: ConversationalVocabulary | None = None, seed: int = 0, active_dims: int = 2,
                          n_sig_buckets: int = 4096) -> tuple[np.ndarray, np.ndarray]:
    """Deterministic synthetic targets: ``active_dims`` random dimensions per row get a random term."""
    vocab = _vocab(vocab)
    rng = np.random.RandomState(seed)
    ids = np.arange(n, dtype=np.int64)
    targets = np.full((n, vocab.vector_dim), SEMANTIC_IGNORE_INDEX, dtype=np.int64)
    k = max(1, min(int(active_dims), vocab.num_vocab_dims))
    for r in range(n):
        for di in np.sort(rng.choice(vocab.num_vocab_dims, size=k, replace=False)):
            nt = len(vocab.terms(vocab.dim_names[int(di)]))
            targets[r, int(di)] = int(rng.randint(0, max(nt, 1))) if nt > 0 else 0
        targets[r, vocab.num_vocab_dims] = signature_to_bucket(build_semantic_signature(targets[r], vocab=vocab), n_sig_buckets)
    return ids, targets


def load_training_data(n: int = 100_000, *, vocab: ConversationalVocabulary | None = None, seed: int = 0, active_dims: int = 2,
                       n_sig_buckets: int = 4096) -> tuple[np.ndarray, np.ndarray]:
    ids, targets = load_training_targets(n, vocab=vocab, seed=seed, active_dims=active_dims, n_sig_buckets=n_sig_buckets)
    return ids, semantic_targets_to_vectors(targets, vocab=vocab, n_sig_buckets=n_sig_buckets)


class SemanticHasher:
    """Multi-table random-hyperplane LSH (``tables`` x ``planes`` sign bits) with exact
    cosine re-ranking of the candidate union."""

    def __init__(self, dim: int, tables: int = 8, planes: int = 12, seed: int = 42) -> None:
        self.dim, self.n_tables, self.n_planes = dim, tables, planes
        self.proj = np.random.RandomState(seed).randn(tables, planes, dim).astype(np.float32)
        self._buckets: list[dict[bytes, list[int]]] = [defaultdict(list) for _ in range(tables)]
        self._ids: np.ndarray | None = None
        self._vecs: np.ndarray | None = None

    def hash(self, vec: np.ndarray) -> tuple[bytes, ...]:
        bits = (self.proj @ np.asarray(vec, dtype=np.float32).ravel()) > 0
        return tuple(bits[t].tobytes() for t in range(self.n_tables))

    def index(self, ids: np.ndarray, vecs: np.ndarray) -> None:
        self._ids, self._vecs = np.asarray(ids), np.asarray(vecs, dtype=np.float32)
        bits = np.einsum("tpd,nd->ntp", self.proj, self._vecs) > 0
        for i in range(len(self._ids)):
            for t in range(self.n_tables):
                self._buckets[t][bits[i, t].tobytes()].append(i)

    def query(self, vec: np.ndarray, k: int = 128) -> tuple[np.ndarray, np.ndarray]:
        if self._ids is None or self._vecs is None:
            raise RuntimeError("Hasher has no indexed data. Call index() first.")
        cand: set[int] = set()
        for t, key in enumerate(self.hash(vec)):
            cand.update(self._buckets[t].get(key, ()))
        if not cand:
            return np.array([], dtype=np.int64), np.array([], dtype=np.float32)
        ci = np.array(sorted(cand), dtype=np.int64)
        q = np.asarray(vec, dtype=np.float32).ravel()
        nrm = np.linalg.norm(q)
        scores = self._vecs[ci] @ (q / nrm if nrm > 0 else q)
        top = np.argsort(-scores, kind="stable")[:min(k, len(scores))]
        return self._ids[ci[top]], scores[top]

    def get_projection_planes(self) -> np.ndarray:
        return self.proj.copy()


class SemanticMatrix:
    """``.npz`` with ``ids`` (N,) and ``vectors`` (N, dim); brute-force neighbours and an LSH index."""

    def __init__(self, path: str | Path) -> None:
        data = np.load(Path(path))
        self.ids, self.vectors = data["ids"], data["vectors"].astype(np.float32)
        nrm = np.linalg.norm(self.vectors, axis=1, keepdims=True)
        self._unit = self.vectors / np.where(nrm > 0, nrm, 1.0)

    def neighbors(self, vec: np.ndarray, k: int = 128) -> tuple[np.ndarray, np.ndarray]:
        q = np.asarray(vec, dtype=np.float32).ravel()
        nrm = np.linalg.norm(q)
        scores = self._unit @ (q / nrm if nrm > 0 else q)
        top = np.argsort(-scores, kind="stable")[:min(k, len(scores))]
        return self.ids[top], scores[top]

    def build_hasher(self, tables: int = 8, planes: int = 12, seed: int = 42) -> SemanticHasher:
        h = SemanticHasher(self.vectors.shape[1], tables, planes, seed)
        h.index(self.ids, self.vectors)
        return h


def generate_synthetic_semantic_data(n: int = 100_000, seed: int = 0, out_dir: str | Path = ".", *,
                                     vocab: ConversationalVocabulary | None = None) -> Path:
    ids, vecs = load_training_data(n, vocab=vocab, seed=seed)
    out = Path(out_dir) / "semantic_vectors.npz"
    out.parent.mkdir(parents=True, exist_ok=True)
    np.savez(out, ids=ids, vectors=vecs)
    return out
