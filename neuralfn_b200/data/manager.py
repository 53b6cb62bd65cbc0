"""Dataset manager: turns text (or ready token arrays) into cached native shard directories and
keeps a manifest per dataset.

A dataset lives in ``<cache>/<name>/<variant>/`` and holds ``fineweb_train_%06d.bin`` /
``fineweb_val_%06d.bin`` shards in the v2 format (the C++ loader opens the directory as is),
plus ``manifest.json``: tokenizer name and digest, vocabulary size, token counts per split, the
source files with their SHA-256, and the shard list. A *variant* is one tokenisation of the
same sources (``bytes``, ``tiktoken:gpt2``, a ``tokenizer.json`` ...). Preparing an existing
variant is refused unless ``overwrite=True``; nothing is downloaded - sources are local files.

Behavioural counterpart: ``server/dataset_manager.py`` (download + tokenise + cache under
``~/.cache/nfn/datasets``, variants).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import time
from pathlib import Path
from typing import Iterable, Sequence

import numpy as np

from .shards import write_v2_shard

__all__ = ["DatasetManager", "DatasetError", "default_cache_dir"]


class DatasetError(RuntimeError):
    pass


def default_cache_dir() -> Path:
    return Path(os.environ.get("NFN_DATASET_CACHE", Path.home() / ".cache" / "nfn" / "datasets"))


def _sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def _variant_dir_name(tokenizer: str) -> str:
    return "".join(c if c.isalnum() or c in "-_." else "_" for c in tokenizer)


class DatasetManager:
    def __init__(self, cache_dir: str | Path | None = None) -> None:
        self.root = Path(cache_dir) if cache_dir is not None else default_cache_dir()

    # -- queries ---------------------------------------------------------------------------
    def list(self) -> list[dict]:
        out = []
        if not self.root.is_dir():
            return out
        for d in sorted(p for p in self.root.iterdir() if p.is_dir()):
            variants = [v.name for v in sorted(d.iterdir()) if (v / "manifest.json").is_file()]
            if variants:
                out.append({"name": d.name, "variants": variants})
        return out

    def path(self, name: str, variant: str | None = None) -> Path:
        base = self.root / name
        if variant is None:
            found = [v for v in sorted(base.iterdir()) if (v / "manifest.json").is_file()] if base.is_dir() else []
            if len(found) != 1:
                raise DatasetError(f"dataset {name!r} has {len(found)} variants; name one")
            return found[0]
        p = base / _variant_dir_name(variant)
        if not (p / "manifest.json").is_file():
            raise DatasetError(f"dataset {name!r} has no variant {variant!r}")
        return p

    def info(self, name: str, variant: str | None = None) -> dict:
        return json.loads((self.path(name, variant) / "manifest.json").read_text(encoding="utf-8"))

    def delete(self, name: str, variant: str | None = None) -> None:
        target = self.path(name, variant) if variant is not None else self.root / name
        if not target.is_dir() or self.root not in target.parents:
            raise DatasetError(f"no such dataset directory: {target}")
        shutil.rmtree(target)

    # -- preparation -----------------------------------------------------------------------
    def prepare_text(self, name: str, sources: Sequence[str | Path], *, tokenizer: str = "bytes", val_fraction: float = 0.05,
                     shard_tokens: int = 1 << 26, document_separator: Sequence[int] | None = None, overwrite: bool = False) -> dict:
        """Tokenises local text files (one document per file, or per blank-line-separated block
        for ``.txt``) into train / val shards. The last ``val_fraction`` of the documents of each
        source goes to validation."""
        from ..serving.chat import load_text_codec
        codec = load_text_codec(tokenizer if tokenizer != "bytes" else "bytes:0")
        vocab = int(codec.vocab_size or 0)
        if vocab <= 0:
            raise DatasetError(f"tokenizer {tokenizer!r} does not report a vocabulary size")
        sep = list(document_separator) if document_separator is not None else []
        train: list[np.ndarray] = []
        val: list[np.ndarray] = []
        src_meta = []
        for src in sources:
            p = Path(src)
            if not p.is_file():
                raise DatasetError(f"source {p} is not a file")
            text = p.read_text(encoding="utf-8")
            docs = [d for d in text.split("\n\n") if d.strip()] if p.suffix == ".txt" else [text]
            n_val = int(round(len(docs) * val_fraction)) if len(docs) > 1 else 0
            for i, d in enumerate(docs):
                ids = np.asarray(list(codec.encode(d)) + sep, dtype=np.uint32)
                (val if i >= len(docs) - n_val else train).append(ids)
            src_meta.append({"path": str(p), "bytes": p.stat().st_size, "sha256": _sha256_file(p), "documents": len(docs)})
        tok_digest = hashlib.sha256(f"{codec.name}:{tokenizer}:{vocab}".encode()).hexdigest()
        return self.prepare_tokens(name, np.concatenate(train) if train else np.zeros(0, np.uint32),
                                   np.concatenate(val) if val else np.zeros(0, np.uint32), vocab_size=vocab, variant=tokenizer,
                                   tokenizer_name=codec.name, tokenizer_sha256=tok_digest, shard_tokens=shard_tokens, sources=src_meta,
                                   overwrite=overwrite)

    def prepare_tokens(self, name: str, train_tokens: Iterable[int], val_tokens: Iterable[int], *, vocab_size: int, variant: str = "tokens",
                       tokenizer_name: str = "external", tokenizer_sha256: str = "0" * 64, shard_tokens: int = 1 << 26,
                       sources: list | None = None, overwrite: bool = False) -> dict:
        if not name or any(c in name for c in "/\\") or name.startswith("."):
            raise DatasetError("dataset names are single path components")
        out = self.root / name / _variant_dir_name(variant)
        if out.exists():
            if not overwrite:
                raise DatasetError(f"{out} exists (pass overwrite=True to rebuild it)")
            shutil.rmtree(out)
        staging = out.with_name(out.name + ".staging")
        if staging.exists():
            shutil.rmtree(staging)
        staging.mkdir(parents=True)
        tr = np.asarray(train_tokens, dtype=np.uint32)
        va = np.asarray(val_tokens, dtype=np.uint32)
        if tr.size < 2:
            raise DatasetError("a dataset needs at least two training tokens")
        if tr.size and int(tr.max()) >= vocab_size or va.size and int(va.max()) >= vocab_size:
            raise DatasetError("token id outside the vocabulary")
        shards = []
        for split, arr in (("train", tr), ("val", va)):
            for i, lo in enumerate(range(0, arr.size, shard_tokens)):
                part = arr[lo:lo + shard_tokens]
                fname = f"fineweb_{split}_{i:06d}.bin"
                write_v2_shard(staging / fname, part, vocab_size, tokenizer_sha256=tokenizer_sha256, tokenizer_revision="local",
                               split="validation" if split == "val" else split,
                               objective="pretrain", tokenizer_name=tokenizer_name[:31])
                shards.append({"file": fname, "split": split, "tokens": int(part.size), "sha256": _sha256_file(staging / fname)})
        manifest = {"schema": "neuralfn_b200.dataset.v1", "name": name, "variant": variant, "created": int(time.time()), "vocab_size": vocab_size,
                    "tokenizer": {"name": tokenizer_name, "sha256": tokenizer_sha256}, "train_tokens": int(tr.size), "val_tokens": int(va.size),
                    "shards": shards, "sources": sources or []}
        (staging / "manifest.json").write_text(json.dumps(manifest, indent=2), encoding="utf-8")
        os.rename(staging, out)
        return manifest

    def verify(self, name: str, variant: str | None = None) -> dict:
        """Re-hashes every shard against the manifest."""
        d = self.path(name, variant)
        man = json.loads((d / "manifest.json").read_text(encoding="utf-8"))
        for s in man["shards"]:
            if _sha256_file(d / s["file"]) != s["sha256"]:
                raise DatasetError(f"{s['file']} does not match its recorded digest")
        return man
