"""Python front-ends of the native data readers.

``TokenDataset`` / ``ByteDataset`` resolve a dataset alias or path and validate every
shard; ``TokenSampler`` yields ``(tokens, targets)`` int32 batches in the sequential window
order of the reference's ``SequentialTokenBatchSampler32`` (``token_shards.cpp:1278-1390``)
with data-parallel rank striding and ``seek`` for resume; ``PrefetchingLoader`` keeps a ring
of pinned host buffers filled by a native thread; ``RecordReader`` reads structured SFT /
preference / PPO-prompt records (``token_shards.h:76-233``).
"""
from __future__ import annotations

import ctypes as C
from typing import Iterator

import numpy as np
import torch

from . import _rt

TRAIN, VAL = 0, 1
_SPLIT = {"train": 0, "val": 1, "validation": 1, 0: 0, 1: 1}
_ZERO_SHA = "0" * 64


class _Dataset:
    _kind = 0

    def __init__(self, alias_or_path: str, *, allow_train_as_val: bool = False, require_validation: bool = True) -> None:
        self._h = _rt.handle(_rt.lib().nfn_dataset_open(str(alias_or_path).encode(), self._kind, int(allow_train_as_val),
                                                        int(require_validation)), "dataset_open")

    def close(self) -> None:
        if getattr(self, "_h", None):
            _rt.lib().nfn_dataset_close(self._h)
            self._h = None

    __del__ = close

    def describe(self, seq_len: int = 0, batch_size: int = 0, train_batch_tokens: int = 0) -> dict:
        return _rt.read_json(_rt.lib().nfn_dataset_json, self._h, seq_len, batch_size, train_batch_tokens)

    def tokens(self, split="train") -> int:
        return int(_rt.lib().nfn_dataset_tokens(self._h, _SPLIT[split]))

    def max_token(self, split="train") -> int:
        return int(_rt.lib().nfn_dataset_max_token(self._h, _SPLIT[split]))

    def sampler(self, split, seq_len: int, batch_size: int, rank: int = 0, world: int = 1) -> "TokenSampler":
        return TokenSampler(self, split, seq_len, batch_size, rank, world)


class TokenDataset(_Dataset):
    _kind = 0


class ByteDataset(_Dataset):
    _kind = 1


class TokenSampler:
    def __init__(self, dataset: _Dataset, split, seq_len: int, batch_size: int, rank: int = 0, world: int = 1) -> None:
        self.dataset, self.seq_len, self.batch_size = dataset, int(seq_len), int(batch_size)
        self._h = _rt.handle(_rt.lib().nfn_sampler_open(dataset._h, _SPLIT[split], seq_len, batch_size, rank, world),
                             "sampler_open")

    def close(self) -> None:
        if getattr(self, "_h", None):
            _rt.lib().nfn_sampler_close(self._h)
            self._h = None

    __del__ = close

    @property
    def total_batches(self) -> int:
        return int(_rt.lib().nfn_sampler_total_batches(self._h))

    @property
    def position(self) -> int:
        return int(_rt.lib().nfn_sampler_position(self._h))

    def seek(self, batch_index: int) -> None:
        _rt.check(_rt.lib().nfn_sampler_seek(self._h, batch_index), "sampler_seek")

    def reset(self) -> None:
        _rt.lib().nfn_sampler_reset(self._h)

    def next_into(self, tokens: torch.Tensor, targets: torch.Tensor, wrap: bool = False) -> bool:
        assert tokens.dtype == torch.int32 and targets.dtype == torch.int32 and tokens.device.type == "cpu"
        assert tokens.is_contiguous() and targets.is_contiguous()
        fn = _rt.lib().nfn_sampler_next_wrap_i32 if wrap else _rt.lib().nfn_sampler_next_i32
        return _rt.check(fn(self._h, tokens.data_ptr(), targets.data_ptr(), tokens.numel()), "sampler_next") == 1

    def next(self, wrap: bool = False):
        tok = torch.empty(self.batch_size, self.seq_len, dtype=torch.int32)
        tgt = torch.empty_like(tok)
        return (tok, tgt) if self.next_into(tok, tgt, wrap) else None

    def __iter__(self) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
        while (b := self.next()) is not None:
            yield b


class PrefetchingLoader:
    """Endless iterator over a sampler through ``slots`` pinned staging buffers filled by a
    native background thread. The tensors yielded alias the ring: they stay valid until
    the next ``__next__`` call (which hands the slot back)."""

    def __init__(self, sampler: TokenSampler, slots: int = 3, pin: bool | None = None) -> None:
        self.sampler = sampler
        pin = torch.cuda.is_available() if pin is None else pin
        shape = (sampler.batch_size, sampler.seq_len)
        mk = (lambda: torch.empty(shape, dtype=torch.int32).pin_memory()) if pin else (lambda: torch.empty(shape, dtype=torch.int32))
        self.tokens = [mk() for _ in range(slots)]
        self.targets = [mk() for _ in range(slots)]
        arr = C.c_void_p * slots
        self._h = _rt.handle(_rt.lib().nfn_prefetcher_open(sampler._h, slots, arr(*[t.data_ptr() for t in self.tokens]),
                                                           arr(*[t.data_ptr() for t in self.targets]), self.tokens[0].numel()),
                             "prefetcher_open")
        self._held = -1
        self.batch_index = -1

    def __iter__(self):
        return self

    def __next__(self):
        L = _rt.lib()
        if self._held >= 0:
            _rt.check(L.nfn_prefetcher_release(self._h, self._held), "prefetcher_release")
            self._held = -1
        idx = C.c_int64(0)
        slot = _rt.check(L.nfn_prefetcher_acquire(self._h, C.byref(idx)), "prefetcher_acquire")
        self._held, self.batch_index = slot, int(idx.value)
        return self.tokens[slot], self.targets[slot]

    def close(self) -> None:
        if getattr(self, "_h", None):
            _rt.lib().nfn_prefetcher_close(self._h)
            self._h = None

    __del__ = close


class RecordReader:
    KINDS = {"sft": 0, "preference": 1, "ppo_prompt": 2}

    def __init__(self, alias_or_path: str, kind: str, split="train", batch_size: int = 1, *, allow_train_as_val: bool = False,
                 rank: int = 0, world: int = 1) -> None:
        self.kind, self.batch_size = kind, int(batch_size)
        self._h = _rt.handle(_rt.lib().nfn_records_open(str(alias_or_path).encode(), self.KINDS[kind], _SPLIT[split],
                                                        int(allow_train_as_val), batch_size, rank, world), "records_open")
        self.seq_len = int(_rt.lib().nfn_records_seq_len(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            _rt.lib().nfn_records_close(self._h)
            self._h = None

    __del__ = close

    def describe(self) -> dict:
        return _rt.read_json(_rt.lib().nfn_records_json, self._h)

    @property
    def total_batches(self) -> int:
        return int(_rt.lib().nfn_records_total_batches(self._h))

    def seek(self, batch_index: int) -> None:
        _rt.check(_rt.lib().nfn_records_seek(self._h, batch_index), "records_seek")

    def reset(self) -> None:
        _rt.lib().nfn_records_reset(self._h)

    def next(self) -> dict | None:
        """SFT: dict of (B, T) tensors. Preference: ``chosen_*`` / ``rejected_*`` entries.
        PPO prompt: ``input_ids`` and ``attention_mask``."""
        B, T = self.batch_size, self.seq_len
        rows = 2 * B if self.kind == "preference" else B
        ids = torch.empty(rows, T, dtype=torch.int32)
        mask = torch.empty(rows, T, dtype=torch.float32)
        tg = torch.empty(rows, T, dtype=torch.int32)
        seg = torch.empty(rows, T, dtype=torch.int32)
        got = _rt.check(_rt.lib().nfn_records_next(self._h, ids.data_ptr(), tg.data_ptr(), mask.data_ptr(), seg.data_ptr(),
                                                   ids.numel()), "records_next")
        if got == 0:
            return None
        if self.kind == "ppo_prompt":
            return {"input_ids": ids, "attention_mask": mask}
        if self.kind == "sft":
            return {"input_ids": ids, "targets": tg, "loss_mask": mask, "sequence_ids": seg}
        out = {}
        for name, sl in (("chosen", slice(0, B)), ("rejected", slice(B, 2 * B))):
            out.update({f"{name}_input_ids": ids[sl], f"{name}_targets": tg[sl], f"{name}_loss_mask": mask[sl],
                        f"{name}_sequence_ids": seg[sl]})
        return out

    def __iter__(self):
        while (b := self.next()) is not None:
            yield b


# ---- writers -----------------------------------------------------------------------------

def write_legacy_shard(path, tokens, with_header: bool = False) -> None:
    arr = np.ascontiguousarray(np.asarray(tokens, dtype=np.uint16))
    _rt.check(_rt.lib().nfn_write_legacy_shard(str(path).encode(), arr.ctypes.data, arr.size, int(with_header)), "write_legacy_shard")


def write_v2_shard(path, tokens, vocab_size: int, *, tokenizer_sha256: str = _ZERO_SHA, tokenizer_revision: str = "local",
                   split: str = "train", objective: str = "pretrain", tokenizer_name: str = "synthetic") -> None:
    arr = np.ascontiguousarray(np.asarray(tokens, dtype=np.uint32))
    _rt.check(_rt.lib().nfn_write_v2_shard(str(path).encode(), arr.ctypes.data, arr.size, vocab_size, tokenizer_sha256.encode(),
                                           tokenizer_revision.encode(), split.encode(), objective.encode(),
                                           tokenizer_name.encode()), "write_v2_shard")


def _sft_payload(input_ids, targets, loss_mask, sequence_ids) -> np.ndarray:
    ids = np.asarray(input_ids, dtype="<u4")
    n, T = ids.shape
    rec = np.empty((n, 4, T), dtype="<u4")
    rec[:, 0] = ids
    rec[:, 1] = np.asarray(targets, dtype="<i4").view("<u4")
    rec[:, 2] = np.asarray(loss_mask, dtype="<f4").view("<u4")
    rec[:, 3] = np.asarray(sequence_ids if sequence_ids is not None else np.zeros((n, T)), dtype="<i4").view("<u4")
    return rec


def _write_records(path, kind: int, payload: np.ndarray, n: int, T: int, vocab_size: int, pad_token_id: int, split: str,
                   tokenizer_sha256: str, chat_template_sha256: str, tokenizer_revision: str) -> None:
    payload = np.ascontiguousarray(payload)
    _rt.check(_rt.lib().nfn_write_records(str(path).encode(), kind, n, T, vocab_size, pad_token_id, tokenizer_sha256.encode(),
                                          chat_template_sha256.encode(), tokenizer_revision.encode(), split.encode(),
                                          payload.ctypes.data, payload.nbytes), "write_records")


def write_sft_records(path, input_ids, targets, loss_mask, sequence_ids=None, *, vocab_size: int, pad_token_id: int = 0,
                      split: str = "train", tokenizer_sha256: str = _ZERO_SHA, chat_template_sha256: str = _ZERO_SHA,
                      tokenizer_revision: str = "local") -> None:
    rec = _sft_payload(input_ids, targets, loss_mask, sequence_ids)
    _write_records(path, 0, rec, rec.shape[0], rec.shape[2], vocab_size, pad_token_id, split, tokenizer_sha256,
                   chat_template_sha256, tokenizer_revision)


def write_preference_records(path, chosen: dict, rejected: dict, *, vocab_size: int, pad_token_id: int = 0, split: str = "train",
                             tokenizer_sha256: str = _ZERO_SHA, chat_template_sha256: str = _ZERO_SHA,
                             tokenizer_revision: str = "local") -> None:
    a = _sft_payload(chosen["input_ids"], chosen["targets"], chosen["loss_mask"], chosen.get("sequence_ids"))
    b = _sft_payload(rejected["input_ids"], rejected["targets"], rejected["loss_mask"], rejected.get("sequence_ids"))
    rec = np.stack([a, b], axis=1)  # (n, 2, 4, T)
    _write_records(path, 1, rec, rec.shape[0], rec.shape[3], vocab_size, pad_token_id, split, tokenizer_sha256,
                   chat_template_sha256, tokenizer_revision)


def write_ppo_prompt_records(path, input_ids, attention_mask, *, vocab_size: int, pad_token_id: int = 0, split: str = "train",
                             tokenizer_sha256: str = _ZERO_SHA, chat_template_sha256: str = _ZERO_SHA,
                             tokenizer_revision: str = "local") -> None:
    ids = np.asarray(input_ids, dtype="<u4")
    n, T = ids.shape
    rec = np.empty((n, 2, T), dtype="<u4")
    rec[:, 0] = ids
    rec[:, 1] = np.asarray(attention_mask, dtype="<f4").view("<u4")
    _write_records(path, 2, rec, n, T, vocab_size, pad_token_id, split, tokenizer_sha256, chat_template_sha256, tokenizer_revision)
