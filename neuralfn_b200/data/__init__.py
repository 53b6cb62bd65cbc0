"""Training-data readers backed by the native runtime library (memory-mapped token / byte
shards, structured post-training records, background prefetch into pinned buffers)."""
from .shards import (ByteDataset, PrefetchingLoader, RecordReader, TokenDataset, TokenSampler, write_legacy_shard,
                     write_ppo_prompt_records, write_preference_records, write_sft_records, write_v2_shard)

__all__ = ["TokenDataset", "ByteDataset", "TokenSampler", "PrefetchingLoader", "RecordReader", "write_legacy_shard",
           "write_v2_shard", "write_sft_records", "write_preference_records", "write_ppo_prompt_records"]
