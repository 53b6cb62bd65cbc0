"""Checkpoint formats: dense GPT (model / fp32 parameters / optimizer / rank-sharded
optimizer + manifest), Glimmer directories, GGUF import, native IR manifests."""
from .container import peek_header, publish_dir, read_container, write_container
from .dense import (consolidate_sharded_optimizer, inspect_dense_model, latest_step, load_dense_checkpoint,
                    read_dense_model, save_dense_checkpoint, write_dense_model)

__all__ = ["write_container", "read_container", "peek_header", "publish_dir", "write_dense_model", "read_dense_model",
           "inspect_dense_model", "save_dense_checkpoint", "load_dense_checkpoint", "consolidate_sharded_optimizer",
           "latest_step"]
