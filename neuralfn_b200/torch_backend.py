"""Public tensor-runtime names in one place (``CompiledTorchGraph``, ``TorchTrainer``,
``TorchTrainConfig``, ``build_module`` and every ``*Stage`` class), mirroring the import
surface of the reference's ``neuralfn/torch_backend.py``. The implementation lives in
``neuralfn_b200.tensor``."""
from __future__ import annotations

from .tensor import (stages_attention, stages_attention_blocks, stages_core, stages_linear,  # noqa: F401
                     stages_losses, stages_misc, stages_moe)
from .tensor.compiler import CompiledTorchGraph, build_function_module
from .tensor.stages_core import STAGE_REGISTRY, build_module
from .tensor.trainer import Muon, TorchTrainConfig, TorchTrainer, graph_topology_sha256, resolve_amp_settings
from .tensor.stages_attention import (apply_rotary_emb, apply_rotary_emb_hf, apply_rotary_interleaved,
                                      rope_inv_freq, sparse_attention_mask)

_g = globals()
for _mod in (stages_core, stages_linear, stages_attention, stages_attention_blocks, stages_moe,
             stages_losses, stages_misc):
    for _name, _obj in vars(_mod).items():
        if _name.endswith("Stage") and isinstance(_obj, type):
            _g[_name] = _obj
del _g, _mod, _name, _obj
