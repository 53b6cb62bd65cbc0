"""Media in the resident engine's prompt: the vision tower (``neuralfn_b200.vision`` / the ``muse_glimmer_vision_tower`` stage)
turns images and video frames into feature rows of the model width; here they replace the embedding rows of the media
placeholder tokens, and the fused rows go to the engine as the prompt's layer-0 inputs (``ResidentEngine.prefill_rows``).

Order of operations, as in the reference's fusion graph (``neuralfn/torch_templates.py:1290-1325``): token embeddings are
normalised by the model's weightless embedding norm, media features by the perception norm with the same epsilon, then image
rows and video rows are scattered, in order, over their placeholder positions. From there on the prompt is ordinary: the
KV cache, decoding, verification blocks and hidden-state taps do not know which rows were media.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .engine import EngineConfig

__all__ = ["fuse_media_rows", "prefill_with_media"]


def _weightless_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)


def fuse_media_rows(config: EngineConfig, embed: torch.Tensor, token_ids: Sequence[int], media: dict[int, torch.Tensor], *,
                    features_normalised: bool = False) -> torch.Tensor:
    """bf16 [n, d_model] layer-0 input rows. ``embed``: the embedding table [vocab, d]; ``media``: placeholder token id ->
    feature rows [count, d] in prompt order (e.g. ``{image_token_id: image_features, video_token_id: video_features}``)."""
    ids = torch.as_tensor(list(token_ids), dtype=torch.long, device=embed.device)
    rows = embed[ids].float() * float(getattr(config, "embed_scale", 1.0) or 1.0)
    if getattr(config, "embed_norm", 0):
        rows = _weightless_rms(rows, config.norm_eps)
    for token_id, feats in media.items():
        at = (ids == int(token_id)).nonzero().flatten()
        if feats.dim() != 2 or feats.shape[1] != rows.shape[1] or at.numel() != feats.shape[0]:
            raise ValueError(f"{at.numel()} placeholders of token {token_id} but {tuple(feats.shape)} media features")
        f = feats.to(rows.device).float()
        rows[at] = f if features_normalised else _weightless_rms(f, config.norm_eps)
    return rows.to(torch.bfloat16)


def prefill_with_media(session, embed: torch.Tensor, token_ids: Sequence[int], media: dict[int, torch.Tensor], **kw) -> dict[str, int]:
    """``NativeInferenceSession.prefill`` for a prompt with media placeholders. The session must be empty (the engine starts
    row prompts at position 0); afterwards it decodes, forks and truncates like any other."""
    if session.token_ids:
        raise ValueError("media prompts start a session: reset it first")
    eng = session.model.engine
    if eng.config.family != 1:
        raise ValueError("media prompts need a Llama-family (Glimmer) engine layout")
    ids = [int(t) for t in token_ids]
    rows = fuse_media_rows(eng.config, embed, ids, media, **kw)
    with session.model._lock:
        session._next_greedy = eng.prefill_rows(session.slot, rows)
        session._tokens = ids
        session._pending = None
    session._stats["prefill_tokens"] += len(ids)
    return {"prompt_tokens": len(ids), "total_tokens": len(ids), "media_rows": sum(int(v.shape[0]) for v in media.values())}
