"""Vision stages of the Glimmer multimodal graphs: the packed image / video tower, the weightless
perception norm and the scatter of media features into placeholder token positions.

Same parameters, inputs and outputs as the reference's ``MuseGlimmerVisionTowerStage``,
``MuseGlimmerPerceptionNormStage`` and ``MuseGlimmerMediaScatterStage``
(``neuralfn/torch_backend.py:2013-2233``). The structure differs: all media of a batch are one packed
sequence, and window / full attention are the *same* packed attention call with a different
segment-id vector, so that on a B200 each layer is one flash-attention launch over every window of
every image instead of a Python loop with one launch per window. The learned position table is
resampled with ``grid_sample`` (bilinear, zeros outside), which is the same arithmetic as four
gathered corners with validity weights.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from . import kernel_bridge as KB
from .stages_core import stage


def vision_segments(grid_thw: Tensor, window: int) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """For media grids ``[n, 3]`` (frames, patch rows, patch columns), on the host:

    * ``order`` – permutation that makes every ``window x window`` tile of a frame contiguous
      (tiles in row-major order, row-major inside a tile),
    * ``window_ids`` / ``media_ids`` – segment id per position *in that order* (one id per tile, one
      id per medium),
    * ``yx`` – (row, column) of each patch inside its frame, in the original order.
    """
    g = grid_thw.detach().to("cpu", torch.int64)
    order, wid, mid, yx = [], [], [], []
    offset, next_window = 0, 0
    for m, (t, h, w) in enumerate(g.tolist()):
        f = torch.arange(t).view(t, 1, 1).expand(t, h, w)
        y = torch.arange(h).view(1, h, 1).expand(t, h, w)
        x = torch.arange(w).view(1, 1, w).expand(t, h, w)
        wh, ww = -(-h // window), -(-w // window)
        tile = (f * wh + y // window) * ww + x // window
        key = (tile * window + y % window) * window + x % window
        perm = torch.argsort(key.reshape(-1), stable=True)
        order.append(perm + offset)
        wid.append(tile.reshape(-1)[perm] + next_window)
        mid.append(torch.full((t * h * w,), m, dtype=torch.int64))
        yx.append(torch.stack((y.reshape(-1), x.reshape(-1)), dim=-1))
        offset += t * h * w
        next_window += t * wh * ww
    return torch.cat(order), torch.cat(wid), torch.cat(mid), torch.cat(yx)


def resample_position_table(table: Tensor, grid_thw: Tensor) -> Tensor:
    """Bilinear resampling of a square learned table ``[side * side, C]`` to every medium's patch
    grid (half-pixel centres, zero outside the table), repeated over frames: ``[sum t*h*w, C]``."""
    side = int(round(table.shape[0] ** 0.5))
    if side * side != table.shape[0]:
        raise ValueError("vision position table must be square")
    img = table.float().t().reshape(1, -1, side, side)
    out = []
    for t, h, w in grid_thw.detach().to("cpu", torch.int64).tolist():
        ys = ((torch.arange(h, device=table.device, dtype=torch.float32) + 0.5) / h) * 2 - 1
        xs = ((torch.arange(w, device=table.device, dtype=torch.float32) + 0.5) / w) * 2 - 1
        grid = torch.stack((xs.view(1, w).expand(h, w), ys.view(h, 1).expand(h, w)), dim=-1).unsqueeze(0)
        sampled = F.grid_sample(img, grid, mode="bilinear", padding_mode="zeros", align_corners=False)
        out.append(sampled.reshape(-1, h * w).t().to(table.dtype).repeat(t, 1))
    return torch.cat(out, dim=0)


class _VisionAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, rope_theta: float) -> None:
        super().__init__()
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim = self.hidden_size // self.num_heads
        self.rope_theta = float(rope_theta)
        self.q_proj = nn.Linear(hidden_size, hidden_size, bias=True)
        self.k_proj = nn.Linear(hidden_size, hidden_size, bias=True)
        self.v_proj = nn.Linear(hidden_size, hidden_size, bias=True)
        self.proj = nn.Linear(hidden_size, hidden_size, bias=True)

    def rope_tables(self, xy: Tensor, dtype) -> tuple[Tensor, Tensor]:
        """2-D rotary tables for (column, row) positions ``[n, 2]``: a quarter of the head for each of
        column / row, the pattern repeated for the second half that ``rotate_half`` pairs with."""
        quarter = self.head_dim // 2
        inv = 1.0 / (self.rope_theta ** (torch.arange(0, quarter, 2, device=xy.device, dtype=torch.float32) / quarter))
        fx, fy = xy[:, 0:1].float() * inv, xy[:, 1:2].float() * inv
        ang = torch.cat((fx, fy, fx, fy), dim=-1)
        return ang.cos().to(dtype), ang.sin().to(dtype)

    @staticmethod
    def _rotate(t: Tensor, cos: Tensor, sin: Tensor) -> Tensor:      # t [n, H, D]
        a, b = t.chunk(2, dim=-1)
        return t * cos[:, None, :] + torch.cat((-b, a), dim=-1) * sin[:, None, :]

    def forward(self, x: Tensor, seg: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        n = x.shape[0]
        q = self._rotate(KB.linear(x, self.q_proj.weight, self.q_proj.bias).view(n, self.num_heads, self.head_dim), cos, sin)
        k = self._rotate(KB.linear(x, self.k_proj.weight, self.k_proj.bias).view(n, self.num_heads, self.head_dim), cos, sin)
        v = KB.linear(x, self.v_proj.weight, self.v_proj.bias).view(n, self.num_heads, self.head_dim)
        o = KB.segment_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0),
                                 seg.view(1, n), causal=False, scale=self.head_dim ** -0.5)
        return KB.linear(o.squeeze(0).transpose(0, 1).reshape(n, self.hidden_size), self.proj.weight, self.proj.bias)


class _VisionLayer(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, num_heads: int, rope_theta: float, eps: float) -> None:
        super().__init__()
        self.norm1 = nn.LayerNorm(hidden_size, eps=eps)
        self.norm2 = nn.LayerNorm(hidden_size, eps=eps)
        self.attn = _VisionAttention(hidden_size, num_heads, rope_theta)
        self.fc1 = nn.Linear(hidden_size, intermediate_size, bias=True)
        self.fc2 = nn.Linear(intermediate_size, hidden_size, bias=True)

    def forward(self, x: Tensor, seg: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        x = x + self.attn(self.norm1(x), seg, cos, sin)
        return x + KB.linear(F.gelu(KB.linear(self.norm2(x), self.fc1.weight, self.fc1.bias)), self.fc2.weight, self.fc2.bias)


@stage("muse_glimmer_vision_tower")
class MuseGlimmerVisionTowerStage(nn.Module):
    """(packed patches ``[n, temporal * 3 * patch * patch]``, grids ``[media, 3]``) -> merged patch
    features ``[n / merge^2, hidden * merge^2]``. Every fourth layer and the last attend over the
    whole medium, the others inside ``pos_emb_height``-patch windows."""

    def __init__(self, *, hidden_size: int = 1536, intermediate_size: int = 8960, num_heads: int = 16, num_layers: int = 50,
                 patch_size: int = 14, patch_temporal: int = 2, merge_size: int = 2, pos_emb_height: int = 32,
                 pos_emb_width: int = 32, rope_theta: float = 10000.0, eps: float = 1e-5) -> None:
        super().__init__()
        if pos_emb_height != pos_emb_width or hidden_size % num_heads != 0 or (hidden_size // num_heads) % 4 != 0:
            raise ValueError("invalid Muse Glimmer vision tower geometry")
        self.hidden_size, self.patch_size = int(hidden_size), int(patch_size)
        self.patch_temporal, self.merge_size = int(patch_temporal), int(merge_size)
        self.patch_embedding = nn.Linear(self.patch_temporal * 3 * self.patch_size ** 2, self.hidden_size, bias=False)
        self.position_embedding = nn.Embedding(pos_emb_height * pos_emb_width, self.hidden_size)
        self.pre_norm = nn.LayerNorm(self.hidden_size, eps=eps)
        self.layers = nn.ModuleList(_VisionLayer(self.hidden_size, intermediate_size, num_heads, rope_theta, eps)
                                    for _ in range(num_layers))
        self.post_norm = nn.LayerNorm(self.hidden_size, eps=eps)
        self.window_patches = int(pos_emb_height)

    @classmethod
    def from_config(cls, cfg):
        keys = ("hidden_size", "intermediate_size", "num_heads", "num_layers", "patch_size", "patch_temporal", "merge_size",
                "pos_emb_height", "pos_emb_width")
        kw = {k: int(cfg[k]) for k in keys if k in cfg}
        for k in ("rope_theta", "eps"):
            if k in cfg:
                kw[k] = float(cfg[k])
        return cls(**kw)

    def merge_patches(self, hidden: Tensor, grid_thw: Tensor) -> Tensor:
        """merge x merge neighbouring patches -> one row, channel-major ([C, merge^2] flattened)."""
        m, out, off = self.merge_size, [], 0
        for t, h, w in grid_thw.detach().to("cpu", torch.int64).tolist():
            n = t * h * w
            blk = hidden[off:off + n].view(t, h // m, m, w // m, m, self.hidden_size)
            out.append(blk.permute(0, 1, 3, 5, 2, 4).reshape(t * (h // m) * (w // m), self.hidden_size * m * m))
            off += n
        return torch.cat(out, dim=0)

    def forward(self, pixel_values: Tensor, grid_thw: Tensor) -> Tensor:
        if grid_thw.ndim != 2 or grid_thw.shape[1] != 3 or pixel_values.ndim < 2:
            raise ValueError("Muse Glimmer vision expects packed patches and [media,3] grids")
        flat = pixel_values.reshape(pixel_values.shape[0], -1)
        if flat.shape[1] != self.patch_embedding.in_features:
            raise ValueError("Muse Glimmer packed patch width is incorrect")
        grid = grid_thw.detach().to("cpu", torch.int64)
        if bool((grid <= 0).any()) or bool((grid[:, 1:] % self.merge_size != 0).any()) or int(grid.prod(-1).sum()) != flat.shape[0]:
            raise ValueError("Muse Glimmer grid and packed-patch geometry differ")
        dev = flat.device
        order, window_ids, media_ids, yx = (t.to(dev) for t in vision_segments(grid, self.window_patches))
        x = KB.linear(flat.to(self.patch_embedding.weight.dtype), self.patch_embedding.weight, None)
        x = self.pre_norm(x + resample_position_table(self.position_embedding.weight, grid).to(x.dtype))
        x = x[order]
        xy = (yx.flip(-1) + 1)[order]                       # 1-based (column, row)
        cos, sin = self.layers[0].attn.rope_tables(xy, x.dtype) if len(self.layers) else (None, None)
        last = len(self.layers) - 1
        for i, layer in enumerate(self.layers):
            full = (i + 1) % 4 == 0 or i == last
            x = layer(x, media_ids if full else window_ids, cos, sin)
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(order.numel(), device=dev)
        return self.merge_patches(self.post_norm(x[inverse]), grid)


@stage("muse_glimmer_perception_norm")
class MuseGlimmerPerceptionNormStage(nn.Module):
    """Weightless RMS norm (fp32 statistics) of the projected media features."""

    def __init__(self, eps: float = 1e-5) -> None:
        super().__init__()
        self.eps = float(eps)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("eps", 1e-5)))

    def forward(self, features: Tensor) -> Tensor:
        return KB.rms_norm(features, None, self.eps)


@stage("muse_glimmer_media_scatter")
class MuseGlimmerMediaScatterStage(nn.Module):
    """Writes media feature rows, in order, into the embedding rows whose token id is the media
    placeholder. The count check is one host read of a device scalar."""

    def __init__(self, token_id: int) -> None:
        super().__init__()
        self.token_id = int(token_id)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["token_id"]))

    def forward(self, embeddings: Tensor, token_ids: Tensor, features: Tensor) -> Tensor:
        if (embeddings.ndim != 3 or token_ids.shape != embeddings.shape[:2] or features.ndim != 2
                or features.shape[1] != embeddings.shape[-1]):
            raise ValueError("Muse Glimmer media scatter geometry mismatch")
        mask = (token_ids == self.token_id).reshape(-1)
        if int(mask.sum()) != features.shape[0]:
            raise ValueError("Muse Glimmer media placeholders and features do not match")
        if features.shape[0] == 0:
            return embeddings.clone()
        slot = (mask.long().cumsum(0) - 1).clamp(min=0)     # feature row for each placeholder position
        flat = embeddings.reshape(-1, embeddings.shape[-1])
        picked = features.to(device=flat.device, dtype=flat.dtype)[slot]
        return torch.where(mask.unsqueeze(-1), picked, flat).view_as(embeddings)
