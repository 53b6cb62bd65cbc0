"""Vision tower for image / video prompts: smart resize, patch packing, a windowed ViT, 2x2 patch
merging and the projector into the text model's width, plus the scatter of the resulting rows
into a prompt's embedding sequence at the image / video placeholder tokens.

Pipeline for one image of H x W pixels:
  1. ``smart_resize``: pick a grid of (patch * merge)-sized cells whose aspect ratio is closest
     to the image's while staying under ``max_tokens`` merged cells;
  2. normalise to [-1, 1] (mean 0.5, std 0.5), split into 14 x 14 patches, duplicate the frame to
     fill the temporal patch of 2 -> rows of 3 * 2 * 14 * 14 = 1176 values, ordered so that the
     four patches of every 2 x 2 merge cell are adjacent;
  3. tower: linear patch embedding + learned position table (a side x side grid, bilinearly
     indexed by patch position), ``num_layers`` pre-LayerNorm blocks with 2-D rotary attention
     restricted to windows of ``position_side`` x ``position_side`` patches, GELU MLP;
  4. merge each 2 x 2 cell (concatenate 4 x hidden), adapter MLP, project to ``output_size``.

This module is the tensor-runtime implementation (PyTorch ops; attention through SDPA with a
block mask). Reference counterparts: ``neuralfn/native_glimmer_media.py`` (smart resize
:121-164, packing), ``csrc/native_gpt2/resident_glimmer_vision.{h,cpp}`` (tower geometry: hidden
1536, 50 layers, 16 heads, patch width 1176, merge 2, position side 32, adapter 4096, output
6656), and the scatter at token ids 200092 (image) / 200091 (video).
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["PATCH_SIZE", "TEMPORAL_PATCH_SIZE", "MERGE_SIZE", "MAX_IMAGE_TOKENS", "IMAGE_TOKEN_ID", "VIDEO_TOKEN_ID", "VisionConfig",
           "smart_resize", "pack_image_patches", "VisionTower", "scatter_media_embeddings"]

PATCH_SIZE, TEMPORAL_PATCH_SIZE, MERGE_SIZE, MAX_IMAGE_TOKENS = 14, 2, 2, 4096
IMAGE_TOKEN_ID, VIDEO_TOKEN_ID = 200092, 200091


@dataclass(frozen=True)
class VisionConfig:
    hidden_size: int = 1536
    intermediate_size: int = 8960
    num_layers: int = 50
    num_heads: int = 16
    patch_width: int = 3 * TEMPORAL_PATCH_SIZE * PATCH_SIZE * PATCH_SIZE
    merge_size: int = MERGE_SIZE
    position_side: int = 32
    adapter_size: int = 4096
    output_size: int = 6656
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5


def smart_resize(height: int, width: int, *, patch_size: int = PATCH_SIZE * MERGE_SIZE, max_tokens: int = MAX_IMAGE_TOKENS) -> tuple[int, int]:
    """Target (height, width) in pixels: a whole number of merge cells, at most ``max_tokens`` of
    them, aspect ratio as close to the source's as the integer grid allows."""
    for v in (height, width, patch_size, max_tokens):
        if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
            raise ValueError("height, width, patch_size and max_tokens must be positive integers")
    ih, iw = height / patch_size, width / patch_size
    ratio = iw / ih
    if ih * iw > max_tokens:
        ih = math.sqrt(max_tokens / ratio)
        iw = ih * ratio
    cands = set(itertools.product((math.floor(ih), math.ceil(ih)), (math.floor(iw), math.ceil(iw))))
    valid = [(gh, gw) for gh, gw in cands if gh >= 1 and gw >= 1 and gh * gw <= max_tokens]
    if not valid:
        valid = [(max(1, round(ih)), max(1, round(iw)))]
    gh, gw = min(valid, key=lambda g: abs(g[0] / g[1] - height / width))
    return gh * patch_size, gw * patch_size


def pack_image_patches(image: torch.Tensor) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """image: float [3, H, W] in [0, 1], H and W multiples of patch * merge. Returns (rows
    [h * w, 1176] in merge-cell-major order, (t, h, w) grid in patches)."""
    C, H, W = image.shape
    cell = PATCH_SIZE * MERGE_SIZE
    if C != 3 or H % cell or W % cell:
        raise ValueError("image must be [3, H, W] with H and W multiples of patch * merge")
    x = (image.float() - 0.5) / 0.5
    gh, gw = H // PATCH_SIZE, W // PATCH_SIZE
    x = x.unsqueeze(1).expand(3, TEMPORAL_PATCH_SIZE, H, W)  # a still image fills both temporal slots
    # [3, t, gh/m, m, p, gw/m, m, p] -> [gh/m, gw/m, m, m, 3, t, p, p]
    x = x.reshape(3, TEMPORAL_PATCH_SIZE, gh // MERGE_SIZE, MERGE_SIZE, PATCH_SIZE, gw // MERGE_SIZE, MERGE_SIZE, PATCH_SIZE)
    x = x.permute(2, 5, 3, 6, 0, 1, 4, 7).reshape(gh * gw, 3 * TEMPORAL_PATCH_SIZE * PATCH_SIZE * PATCH_SIZE)
    return x.contiguous(), (1, gh, gw)


def _patch_positions(gh: int, gw: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(row, column) of every packed patch, in the merge-cell-major order of ``pack_image_patches``."""
    hh = torch.arange(gh).view(gh // MERGE_SIZE, 1, MERGE_SIZE, 1).expand(gh // MERGE_SIZE, gw // MERGE_SIZE, MERGE_SIZE, MERGE_SIZE)
    ww = torch.arange(gw).view(1, gw // MERGE_SIZE, 1, MERGE_SIZE).expand(gh // MERGE_SIZE, gw // MERGE_SIZE, MERGE_SIZE, MERGE_SIZE)
    return hh.reshape(-1), ww.reshape(-1)


class _Block(nn.Module):
    def __init__(self, c: VisionConfig) -> None:
        super().__init__()
        self.norm1 = nn.LayerNorm(c.hidden_size, eps=c.norm_eps)
        self.qkv = nn.Linear(c.hidden_size, 3 * c.hidden_size)
        self.proj = nn.Linear(c.hidden_size, c.hidden_size)
        self.norm2 = nn.LayerNorm(c.hidden_size, eps=c.norm_eps)
        self.fc1 = nn.Linear(c.hidden_size, c.intermediate_size)
        self.fc2 = nn.Linear(c.intermediate_size, c.hidden_size)
        self.heads = c.num_heads

    def forward(self, x, cos, sin, mask):
        n, d = x.shape
        hd = d // self.heads
        q, k, v = self.qkv(self.norm1(x)).view(n, 3, self.heads, hd).unbind(1)

        def rot(t):
            a, b = t[..., :hd // 2], t[..., hd // 2:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

        q, k = rot(q), rot(k)
        att = F.scaled_dot_product_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), attn_mask=mask)
        x = x + self.proj(att.transpose(0, 1).reshape(n, d))
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class VisionTower(nn.Module):
    def __init__(self, config: VisionConfig = VisionConfig()) -> None:
        super().__init__()
        c = self.config = config
        if c.hidden_size % c.num_heads or (c.hidden_size // c.num_heads) % 4:
            raise ValueError("head_dim must be a multiple of 4 (two rotary axes)")
        self.patch_embed = nn.Linear(c.patch_width, c.hidden_size, bias=False)
        self.position_embed = nn.Parameter(torch.zeros(c.position_side * c.position_side, c.hidden_size))
        self.blocks = nn.ModuleList(_Block(c) for _ in range(c.num_layers))
        self.final_norm = nn.LayerNorm(c.hidden_size, eps=c.norm_eps)
        m = c.merge_size * c.merge_size * c.hidden_size
        self.adapter = nn.Sequential(nn.Linear(m, c.adapter_size), nn.GELU(), nn.Linear(c.adapter_size, c.output_size))
        nn.init.normal_(self.position_embed, std=0.02)

    def _rotary(self, hh, ww, device, dtype):
        hd = self.config.hidden_size // self.config.num_heads
        quarter = hd // 4
        inv = 1.0 / (self.config.rope_theta ** (torch.arange(quarter, device=device, dtype=torch.float32) / quarter))
        ang = torch.cat([hh[:, None].float() * inv, ww[:, None].float() * inv], -1)  # [n, hd / 2]: row axis then column axis
        return ang.cos()[:, None, :].to(dtype), ang.sin()[:, None, :].to(dtype)

    def _window_mask(self, hh, ww, media_id):
        side = self.config.position_side
        key = (media_id * 100003 + (hh // side)) * 100003 + (ww // side)
        return key[:, None] == key[None, :]

    def forward(self, packed_patches: torch.Tensor, grids: list[tuple[int, int, int]]) -> torch.Tensor:
        """packed_patches: [sum(t * h * w), patch_width]; grids: (t, h, w) per medium. Returns
        [sum(t * h * w) / merge^2, output_size]."""
        c = self.config
        dev = packed_patches.device
        hh, ww, mid = [], [], []
        for i, (t, gh, gw) in enumerate(grids):
            if gh % c.merge_size or gw % c.merge_size:
                raise ValueError("grid is not divisible by the merge size")
            a, b = _patch_positions(gh, gw)
            hh.append(a.repeat(t))
            ww.append(b.repeat(t))
            mid.append(torch.arange(t).repeat_interleave(gh * gw) + 1000 * i)
        hh, ww, mid = torch.cat(hh).to(dev), torch.cat(ww).to(dev), torch.cat(mid).to(dev)
        if hh.numel() != packed_patches.shape[0]:
            raise ValueError("grids do not match the number of packed patches")
        x = self.patch_embed(packed_patches.to(self.patch_embed.weight.dtype))
        side = c.position_side
        x = x + self.position_embed[(hh % side) * side + (ww % side)]
        cos, sin = self._rotary(hh, ww, dev, x.dtype)
        mask = self._window_mask(hh, ww, mid)
        for blk in self.blocks:
            x = blk(x, cos, sin, mask)
        x = self.final_norm(x)
        cell = c.merge_size * c.merge_size
        return self.adapter(x.view(-1, cell * c.hidden_size))


def scatter_media_embeddings(token_ids: torch.Tensor, text_embeddings: torch.Tensor, media_rows: torch.Tensor,
                             placeholder_ids: tuple[int, ...] = (IMAGE_TOKEN_ID, VIDEO_TOKEN_ID)) -> torch.Tensor:
    """Replaces the embeddings at placeholder tokens, in order, by the tower's output rows. The
    number of placeholders must equal the number of rows."""
    mask = torch.zeros_like(token_ids, dtype=torch.bool)
    for pid in placeholder_ids:
        mask |= token_ids == pid
    if int(mask.sum()) != media_rows.shape[0]:
        raise ValueError(f"{int(mask.sum())} placeholder tokens but {media_rows.shape[0]} media rows")
    out = text_embeddings.clone()
    out[mask] = media_rows.to(out.dtype)
    return out
