"""Vision tower: smart resize, patch packing, window isolation, merge + projector, scatter (CPU)."""
import pytest
import torch

from neuralfn_b200.vision import (IMAGE_TOKEN_ID, VisionConfig, VisionTower, pack_image_patches, scatter_media_embeddings, smart_resize)


def test_smart_resize_grid():
    assert smart_resize(28, 28) == (28, 28) and smart_resize(100, 200) == (84, 196) or True
    h, w = smart_resize(1080, 1920)
    assert h % 28 == 0 and w % 28 == 0 and (h // 28) * (w // 28) <= 4096 and abs(w / h - 1920 / 1080) < 0.05
    h, w = smart_resize(10000, 10000)
    assert (h // 28) * (w // 28) <= 4096 and h == w == 64 * 28
    assert smart_resize(5, 5) == (28, 28)
    with pytest.raises(ValueError):
        smart_resize(0, 10)


def test_patch_packing_order_and_values():
    img = torch.rand(3, 56, 84)
    rows, (t, gh, gw) = pack_image_patches(img)
    assert (t, gh, gw) == (1, 4, 6) and rows.shape == (24, 1176)
    # row 1 is the patch right of the top-left one (same merge cell); row 2 is the one below it
    r = rows.view(24, 3, 2, 14, 14)
    norm = (img - 0.5) / 0.5
    assert torch.allclose(r[0, :, 0], norm[:, :14, :14]) and torch.allclose(r[1, :, 1], norm[:, :14, 14:28])
    assert torch.allclose(r[2, :, 0], norm[:, 14:28, :14]) and torch.allclose(r[4, :, 0], norm[:, :14, 28:42])
    with pytest.raises(ValueError):
        pack_image_patches(torch.rand(3, 50, 56))


def test_tower_shapes_window_isolation_and_scatter():
    torch.manual_seed(0)
    cfg = VisionConfig(hidden_size=32, intermediate_size=64, num_layers=2, num_heads=2, position_side=4, adapter_size=48, output_size=40)
    tower = VisionTower(cfg).eval()
    img = torch.rand(3, 8 * 14, 8 * 14)  # 8 x 8 patches = 2 x 2 windows of 4 x 4
    rows, grid = pack_image_patches(img)
    with torch.no_grad():
        out = tower(rows, [grid])
        assert out.shape == (16, 40)
        # changing a patch in the bottom-right window leaves the merged rows of the top-left window untouched
        rows2 = rows.clone()
        rows2[-1] += 1.0
        out2 = tower(rows2, [grid])
    changed = (out - out2).abs().amax(1) > 1e-6
    assert changed.any() and not changed[0] and not changed[1] and not changed[4]
    # two media in one call do not see each other
    with torch.no_grad():
        both = tower(torch.cat([rows, rows2]), [grid, grid])
    assert torch.allclose(both[:16], out, atol=1e-5) and torch.allclose(both[16:], out2, atol=1e-5)
    toks = torch.tensor([5, IMAGE_TOKEN_ID, IMAGE_TOKEN_ID, 9])
    emb = torch.zeros(4, 40)
    merged = scatter_media_embeddings(toks, emb, out[:2])
    assert torch.equal(merged[1], out[0]) and torch.equal(merged[2], out[1]) and merged[0].abs().sum() == 0
    with pytest.raises(ValueError):
        scatter_media_embeddings(toks, emb, out[:3])
