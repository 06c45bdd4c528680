"""Image preprocessing: decode with alpha on white, smart resize bounds, canvas variant, patch layout."""
import io

import numpy as np
import pytest
import torch

from volta_engine_b200.loader.image import VisionParams, canvas_size, decode_image, prepare_image, smart_resize


def _png(arr, mode):
    from PIL import Image
    b = io.BytesIO()
    Image.fromarray(arr, mode).save(b, format="PNG")
    return b.getvalue()


def test_decode_composites_alpha_on_white():
    rgba = np.zeros((4, 4, 4), dtype=np.uint8)
    rgba[..., 0] = 200
    rgba[:2, :, 3] = 255            # top half opaque red-ish, bottom half transparent
    out = decode_image(_png(rgba, "RGBA"))
    assert out.shape == (4, 4, 3)
    assert tuple(out[0, 0]) == (200, 0, 0) and tuple(out[3, 3]) == (255, 255, 255)
    rgb = np.random.default_rng(0).integers(0, 255, (5, 7, 3), dtype=np.uint8)
    assert np.array_equal(decode_image(_png(rgb, "RGB")), rgb)


def test_smart_resize_rules():
    f = 32
    for (h, w) in [(480, 640), (1080, 1920), (3000, 4000), (20, 30), (33, 1000)]:
        oh, ow = smart_resize(h, w, f, 65536, 1048576)
        assert oh % f == 0 and ow % f == 0 and 65536 <= oh * ow <= 1048576
        if min(h, w) >= 2 * f:
            assert abs(oh / ow - h / w) / (h / w) < 0.25
    assert smart_resize(480, 640, 32, 65536, 1048576) == (480, 640)
    assert smart_resize(1080, 1920, 32, 65536, 1048576) == (768, 1344)
    with pytest.raises(ValueError):
        smart_resize(10, 3000, 32, 65536, 1048576)


def test_canvas_keeps_aspect_and_budget():
    ch, cw, ih, iw = canvas_size(1080, 1920, 32, 65536, 1048576)
    assert ch % 32 == 0 and cw % 32 == 0 and ch * cw <= 1048576 and ih <= ch and iw <= cw
    assert abs(ih / iw - 1080 / 1920) < 0.01


def test_patch_layout_matches_block_order():
    p = VisionParams(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=64, max_pixels=4096)
    # a 16x16 image whose red channel encodes the pixel index; mean 0 / std 1 keeps values readable
    p.mean, p.std = (0.0, 0.0, 0.0), (1.0, 1.0, 1.0)
    rgb = np.zeros((16, 16, 3), dtype=np.uint8)
    rgb[..., 0] = np.arange(256, dtype=np.uint8).reshape(16, 16)
    pre = prepare_image(rgb, p)
    assert (pre.grid_h, pre.grid_w) == (4, 4) and pre.patches.shape == (16, 3 * 2 * 16) and pre.tokens(2) == 4
    img = torch.from_numpy(rgb[..., 0].astype(np.float32) / 255.0)
    # merge-block order: patches (0,0) (0,1) (1,0) (1,1) of block (0,0), then block (0,1) ...
    order = [(0, 0), (0, 1), (1, 0), (1, 1), (0, 2), (0, 3), (1, 2), (1, 3)]
    for i, (py, px) in enumerate(order):
        want = img[py * 4:(py + 1) * 4, px * 4:(px + 1) * 4].reshape(-1)
        got = pre.patches[i].reshape(3, 2, 16)
        assert torch.allclose(got[0, 0], want, atol=1e-6) and torch.allclose(got[0, 1], want, atol=1e-6)
        assert float(got[1].abs().sum()) == 0.0
    assert prepare_image(rgb, p).hash == pre.hash
    pc = VisionParams(patch_size=4, merge_size=2, min_pixels=64, max_pixels=4096, canvas=True)
    prec = prepare_image(np.full((10, 30, 3), 255, dtype=np.uint8), pc)
    assert prec.grid_h * 4 >= 10 and prec.grid_w * 4 >= 30 and prec.grid_h % 2 == 0 and prec.grid_w % 2 == 0
