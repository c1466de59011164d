"""BMP and GIF readers (``csrc/server/image_misc.cpp``) against Pillow."""
import io

import numpy as np
import pytest

from agens_engine_b200.serve import vision as V

PIL = pytest.importorskip("PIL.Image")


def _img(h, w, seed=0):
    rng = np.random.default_rng(seed)
    y, x = np.mgrid[0:h, 0:w]
    a = np.stack([(x * 255 // max(w - 1, 1)), (y * 255 // max(h - 1, 1)), ((x + y) % 256)], -1).astype(np.uint8)
    a[h // 4: h // 2, w // 3: w // 2] = rng.integers(0, 256, 3)
    return a


def _save(arr, fmt, mode="RGB", **kw):
    buf = io.BytesIO()
    im = PIL.fromarray(arr)
    if mode != "RGB":
        im = im.convert(mode) if mode != "P" else im.quantize(64)
    im.save(buf, fmt, **kw)
    return buf.getvalue()


def _pil(data):
    im = PIL.open(io.BytesIO(data))
    im.seek(0)
    return np.asarray(im.convert("RGB"))


@pytest.mark.parametrize("h,w", [(5, 7), (32, 33), (1, 1)])
@pytest.mark.parametrize("mode", ["RGB", "P", "RGBA"])
def test_bmp(h, w, mode):
    data = _save(_img(h, w, h * w), "BMP", mode)
    assert np.array_equal(V.decode_image(data), _pil(data))


@pytest.mark.parametrize("h,w", [(9, 13), (64, 40), (1, 3), (200, 150)])
@pytest.mark.parametrize("interlace", [False, True])
def test_gif_first_frame(h, w, interlace):
    data = _save(_img(h, w, h + w), "GIF", "P", interlace=interlace)
    assert np.array_equal(V.decode_image(data), _pil(data))


def test_gif_noise_exercises_table_resets():
    rng = np.random.default_rng(4)
    arr = rng.integers(0, 256, (90, 120, 3), dtype=np.uint8)        # incompressible: the 4096-entry table fills and clears
    data = _save(arr, "GIF", "P")
    assert np.array_equal(V.decode_image(data), _pil(data))


def test_bad_files_are_refused():
    for bad in (b"BM" + b"\x00" * 20, b"GIF89a" + b"\x00" * 3, b"GIF89a\x02\x00\x02\x00\x00\x00\x00\x2c" + b"\x00" * 4):
        with pytest.raises(ValueError):
            V.decode_image(bad)


# ---- WebP, lossless (csrc/server/webp.cpp) -----------------------------------------------------------------------------
def _webp_ok():
    from PIL import features
    return features.check("webp")


def _webp(arr, mode="RGB", **kw):
    buf = io.BytesIO()
    PIL.fromarray(arr, mode).save(buf, "WEBP", lossless=True, **kw)
    return buf.getvalue()


@pytest.mark.skipif(not _webp_ok(), reason="Pillow without WebP support")
def test_webp_lossless_matches_the_source_pixels():
    """Lossless WebP files written by Pillow (libwebp) at several encoder efforts: noise (literals), gradients and a
    smooth random walk (predictor, cross-colour, subtract-green transforms), palettes of 2 / 5 / 40 colours (colour
    indexing with 8 / 2 / 1 pixels per byte), a tiled pattern (backward references, colour cache), one pixel."""
    rng = np.random.default_rng(0)
    yy, xx = np.mgrid[0:120, 0:200]
    pal = rng.integers(0, 256, (40, 3), dtype=np.uint8)
    walk = np.cumsum(rng.integers(-3, 4, (150, 210, 3)), axis=1)
    cases = {
        "noise": rng.integers(0, 256, (29, 37, 3), dtype=np.uint8),
        "gradient": np.stack([(xx * 255 // 199), (yy * 255 // 119), ((xx + yy) % 256)], -1).astype(np.uint8),
        "palette 2": pal[:2][rng.integers(0, 2, (17, 33))],
        "palette 5": pal[:5][rng.integers(0, 5, (48, 64))],
        "palette 40": pal[rng.integers(0, 40, (50, 50))],
        "tiled": np.tile(rng.integers(0, 256, (8, 8, 3), dtype=np.uint8), (12, 20, 1)),
        "walk": ((walk - walk.min()) * 255 // max(1, walk.max() - walk.min())).astype(np.uint8),
        "one pixel": np.array([[[10, 200, 30]]], dtype=np.uint8),
        "flat": np.full((40, 70, 3), 77, dtype=np.uint8),
        "mixed": _img(97, 131, seed=3),
    }
    for name, arr in cases.items():
        for q, method in ((0, 0), (75, 4), (100, 6)):
            data = _webp(arr, quality=q, method=method)
            got = V.decode_image(data)
            assert got.shape == arr.shape and np.array_equal(got, arr), (name, q)


@pytest.mark.skipif(not _webp_ok(), reason="Pillow without WebP support")
def test_webp_alpha_container_and_refusals():
    rng = np.random.default_rng(1)
    rgba = rng.integers(0, 256, (20, 30, 4), dtype=np.uint8)
    rgba[..., 3] = np.maximum(rgba[..., 3], 1)              # no fully transparent pixel (their colour may be rewritten)
    data = _webp(rgba, "RGBA", exact=True)
    assert np.array_equal(V.decode_image(data), rgba[..., :3])            # alpha is dropped
    # the same lossless payload inside the extended container
    vp8l = data[12:]
    x = b"VP8X" + (10).to_bytes(4, "little") + bytes([0x10, 0, 0, 0]) + (29).to_bytes(3, "little") + (19).to_bytes(3, "little")
    body = b"WEBP" + x + vp8l
    ext = b"RIFF" + len(body).to_bytes(4, "little") + body
    assert np.array_equal(V.decode_image(ext), rgba[..., :3])
    # lossy WebP: recognised, refused with a message
    buf = io.BytesIO()
    PIL.fromarray(rgba[..., :3].copy()).save(buf, "WEBP", quality=80)
    with pytest.raises(ValueError, match="lossy"):
        V.decode_image(buf.getvalue())
    # damaged files fail cleanly
    for cut in (len(data) // 2, 24, 13):
        with pytest.raises(ValueError):
            V.decode_image(data[:cut])
    broken = bytearray(data); broken[12 + 8] = 0x00            # the lossless signature byte
    with pytest.raises(ValueError):
        V.decode_image(bytes(broken))
