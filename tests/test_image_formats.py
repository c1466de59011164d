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
