"""The host JPEG decoder (``csrc/server/jpeg.cpp``) against Pillow's decoder on synthetic images: grey, 4:4:4, 4:2:2,
4:2:0, odd sizes, restart intervals, an Adobe RGB file, progressive files."""
import io

import numpy as np
import pytest

from agens_engine_b200.serve import vision as V

PIL = pytest.importorskip("PIL.Image")


def _image(h, w, seed=0):
    """Smooth gradients + a few hard edges + mild noise: exercises DC prediction, AC runs and chroma edges."""
    rng = np.random.default_rng(seed)
    y, x = np.mgrid[0:h, 0:w].astype(np.float32)
    img = np.stack([127 + 120 * np.sin(x / 9.0 + y / 23.0), 127 + 120 * np.cos(y / 7.0), 255 * (x / max(w - 1, 1))], -1)
    img[h // 3: h // 2, w // 4: w // 2] = (250, 20, 30)
    img[h // 2:, : w // 5] = (10, 240, 200)
    img += rng.normal(0, 3, img.shape)
    return np.clip(img, 0, 255).astype(np.uint8)


def _encode(arr, mode="RGB", **kw):
    buf = io.BytesIO()
    PIL.fromarray(arr if mode == "RGB" else arr[..., 0], mode).save(buf, "JPEG", **kw)
    return buf.getvalue()


def _pil(data):
    return np.asarray(PIL.open(io.BytesIO(data)).convert("RGB"))


@pytest.mark.parametrize("h,w", [(64, 64), (37, 53), (8, 8), (1, 1), (200, 17)])
@pytest.mark.parametrize("sub", [0, 1, 2])          # 4:4:4, 4:2:2, 4:2:0
def test_colour_matches_pillow(h, w, sub):
    data = _encode(_image(h, w, seed=h + w), quality=92, subsampling=sub)
    ours, ref = V.decode_image(data), _pil(data)
    assert ours.shape == ref.shape == (h, w, 3)
    diff = np.abs(ours.astype(np.int32) - ref.astype(np.int32))
    assert diff.mean() < 1.0 and diff.max() <= 12, (diff.mean(), diff.max())


def test_grey_and_low_quality():
    for q in (95, 30):
        data = _encode(_image(50, 70, seed=q), mode="L", quality=q)
        ours, ref = V.decode_image(data), _pil(data)
        diff = np.abs(ours.astype(np.int32) - ref.astype(np.int32))
        assert diff.max() <= 2, diff.max()


def test_restart_intervals():
    img = _image(96, 80, seed=3)
    try:
        data = _encode(img, quality=90, subsampling=2, restart_marker_blocks=3)
    except TypeError:
        pytest.skip("this Pillow cannot write restart markers")
    if b"\xff\xdd" not in data:
        pytest.skip("this Pillow ignored restart_marker_blocks")
    ours, ref = V.decode_image(data), _pil(data)
    diff = np.abs(ours.astype(np.int32) - ref.astype(np.int32))
    assert diff.mean() < 1.0 and diff.max() <= 12


@pytest.mark.parametrize("h,w", [(64, 64), (37, 53), (8, 8), (1, 1), (200, 17), (131, 97)])
@pytest.mark.parametrize("sub", [0, 1, 2])
def test_progressive_matches_pillow(h, w, sub):
    """Progressive files (DC and AC scans, first passes and refinements, one component per AC scan) decode to what
    Pillow's decoder gives for the same file, as closely as the sequential files do."""
    for q in (92, 40):
        data = _encode(_image(h, w, seed=h * 3 + w), quality=q, subsampling=sub, progressive=True)
        assert b"\xff\xc2" in data                                    # a progressive frame header
        ours, ref = V.decode_image(data), _pil(data)
        assert ours.shape == ref.shape == (h, w, 3)
        diff = np.abs(ours.astype(np.int32) - ref.astype(np.int32))
        assert diff.mean() < 1.0 and diff.max() <= 12, (q, diff.mean(), diff.max())


def test_progressive_grey_restarts_and_truncation():
    data = _encode(_image(50, 70, seed=1), mode="L", quality=85, progressive=True)
    diff = np.abs(V.decode_image(data).astype(np.int32) - _pil(data).astype(np.int32))
    assert diff.max() <= 2, diff.max()
    img = _image(96, 80, seed=3)
    try:
        data = _encode(img, quality=90, subsampling=2, progressive=True, restart_marker_blocks=2)
    except TypeError:
        data = None
    if data is not None and b"\xff\xdd" in data:
        diff = np.abs(V.decode_image(data).astype(np.int32) - _pil(data).astype(np.int32))
        assert diff.mean() < 1.0 and diff.max() <= 12
    # a progressive file cut after its first scans still gives an image (coarser), never a crash
    data = _encode(_image(64, 64, seed=2), quality=90, progressive=True)
    cut = data[: len(data) * 2 // 3]
    try:
        out = V.decode_image(cut)
        assert out.shape == (64, 64, 3)
    except ValueError:
        pass


def test_truncated_and_garbage_inputs_fail_cleanly():
    data = _encode(_image(40, 40), quality=90)
    for bad in (data[:20], data[: len(data) // 2][:-1] + b"\xff", b"\xff\xd8\xff\xe0\x00\x02" + b"\x00" * 50, b"\xff\xd8"):
        try:
            out = V.decode_image(bad)
        except ValueError:
            continue
        assert out.shape[2] == 3            # a truncated scan may still decode (missing data reads as zeros)


def test_cmyk_files_match_pillow():
    """Four-component Adobe files (inverted ink values): converted to RGB as common viewers do; sequential and
    progressive."""
    img = PIL.fromarray(_image(60, 90, seed=9)).convert("CMYK")
    for kw in ({}, {"progressive": True}):
        buf = io.BytesIO()
        img.save(buf, "JPEG", quality=92, **kw)
        data = buf.getvalue()
        ours, ref = V.decode_image(data), _pil(data)
        diff = np.abs(ours.astype(np.int32) - ref.astype(np.int32))
        assert ours.shape == (60, 90, 3) and diff.mean() < 1.0 and diff.max() <= 12, (kw, diff.mean(), diff.max())
