"""Damaged image files through the host decoders: every input either decodes or is refused with a ValueError.  The
mutations are seeded, so a failure names a reproducible input.  (The same corpus is what the decoders are run against
under AddressSanitizer / UBSan during development.)"""
import io
import random

import numpy as np
import pytest

from agens_engine_b200.serve import vision as V

Image = pytest.importorskip("PIL.Image")


def _seeds():
    rng = np.random.default_rng(5)
    y, x = np.mgrid[0:36, 0:44]
    a = (np.stack([(x * 7 + y * 3) % 256, (x * 2 + y * 5) % 256, (x + y) % 256], -1) // 2 + rng.integers(0, 128, (36, 44, 3))).astype(np.uint8)
    im = Image.fromarray(a)
    out = []

    def add(fmt, img=im, **kw):
        b = io.BytesIO()
        img.save(b, fmt, **kw)
        out.append((fmt, b.getvalue()))
    add("JPEG", quality=80)
    add("JPEG", progressive=True, quality=70, subsampling=2)
    add("JPEG", img=im.convert("L"))
    add("JPEG", img=im.convert("CMYK"))
    add("PNG")
    add("PNG", img=im.quantize(16))
    add("PNG", img=im.convert("LA"))
    add("GIF", img=im.quantize(64))
    add("GIF", img=im.quantize(256), interlace=True)
    add("BMP")
    add("BMP", img=im.quantize(16))
    add("WEBP", lossless=True)
    add("WEBP", img=im.quantize(8).convert("RGB"), lossless=True)
    return out


def _try(data: bytes):
    try:
        img = V.decode_image(data)
    except ValueError:
        return None
    assert img.dtype == np.uint8 and img.ndim == 3 and img.shape[2] == 3
    return img


def test_every_prefix_of_a_file_decodes_or_is_refused():
    for fmt, data in _seeds():
        assert _try(data) is not None, fmt
        step = max(1, len(data) // 400)
        for n in list(range(0, min(len(data), 64))) + list(range(64, len(data), step)):
            _try(data[:n])


def test_mutated_files_decode_or_are_refused():
    rng = random.Random(11)
    seeds = _seeds()
    decoded = 0
    for _ in range(3000):
        fmt, data = rng.choice(seeds)
        b = bytearray(data)
        for _ in range(rng.randint(1, 4)):
            i, r = rng.randrange(len(b)), rng.random()
            if r < 0.35:
                b[i] = rng.randrange(256)
            elif r < 0.6:
                b[i] ^= 1 << rng.randrange(8)
            elif r < 0.75:
                b[i:i + rng.randint(1, 12)] = bytes(rng.choice((0, 255)) for _ in range(rng.randint(1, 12)))
            elif r < 0.9:
                j = rng.randrange(len(b))
                b[i:i + 16] = b[j:j + 16]
            else:
                del b[i:i + rng.randint(1, 24)]
            if not b:
                break
        decoded += _try(bytes(b)) is not None
    assert decoded > 300                                     # many damaged files still decode (to something)
