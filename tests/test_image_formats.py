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


# ---- PNG (chunks and zlib in Python, scanlines in csrc/server/image_misc.cpp) -----------------------------------------------
def _png(arr, mode, **kw):
    buf = io.BytesIO()
    PIL.fromarray(arr, mode).save(buf, "PNG", **kw)
    return buf.getvalue()


def test_png_colour_types_and_bit_depths_match_pillow():
    rng = np.random.default_rng(2)
    rgb = _img(53, 71, seed=5)
    rgba = np.concatenate([rgb, rng.integers(0, 256, (53, 71, 1), dtype=np.uint8)], -1)
    grey = rgb[..., 0].copy()
    la = np.stack([grey, rgba[..., 3]], -1)
    for name, data in {"rgb": _png(rgb, "RGB"), "rgba": _png(rgba, "RGBA"), "grey": _png(grey, "L"), "grey+alpha": _png(la, "LA"),
                       "rgb optimised": _png(rgb, "RGB", optimize=True)}.items():
        assert np.array_equal(V.decode_image(data), _pil(data)), name
    # palette images at 8, 4, 2 and 1 bits per pixel
    for colours, bits in ((200, 8), (16, 4), (4, 2), (2, 1)):
        pal = rng.integers(0, 256, (colours, 3), dtype=np.uint8)
        idx = rng.integers(0, colours, (37, 45), dtype=np.uint8)
        im = PIL.fromarray(idx, "P")
        im.putpalette(pal.reshape(-1).tolist())
        buf = io.BytesIO()
        im.save(buf, "PNG", bits=bits)
        assert np.array_equal(V.decode_image(buf.getvalue()), pal[idx]), bits
    # bilevel and 16-bit grey (the high byte is kept)
    one = rng.integers(0, 2, (19, 27)).astype(np.uint8) * 255
    buf = io.BytesIO()
    PIL.fromarray(one, "L").convert("1", dither=0).save(buf, "PNG")
    assert np.array_equal(V.decode_image(buf.getvalue())[..., 0], one) and np.array_equal(V.decode_image(buf.getvalue()), _pil(buf.getvalue()))
    g16 = rng.integers(0, 65536, (21, 33)).astype(np.uint16)
    buf = io.BytesIO()
    PIL.fromarray(g16).save(buf, "PNG")
    assert np.array_equal(V.decode_image(buf.getvalue())[..., 1], (g16 >> 8).astype(np.uint8))


def test_png_adam7_interlaced_and_every_filter():
    """Interlaced files (Pillow does not write them): built here pass by pass, each scanline with one of the five filter
    types, for RGB, RGBA, 16-bit RGB and a 2-bit palette."""
    import struct
    import zlib
    rng = np.random.default_rng(3)

    def chunk(kind, body):
        return struct.pack(">I", len(body)) + kind + body + struct.pack(">I", zlib.crc32(kind + body))

    def filtered(rows, bpp):            # rows: list of bytes objects; cycles through filter types 0..4
        out, prev = b"", bytes(len(rows[0])) if rows else b""
        for j, row in enumerate(rows):
            f = j % 5
            enc = bytearray(len(row))
            for i, v in enumerate(row):
                a = row[i - bpp] if i >= bpp else 0
                b = prev[i]
                c = prev[i - bpp] if i >= bpp else 0
                if f == 0: pr = 0
                elif f == 1: pr = a
                elif f == 2: pr = b
                elif f == 3: pr = (a + b) >> 1
                else:
                    pa, pb, pc = abs(b - c), abs(a - c), abs(a + b - 2 * c)
                    pr = a if pa <= pb and pa <= pc else (b if pb <= pc else c)
                enc[i] = (v - pr) & 255
            out += bytes([f]) + bytes(enc)
            prev = row
        return out

    def pack_rows(px, depth):           # px: [h, w, ch] integer samples -> list of scanline bytes
        rows = []
        for r in px:
            flat = r.reshape(-1)
            if depth == 8:
                rows.append(bytes(flat.astype(np.uint8)))
            elif depth == 16:
                rows.append(flat.astype(">u2").tobytes())
            else:
                bits = "".join(format(int(v), f"0{depth}b") for v in flat)
                bits += "0" * (-len(bits) % 8)
                rows.append(bytes(int(bits[i:i + 8], 2) for i in range(0, len(bits), 8)))
        return rows

    passes = [(0, 0, 8, 8), (4, 0, 8, 8), (0, 4, 4, 8), (2, 0, 4, 4), (0, 2, 2, 4), (1, 0, 2, 2), (0, 1, 1, 2)]
    for w, h in ((23, 17), (3, 2), (8, 8), (1, 1)):
        for ctype, depth, ch in ((2, 8, 3), (6, 8, 4), (2, 16, 3), (3, 2, 1)):
            hi = 4 if ctype == 3 else (65536 if depth == 16 else 256)
            px = rng.integers(0, hi, (h, w, ch))
            raw = b""
            for x0, y0, dx, dy in passes:
                sub = px[y0::dy, x0::dx]
                if sub.size:
                    raw += filtered(pack_rows(sub, depth), max(1, ch * depth // 8))
            pal = rng.integers(0, 256, (4, 3), dtype=np.uint8)
            data = b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, depth, ctype, 0, 0, 1))
            if ctype == 3:
                data += chunk(b"PLTE", pal.tobytes())
            data += chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b"")
            got = V.decode_image(data)
            if ctype == 3:
                want = pal[px[..., 0]]
            elif depth == 16:
                want = (px[..., :3] >> 8).astype(np.uint8)
            else:
                want = px[..., :3].astype(np.uint8)
            assert np.array_equal(got, want), (w, h, ctype, depth)
            assert np.array_equal(got, _pil(data)) or depth == 16          # Pillow reads it the same way (16-bit RGB aside)
    with pytest.raises(ValueError):
        V.decode_image(b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", 4, 4, 8, 2, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(b"\0" * 10)) + chunk(b"IEND", b""))


def test_oversized_and_expanding_images_are_refused():
    """Headers that claim more pixels than a request may make the host decode are refused before any buffer is made,
    and a PNG's compressed stream is inflated only as far as its scanlines can hold."""
    import struct
    import zlib
    from agens_engine_b200.serve import vision as V

    def chunk(kind, body):
        return struct.pack(">I", len(body)) + kind + body + struct.pack(">I", zlib.crc32(kind + body))
    bomb = zlib.compress(b"\0" * (64 << 20), 9)                  # 64 MiB of zeros in about 64 KiB
    png = b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", 4, 4, 8, 2, 0, 0, 0)) + chunk(b"IDAT", bomb) + chunk(b"IEND", b"")
    img = V.decode_image(png)                                    # only the first rows are inflated; the rest is ignored
    assert img.shape == (4, 4, 3) and not img.any()
    huge = b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", 60000, 60000, 8, 2, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(b"\0")) + chunk(b"IEND", b"")
    with pytest.raises(ValueError, match="too large"):
        V.decode_image(huge)
    gif = b"GIF89a" + struct.pack("<HH", 16000, 16000) + b"\x00\x00\x00" + b"\x3b"
    with pytest.raises(ValueError, match="too large"):
        V.decode_image(gif)
    bmp = b"BM" + struct.pack("<IHHI", 54, 0, 0, 54) + struct.pack("<IiiHHIIiiII", 40, 30000, 30000, 1, 24, 0, 0, 0, 0, 0, 0)
    with pytest.raises(ValueError):
        V.decode_image(bmp)
