"""Image input, host side (bindings of ``csrc/server/vision.cpp``): smart_resize, antialiased bicubic resize +
normalisation + patch layout, placeholder expansion, multi-axis rotary positions, and a few pure-Python decoders for
the image containers a request may carry."""
from __future__ import annotations

import base64
import ctypes as C
import hashlib
import struct
import zlib
from typing import List, Sequence, Tuple

import numpy as np

from .. import _lib

PATCH = 16
MERGE = 2
FACTOR = PATCH * MERGE
MIN_PIXELS = 64 * 64
MAX_PIXELS = 4_194_304
MAX_DECODE_PIXELS = 1 << 26          # largest image a request may make the host decode (192 MiB of RGB)
MAX_IMAGES = 16
_sig = False


def _h():
    global _sig
    h = _lib.host_lib()
    if not _sig:
        i, ll, vp = C.c_int, C.c_longlong, C.c_void_p
        ip = C.POINTER(C.c_int)
        h.b2h_smart_resize.argtypes, h.b2h_smart_resize.restype = [i, i, i, ll, ll, ip, ip], i
        h.b2h_image_preprocess.argtypes, h.b2h_image_preprocess.restype = [vp, i, i, i, i, i, vp, vp], i
        h.b2h_ppm_header.argtypes, h.b2h_ppm_header.restype = [vp, C.c_long, ip, ip], i
        h.b2h_expand_placeholders.argtypes, h.b2h_expand_placeholders.restype = [ip, i, i, ip, i, ip, i], i
        h.b2h_mrope_positions.argtypes, h.b2h_mrope_positions.restype = [ip, i, i, ip, i, ip], i
        h.b2h_jpeg_info.argtypes, h.b2h_jpeg_info.restype = [vp, C.c_long, ip, ip, ip], i
        h.b2h_jpeg_decode.argtypes, h.b2h_jpeg_decode.restype = [vp, C.c_long, vp], i
        h.b2h_jpeg_error.argtypes, h.b2h_jpeg_error.restype = [], C.c_char_p
        for nm in ("b2h_bmp_info", "b2h_gif_info", "b2h_webp_info"):
            getattr(h, nm).argtypes, getattr(h, nm).restype = [vp, C.c_long, ip, ip], i
        for nm in ("b2h_bmp_decode", "b2h_gif_decode", "b2h_webp_decode"):
            getattr(h, nm).argtypes, getattr(h, nm).restype = [vp, C.c_long, vp], i
        h.b2h_image_error.argtypes, h.b2h_image_error.restype = [], C.c_char_p
        h.b2h_webp_error.argtypes, h.b2h_webp_error.restype = [], C.c_char_p
        h.b2h_png_unfilter.argtypes, h.b2h_png_unfilter.restype = [vp, C.c_long, i, i, i, i, i, vp, i, vp], i
        _sig = True
    return h


def smart_resize(h: int, w: int, factor: int = FACTOR, min_pixels: int = MIN_PIXELS, max_pixels: int = MAX_PIXELS) -> Tuple[int, int]:
    oh, ow = C.c_int(), C.c_int()
    if _h().b2h_smart_resize(h, w, factor, min_pixels, max_pixels, C.byref(oh), C.byref(ow)) != 0:
        raise ValueError("absolute aspect ratio must be smaller than 200")
    return oh.value, ow.value


def preprocess(rgb: np.ndarray, size: Tuple[int, int] = None, want_resized: bool = False):
    """rgb: uint8 [h, w, 3].  Returns (patches fp32 [gh*gw, 1536] in merge-block order, (gh, gw)[, resized fp32 [3, oh, ow]])."""
    rgb = np.ascontiguousarray(rgb, dtype=np.uint8)
    h, w, _ = rgb.shape
    oh, ow = size or smart_resize(h, w)
    gh, gw = oh // PATCH, ow // PATCH
    patches = np.empty((gh * gw, 3 * 2 * PATCH * PATCH), dtype=np.float32)
    resized = np.empty((3, oh, ow), dtype=np.float32) if want_resized else None
    rc = _h().b2h_image_preprocess(rgb.ctypes.data, h, w, oh, ow, PATCH, resized.ctypes.data if want_resized else None,
                                   patches.ctypes.data)
    if rc != 0:
        raise ValueError("bad image or target size")
    return (patches, (gh, gw), resized) if want_resized else (patches, (gh, gw))


def expand_placeholders(ids: Sequence[int], pad_id: int, counts: Sequence[int]) -> List[int]:
    cap = len(ids) + sum(counts)
    out = (C.c_int * cap)()
    n = _h().b2h_expand_placeholders((C.c_int * len(ids))(*ids), len(ids), pad_id, (C.c_int * max(len(counts), 1))(*counts),
                                     len(counts), out, cap)
    if n < 0:
        raise ValueError("number of image placeholders does not match the number of images")
    return list(out[:n])


def mrope_positions(ids: Sequence[int], pad_id: int, grids: Sequence[Tuple[int, int]]):
    """Returns (positions int32 [3, n], next running position); ``grids`` are the merged (gh/2, gw/2) sizes."""
    n = len(ids)
    pos = np.zeros((3, n), dtype=np.int32)
    flat = [v for g in grids for v in g]
    nxt = _h().b2h_mrope_positions((C.c_int * n)(*ids), n, pad_id, (C.c_int * max(len(flat), 1))(*flat), len(grids),
                                   pos.ctypes.data_as(C.POINTER(C.c_int)))
    if nxt < 0:
        raise ValueError("placeholder runs do not match the image grids")
    return pos, nxt


# ---------------------------------------------------------------------------------------------------------------------
def decode_image(data: bytes) -> np.ndarray:
    """uint8 [h, w, 3] from a binary PPM, a PNG (every colour type and bit depth, interlaced or not; alpha is
    dropped) or a JPEG (``csrc/server/jpeg.cpp``: sequential or progressive, grey or three components, 1x / 2x sampling
    factors, restart intervals; arithmetic-coded files are refused with a message), an uncompressed BMP or the first
    frame of a GIF (``csrc/server/image_misc.cpp``), or a lossless WebP (``csrc/server/webp.cpp``)."""
    if data[:2] == b"P6":
        h, w = C.c_int(), C.c_int()
        buf = (C.c_ubyte * len(data)).from_buffer_copy(data)
        off = _h().b2h_ppm_header(buf, len(data), C.byref(h), C.byref(w))
        if off < 0:
            raise ValueError("bad PPM")
        return np.frombuffer(data, dtype=np.uint8, count=h.value * w.value * 3, offset=off).reshape(h.value, w.value, 3).copy()
    if data[:8] == b"\x89PNG\r\n\x1a\n":
        return _decode_png(data)
    if data[:2] == b"\xff\xd8":
        return _decode_jpeg(data)
    if data[:2] == b"BM":
        return _decode_simple(data, "bmp")
    if data[:4] == b"GIF8":
        return _decode_simple(data, "gif")
    if data[:4] == b"RIFF" and data[8:12] == b"WEBP":
        return _decode_simple(data, "webp")
    raise ValueError("unknown image format")


def _decode_jpeg(data: bytes) -> np.ndarray:
    lib = _h()
    buf = (C.c_ubyte * len(data)).from_buffer_copy(data)
    h, w, nc = C.c_int(), C.c_int(), C.c_int()
    if lib.b2h_jpeg_info(buf, len(data), C.byref(h), C.byref(w), C.byref(nc)) != 0:
        raise ValueError(lib.b2h_jpeg_error().decode() or "bad JPEG")
    if h.value * w.value > MAX_DECODE_PIXELS:
        raise ValueError("jpeg: image too large")
    out = np.empty((h.value, w.value, 3), dtype=np.uint8)
    if lib.b2h_jpeg_decode(buf, len(data), out.ctypes.data_as(C.c_void_p)) != 0:
        raise ValueError(lib.b2h_jpeg_error().decode() or "bad JPEG")
    return out


def _decode_simple(data: bytes, kind: str) -> np.ndarray:
    """BMP (uncompressed 8 / 24 / 32-bit) and GIF (first frame) through ``csrc/server/image_misc.cpp``; lossless WebP
    through ``csrc/server/webp.cpp`` (lossy WebP is refused with a message)."""
    lib = _h()
    info, dec, err = {"bmp": (lib.b2h_bmp_info, lib.b2h_bmp_decode, lib.b2h_image_error),
                      "gif": (lib.b2h_gif_info, lib.b2h_gif_decode, lib.b2h_image_error),
                      "webp": (lib.b2h_webp_info, lib.b2h_webp_decode, lib.b2h_webp_error)}[kind]
    buf = (C.c_ubyte * len(data)).from_buffer_copy(data)
    h, w = C.c_int(), C.c_int()
    if info(buf, len(data), C.byref(h), C.byref(w)) != 0:
        raise ValueError(err().decode() or f"bad {kind}")
    if h.value * w.value > MAX_DECODE_PIXELS:
        raise ValueError(f"{kind}: image too large")
    out = np.empty((h.value, w.value, 3), dtype=np.uint8)
    if dec(buf, len(data), out.ctypes.data_as(C.c_void_p)) != 0:
        raise ValueError(err().decode() or f"bad {kind}")
    return out


def _decode_png(data: bytes) -> np.ndarray:
    """PNG: the chunks are read and the IDAT stream inflated here (zlib), the scanlines are reconstructed by
    ``b2h_png_unfilter`` (``csrc/server/image_misc.cpp``): every filter type, bit depths 1 to 16, every colour type,
    Adam7 interlacing; alpha is dropped."""
    p, idat, pal = 8, [], b""
    w = h = depth = ctype = interlace = 0
    while p + 8 <= len(data):
        n, kind = struct.unpack(">I4s", data[p:p + 8])
        body = data[p + 8:p + 8 + n]
        if kind == b"IHDR":
            if len(body) < 13:
                raise ValueError("png: truncated header")
            w, h, depth, ctype, _, _, interlace = struct.unpack(">IIBBBBB", body[:13])
        elif kind == b"PLTE":
            pal = bytes(body[:len(body) // 3 * 3])
        elif kind == b"IDAT":
            idat.append(body)
        elif kind == b"IEND":
            break
        p += 12 + n
    if w <= 0 or h <= 0 or ctype not in (0, 2, 3, 4, 6) or depth not in (1, 2, 4, 8, 16):
        raise ValueError("bad PNG header")
    if w * h > MAX_DECODE_PIXELS:
        raise ValueError("png: image too large")
    # inflate no more than the scanlines can hold (filter bytes and Adam7 row padding included): a small file may
    # expand a thousandfold
    limit = h * (1 + (w * 8 * depth + 7) // 8) + 16 * (h + 7) + 64
    try:
        z = zlib.decompressobj()
        raw = z.decompress(b"".join(idat), limit)
    except zlib.error as e:
        raise ValueError(f"png: {e}")
    lib = _h()
    out = np.empty((h, w, 3), dtype=np.uint8)
    buf = (C.c_ubyte * len(raw)).from_buffer_copy(raw)
    pbuf = (C.c_ubyte * max(len(pal), 1)).from_buffer_copy(pal or b"\0")
    if lib.b2h_png_unfilter(buf, len(raw), w, h, depth, ctype, interlace, pbuf, len(pal) // 3, out.ctypes.data_as(C.c_void_p)) != 0:
        raise ValueError(lib.b2h_image_error().decode() or "bad PNG")
    return out


def load_url(url: str) -> bytes:
    """Only ``data:`` URLs are accepted (the server has no outbound network)."""
    if not url.startswith("data:"):
        raise ValueError("only data: URLs are supported for images")
    head, _, payload = url.partition(",")
    return base64.b64decode(payload) if head.endswith(";base64") else payload.encode()


def image_key(data: bytes) -> int:
    """Prefix-cache salt of an image: the first 8 bytes of its SHA-256."""
    return int.from_bytes(hashlib.sha256(data).digest()[:8], "little")


# ---------------------------------------------------------------------------------------------------------------------
class VisionFrontEnd:
    """Turns the ``image_url`` parts of a chat request into what the model's prefill takes: the prompt with every image
    placeholder expanded to one token per merged patch, the encoder's rows for those tokens, multi-axis rotary
    positions and the running position after the prompt (reference: crates/agens-cli/src/mm.rs ``encode`` /
    ``prefill_prompt_with`` and crates/agens-server/src/vision.rs).  Runs on the engine thread: the tower launches
    kernels on the model's device."""

    def __init__(self, tower, pad_id: int, head_dim: int, sections: Sequence[int] = (24, 20, 20), interleaved: bool = True,
                 max_images: int = 16):
        from ..ops import basic
        self.tower, self.pad_id, self.max_images = tower, int(pad_id), max_images
        sections = list(sections)
        if sum(sections) != head_dim // 2:                     # scale the split to this head size, keeping the shares
            half = head_dim // 2
            sections = [half * s // sum(sections) for s in sections]
            sections[0] += half - sum(sections)
        self.pair_axis = basic.mrope_pair_axis(head_dim, sections, interleaved)

    def prepare(self, prompt: Sequence[int], urls: Sequence[str]) -> dict:
        import torch
        if len(urls) > self.max_images:
            raise ValueError(f"at most {self.max_images} images per request")
        rows, counts, grids, keys = [], [], [], []
        for u in urls:
            data = load_url(u)
            patches, (gh, gw) = preprocess(decode_image(data))
            rows.append(self.tower.encode(torch.from_numpy(patches), (gh, gw)))
            counts.append(gh * gw // 4)
            grids.append((gh // 2, gw // 2))
            keys.append(image_key(data))
        ids = expand_placeholders(list(prompt), self.pad_id, counts)
        pos3, nxt = mrope_positions(ids, self.pad_id, grids)
        return {"ids": ids, "rows": torch.cat(rows, 0), "pos3": torch.from_numpy(pos3), "pair_axis": self.pair_axis,
                "rope_next": int(nxt), "pad_id": self.pad_id, "keys": keys}
