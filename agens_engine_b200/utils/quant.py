"""Mixed 2/3/4-bit group quantisation: checkpoint containers, the kernel ("FM") layout and fp32 references.

Two layouts exist for one quantised linear ``W[n, k]``:

* **Checkpoint container** (public format; superset of the reference's compressed-tensors ``pack-quantized``
  container, reference ``crates/agens-core/src/reference.rs:16-72`` and ``crates/agens-core/src/weights.rs:15-24``):
  ``weight_packed`` int32 ``[n, k*bits/32]`` holding a little-endian bit stream of unsigned ``bits``-wide codes
  along k (for 4 bits: 8 nibbles per word, lowest nibble = lowest k, code = q + 8 when symmetric),
  ``weight_scale`` bf16 or fp16 ``[n, k/group]`` and, for asymmetric tensors, ``weight_zero_point`` fp16
  ``[n, k/group]`` in code units.  ``w = scale * (code - zero)``; symmetric tensors use ``zero = 2**(bits-1)``.

* **FM (fragment-major) kernel layout**, consumed by ``csrc/kernels/sm100/wq_gemv.cu``.  Rows are cut into blocks
  of 16, k into chunks (64 codes for 4 bits, 128 for 2 and 3 bits).  The tensor is stored panel-major: for every
  panel of 32 rows and every batch of 128 k one contiguous block holds the records of its two row blocks followed by
  their (scale, zero) pairs, so one bulk copy brings everything a warp needs for that tile.  One chunk of one row
  block is a record of
  ``32 lanes x 16 B`` (plus ``32 x 8 B`` of high bits for 3-bit tensors) in which lane ``(g, t)`` (``g = lane >> 2``,
  ``t = lane & 3``) finds exactly the codes of rows ``g`` and ``g + 8`` that its ``mma.m16n8k16`` A fragments need,
  positioned so that a single ``lop3`` turns two codes into two fp16 numbers ``1024 + c * code``.  The power of two
  ``c`` is undone by staging the activation of that k slot as ``x / c``; the constant ``1024`` is removed per group
  with a precomputed activation sum.  Scales and zero points are stored per row block and group as fp16 pairs.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

BITS = (2, 3, 4)


def chunk_k(bits: int) -> int:
    """k codes covered by one FM record."""
    return 64 if bits == 4 else 128


def record_bytes(bits: int) -> int:
    return {4: 512, 2: 512, 3: 768}[bits]


@dataclasses.dataclass
class QuantLinear:
    """A quantised linear in checkpoint form (all tensors on CPU or GPU, any device)."""
    n: int
    k: int
    bits: int
    group: int
    codes: torch.Tensor          # uint8 [n, k] unpacked codes (kept for tests / repacking)
    scale: torch.Tensor          # fp16 [n, k/group]
    zero: torch.Tensor           # fp16 [n, k/group] (code units)

    def dequant(self, dtype=torch.float32) -> torch.Tensor:
        return dequant_codes(self.codes, self.scale, self.zero, self.group).to(dtype)


def quantize(w: torch.Tensor, bits: int, group: int, symmetric: bool = False,
             scale_dtype=torch.float16) -> QuantLinear:
    """Round-to-nearest group quantisation of ``w[n, k]`` (fp32).

    Asymmetric: ``scale = (max - min) / (2**bits - 1)``, ``zero = -min / scale`` kept as an fp16 real number.
    Symmetric: ``scale = amax / (2**(bits-1) - 1)`` and ``zero = 2**(bits-1)`` (the reference's convention,
    ``reference.rs:40-52``).  Scales are rounded to ``scale_dtype`` before the codes are chosen, so the stored
    tensors reproduce the quantiser's own decision exactly.
    """
    assert bits in BITS and w.dim() == 2
    n, k = w.shape
    assert k % group == 0, (k, group)
    wf = w.float().reshape(n, k // group, group)
    qmax = (1 << bits) - 1
    if symmetric:
        amax = wf.abs().amax(dim=-1)
        half = float((1 << (bits - 1)) - 1)
        scale = torch.where(amax > 0, amax / half, torch.ones_like(amax))
        scale = scale.to(scale_dtype).float()
        zero = torch.full_like(scale, float(1 << (bits - 1)))
    else:
        lo = wf.amin(dim=-1)
        hi = wf.amax(dim=-1)
        scale = (hi - lo) / qmax
        scale = torch.where(scale > 0, scale, torch.ones_like(scale))
        scale = scale.to(scale_dtype).float()
        zero = (-lo / scale).to(torch.float16).float()
    q = torch.round(wf / scale.unsqueeze(-1) + zero.unsqueeze(-1)).clamp_(0, qmax)
    return QuantLinear(n=n, k=k, bits=bits, group=group,
                       codes=q.reshape(n, k).to(torch.uint8),
                       scale=scale.to(torch.float16), zero=zero.to(torch.float16))


def dequant_codes(codes: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, group: int) -> torch.Tensor:
    n, k = codes.shape
    c = codes.float().reshape(n, k // group, group)
    return ((c - zero.float().unsqueeze(-1)) * scale.float().unsqueeze(-1)).reshape(n, k)


# ---------------------------------------------------------------------------------------------------------------
# Checkpoint container: little-endian bit stream along k
# ---------------------------------------------------------------------------------------------------------------

def pack_stream(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 codes ``[n, k]`` -> int32 ``[n, k*bits/32]`` (bit i*bits of the row stream = bit 0 of code i)."""
    n, k = codes.shape
    assert (k * bits) % 32 == 0
    c = codes.to(torch.int64)
    bitpos = torch.arange(bits, dtype=torch.int64, device=codes.device)
    bitsm = ((c.unsqueeze(-1) >> bitpos) & 1).reshape(n, k * bits)          # [n, k*bits] of 0/1
    words = bitsm.reshape(n, -1, 32)
    weights = (1 << torch.arange(32, dtype=torch.int64, device=codes.device))
    packed = (words * weights).sum(dim=-1)                                  # [n, words] in 0..2^32-1
    packed = torch.where(packed >= (1 << 31), packed - (1 << 32), packed)
    return packed.to(torch.int32)


def unpack_stream(packed: torch.Tensor, bits: int, k: int) -> torch.Tensor:
    n = packed.shape[0]
    p = packed.to(torch.int64) & 0xFFFFFFFF
    bitpos = torch.arange(32, dtype=torch.int64, device=packed.device)
    bitsm = ((p.unsqueeze(-1) >> bitpos) & 1).reshape(n, -1)[:, : k * bits].reshape(n, k, bits)
    weights = (1 << torch.arange(bits, dtype=torch.int64, device=packed.device))
    return (bitsm * weights).sum(dim=-1).to(torch.uint8)


# ---------------------------------------------------------------------------------------------------------------
# FM layout (CPU/torch restatement of what the device repack kernel writes)
# ---------------------------------------------------------------------------------------------------------------

def _slot_tables(bits: int):
    """For one FM record return, for every code of a lane, ``(word, bit, row_half, step, slot, c_log2)``.

    ``step`` is the mma k-step inside the chunk (16 codes of k each), ``slot`` in 0..3 the lane's k slot inside
    the step (logical k = chunk*CK + step*16 + t*4 + slot), ``row_half`` 0 for row g and 1 for row g+8, and
    ``c_log2`` the power of two the extraction multiplies the code by.  High bits of 3-bit codes are handled by
    :func:`_hi_tables`.
    """
    ent = []
    if bits == 4:
        # word j = step j.  extraction e -> (slots pair, row half): shifts (0, 8) x positions (0, 4)
        for j in range(4):
            for row_half in (0, 1):
                for pair in (0, 1):           # pair 0 = slots (0,1) at c=1 ; pair 1 = slots (2,3) at c=16
                    pos = 4 * pair + 8 * row_half
                    for hi16 in (0, 1):
                        ent.append((j, pos + 16 * hi16, row_half, j, 2 * pair + hi16, 4 * pair))
    else:
        # 2-bit fields (also the low plane of 3-bit): word u holds steps 2u, 2u+1.
        # field position p in {0,2,4,6} (c = 1,4,16,64); +8 selects the row half.
        for u in range(4):
            for row_half in (0, 1):
                for q in range(4):            # q -> c = 4**q ; step = 2u + (q >> 1) ; pair = q & 1
                    pos = 2 * q + 8 * row_half
                    for hi16 in (0, 1):
                        ent.append((u, pos + 16 * hi16, row_half, 2 * u + (q >> 1), 2 * (q & 1) + hi16, 2 * q))
    return ent


# 3-bit high plane: hi word h (0,1) serves low words 2h, 2h+1; each low word has two rounds (row half 0 / 1) of
# four fields.  Round r = 2*(u & 1) + row_half uses source bit set SRC[r] so that after one shift the four bits sit
# at positions {2,4,6,8} of each 16-bit half, directly above their 2-bit fields.
_HI_SRC = ((0, 2, 4, 6), (1, 3, 5, 7), (8, 10, 12, 14), (9, 11, 13, 15))


def _hi_tables():
    ent = []  # (hi_word, bit, low_word u, row_half, q, hi16)
    for u in range(4):
        for row_half in (0, 1):
            r = 2 * (u & 1) + row_half
            for q in range(4):
                for hi16 in (0, 1):
                    ent.append((u >> 1, _HI_SRC[r][q] + 16 * hi16, u, row_half, q, hi16))
    return ent


def slot_scales(bits: int) -> torch.Tensor:
    """``c`` for every (step, slot) of a chunk: the activation of that k position is staged as ``x / c``."""
    ck = chunk_k(bits)
    out = torch.ones(ck // 16, 4)
    for (_, _, _, step, slot, c_log2) in _slot_tables(bits):
        out[step, slot] = float(1 << c_log2)
    return out


def w_batch_bytes(bits: int) -> int:
    """Weight bytes of one 128-k batch of one 16-row block."""
    return (128 // chunk_k(bits)) * record_bytes(bits)


def block_bytes(bits: int, group: int) -> int:
    """Bytes of one (32-row panel, 128-k batch) block: two row blocks of records + their (scale, zero) pairs."""
    return 2 * w_batch_bytes(bits) + 2 * (128 // group) * 64


def _records(ql: QuantLinear) -> torch.Tensor:
    """uint8 [n/16, k/CK, record_bytes]: the per-(row block, chunk) records."""
    n, k, bits = ql.n, ql.k, ql.bits
    ck = chunk_k(bits)
    nrb, nch = n // 16, k // ck
    codes = ql.codes.to(torch.int64).cpu().reshape(nrb, 16, nch, ck // 16, 4, 4)   # rb, row, chunk, step, t, slot
    lanes_g = torch.arange(32) >> 2
    lanes_t = torch.arange(32) & 3
    words = torch.zeros(nrb, nch, 32, 4, dtype=torch.int64)
    lo_bits = 2 if bits == 3 else bits
    lo_mask = (1 << lo_bits) - 1
    for (word, bit, row_half, step, slot, _c) in _slot_tables(bits):
        rows = lanes_g + 8 * row_half
        v = codes[:, rows, :, step, lanes_t, slot]               # [32(lane), nrb, nch] (advanced indexing first)
        v = v.permute(1, 2, 0) & lo_mask                          # [nrb, nch, 32]
        words[:, :, :, word] |= v << bit
    rec = [words]
    if bits == 3:
        hi = torch.zeros(nrb, nch, 32, 2, dtype=torch.int64)
        for (hword, bit, u, row_half, q, hi16) in _hi_tables():
            step, slot = 2 * u + (q >> 1), 2 * (q & 1) + hi16
            rows = lanes_g + 8 * row_half
            v = codes[:, rows, :, step, lanes_t, slot].permute(1, 2, 0) >> 2
            hi[:, :, :, hword] |= (v & 1) << bit
        rec.append(hi)
    flat = []
    for w in rec:                                                 # [nrb, nch, 32, W] -> bytes little endian
        w8 = torch.stack([(w >> (8 * b)) & 0xFF for b in range(4)], dim=-1).to(torch.uint8)
        flat.append(w8.reshape(nrb, nch, -1))
    out = torch.cat(flat, dim=-1).contiguous()
    assert out.shape[-1] == record_bytes(bits)
    return out


def pack_fm(ql: QuantLinear) -> torch.Tensor:
    """Checkpoint codes -> FM layout: uint8 ``[n/32, k/128, block_bytes]``."""
    n, k, bits, group = ql.n, ql.k, ql.bits, ql.group
    assert n % 32 == 0 and k % 128 == 0 and k % group == 0
    rec = _records(ql)                                            # [n/16, k/CK, REC]
    rpb = 128 // chunk_k(bits)
    npan, nbat = n // 32, k // 128
    w = rec.reshape(npan, 2, nbat, rpb * record_bytes(bits)).permute(0, 2, 1, 3).reshape(npan, nbat, -1)
    gpb = 128 // group
    sz = torch.stack([ql.scale.cpu(), ql.zero.cpu()], dim=-1).to(torch.float16)        # [n, ng, 2]
    sz = sz.reshape(npan, 2, 16, nbat, gpb, 2).permute(0, 3, 1, 4, 2, 5).contiguous()  # pan, bat, rb, g, row, (s,z)
    szb = sz.view(torch.uint8).reshape(npan, nbat, 2 * gpb * 64)
    out = torch.cat([w, szb], dim=-1).contiguous()
    assert out.shape[-1] == block_bytes(bits, group)
    return out


def unpack_fm(wq: torch.Tensor, bits: int, n: int, k: int, group: int) -> QuantLinear:
    """Inverse of :func:`pack_fm` (used by tests and by the dequant oracle)."""
    ck = chunk_k(bits)
    rpb, gpb = 128 // ck, 128 // group
    npan, nbat = n // 32, k // 128
    blk = wq.cpu().reshape(npan, nbat, block_bytes(bits, group))
    wb = 2 * w_batch_bytes(bits)
    rec = blk[:, :, :wb].reshape(npan, nbat, 2, rpb, record_bytes(bits)).permute(0, 2, 1, 3, 4)
    rec = rec.reshape(n // 16, k // ck, record_bytes(bits))
    nrb, nch = n // 16, k // ck
    b = rec.to(torch.int64)
    lo = b[:, :, :512].reshape(nrb, nch, 32, 4, 4)
    words = sum(lo[..., i] << (8 * i) for i in range(4))          # [nrb, nch, 32, 4]
    codes = torch.zeros(nrb, 16, nch, ck // 16, 4, 4, dtype=torch.int64)
    lanes_g = torch.arange(32) >> 2
    lanes_t = torch.arange(32) & 3
    lo_bits = 2 if bits == 3 else bits
    for (word, bit, row_half, step, slot, _c) in _slot_tables(bits):
        v = (words[:, :, :, word] >> bit) & ((1 << lo_bits) - 1)   # [nrb, nch, 32]
        rows = lanes_g + 8 * row_half
        codes[:, rows, :, step, lanes_t, slot] = v.permute(2, 0, 1)
    if bits == 3:
        hib = b[:, :, 512:].reshape(nrb, nch, 32, 2, 4)
        hi = sum(hib[..., i] << (8 * i) for i in range(4))
        for (hword, bit, u, row_half, q, hi16) in _hi_tables():
            step, slot = 2 * u + (q >> 1), 2 * (q & 1) + hi16
            rows = lanes_g + 8 * row_half
            v = ((hi[:, :, :, hword] >> bit) & 1) << 2
            codes[:, rows, :, step, lanes_t, slot] |= v.permute(2, 0, 1)
    szb = blk[:, :, wb:].contiguous().view(torch.float16).reshape(npan, nbat, 2, gpb, 16, 2)
    sz = szb.permute(0, 2, 4, 1, 3, 5).reshape(n, k // group, 2)
    return QuantLinear(n=n, k=k, bits=bits, group=group, codes=codes.reshape(n, k).to(torch.uint8),
                       scale=sz[..., 0].contiguous(), zero=sz[..., 1].contiguous())


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Merge gate_proj and up_proj rows so that every 16-row block holds 8 gate rows followed by the 8 up rows of
    the same output features: rows ``g`` and ``g + 8`` of one mma accumulator are then a (gate, up) pair and the
    GEMV epilogue applies SwiGLU in registers.  The reference merges gate and up at load as well
    (``crates/agens-cli/src/m1.rs`` weight loop), but keeps them as two halves."""
    f, k = gate.shape
    assert up.shape == gate.shape and f % 8 == 0
    g = gate.reshape(f // 8, 8, k)
    u = up.reshape(f // 8, 8, k)
    return torch.cat([g, u], dim=1).reshape(2 * f, k)


def seeded_bit_assignment(names, seed: int, choices=(2, 3, 4)) -> dict:
    """Per-linear bit width drawn from a seeded generator (the benchmark configs' "seeded assignment")."""
    gen = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, len(choices), (len(names),), generator=gen).tolist()
    return {nm: choices[i] for nm, i in zip(names, idx)}
