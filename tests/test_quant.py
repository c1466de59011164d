"""CPU tests of the quantisation containers (reference test model: crates/agens-core/src/reference.rs tests,
pack/unpack round trip and gemv vs dequant)."""
import pytest
import torch

from agens_engine_b200.utils import quant


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("symmetric", [False, True])
def test_quantize_error_bound(bits, group, symmetric):
    torch.manual_seed(bits * 10 + group)
    w = torch.randn(32, 256) * 0.02
    ql = quant.quantize(w, bits, group, symmetric=symmetric)
    assert ql.codes.max() <= (1 << bits) - 1
    err = (ql.dequant() - w).abs().reshape(32, 256 // group, group).amax(-1)
    step = ql.scale.float()
    assert torch.all(err <= step * (0.51 if not symmetric else 1.01) + 1e-6)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_stream_roundtrip(bits):
    torch.manual_seed(1)
    codes = torch.randint(0, 1 << bits, (16, 256), dtype=torch.uint8)
    packed = quant.pack_stream(codes, bits)
    assert packed.dtype == torch.int32 and packed.shape == (16, 256 * bits // 32)
    assert torch.equal(quant.unpack_stream(packed, bits, 256), codes)


def test_stream_w4_matches_reference_nibble_order():
    # reference.rs:21-33: 8 nibbles per word, lowest nibble = lowest input index
    codes = torch.arange(8, dtype=torch.uint8).reshape(1, 8).repeat(1, 4)
    packed = quant.pack_stream(codes, 4)
    assert (packed[0, 0].item() & 0xFFFFFFFF) == 0x76543210


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("group", [64, 128])
def test_fm_roundtrip(bits, group):
    torch.manual_seed(7)
    w = torch.randn(64, 384) * 0.02
    ql = quant.quantize(w, bits, group)
    wq = quant.pack_fm(ql)
    assert wq.shape == (2, 3, quant.block_bytes(bits, group))
    back = quant.unpack_fm(wq, bits, 64, 384, group)
    assert torch.equal(back.codes, ql.codes)
    assert torch.equal(back.scale, ql.scale) and torch.equal(back.zero, ql.zero)


def test_fm_every_bit_used_once():
    for bits in (2, 3, 4):
        n, k = 32, 128
        total = torch.zeros(quant.block_bytes(bits, 64) * 8, dtype=torch.int32)
        for r in range(0, n, 5):
            for c in range(0, k, 7):
                codes = torch.zeros(n, k, dtype=torch.uint8)
                codes[r, c] = (1 << bits) - 1
                ql = quant.QuantLinear(n, k, bits, 64, codes, torch.zeros(n, k // 64).half(), torch.zeros(n, k // 64).half())
                b = quant.pack_fm(ql).reshape(-1)
                setbits = sum(bin(int(x)).count("1") for x in b.tolist())
                assert setbits == bits
                idx = torch.nonzero(b).reshape(-1)
                for i in idx.tolist():
                    for j in range(8):
                        if (int(b[i]) >> j) & 1:
                            total[i * 8 + j] += 1
        assert total.max() <= 1


def test_slot_scales_table():
    assert quant.slot_scales(4).tolist() == [[1.0, 1.0, 16.0, 16.0]] * 4
    s2 = quant.slot_scales(2)
    assert s2[0].tolist() == [1.0, 1.0, 4.0, 4.0] and s2[1].tolist() == [16.0, 16.0, 64.0, 64.0]


def test_interleave_gate_up():
    g = torch.arange(16 * 4, dtype=torch.float32).reshape(16, 4)
    u = -g
    m = quant.interleave_gate_up(g, u)
    assert torch.equal(m[:8], g[:8]) and torch.equal(m[8:16], u[:8]) and torch.equal(m[16:24], g[8:])


def test_seeded_bit_assignment_is_deterministic():
    names = [f"l{i}" for i in range(20)]
    a = quant.seeded_bit_assignment(names, 3)
    assert a == quant.seeded_bit_assignment(names, 3) and set(a.values()) <= {2, 3, 4}
