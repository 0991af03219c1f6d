"""The CPU oracle against every known-answer unit test the reference keeps for the quant
formats on this path (src/quant/{half,q4_0,q4_k,q5_k,q6_k,q8_0,iq4_xs}.rs); the vectors are
in tests/golden/quant_kats.json with the file:line each one comes from."""
import json
import struct
from pathlib import Path

import numpy as np
import pytest

import oracle as ro
from reinstinct_b200.synth import Lcg

KATS = json.loads((Path(__file__).parent / "golden" / "quant_kats.json").read_text())


def f16(v: float) -> bytes:
    return struct.pack("<H", ro.f32_to_f16(v))


def k_scales(sc: int, m: int) -> bytes:
    """12 packed bytes with all eight 6-bit (scale, min) pairs equal to (sc, m)."""
    a = (sc & 63) | (((sc >> 4) & 3) << 6)
    b = (m & 63) | (((m >> 4) & 3) << 6)
    c = (sc & 15) | ((m & 15) << 4)
    return bytes([a] * 4 + [b] * 4 + [c] * 4)


def q4k_block(d, dmin, sc, m, nibble) -> bytearray:
    return bytearray(f16(d) + f16(dmin) + k_scales(sc, m) + bytes([nibble | (nibble << 4)] * 128))


def q5k_block(d, dmin, sc, m, nibble, high) -> bytearray:
    return bytearray(f16(d) + f16(dmin) + k_scales(sc, m) + bytes([0xFF if high else 0] * 32)
                     + bytes([nibble | (nibble << 4)] * 128))


def q6k_block(d, scale, q) -> bytearray:
    lo, pair = q & 15, (q >> 4) & 3
    return bytearray(bytes([lo | (lo << 4)] * 128) + bytes([pair * 0x55] * 64)
                     + bytes([scale & 0xFF] * 16) + f16(d))


def iq4xs_block(d, ls, nibble) -> bytearray:
    hi2, lo4 = (ls >> 4) & 3, ls & 15
    sh = sum(hi2 << (2 * i) for i in range(8))
    return bytearray(f16(d) + struct.pack("<H", sh) + bytes([lo4 | (lo4 << 4)] * 4)
                     + bytes([nibble | (nibble << 4)] * 128))


def deq(t, block, n=256):
    return ro.dequantize(t, np.frombuffer(bytes(block), dtype=np.uint8), n)


def test_f16_known_values():
    for bits, want in KATS["f16_to_f32"]["cases"]:
        got = struct.unpack("<I", struct.pack("<f", ro.f16_to_f32(bits)))[0]
        assert got == int(want, 16), hex(bits)
    assert np.isnan(ro.f16_to_f32(KATS["f16_nan"]["bits"]))
    for bits in KATS["f16_round_trip"]["bits"]:
        assert ro.f32_to_f16(ro.f16_to_f32(bits)) == bits
    for v in KATS["bf16"]["values"]:
        bits = struct.unpack("<I", struct.pack("<f", v))[0] >> 16
        assert float(ro.lib().ro_bf16_to_f32(bits)) == v


def test_f16_matches_ieee_on_all_normals_and_truncates_subnormals():
    # f16 -> f32 is exact for every one of the 65536 patterns
    bits = np.arange(65536, dtype=np.uint16)
    ours = np.array([ro.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    ieee = bits.view(np.float16).astype(np.float32)
    assert np.array_equal(ours.view(np.uint32)[~np.isnan(ieee)], ieee.view(np.uint32)[~np.isnan(ieee)])
    # f32 -> f16: nearest-even on normals (as numpy), truncation on subnormal results
    rng = np.random.default_rng(1)
    v = (rng.standard_normal(20000) * 10.0 ** rng.uniform(-4, 4, 20000)).astype(np.float32)
    normal = np.abs(v) >= 6.2e-5
    ours16 = np.array([ro.f32_to_f16(float(x)) for x in v], dtype=np.uint16)
    assert np.array_equal(ours16[normal], v[normal].astype(np.float16).view(np.uint16))
    # 1.5 * 2^-24 is halfway between subnormals 1 and 2: the reference truncates to 1
    assert ro.f32_to_f16(1.5 * 2.0 ** -24) == 1
    assert ro.f32_to_f16(1.99 * 2.0 ** -24) == 1


def test_q4_k_vectors():
    for case in KATS["q4_k"]:
        for nib in case["nibbles"]:
            out = deq(ro.Q4_K, q4k_block(case["d"], case["dmin"], case["sc"], case["m"], nib))
            want = float(nib) if case.get("expect") == "nibble" else case["expect_value"]
            assert np.all(out == want), case["ref"]
    c = KATS["q4_k_low_high"]
    b = q4k_block(1.0, 0.0, 1, 0, 0)
    b[16:144] = bytes([c["low"] | (c["high"] << 4)] * 128)
    out = deq(ro.Q4_K, b).reshape(4, 2, 32)
    assert np.all(out[:, 0] == c["low"]) and np.all(out[:, 1] == c["high"])


def test_q4_k_repack_decodes_like_the_kernel():
    c = KATS["q4_k_repack"]
    raw = bytearray()
    for blk in range(c["n_blocks"]):
        b = q4k_block(c["d"], c["dmin"], c["sc"], c["m"], 0)
        for i in range(128):
            b[16 + i] = ((blk * 128 + i) * c["qs_mul"] + c["qs_add"]) & 0xFF
        raw += b
    in_dim = c["n_blocks"] * 256
    raw = np.frombuffer(bytes(raw), dtype=np.uint8)
    want = ro.dequantize(ro.Q4_K, raw, in_dim)
    packed = ro.repack(ro.Q4_K, raw, in_dim, 1)
    nsp = ro.nsp(in_dim)
    nib_len, sm_len = nsp * 16, nsp * 2
    got = np.zeros(in_dim, dtype=np.float32)
    for gsb in range(in_dim // 32):
        nib = packed[gsb * 16:gsb * 16 + 16]
        sc, m = float(packed[nib_len + gsb * 2]), float(packed[nib_len + gsb * 2 + 1])
        dd = nib_len + sm_len + (gsb // 8) * 4
        d = ro.f16_to_f32(int(packed[dd]) | int(packed[dd + 1]) << 8)
        dmin = ro.f16_to_f32(int(packed[dd + 2]) | int(packed[dd + 3]) << 8)
        blk, s = divmod(gsb, 8)
        base = blk * 256 + (s // 2) * 64 + (s & 1) * 32
        for k in range(32):
            q = nib[k] & 15 if k < 16 else nib[k - 16] >> 4
            got[base + k] = np.float32(d * sc) * np.float32(q) - np.float32(dmin * m)
    assert np.max(np.abs(got - want)) < c["tol"]


def test_q5_k_vectors():
    for case in KATS["q5_k"]:
        out = deq(ro.Q5_K, q5k_block(case["d"], case["dmin"], case["sc"], case["m"], case["nibble"], case["high_bit"]))
        assert np.all(out == case["expect_value"]), case["ref"]
    c = KATS["q5_k_equals_q4_k"]
    q5 = deq(ro.Q5_K, q5k_block(c["d"], c["dmin"], c["sc"], c["m"], c["nibble"], False))
    q4 = deq(ro.Q4_K, q4k_block(c["d"], c["dmin"], c["sc"], c["m"], c["nibble"]))
    assert np.array_equal(q5, q4)
    for case in KATS["q5_k_qh_bits"]["cases"]:
        b = q5k_block(1.0, 0.0, 1, 0, 0, False)
        b[16 + case["qh_index"]] = case["qh_value"]
        out = deq(ro.Q5_K, b)
        assert out[case["weight"]] == 16.0 and np.count_nonzero(out) == 1


def test_q6_k_vectors():
    for case in KATS["q6_k"]:
        for q in case["q"]:
            out = deq(ro.Q6_K, q6k_block(case["d"], case["scale"], q))
            want = float(q - 32) if case.get("expect") == "q_minus_32" else case["expect_value"]
            assert np.all(out == want), (case["ref"], q)
    c = KATS["q6_k_scale_index"]
    b = q6k_block(c["d"], 0, c["q"])
    b[192:208] = bytes(range(16))
    out = deq(ro.Q6_K, b)
    for idx in range(256):
        chunk, inner = divmod(idx, 128)
        group, l = divmod(inner, 32)
        assert out[idx] == chunk * 8 + l // 16 + group * 2


def test_q8_0_vectors():
    b = f16(1.0) + bytes(range(32))
    assert np.array_equal(deq(ro.Q8_0, b, 32), np.arange(32, dtype=np.float32))
    c = KATS["q8_0"]["negative"]
    assert np.all(deq(ro.Q8_0, f16(c["d"]) + bytes([c["q"]] * 32), 32) == c["expect_value"])
    d1, d2 = KATS["q8_0"]["multi"]["d"]
    out = deq(ro.Q8_0, f16(d1) + bytes([1] * 32) + f16(d2) + bytes([1] * 32), 64)
    assert np.all(out[:32] == d1) and np.all(out[32:] == d2)


def test_q4_0_vectors():
    b = f16(1.0) + bytes([k | ((15 - k) << 4) for k in range(16)])
    out = deq(ro.Q4_0, b, 32)
    for k in range(16):
        assert out[k] == k - 8 and out[k + 16] == (15 - k) - 8
    for in_dim, want in KATS["q4_0"]["pad"]["cases"]:
        assert ro.nsp(in_dim) == want
    # repack: nibbles verbatim, scales split out, tight stride when not a power of two
    c = KATS["q4_0"]["repack_copy"]
    in_dim, out_dim = c["in_dim"], c["out_dim"]
    nb = in_dim // 32
    assert ro.nsp(in_dim) == nb
    raw = np.array([i % c["mod"] for i in range(out_dim * nb * 18)], dtype=np.uint8)
    for blk in range(out_dim * nb):
        raw[blk * 18:blk * 18 + 2] = np.frombuffer(f16(blk + 1.0), dtype=np.uint8)
    packed = ro.repack(ro.Q4_0, raw, in_dim, out_dim)
    assert packed.size == ro.repacked_len(ro.Q4_0, in_dim, out_dim)
    for i in range(out_dim * nb):
        assert np.array_equal(packed[i * 16:i * 16 + 16], raw[i * 18 + 2:i * 18 + 18])
        assert np.array_equal(packed[out_dim * nb * 16 + i * 2:][:2], raw[i * 18:i * 18 + 2])


def test_q4_0_repack_reads_back_bit_exact():
    c = KATS["q4_0"]["repack_dequant"]
    in_dim, out_dim = c["in_dim"], c["out_dim"]
    nb, nsp = in_dim // 32, ro.nsp(in_dim)
    assert nsp == nb + 1
    rng = Lcg(c["seed"], c["inc"])
    raw = np.zeros(out_dim * nb * 18, dtype=np.uint8)
    for blk in range(out_dim * nb):
        raw[blk * 18:blk * 18 + 2] = np.frombuffer(f16(np.float32(c["d_step"]) * np.float32(blk + 1.0)), dtype=np.uint8)
        raw[blk * 18 + 2:blk * 18 + 18] = rng.bytes(16)
    direct = ro.dequantize(ro.Q4_0, raw, out_dim * in_dim)
    packed = ro.repack(ro.Q4_0, raw, in_dim, out_dim)
    nib_len = out_dim * nsp * 16
    for row in range(out_dim):
        for blk in range(nb):
            dd = nib_len + (row * nsp + blk) * 2
            d = np.float32(ro.f16_to_f32(int(packed[dd]) | int(packed[dd + 1]) << 8))
            for k in range(16):
                byte = int(packed[(row * nsp + blk) * 16 + k])
                base = row * in_dim + blk * 32
                assert direct[base + k] == d * np.float32((byte & 15) - 8)
                assert direct[base + k + 16] == d * np.float32((byte >> 4) - 8)


def test_iq4_xs_vectors():
    K = KATS["iq4_xs"]
    lut = K["kvalues"]["values"]
    c = K["zero_scale"]
    assert np.all(deq(ro.IQ4_XS, iq4xs_block(c["d"], c["ls"], c["nibble"])) == 0.0)
    for nib in range(16):
        assert np.all(deq(ro.IQ4_XS, iq4xs_block(1.0, K["lut"]["ls"], nib)) == lut[nib])
    c = K["negative"]
    assert np.all(deq(ro.IQ4_XS, iq4xs_block(c["d"], c["ls"], c["nibble"])) == c["expect_value"])
    c = K["low_high"]
    b = iq4xs_block(1.0, 33, 0)
    b[8:136] = bytes([c["low"] | (c["high"] << 4)] * 128)
    out = deq(ro.IQ4_XS, b).reshape(8, 2, 16)
    assert np.all(out[:, 0] == lut[c["low"]]) and np.all(out[:, 1] == lut[c["high"]])
    b = iq4xs_block(1.0, 32, 8)
    sh, sl = 0, [0, 0, 0, 0]
    for sb in range(8):
        ls = 33 + sb
        sh |= ((ls >> 4) & 3) << (2 * sb)
        sl[sb // 2] |= (ls & 15) << (4 * (sb & 1))
    b[2:4] = struct.pack("<H", sh)
    b[4:8] = bytes(sl)
    out = deq(ro.IQ4_XS, b).reshape(8, 32)
    for sb in range(8):
        assert np.all(out[sb] == 1 + sb)


def test_iq4_xs_repack_reads_back_within_f16_fold():
    c = KATS["iq4_xs"]["repack_dequant"]
    in_dim, out_dim = c["in_dim"], c["out_dim"]
    nblk, nsp = in_dim // 256, ro.nsp(in_dim)
    assert nsp == c["nsp"]
    rng = Lcg(c["seed"], c["inc"])
    raw = np.zeros(out_dim * nblk * 136, dtype=np.uint8)
    for blk in range(out_dim * nblk):
        raw[blk * 136:blk * 136 + 2] = np.frombuffer(f16(np.float32(c["d_step"]) * np.float32(blk + 1.0)), dtype=np.uint8)
        raw[blk * 136 + 2:blk * 136 + 136] = rng.bytes(134)
    direct = ro.dequantize(ro.IQ4_XS, raw, out_dim * in_dim).reshape(out_dim, in_dim // 32, 2, 16)
    packed = ro.repack(ro.IQ4_XS, raw, in_dim, out_dim)
    assert packed.size == ro.repacked_len(ro.IQ4_XS, in_dim, out_dim)
    lut = np.array(KATS["iq4_xs"]["kvalues"]["values"], dtype=np.float32)
    nib_len = out_dim * nsp * 16
    worst = 0.0
    for row in range(out_dim):
        for sb in range(in_dim // 32):
            dd = nib_len + (row * nsp + sb) * 2
            dl = np.float32(ro.f16_to_f32(int(packed[dd]) | int(packed[dd + 1]) << 8))
            q = packed[(row * nsp + sb) * 16:][:16]
            for got, want in ((dl * lut[q & 15], direct[row, sb, 0]), (dl * lut[q >> 4], direct[row, sb, 1])):
                worst = max(worst, float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30))))
    assert worst < c["tol"]


@pytest.mark.parametrize("t,expected", [(ro.Q4_0, (18, 32)), (ro.Q8_0, (34, 32)), (ro.Q4_K, (144, 256)),
                                        (ro.Q5_K, (176, 256)), (ro.Q6_K, (210, 256)), (ro.IQ4_XS, (136, 256))])
def test_block_sizes(t, expected):
    assert (ro.block_bytes(t), ro.block_weights(t)) == expected
