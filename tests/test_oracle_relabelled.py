"""Relabelled source formats (Q3_K -> Q6_K, IQ4_NL -> IQ4_XS planes, BF16 -> Q8_0): the oracle against
the reference's own unit tests for them (src/quant/q3_k.rs:175-212, src/quant/iq4_nl.rs:80-117), restated
with the same generators, and against exact identities."""
import numpy as np

import oracle as ro

M64 = (1 << 64) - 1


def lcg_bytes(seed: int, n: int):
    """The reference tests' byte generator: seed = seed * 6364136223846793005 + 1, byte = seed >> 56."""
    out = np.empty(n, dtype=np.uint8)
    for i in range(n):
        seed = (seed * 6364136223846793005 + 1) & M64
        out[i] = seed >> 56
    return out, seed


def test_q3k_scales_of_32_give_a_zero_block():
    """scale_unpack_and_zero_factor_block (q3_k.rs:175-190): sixteen 6-bit scales of 32 are bytes
    0..7 = 0x00, 8..11 = 0xAA; the factor (32 - 32) makes every weight zero whatever the quants."""
    blk = np.full(110, 0xA5, dtype=np.uint8)
    blk[96:104] = 0
    blk[104:108] = 0xAA
    blk[108:110] = np.frombuffer(np.uint16(ro.f32_to_f16(1.0)).tobytes(), dtype=np.uint8)
    out = ro.dequantize_src(ro.Q3_K, blk, 256)
    assert np.all(out == 0.0)
    q6 = ro.q3k_to_q6k(blk, 256)
    assert np.all(q6[192:208] == 0)                      # sc6 = 32 - 32
    assert np.all(ro.dequantize(ro.Q6_K, q6, 256) == 0.0)


def test_q3k_to_q6k_is_bit_exact():
    """transcode_to_q6_k_is_bit_exact (q3_k.rs:192-212): 32 blocks of generator bytes with
    d = 0.02 * (1 + b/32); the Q6_K decode of the transcode equals the direct decode bit for bit."""
    n_blocks, seed = 32, 0x0A3E0000
    raw = np.empty(n_blocks * 110, dtype=np.uint8)
    for b in range(n_blocks):
        raw[b * 110:b * 110 + 108], seed = lcg_bytes(seed, 108)
        d = np.float32(0.02) * (np.float32(1.0) + np.float32(b) / np.float32(32.0))
        raw[b * 110 + 108:b * 110 + 110] = np.frombuffer(np.uint16(ro.f32_to_f16(float(d))).tobytes(), dtype=np.uint8)
    n = n_blocks * 256
    direct = ro.dequantize_src(ro.Q3_K, raw, n)
    via = ro.dequantize(ro.Q6_K, ro.q3k_to_q6k(raw, n), n)
    assert np.array_equal(direct.view(np.uint32), via.view(np.uint32))
    assert np.any(direct != 0)
    # quants land in 28..35 and scales in -32..31
    q6 = ro.q3k_to_q6k(raw, n).reshape(n_blocks, 210)
    assert q6[:, 192:208].view(np.int8).min() >= -32 and q6[:, 192:208].view(np.int8).max() <= 31


def test_iq4nl_repack_is_bit_exact_against_dequant():
    """repack_is_bit_exact_against_dequant (iq4_nl.rs:80-117): in_dim 128 (nsp = 5), 3 rows,
    d = 0.01 * (b - 5); reading the repacked planes back with the IQ4_XS index arithmetic
    reproduces the direct decode exactly."""
    in_dim, out_dim, n_sub = 128, 3, 4
    assert ro.nsp(in_dim) == 5
    seed = 0x1A4A1000
    raw = np.empty(out_dim * n_sub * 18, dtype=np.uint8)
    for b in range(out_dim * n_sub):
        d = np.float32(0.01) * (np.float32(b) - np.float32(5.0))
        raw[b * 18:b * 18 + 2] = np.frombuffer(np.uint16(ro.f32_to_f16(float(d))).tobytes(), dtype=np.uint8)
        raw[b * 18 + 2:b * 18 + 18], seed = lcg_bytes(seed, 16)
    direct = ro.dequantize_src(ro.IQ4_NL, raw, in_dim * out_dim).reshape(out_dim, in_dim)
    packed = ro.repack_any(ro.IQ4_NL, raw, in_dim, out_dim)
    assert ro.kernel_type(ro.IQ4_NL) == ro.IQ4_XS
    nsp, nib_len = 5, out_dim * 5 * 16
    assert packed.size == nib_len + out_dim * nsp * 2
    kv = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)
    for row in range(out_dim):
        for sb in range(n_sub):
            nib = packed[(row * nsp + sb) * 16:(row * nsp + sb) * 16 + 16]
            d_off = nib_len + (row * nsp + sb) * 2
            d = np.float32(ro.f16_to_f32(int(packed[d_off]) | (int(packed[d_off + 1]) << 8)))
            lo, hi = d * kv[nib & 15], d * kv[nib >> 4]
            assert np.array_equal(lo, direct[row, sb * 32:sb * 32 + 16])
            assert np.array_equal(hi, direct[row, sb * 32 + 16:sb * 32 + 32])
        assert np.all(packed[(row * nsp + 4) * 16:(row * nsp + 5) * 16] == 0)   # the pad sub-block


def test_q3k_relabel_through_the_matvec_oracle():
    """A Q3_K tensor relabelled and repacked gives the matvec its direct decode defines."""
    rng = np.random.default_rng(11)
    in_dim, out_dim = 512, 24
    raw = rng.integers(0, 256, out_dim * (in_dim // 256) * 110, dtype=np.uint8)
    blocks = raw.reshape(-1, 110)
    blocks[:, 108:110] = np.frombuffer(np.array([ro.f32_to_f16(0.01 + 0.001 * i) for i in range(blocks.shape[0])],
                                                dtype=np.uint16).tobytes(), dtype=np.uint8).reshape(-1, 2)
    w = ro.dequantize_src(ro.Q3_K, raw, in_dim * out_dim).reshape(out_dim, in_dim).astype(np.float64)
    x = rng.standard_normal((1, in_dim)).astype(np.float32)
    xq = ro.quantize_q8(x)
    xd = ro.dequantize_q8(xq, in_dim, 1).astype(np.float64)
    _, y64, _ = ro.matvec_q8(ro.Q6_K, ro.repack_any(ro.Q3_K, raw, in_dim, out_dim), xq, in_dim, out_dim, 1)
    assert ro.rel_l2(y64, xd @ w.T) < 1e-6   # the decoded f32 weights carry one rounding the integer form does not


def test_bf16_requantizes_to_q8_0():
    """BF16 -> Q8_0 (qwen35.rs:296-307, q8_0.rs:45-61): d = amax/127 stored as f16, round half away
    from zero, clamp; one step of error at most, zeros stay zeros."""
    rng = np.random.default_rng(12)
    in_dim, out_dim = 64, 5
    f = (rng.standard_normal(in_dim * out_dim) * 0.05).astype(np.float32)
    f[:32] = 0.0
    f[32:64] = 0.0
    f[32] = 127.0 / 256.0             # amax: d = 2^-8, 1/d = 256, all exact in bf16
    f[33] = 0.5 / 256.0               # v / d = 0.5 -> rounds away from zero to 1
    f[34] = -0.5 / 256.0              # -> -1
    f[35] = 2.5 / 256.0               # -> 3 (round-half-even would give 2)
    bf = (f.view(np.uint32) >> 16).astype(np.uint16)
    vals = ro.dequantize_src(ro.BF16, bf.view(np.uint8), f.size)
    q8 = ro.quantize_q8_0(vals).reshape(-1, 34)
    assert np.all(q8[0] == 0)
    assert list(q8[1, 2:6].view(np.int8)) == [127, 1, -1, 3]
    assert (int(q8[1, 0]) | (int(q8[1, 1]) << 8)) == ro.f32_to_f16(1.0 / 256.0)
    deq = ro.dequantize(ro.Q8_0, q8.reshape(-1), f.size)
    d = np.array([ro.f16_to_f32(int(b[0]) | (int(b[1]) << 8)) for b in q8], dtype=np.float32)
    assert np.all(np.abs(deq.reshape(-1, 32) - vals.reshape(-1, 32)) <= 0.51 * np.abs(d)[:, None] + 1e-9)
    assert ro.kernel_type(ro.BF16) == ro.Q8_0
    packed = ro.repack_any(ro.BF16, bf.view(np.uint8), in_dim, out_dim)
    assert np.array_equal(packed, ro.repack(ro.Q8_0, q8.reshape(-1), in_dim, out_dim))


def test_iq3s_kernel_type_is_iq4xs_planes_with_linear_codebook():
    """IQ3_S runs as its own kernel type on the IQ4_XS planes with the codebook 2n - 15
    (src/runtime/qwen35.rs:281-286, src/quant/iq3_s.rs:193-214): same plane sizes as IQ4_XS, the
    integer dots are sum((2n - 15) * xq), and the f32 result is the weights db * (2n - 15) against the
    dequantized activations."""
    import cases
    in_dim, out_dim, rows = 512, 37, 3
    assert ro.kernel_type(ro.IQ3_S) == ro.IQ3_S
    assert ro.repacked_len(ro.IQ3_S, in_dim, out_dim) == ro.repacked_len(ro.IQ4_XS, in_dim, out_dim)
    assert ro.block_bytes(ro.IQ3_S) == 110 and ro.block_weights(ro.IQ3_S) == 256
    planes, w = cases.iq3s_planes(in_dim, out_dim, seed=3)
    assert planes.size == ro.repacked_len(ro.IQ3_S, in_dim, out_dim)
    x = np.random.default_rng(4).standard_normal((rows, in_dim)).astype(np.float32)
    xq = ro.quantize_q8(x)
    y32, y64, idots = ro.matvec_q8(ro.IQ3_S, planes, xq, in_dim, out_dim, rows, want_idots=True)
    recs = xq.reshape(rows, in_dim // 32, 40)
    q = recs[:, :, 8:].view(np.int8).astype(np.int64)                       # [rows, n_sub, 32]
    nib = planes[:out_dim * ro.nsp(in_dim) * 16].reshape(out_dim, ro.nsp(in_dim), 16)[:, :in_dim // 32]
    v = 2 * np.concatenate([nib & 15, nib >> 4], axis=2).astype(np.int64) - 15
    want = np.einsum("osk,rsk->ros", v, q)
    assert np.array_equal(idots.reshape(rows, out_dim, in_dim // 32, 2)[..., 0], want)
    xd = ro.dequantize_q8(xq, in_dim, rows).astype(np.float64)
    assert ro.rel_l2(y64, xd @ w.T) < 1e-6
    assert ro.rel_l2(y32, y64) < 1e-5


def test_q5_1_repack_is_bit_exact_against_dequant():
    """repack_is_bit_exact_against_dequant (q5_1.rs:108-157): in_dim 256 (nsp = 9), 5 rows,
    d = 0.01 * (b + 1), m = -0.1 * (b % 7), the other 20 bytes of every block from the test's LCG;
    reading the planes back the way the kernels do (nibble k low / k + 16 high, qh bit 4g + b,
    dsc = d, deff = -m) reproduces the direct decode bit for bit."""
    in_dim, out_dim, n_sub = 256, 5, 8
    nsp = ro.nsp(in_dim)
    assert nsp == 9
    seed = 0x05100001
    raw = np.empty(out_dim * n_sub * 24, dtype=np.uint8)
    for b in range(out_dim * n_sub):
        o = b * 24
        d = np.float32(0.01) * (np.float32(b) + np.float32(1.0))
        m = np.float32(-0.1) * np.float32(b % 7)
        raw[o:o + 2] = np.frombuffer(np.uint16(ro.f32_to_f16(float(d))).tobytes(), dtype=np.uint8)
        raw[o + 2:o + 4] = np.frombuffer(np.uint16(ro.f32_to_f16(float(m))).tobytes(), dtype=np.uint8)
        raw[o + 4:o + 24], seed = lcg_bytes(seed, 20)
    assert ro.block_bytes(ro.Q5_1) == 24 and ro.block_weights(ro.Q5_1) == 32
    direct = ro.dequantize(ro.Q5_1, raw, in_dim * out_dim).reshape(out_dim, in_dim)
    packed = ro.repack(ro.Q5_1, raw, in_dim, out_dim)
    nib_len, qh_len = out_dim * nsp * 16, out_dim * nsp * 4
    assert packed.size == nib_len + qh_len + out_dim * nsp * 4 == ro.repacked_len(ro.Q5_1, in_dim, out_dim)
    for row in range(out_dim):
        for sb in range(n_sub):
            i = row * nsp + sb
            nib = packed[i * 16:i * 16 + 16]
            qh = int.from_bytes(packed[nib_len + i * 4:nib_len + i * 4 + 4].tobytes(), "little")
            dm = nib_len + qh_len + i * 4
            dsc = np.float32(ro.f16_to_f32(int(packed[dm]) | (int(packed[dm + 1]) << 8)))
            deff = -np.float32(ro.f16_to_f32(int(packed[dm + 2]) | (int(packed[dm + 3]) << 8)))
            for w in range(32):
                g, b = w // 4, w % 4
                byte = int(nib[(g // 2) * 4 + b])
                q5 = ((byte & 15) if g % 2 == 0 else (byte >> 4)) | (((qh >> (4 * g + b)) & 1) << 4)
                widx = (g // 2) * 4 + b if g % 2 == 0 else 16 + (g // 2) * 4 + b
                assert dsc * np.float32(q5) - deff == direct[row, sb * 32 + widx], (row, sb, widx)
        assert np.all(packed[(row * nsp + 8) * 16:(row * nsp + 9) * 16] == 0)   # the pad sub-block


def test_q5_1_matvec_oracle_against_dequantized_weights():
    """The Q5_K body with dsc = d, deff = -m (kernels/moe_matvec_q5k_repacked.cpp:86-101) gives the
    dequantized weights times the dequantized activations: d * q5 . x + m * sum(x)."""
    from reinstinct_b200 import synth
    in_dim, out_dim, rows = 160, 23, 2          # five sub-blocks: not a multiple of 256
    raw = synth.synth_blocks(ro.Q5_1, in_dim, out_dim, seed=51, signed_scales=True)
    x = np.random.default_rng(52).standard_normal((rows, in_dim)).astype(np.float32)
    xq = ro.quantize_q8(x)
    planes = ro.repack(ro.Q5_1, raw, in_dim, out_dim)
    y32, y64, _ = ro.matvec_q8(ro.Q5_1, planes, xq, in_dim, out_dim, rows)
    w = ro.dequantize(ro.Q5_1, raw, in_dim * out_dim).reshape(out_dim, in_dim).astype(np.float64)
    # the kernel's "- deff * xsum" uses the sum of the UNquantized activations of the block
    recs = xq.reshape(rows, in_dim // 32, 40)
    dx = recs[:, :, 0:4].copy().view(np.float32)[..., 0].astype(np.float64)
    xsum = recs[:, :, 4:8].copy().view(np.float32)[..., 0].astype(np.float64)
    q = recs[:, :, 8:].view(np.int8).astype(np.float64)
    blocks = raw.reshape(out_dim, in_dim // 32, 24)
    d = blocks[:, :, 0:2].copy().view(np.float16)[..., 0].astype(np.float64)
    m = blocks[:, :, 2:4].copy().view(np.float16)[..., 0].astype(np.float64)
    q5 = ((w.reshape(out_dim, -1, 32) - m[..., None]) / np.where(d == 0, 1, d)[..., None]).round()
    want = np.einsum("os,rs,osk,rsk->ro", d, dx, q5, q) + np.einsum("os,rs->ro", m, xsum)
    assert ro.rel_l2(y64, want) < 1e-6
    assert ro.rel_l2(y32, y64) < 1e-5
