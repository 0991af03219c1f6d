"""Properties that pin the oracle's int8 path, for which the reference has no CPU code and no
test vector: exact identities against its (pinned) dequantizers, the reference's own
tolerance test against the f32 path, and invariants of the quantizer, sort and router."""
import numpy as np
import pytest

import cases
import oracle as ro


@pytest.mark.parametrize("t", ro.ALL_TYPES)
@pytest.mark.parametrize("in_dim,out_dim", [(256, 5), (512, 3), (1024, 4), (768, 7)])
def test_int8_path_equals_dequantized_dot(t, in_dim, out_dim):
    """With xsum made consistent with the quants (xsum := dx * sum(xq)), the int8-path result
    is, in exact arithmetic, the dot of the dequantized weights with the dequantized
    activations.  IQ4_XS differs by its folded f16 scale (one f16 rounding)."""
    raw, x = cases.synth_case(t, in_dim, out_dim, 2, seed=100 + t)
    xq = ro.quantize_q8(x).reshape(-1, 40).copy()
    d = xq[:, 0:4].copy().view(np.float32).reshape(-1)
    qs = xq[:, 8:40].view(np.int8).astype(np.int32)
    xq[:, 4:8] = (d * qs.sum(axis=1).astype(np.float32)).astype(np.float32).view(np.uint8).reshape(-1, 4)
    w = ro.repack(t, raw, in_dim, out_dim)
    _, y64, _ = ro.matvec_q8(t, w, xq.reshape(-1), in_dim, out_dim, 2)
    wf = ro.dequantize(t, raw, in_dim * out_dim).astype(np.float64).reshape(out_dim, in_dim)
    xhat = ro.dequantize_q8(xq.reshape(-1), in_dim, 2).astype(np.float64)
    want = xhat @ wf.T
    tol = 6e-4 if t == ro.IQ4_XS else 2e-6
    assert ro.rel_l2(y64, want) < tol


@pytest.mark.parametrize("t", ro.ALL_TYPES)
def test_block_integers_match_plain_integer_dots(t):
    """The per-block integers are sum(w_int * xq) with w_int the format's integer weight."""
    in_dim, out_dim = 512, 6
    raw, x = cases.synth_case(t, in_dim, out_dim, 1, seed=7 + t)
    xq = ro.quantize_q8(x)
    qs = xq.reshape(-1, 40)[:, 8:].view(np.int8).astype(np.int64)  # [n_sub, 32]
    w = ro.repack(t, raw, in_dim, out_dim)
    _, _, idots = ro.matvec_q8(t, w, xq, in_dim, out_dim, 1, want_idots=True)
    # integer weights recovered from the f32 dequantizer with unit scales
    unit = raw.copy().reshape(-1, ro.block_bytes(t))
    one = cases.f16b(1.0)
    if t in (ro.Q4_0, ro.Q8_0):
        unit[:, 0:2] = one
        wi = np.rint(ro.dequantize(t, unit.reshape(-1), in_dim * out_dim)).astype(np.int64)
    elif t == ro.Q6_K:
        unit[:, 208:210] = one
        unit[:, 192:208] = 1
        wi = np.rint(ro.dequantize(t, unit.reshape(-1), in_dim * out_dim)).astype(np.int64)
    elif t in (ro.Q4_K, ro.Q5_K):
        unit[:, 0:2] = one
        unit[:, 2:4] = 0
        unit[:, 4:8] = 1   # sc = 1 for sub-blocks 0..3, high bits 0
        unit[:, 8:12] = 0
        unit[:, 12:16] = 1  # sc = 1 for sub-blocks 4..7
        wi = np.rint(ro.dequantize(t, unit.reshape(-1), in_dim * out_dim)).astype(np.int64)
    else:  # IQ4_XS: ls = 33 everywhere -> dl = d
        unit[:, 0:2] = one
        unit[:, 2:4] = np.frombuffer((0xAAAA).to_bytes(2, "little"), dtype=np.uint8)
        unit[:, 4:8] = 0x11
        wi = np.rint(ro.dequantize(t, unit.reshape(-1), in_dim * out_dim)).astype(np.int64)
    wi = wi.reshape(out_dim, in_dim // 32, 32)
    full = np.einsum("rsk,sk->rs", wi, qs)
    if t == ro.Q6_K:
        lo = np.einsum("rsk,sk->rs", wi[:, :, :16], qs[:, :16])
        hi = np.einsum("rsk,sk->rs", wi[:, :, 16:], qs[:, 16:])
        assert np.array_equal(idots[0, :, :, 0], lo) and np.array_equal(idots[0, :, :, 1], hi)
    else:
        assert np.array_equal(idots[0, :, :, 0], full) and not idots[0, :, :, 1].any()


@pytest.mark.parametrize("t,seed,inc", [(ro.Q4_K, 0xD4A40001, 1442695040888963407),
                                        (ro.Q5_K, 0xD5A51234, 1), (ro.Q6_K, 0xD6A65678, 1)])
def test_reference_tolerance_case_2048x384(t, seed, inc):
    """matvec_q4k_repacked_matches_dequant_path (src/runtime/kernels.rs:3021-3118): the
    int8 path within 1.5e-2 rel-L2 of dequant + f32 matvec on the same seeded case."""
    in_dim, out_dim = 2048, 384
    raw = cases.lcg_case(t, in_dim, out_dim, seed, inc)
    x = cases.lcg_x(in_dim, 0x13579BDF)
    want = cases.f32_path(t, raw, x, in_dim, out_dim)[0]
    y32, y64, _ = ro.matvec_q8(t, ro.repack(t, raw, in_dim, out_dim), ro.quantize_q8(x), in_dim, out_dim)
    e = ro.rel_l2(y32[0], want)
    assert e < 1.5e-2, e
    assert ro.rel_l2(y32, y64) < 1e-5


def test_quantize_q8_definition():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 256)).astype(np.float32)
    x[0, 32:64] = 0.0            # an all-zero block
    x[1, 0] = 1e30               # a huge value
    x[2, 64:96] = 0.5            # ties: 0.5 * 127 / 0.5 = 127 exactly
    blk = ro.quantize_q8(x).reshape(3, 8, 40)
    d = blk[:, :, 0:4].copy().view(np.float32).reshape(3, 8)
    xsum = blk[:, :, 4:8].copy().view(np.float32).reshape(3, 8)
    q = blk[:, :, 8:].view(np.int8)
    xb = x.reshape(3, 8, 32)
    amax = np.abs(xb).max(axis=2)
    assert np.array_equal(d, np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32))
    assert d[0, 1] == 1.0 and not q[0, 1].any() and xsum[0, 1] == 0.0
    assert np.abs(q.astype(np.int32)).max() <= 127
    with np.errstate(divide="ignore"):
        inv = np.where(amax > 0, np.float32(127.0) / amax, np.float32(0.0)).astype(np.float32)
    want = np.clip(np.rint(xb * inv[:, :, None]), -127, 127).astype(np.int8)
    assert np.array_equal(q, want)
    # xsum is the 16,8,4,2,1 xor-butterfly sum in f32
    s = xb.copy()
    for off in (16, 8, 4, 2, 1):
        s = s + s[:, :, np.arange(32) ^ off]
    assert np.array_equal(xsum, s[:, :, 0])


def test_round_half_even_in_quantizer():
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, 0] = 127.0   # amax = 127 -> inv = 1 exactly
    x[0, 1:5] = [0.5, 1.5, 2.5, -0.5]
    q = ro.quantize_q8(x).reshape(-1, 40)[0, 8:].view(np.int8)
    assert list(q[:5]) == [127, 0, 2, 2, 0]


@pytest.mark.parametrize("n_entries,n_expert,bn", [(0, 4, 16), (1, 1, 16), (4096, 256, 16), (777, 60, 32), (100, 128, 64)])
def test_moe_sort_invariants(n_entries, n_expert, bn):
    """verify_moe_sort (src/runtime/qwen35.rs:2943-2995)."""
    rng = np.random.default_rng(n_entries + n_expert)
    ids = rng.integers(0, n_expert, n_entries, dtype=np.int32)
    if n_entries > 10:
        ids[3] = -1
        ids[7] = n_expert  # out-of-range ids are dropped
    count, eoff, toff, perm = ro.moe_sort(ids, n_expert, bn)
    valid = (ids >= 0) & (ids < n_expert)
    assert np.array_equal(count, np.bincount(ids[valid], minlength=n_expert))
    assert np.array_equal(eoff, np.concatenate([[0], np.cumsum(count)]))
    assert np.array_equal(toff, np.concatenate([[0], np.cumsum((count + bn - 1) // bn)]))
    total = int(eoff[-1])
    assert sorted(perm[:total].tolist()) == np.nonzero(valid)[0].tolist()
    for e in range(n_expert):
        seg = perm[eoff[e]:eoff[e + 1]]
        assert np.all(ids[seg] == e) and np.all(np.diff(seg) > 0)


def test_router_topk():
    rng = np.random.default_rng(5)
    logits = rng.standard_normal((16, 256)).astype(np.float32)
    ids, wts = ro.router_topk(logits, 8)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    want = np.argsort(-p, axis=1, kind="stable")[:, :8]
    assert np.array_equal(ids, want)
    assert np.allclose(wts.sum(axis=1), 1.0, atol=1e-5)
    assert np.allclose(wts, np.take_along_axis(p, want, 1) / np.take_along_axis(p, want, 1).sum(1, keepdims=True), rtol=1e-4)


def test_shapes_rejected():
    assert ro.repacked_len(ro.Q4_K, 96, 4) == 0 and ro.repacked_len(99, 256, 4) == 0
    # Appendix sizes of the benchmark configurations
    assert ro.repacked_len(ro.Q8_0, 4096, 4096) == 17965056
    assert ro.repacked_len(ro.Q4_K, 5120, 17408) == 51527680
    assert ro.repacked_len(ro.Q6_K, 17408, 5120) == 73113600
    assert ro.repacked_len(ro.Q4_K, 2048, 1024) == 1230848
    assert ro.repacked_len(ro.Q6_K, 512, 2048) == 913408


def test_moe_act_q8_is_quantizer_of_activation():
    """ro_moe_act_q8 = gated activation in f32, then the ro_quantize_q8 record stream; both
    activations against f64 formulas (kernels/moe_geglu_q8.cpp:20-32, kernels/swiglu.cpp:11-21)."""
    rng = np.random.default_rng(3)
    ff, n_slot = 256, 5
    gu = (rng.standard_normal((n_slot, 2 * ff)) * 2).astype(np.float32)
    g, u = gu[:, :ff].astype(np.float64), gu[:, ff:].astype(np.float64)
    for act, a64 in ((0, 0.5 * g * (1 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))),
                     (1, g / (1 + np.exp(-g)))):
        q, v = ro.moe_act_q8(gu, act)
        # 1 + tanh cancels for negative gates: the error scales with |gate * up|, not the result
        assert np.all(np.abs(v - a64 * u) <= 2e-6 * np.abs(a64 * u) + 1.5e-7 * np.abs(g * u))
        np.testing.assert_array_equal(q.reshape(-1), ro.quantize_q8(v).reshape(-1))


def test_moe_combine_weighted_sum():
    rng = np.random.default_rng(4)
    n_tok, n_used, hidden, n_expert = 3, 4, 40, 16
    ex = rng.standard_normal((n_tok, n_used, hidden)).astype(np.float32)
    ids = rng.integers(0, n_expert, (n_tok, n_used)).astype(np.int32)
    w = rng.random((n_tok, n_used)).astype(np.float32)
    sc = (rng.random(n_expert) + 0.5).astype(np.float32)
    out = ro.moe_combine(ex, ids, w, sc)
    ref = np.einsum("tj,tjh->th", w.astype(np.float64) * sc[ids], ex.astype(np.float64))
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-6)
    ones = ro.moe_combine(ex, ids, w, np.ones(n_expert, dtype=np.float32))
    np.testing.assert_array_equal(ro.moe_combine(ex, ids, w, None), ones)
    # one slot with weight 1 and scale 1 returns that expert's row unchanged
    np.testing.assert_array_equal(ro.moe_combine(ex[:, :1], ids[:, :1], np.ones((n_tok, 1), np.float32), None), ex[:, 0])


def test_rmsnorm_q8_is_norm_then_quantizer():
    """ro_rmsnorm_q8 = (x + add) * rsqrt(mean + eps) * w in f32 (against f64), then the ro_quantize_q8
    record stream of exactly those values (kernels/rmsnorm_q8.cpp:38-103, qwen35_fused.cpp:66-118)."""
    rng = np.random.default_rng(21)
    for n, n_vec in ((2048, 3), (5120, 1), (96, 2)):
        x = rng.standard_normal((n_vec, n)).astype(np.float32) * 3
        add = rng.standard_normal((n_vec, n)).astype(np.float32)
        w = (rng.random(n) + 0.5).astype(np.float32)
        for a in (None, add):
            hid, y, q = ro.rmsnorm_q8(x, w, 1e-6, a)
            h64 = x.astype(np.float64) + (0 if a is None else a.astype(np.float64))
            np.testing.assert_array_equal(hid, x if a is None else x + a)
            ref = h64 / np.sqrt((h64 ** 2).mean(1, keepdims=True) + 1e-6) * w
            np.testing.assert_allclose(y, ref, rtol=3e-6, atol=1e-7)
            np.testing.assert_array_equal(q, ro.quantize_q8(y))


def test_swiglu_q8_is_activation_then_quantizer():
    rng = np.random.default_rng(22)
    g = (rng.standard_normal(4096) * 3).astype(np.float32)
    u = rng.standard_normal(4096).astype(np.float32)
    v, q = ro.swiglu_q8(g, u)
    g64 = g.astype(np.float64)
    np.testing.assert_allclose(v, g64 / (1 + np.exp(-g64)) * u, rtol=3e-6, atol=1e-7)
    np.testing.assert_array_equal(q, ro.quantize_q8(v.reshape(1, -1)))
