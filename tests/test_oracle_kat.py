"""Pins the CPU oracle: (1) the known-answer vectors the reference's own tests hold for this
path, (2) hand-built single-block quant vectors derived from the format definition,
(3) an independent numpy statement of the block formats on random data.

Reference KAT sources (values retyped from the expectations in those tests):
  crates/tl_cuda/tests/nn_llm_test.rs:123-132,136-147,151-169,173-213,239-289
  crates/tl_cuda/tests/matmul_special_test.rs:17-70
  crates/tl_cuda/tests/new_ops_comprehensive_test.rs:537-616,635-683
  crates/tl_cpu/tests/cpu_tensor_tests.rs:328-340,400-460,488-506
"""
import math
import struct

import numpy as np
import pytest

import npref
from tl_b200 import synth


def h16(x):
    return np.array([x], dtype=np.float16).view(np.uint8).tolist()


def test_rms_norm_kat(orc):
    rms = math.sqrt(14.0 / 3.0)
    r = orc.rms_norm(np.array([[1.0, 2.0, 3.0]]), None, 1e-5)
    np.testing.assert_allclose(r[0], [1 / rms, 2 / rms, 3 / rms], atol=1e-4)
    r = orc.rms_norm(np.array([[1.0, 2.0, 3.0]]), np.array([2.0, 3.0, 0.5]), 1e-5)
    np.testing.assert_allclose(r[0], [2 / rms, 6 / rms, 1.5 / rms], atol=1e-4)
    rms4 = math.sqrt(30.0 / 4.0)
    r = orc.rms_norm(np.array([[1.0, 2.0, 3.0, 4.0]]), np.ones(4), 1e-5)
    np.testing.assert_allclose(r[0], [(i + 1) / rms4 for i in range(4)], atol=1e-3)
    # fused_add_rms_norm KAT: x + residual = [2, 2] -> [1, 1]
    s = orc.add(np.array([1.0, 2.0]), np.array([1.0, 0.0]))
    np.testing.assert_allclose(orc.rms_norm(s[None], np.ones(2), 1e-5)[0], [1.0, 1.0], atol=1e-3)


def test_causal_mask_kat(orc):
    m = orc.causal_mask(3).reshape(-1)
    assert m[0] == 0 and m[3] == 0 and m[4] == 0
    assert np.isneginf(m[1]) and np.isneginf(m[5])


def test_rope_tables_kat(orc):
    c, s = orc.rope_table_half(4, 8, 10000.0)
    assert c.shape == (4, 4)
    np.testing.assert_allclose(c[0], 1.0, atol=1e-5)
    np.testing.assert_allclose(s[0], 0.0, atol=1e-5)
    c2, s2 = orc.rope_table_cpu(4, 8, 10000.0)
    assert c2.shape == (4, 8)
    np.testing.assert_array_equal(c2[:, 0::2], c)  # pair-duplicated layout of the CPU backend
    np.testing.assert_array_equal(c2[:, 1::2], c)
    np.testing.assert_array_equal(s2[:, 0::2], s)
    # values: cos(pos * base^(-2i/dim)) in f32
    f = np.float32(1.0) / np.float32(10000.0) ** (np.float32(2.0) * np.float32(1) / np.float32(8))
    assert abs(c[3, 1] - math.cos(3 * float(f))) < 1e-6


def test_rope_per_position_kat(orc):
    c, s = orc.rope_table_half(4, 4, 10000.0)
    x = np.ones((2, 1, 4), dtype=np.float32)
    r = orc.apply_rope_rotate_half(x, c[:2], s[:2])
    np.testing.assert_allclose(r[0, 0], 1.0, atol=1e-5)  # position 0 unchanged
    assert np.abs(r[0, 0] - r[1, 0]).sum() > 1e-5        # position 1 differs
    # CPU convention: row 0 of the (narrowed) table rotates every vector, adjacent pairs
    c2, s2 = orc.rope_table_cpu(4, 4, 10000.0)
    xx = np.arange(8, dtype=np.float32).reshape(2, 4) + 1
    rc = orc.apply_rope_cpu(xx, c2[1:3], s2[1:3])
    for v in range(2):
        for i in (0, 2):
            cc, ss = c2[1, i], s2[1, i]
            assert rc[v, i] == np.float32(xx[v, i] * cc) - np.float32(xx[v, i + 1] * ss)
            assert rc[v, i + 1] == np.float32(xx[v, i] * ss) + np.float32(xx[v, i + 1] * cc)


def test_matmul_kat(orc):
    np.testing.assert_allclose(orc.matmul(np.array([[1, 2], [3, 4.0]]), np.array([[5, 6], [7, 8.0]])),
                               [[19, 22], [43, 50]], atol=1e-4)
    np.testing.assert_allclose(orc.matmul(np.array([[1, 2, 3], [4, 5, 6.0]]),
                                          np.array([[7, 8], [9, 10], [11, 12.0]])),
                               [[58, 64], [139, 154]], atol=1e-4)


def test_softmax_embedding_argmax_kat(orc):
    s = orc.softmax(np.array([[1.0, 2.0, 3.0]]), -1)[0]
    assert abs(s.sum() - 1.0) < 1e-5 and s[0] < s[1] < s[2]
    e = orc.embedding(np.array([[10, 20], [30, 40], [50, 60.0]]), np.array([0.0, 2.0]))
    np.testing.assert_array_equal(e, [[10, 20], [50, 60]])
    with pytest.raises(IndexError):
        orc.embedding(np.ones((3, 2)), np.array([3.0]))
    assert orc.argmax_last(np.array([1.0, 5.0, 3.0, 2.0])) == 1
    assert orc.argmax_last(np.array([1.0, 5.0, 2.0, 3.0, 4.0])) == 1      # top-k(1) KAT
    assert orc.argmax_last(np.array([1.0, 100.0, 2.0])) == 1               # top-p KAT
    # tie rules: tl_cpu keeps the last maximum, the CUDA kernel the first
    assert orc.argmax_last(np.array([7.0, 1.0, 7.0])) == 2
    assert orc.argmax_first(np.array([7.0, 1.0, 7.0])) == 0


def test_shape_ops_kat(orc):
    np.testing.assert_array_equal(orc.repeat_interleave(np.array([1.0, 2.0, 3.0]), 2, 0),
                                  [1, 1, 2, 2, 3, 3])


def test_repetition_penalty_and_silu_kat(orc):
    r = orc.repetition_penalty(np.array([1.0, 2, 3, 4, 5]), np.array([1.0, 3.0]), 2.0)
    np.testing.assert_allclose(r, [1, 1, 3, 2, 5], atol=1e-4)
    r = orc.repetition_penalty(np.array([-1.0, 2.0]), np.array([0.0, 0.0]), 2.0)
    np.testing.assert_allclose(r, [-2.0, 2.0])
    v = orc.mul(orc.silu(np.array([0.0, 1.0, -1.0, 2.0])), np.ones(4))
    assert abs(v[0]) < 1e-5 and abs(v[1] - 0.7311) < 1e-3


def test_sdpa_kat(orc):
    q = np.array([[[1.0, 0, 0, 0], [0, 1, 0, 0]]])
    v = np.arange(1, 9, dtype=np.float32).reshape(1, 2, 4)
    o = orc.sdpa_cpu(q, q, v)
    assert np.isfinite(o).all()
    p = np.exp([0.5, 0.0])
    p /= p.sum()
    np.testing.assert_allclose(o[0, 0], p[0] * v[0, 0] + p[1] * v[0, 1], rtol=1e-6)


# ---------------------------------------------------------------- hand-built quant blocks

def test_f16_widening_exact(orc):
    L = orc.lib()
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = orc.dequantize(synth.F16, allh.view(np.uint8), 65536)  # all 65536 bit patterns
    nan = np.isnan(ref)
    np.testing.assert_array_equal(got.view(np.uint32)[~nan], ref.view(np.uint32)[~nan])
    assert np.isnan(got[nan]).all()
    vals = np.concatenate([np.random.default_rng(1).standard_normal(4000).astype(np.float32) * 100,
                           np.array([0, -0.0, 65504, 65519.99, 65520, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5, np.inf],
                                    dtype=np.float32)])
    got = np.array([L.orc_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    np.testing.assert_array_equal(got, vals.astype(np.float16).view(np.uint16))


def test_q4_0_handbuilt(orc):
    blk = h16(0.5) + [(j & 15) | (((15 - j) & 15) << 4) for j in range(16)]
    w = orc.dequantize(synth.Q4_0, np.array(blk, dtype=np.uint8), 32)
    np.testing.assert_array_equal(w[:16], [0.5 * (j - 8) for j in range(16)])
    np.testing.assert_array_equal(w[16:], [0.5 * (15 - j - 8) for j in range(16)])


def test_q8_0_handbuilt(orc):
    q = [(-127 + 8 * j) for j in range(32)]
    blk = h16(0.25) + [x & 0xFF for x in q]
    w = orc.dequantize(synth.Q8_0, np.array(blk, dtype=np.uint8), 32)
    np.testing.assert_array_equal(w, [0.25 * x for x in q])


def test_q4_k_handbuilt(orc):
    # d = 1.0 (0x3C00), dmin = 0.5; scales/mins exercise the j>=4 split-bit case; ramp nibbles
    sc = [1, 2, 3, 63, 17, 33, 48, 62]
    mn = [0, 5, 10, 15, 16, 32, 47, 63]
    packed = npref.pack_q4k_scales(sc, mn)
    assert npref.q4k_scales(packed) == (sc, mn)
    qs = [((l % 16)) | (((l * 3) % 16) << 4) for l in range(128)]
    blk = [0x00, 0x3C] + h16(0.5) + packed + qs
    assert len(blk) == 144
    w = orc.dequantize(synth.Q4_K, np.array(blk, dtype=np.uint8), 256)
    for g in range(4):
        for l in range(32):
            b = qs[32 * g + l]
            assert w[64 * g + l] == sc[2 * g] * (b & 15) - 0.5 * mn[2 * g]
            assert w[64 * g + 32 + l] == sc[2 * g + 1] * (b >> 4) - 0.5 * mn[2 * g + 1]


def test_q6_k_handbuilt(orc):
    rng = np.random.default_rng(5)
    ql = rng.integers(0, 256, 128, dtype=np.uint8).tolist()
    qh = rng.integers(0, 256, 64, dtype=np.uint8).tolist()
    sc = list(range(-8, 8))
    blk = ql + qh + [s & 0xFF for s in sc] + h16(2.0)
    assert len(blk) == 210
    w = orc.dequantize(synth.Q6_K, np.array(blk, dtype=np.uint8), 256)
    # element (chunk 1, l = 20, third quarter): low nibble source ql[64+20] >> 4, high bits qh[32+20] >> 4
    l, c = 20, 1
    q = ((ql[64 * c + l] >> 4) | (((qh[32 * c + l] >> 4) & 3) << 4)) - 32
    assert w[128 * c + l + 64] == 2.0 * sc[8 * c + l // 16 + 4] * q
    np.testing.assert_array_equal(w, npref.deq_q6_k(blk))


@pytest.mark.parametrize("t", [synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K])
def test_dequant_matches_independent_numpy(orc, t):
    rng = np.random.default_rng(100 + t)
    w = synth.random_quant(t, 8, 1024, rng).reshape(-1)
    a = orc.dequantize(t, w, 8 * 1024)
    b = npref.DEQ[t](w)
    np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32))


def test_dequant_rejects_bad_sizes(orc):
    with pytest.raises(ValueError):
        orc.dequantize(synth.Q4_K, np.zeros(143, dtype=np.uint8), 256)
    with pytest.raises(ValueError):
        orc.dequantize(synth.Q4_0, np.zeros(18, dtype=np.uint8), 31)
    assert orc.dequantize(synth.Q4_K, np.zeros(0, dtype=np.uint8), 0).size == 0  # empty input


def test_qmatmul_equals_dequant_transpose_matmul(orc):
    # system.rs:193-222: dequantize -> transpose_2d -> matmul; the streaming form must be bit-identical
    rng = np.random.default_rng(3)
    n, k, m = 48, 512, 3
    for t in (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K):
        w = synth.random_quant(t, n, k, rng)
        x = rng.standard_normal((m, k), dtype=np.float32)
        wf = orc.dequantize(t, w.reshape(-1), n * k).reshape(n, k)
        ref = orc.matmul(x, np.ascontiguousarray(wf.T))
        got = orc.qmatmul(t, w.reshape(-1), n, k, x)
        np.testing.assert_array_equal(ref.view(np.uint32), got.view(np.uint32))


def test_llama_driver_matches_op_by_op(orc):
    """The fused driver equals the same forward pass issued op by op through the oracle's
    primitive functions in the TL program's order (chatbot_llama3.tl:66-125)."""
    cfg = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=320,
               eps=1e-5, rope_base=10000.0, attn_scale=0.125)
    tens = synth.llama_tensors(cfg, 7, synth.Q4_K, synth.Q6_K)
    model = orc.Llama(dict(cfg, kv_f16=0, max_seq=16), {k: (t, d) for k, (t, d, s) in tens.items()})
    toks = [5, 17, 300]
    logits = model.forward(toks, 0)
    step = model.forward([9], 3)

    def W(name):
        t, d, shp = tens[name]
        return orc.dequantize(t, d, int(np.prod(shp))).reshape(shp)
    cos, sin = orc.rope_table_cpu(16, 64, 10000.0)

    def run(x, sp, kc, vc):
        sl = x.shape[0]
        for li in range(2):
            p = "blk.%d." % li
            h = orc.rms_norm(x, W(p + "attn_norm.weight"), 1e-5)
            q = orc.matmul(h, np.ascontiguousarray(W(p + "attn_q.weight").T)).reshape(1, sl, 4, 64)
            k = orc.matmul(h, np.ascontiguousarray(W(p + "attn_k.weight").T)).reshape(1, sl, 2, 64)
            v = orc.matmul(h, np.ascontiguousarray(W(p + "attn_v.weight").T)).reshape(1, sl, 2, 64)
            q = orc.apply_rope_cpu(q, cos[sp:sp + sl], sin[sp:sp + sl])
            k = orc.apply_rope_cpu(k, cos[sp:sp + sl], sin[sp:sp + sl])
            kt, vt = k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3)
            if sp:
                kt = np.concatenate([kc[li], kt], axis=2)
                vt = np.concatenate([vc[li], vt], axis=2)
            kc[li], vc[li] = kt, vt
            kw = orc.repeat_interleave(kt, 2, 1)
            vw = orc.repeat_interleave(vt, 2, 1)
            mm = orc.matmul(np.ascontiguousarray(q.transpose(0, 2, 1, 3)),
                            np.ascontiguousarray(kw.transpose(0, 1, 3, 2)))
            sc = orc.scale(mm, 0.125)
            if sl > 1:
                sc = orc.add(sc, np.broadcast_to(orc.causal_mask(sl), sc.shape))
            pr = orc.softmax(sc, 3)
            ao = orc.matmul(pr, vw).transpose(0, 2, 1, 3).reshape(sl, 256)
            x = orc.add(x, orc.matmul(ao, np.ascontiguousarray(W(p + "attn_output.weight").T)))
            h = orc.rms_norm(x, W(p + "ffn_norm.weight"), 1e-5)
            g = orc.silu(orc.matmul(h, np.ascontiguousarray(W(p + "ffn_gate.weight").T)))
            u = orc.matmul(h, np.ascontiguousarray(W(p + "ffn_up.weight").T))
            x = orc.add(x, orc.matmul(orc.mul(g, u), np.ascontiguousarray(W(p + "ffn_down.weight").T)))
        h = orc.rms_norm(x, W("output_norm.weight"), 1e-5)
        return orc.matmul(h, np.ascontiguousarray(W("output.weight").T))[-1]

    kc, vc = {}, {}
    emb = W("token_embd.weight")
    ref = run(orc.embedding(emb, np.array(toks, dtype=np.float32)), 0, kc, vc)
    np.testing.assert_array_equal(ref.view(np.uint32), logits.view(np.uint32))
    ref2 = run(orc.embedding(emb, np.array([9.0])), 3, kc, vc)
    np.testing.assert_array_equal(ref2.view(np.uint32), step.view(np.uint32))
    model.close()


def test_sample_top_p_restatement(orc):
    """sample_impl (crates/tl_cpu/src/tensor.rs:1625-1680) with the random number passed in.  The reference's own
    sampler test only pins the dominated case (one logit far above the rest returns that token, whatever is drawn)."""
    dominated = np.array([1.0, 100.0, 2.0], dtype=np.float32)
    for u in (0.0, 0.3, 0.999):
        assert orc.sample_top_p(dominated, 1.0, 0.9, u) == 1
    # temp <= 0: greedy branch, last maximum
    assert orc.sample_top_p(np.array([7.0, 1.0, 7.0], dtype=np.float32), 0.0, 0.9, 0.5) == 2
    # equal probabilities keep index order in the stable descending sort; the draw walks that order
    x = np.array([0.1, 2.0, 2.0, -1.0, 0.5], dtype=np.float32)
    p = np.exp(x - x.max()); p /= p.sum()
    order = [1, 2, 4, 0, 3]
    cum = np.cumsum(p[order])
    cutoff = int(np.argmax(cum > 0.9))            # first running sum above top_p
    for u in (0.0, 0.2, 0.45, 0.7, 0.95, 0.999):
        r = u * cum[cutoff]
        want = order[int(np.argmax(cum[:cutoff + 1] >= r))]
        assert orc.sample_top_p(x, 1.0, 0.9, u) == want
    # top_p = 1.0: the running sum never exceeds it, every token stays
    assert orc.sample_top_p(x, 1.0, 1.0, 0.9999) in (0, 3)


def test_extra_block_types_hand_built(orc):
    """Q4_1 / Q5_0 / Q5_1 / Q8_1 (no dequantiser in the reference, crates/tl_runtime/src/quantized.rs:108): single blocks
    with d = 2.0, m = 0.5 and ramp quants, worked out by hand from the published block definitions."""
    from tl_b200 import synth
    h = lambda v: np.array([v], dtype=np.float16).view(np.uint8)
    nib = np.array([(j & 15) | (((15 - j) & 15) << 4) for j in range(16)], dtype=np.uint8)   # low nibble j, high nibble 15 - j
    lo, hi = np.arange(16), 15 - np.arange(16)
    q41 = np.concatenate([h(2.0), h(0.5), nib])
    np.testing.assert_array_equal(orc.dequantize(synth.Q4_1, q41, 32), np.concatenate([2.0 * lo + 0.5, 2.0 * hi + 0.5]).astype(np.float32))
    qh = np.array([0x0000FFFF], dtype=np.uint32).view(np.uint8)                              # fifth bit set for the first 16 weights only
    q50 = np.concatenate([h(2.0), qh, nib])
    np.testing.assert_array_equal(orc.dequantize(synth.Q5_0, q50, 32), np.concatenate([2.0 * (lo + 16 - 16), 2.0 * (hi - 16)]).astype(np.float32))
    q51 = np.concatenate([h(2.0), h(0.5), qh, nib])
    np.testing.assert_array_equal(orc.dequantize(synth.Q5_1, q51, 32), np.concatenate([2.0 * (lo + 16) + 0.5, 2.0 * hi + 0.5]).astype(np.float32))
    q = np.arange(-16, 16, dtype=np.int8)
    q81 = np.concatenate([h(2.0), h(123.0), q.view(np.uint8)])
    np.testing.assert_array_equal(orc.dequantize(synth.Q8_1, q81, 32), (2.0 * q).astype(np.float32))
    assert orc.type_nbytes(synth.Q4_1, 64) == 40 and orc.type_nbytes(synth.Q5_0, 64) == 44
    assert orc.type_nbytes(synth.Q5_1, 64) == 48 and orc.type_nbytes(synth.Q8_1, 64) == 72 and orc.type_nbytes(synth.Q5_0, 48) == 0


def test_philox_known_answers(orc):
    """Philox-4x32-10 against the three known-answer vectors published with the algorithm (all-zero, all-ones and the
    digits-of-pi counter / key), and the library's host helper against the oracle's."""
    assert orc.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert orc.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert orc.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    import tl_b200 as tl
    for seed, ctr in ((0, 0), (7, 1), (2 ** 63 + 5, 2 ** 40 + 3)):
        u = orc.rng_uniform(seed, ctr)
        assert 0.0 <= u < 1.0 and u == tl.rng_uniform(seed, ctr)
    x = np.array([0.1, 2.0, 1.5, -1.0, 1.9], dtype=np.float32)
    assert orc.sample_top_k_top_p(x, 1.0, 0, 1.0, 0.999) == 3                   # no limits: the tail token is reachable
    assert orc.sample_top_k_top_p(x, 1.0, 2, 1.0, 0.999) == 4                   # two best tokens only: 1 (2.0) and 4 (1.9)
    assert orc.sample_top_k_top_p(x, 1.0, 2, 1.0, 0.0) == 1
    assert orc.sample_top_k_top_p(x, 1.0, 0, 1.0, 0.3) == orc.sample_top_p(x, 1.0, 1.0, 0.3)
