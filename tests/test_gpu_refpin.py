"""Pins the oracle on outputs of the reference itself: the reference's own CUDA kernels
(crates/tl_cuda/src/cuda_kernels/autograd.cu, compiled unmodified into oracle/_ref/libtlref.so) run on the
same seeded inputs as the oracle's restatement and as libtlb200.

What this pins that no test of the reference holds: the Q4_K and Q6_K bit layouts (every weight of a
tensor extracted through the reference's fused kernel with one-hot activations), the quantized matvec,
RMSNorm and its fused forms, rotate-half RoPE, softmax, argmax ties, attention, and the small glue ops.
The reference kernels are compiled with nvcc's default FMA contraction, so agreement with the FMA-free
oracle is to one rounding of an intermediate (tolerances below), not to the bit, except where no
contraction is possible.
"""
import numpy as np
import pytest

import tl_b200 as tl
from oracle import ref_cuda
from tl_b200 import synth

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libtlref.so not built (needs the TL checkout)")]
T = tl.Tensor.from_numpy
EPS32 = float(np.finfo(np.float32).eps)


def _f16_field(raw, block_bytes, off):
    return raw.reshape(-1, block_bytes)[:, off:off + 2].copy().view(np.float16).astype(np.float32).reshape(-1)


@pytest.mark.parametrize("n,k,seed", [(48, 256, 1), (16, 1024, 2)])
def test_q4k_bit_layout_through_reference_kernel(orc, n, k, seed):
    """Row j of an identity activation makes mul_mv_q4_k_kernel return column j of the dequantised weight:
    out[j][row] = 1 * (d*sc*q - dmin*m) + zeros.  Against the oracle's dequantize_q4_k and against
    tlb_qtensor_dequantize, to one rounding of the largest intermediate |d|*63*15 + |dmin|*63."""
    raw = synth.random_quant(synth.Q4_K, n, k, np.random.default_rng(seed)).reshape(-1)
    got = ref_cuda.mul_mv(synth.Q4_K, raw, n, k, np.eye(k, dtype=np.float32)).T          # [n, k]
    want = orc.dequantize(synth.Q4_K, raw, n * k).reshape(n, k)
    d, dmin = np.abs(_f16_field(raw, 144, 0)), np.abs(_f16_field(raw, 144, 2))
    bound = np.repeat((d * 63 * 15 + dmin * 63).reshape(n, k // 256), 256, axis=1) * EPS32
    assert np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) / np.maximum(bound, 1e-30)))
    assert np.mean(got == want) > 0.5        # most weights come out bit-identical even with contraction
    mine = tl.QTensor.from_gguf_bytes(synth.Q4_K, n, k, raw).dequantize().numpy()
    np.testing.assert_array_equal(mine.view(np.uint32), want.view(np.uint32))
    assert np.all(np.abs(got - mine) <= bound)


@pytest.mark.parametrize("n,k,seed", [(48, 256, 3), (16, 1024, 4)])
def test_q6k_bit_layout_through_reference_kernel(orc, n, k, seed):
    """Same for Q6_K.  With a one-hot activation the kernel evaluates (1 * (d*sc)) * q + 0: the same two
    roundings as dequantize_q6_k, so every non-zero weight compares bit for bit (a weight of -0.0, from a quant of 32
    under a negative scale, comes out of the kernel's running sum as +0.0)."""
    raw = synth.random_quant(synth.Q6_K, n, k, np.random.default_rng(seed)).reshape(-1)
    got = ref_cuda.mul_mv(synth.Q6_K, raw, n, k, np.eye(k, dtype=np.float32)).T
    want = orc.dequantize(synth.Q6_K, raw, n * k).reshape(n, k)
    np.testing.assert_array_equal(got, want)
    nz = want != 0
    assert nz.mean() > 0.9
    np.testing.assert_array_equal(got[nz].view(np.uint32), want[nz].view(np.uint32))
    mine = tl.QTensor.from_gguf_bytes(synth.Q6_K, n, k, raw).dequantize().numpy()
    np.testing.assert_array_equal(mine.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("t", [synth.Q4_K, synth.Q6_K])
@pytest.mark.parametrize("n,k,m", [(64, 1024, 1), (48, 2048, 3), (256, 512, 4)])
def test_quantized_matvec_reference_kernel_vs_oracle_vs_library(orc, t, n, k, m):
    rng = np.random.default_rng(n + k + m + t)
    raw = synth.random_quant(t, n, k, rng).reshape(-1)
    x = rng.standard_normal((m, k), dtype=np.float32)
    ref = ref_cuda.mul_mv(t, raw, n, k, x)
    want = orc.qmatmul(t, raw, n, k, x)
    scale = float(np.max(np.abs(want)))
    assert np.max(np.abs(ref - want)) <= 1e-5 * scale          # same summation order; only FMA contraction differs
    mine = T(x).matmul_quantized(tl.QTensor.from_gguf_bytes(t, n, k, raw)).numpy()
    assert np.max(np.abs(mine - ref)) <= 1e-4 * scale          # the library against the reference's own kernel


def test_rms_norm_family(orc):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((5, 2048), dtype=np.float32) * 3
    r = rng.standard_normal((5, 2048), dtype=np.float32)
    w = rng.standard_normal(2048, dtype=np.float32)
    a = ref_cuda.rms_norm(x, 1e-5)                       # x * rsqrtf(mean + eps); the oracle divides by sqrtf
    np.testing.assert_allclose(a, orc.rms_norm(x, None, 1e-5), rtol=4e-6, atol=0)
    np.testing.assert_allclose(T(x).rms_norm(None, 1e-5).numpy(), a, rtol=4e-6, atol=0)
    b = ref_cuda.fused_rms_norm(x, w, 1e-5)
    np.testing.assert_allclose(b, orc.rms_norm(x, w, 1e-5), rtol=4e-6, atol=1e-30)
    np.testing.assert_allclose(T(x).fused_rms_norm(T(w), 1e-5).numpy(), b, rtol=4e-6, atol=1e-30)
    c = ref_cuda.fused_add_rms_norm(x, r, w, 1e-5)
    np.testing.assert_allclose(c, orc.rms_norm(orc.add(x, r), w, 1e-5), rtol=4e-6, atol=1e-30)
    np.testing.assert_allclose(T(x).fused_add_rms_norm(T(r), T(w), 1e-5).numpy(), c, rtol=4e-6, atol=1e-30)


@pytest.mark.parametrize("dim,base", [(64, 10000.0), (128, 500000.0)])
def test_rotate_half_rope(orc, dim, base):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((9, 6, dim), dtype=np.float32)
    cos_t, sin_t = orc.rope_table_half(16, dim, base)
    a = ref_cuda.apply_rope(x, cos_t, sin_t)
    np.testing.assert_allclose(a, orc.apply_rope_rotate_half(x, cos_t, sin_t), rtol=0, atol=4 * EPS32 * float(np.max(np.abs(x))))
    ct = tl.Tensor.rope_new_cos(dim, 16, base, tl.ROPE_HALF)
    st = tl.Tensor.rope_new_sin(dim, 16, base, tl.ROPE_HALF)
    np.testing.assert_array_equal(ct.numpy(), cos_t)          # host libm tables, as both back ends build them
    np.testing.assert_array_equal(st.numpy(), sin_t)
    mine = T(x).apply_rope(ct, st, tl.ROPE_HALF).numpy()
    np.testing.assert_allclose(mine, a, rtol=0, atol=4 * EPS32 * float(np.max(np.abs(x))))


def test_softmax_argmax_and_glue_ops(orc):
    rng = np.random.default_rng(7)
    s = rng.standard_normal((3, 4, 5, 77), dtype=np.float32) * 4
    for axis in (3, 1):
        a = ref_cuda.softmax(s, axis)
        np.testing.assert_allclose(a, orc.softmax(s, axis), rtol=2e-6, atol=1e-9)
        np.testing.assert_allclose(T(s).softmax(axis).numpy(), a, rtol=4e-6, atol=1e-9)
    lg = rng.standard_normal(32000, dtype=np.float32)
    lg[[17, 9000, 31999]] = 9.0                          # ties: the reference CUDA kernel keeps the first
    assert ref_cuda.argmax_all(lg) == orc.argmax_first(lg) == T(lg).argmax(tl.TIE_FIRST).item_i64() == 17
    assert orc.argmax_last(lg) == T(lg).argmax(tl.TIE_LAST).item_i64() == 31999
    np.testing.assert_array_equal(ref_cuda.causal_mask(9), orc.causal_mask(9))
    np.testing.assert_array_equal(tl.Tensor.new_causal_mask(9).numpy(), ref_cuda.causal_mask(9))
    kv = rng.standard_normal((1, 2, 7, 16), dtype=np.float32)
    np.testing.assert_array_equal(ref_cuda.repeat_interleave(kv, 4, 1), orc.repeat_interleave(kv, 4, 1))
    np.testing.assert_array_equal(T(kv).repeat_interleave(4, 1).numpy(), ref_cuda.repeat_interleave(kv, 4, 1))
    table = rng.standard_normal((50, 24), dtype=np.float32)
    idx = np.array([0, 49, 7, 7], dtype=np.float32)
    np.testing.assert_array_equal(ref_cuda.embedding_f32(table, idx), orc.embedding(table, idx))
    np.testing.assert_array_equal(T(idx).embedding(T(table)).numpy(), ref_cuda.embedding_f32(table, idx))
    pen = ref_cuda.repetition_penalty(lg[:1000], [3, 17, 999], 1.1)
    np.testing.assert_array_equal(pen, orc.repetition_penalty(lg[:1000], np.array([3, 17, 999], dtype=np.float32), 1.1))
    np.testing.assert_array_equal(T(lg[:1000]).repetition_penalty(T(np.array([3, 17, 999], dtype=np.float32)), 1.1).numpy(), pen)
    g = rng.standard_normal(4096, dtype=np.float32) * 3
    u = rng.standard_normal(4096, dtype=np.float32)
    sm = ref_cuda.fused_silu_mul(g, u)                   # x / (1 + expf(-x)) * up; the CPU path multiplies by 1 / (1 + exp(-x))
    np.testing.assert_allclose(sm, orc.mul(orc.silu(g), u), rtol=4e-6, atol=1e-12)
    np.testing.assert_allclose(T(g).fused_silu_mul(T(u)).numpy(), sm, rtol=4e-6, atol=1e-12)


def test_matmul_and_attention(orc):
    rng = np.random.default_rng(8)
    a = rng.standard_normal((2, 3, 5, 64), dtype=np.float32)
    b = rng.standard_normal((2, 3, 64, 9), dtype=np.float32)
    m = ref_cuda.matmul(a.reshape(6, 5, 64), b.reshape(6, 64, 9)).reshape(2, 3, 5, 9)
    np.testing.assert_allclose(m, orc.matmul(a.reshape(6, 5, 64), b.reshape(6, 64, 9)).reshape(2, 3, 5, 9), rtol=0, atol=2e-5)
    np.testing.assert_allclose(T(a).matmul(T(b)).numpy(), m, rtol=0, atol=5e-5)
    for d, sq, sk in ((64, 5, 37), (128, 1, 70)):
        q = rng.standard_normal((1, 4, sq, d), dtype=np.float32)
        k = rng.standard_normal((1, 4, sk, d), dtype=np.float32)
        v = rng.standard_normal((1, 4, sk, d), dtype=np.float32)
        o = ref_cuda.sdpa(q, k, v)
        np.testing.assert_allclose(o, orc.sdpa_cpu(q, k, v), rtol=0, atol=2e-5)
        np.testing.assert_allclose(T(q).sdpa(T(k), T(v)).numpy(), o, rtol=0, atol=2e-5)
        mask = np.where(rng.random((sq, sk)) < 0.3, -np.inf, 0.0).astype(np.float32)
        mask[:, 0] = 0.0                                 # no fully masked row
        om = ref_cuda.sdpa(q, k, v, mask)                # additive mask, the CUDA convention
        np.testing.assert_allclose(T(q).sdpa(T(k), T(v), T(mask), mask_mode=1).numpy(), om, rtol=0, atol=2e-5)
        keep = (mask == 0).astype(np.float32)            # the CPU convention on the equivalent 0/1 mask
        np.testing.assert_allclose(orc.sdpa_cpu(q, k, v, keep), om, rtol=0, atol=2e-5)
