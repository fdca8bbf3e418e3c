"""GPU parity: dequantisation (bit-exact) and the dequant-fused matvec against the CPU oracle,
through the C ABI."""
import numpy as np
import pytest

import tl_b200 as tl
from tl_b200 import synth

pytestmark = pytest.mark.gpu

TYPES = [synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K]
MATVEC_TOL = 1e-4   # our own bar; the required gate is 2e-2 max-abs-rel


def relerr(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("n,k", [(16, 256), (48, 1024), (33, 512), (1, 256)])
def test_dequant_bit_exact(orc, t, n, k):
    rng = np.random.default_rng(1000 + t + n)
    w = synth.random_quant(t, n, k, rng)
    q = tl.QTensor.from_gguf_bytes(t, n, k, w)
    info = q.info()
    assert (info["type"], info["n"], info["k"]) == (t, n, k)
    assert info["device_bytes"] == (n + 15) // 16 * 16 * k * synth.bytes_per_weight(t)
    got = q.dequantize().numpy()
    ref = orc.dequantize(t, w.reshape(-1), n * k).reshape(n, k)
    np.testing.assert_array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_dequant_extreme_blocks(orc):
    """f16 scales that are subnormal, zero, negative and the largest finite value; all-ones quants."""
    for t in TYPES:
        blk, nb = synth.BLOCK[t]
        n, k = 16, 256
        w = np.full((n * k // blk, nb), 0xFF, dtype=np.uint8)
        scales = np.array([0x0001, 0x0000, 0x8001, 0x7BFF, 0x03FF, 0xFBFF, 0x3C00, 0x0400], dtype=np.uint16)
        pos = {synth.Q4_0: 0, synth.Q8_0: 0, synth.Q4_K: 0, synth.Q6_K: 208}[t]
        for i in range(w.shape[0]):
            w[i, pos:pos + 2] = np.array([scales[i % 8]], dtype=np.uint16).view(np.uint8)
            if t == synth.Q4_K:
                w[i, 2:4] = np.array([scales[(i + 3) % 8]], dtype=np.uint16).view(np.uint8)
        got = tl.QTensor.from_gguf_bytes(t, n, k, w).dequantize().numpy()
        ref = orc.dequantize(t, w.reshape(-1), n * k).reshape(n, k)
        np.testing.assert_array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_dequant_full_size_rows_checksum(orc):
    """A Llama-3-8B sized projection (4096 x 4096, Q4_K): bit-exact on sampled rows + u32 checksum of all."""
    rng = np.random.default_rng(7)
    n = k = 4096
    w = synth.random_quant(synth.Q4_K, n, k, rng)
    got = tl.QTensor.from_gguf_bytes(synth.Q4_K, n, k, w).dequantize().numpy()
    ref = orc.dequantize(synth.Q4_K, w.reshape(-1), n * k).reshape(n, k)
    assert int(got.view(np.uint32).sum(dtype=np.uint64)) == int(ref.view(np.uint32).sum(dtype=np.uint64))
    np.testing.assert_array_equal(got[::97].view(np.uint32), ref[::97].view(np.uint32))


def test_qtensor_rejects_bad_input():
    with pytest.raises(tl.TlbError) as e:
        tl.QTensor.from_gguf_bytes(synth.Q4_K, 16, 256, np.zeros(100, dtype=np.uint8))
    assert e.value.code == 1
    with pytest.raises(tl.TlbError) as e:
        tl.QTensor.from_gguf_bytes(synth.Q4_0, 16, 48, np.zeros(16 * 27, dtype=np.uint8))      # K not a whole number of blocks
    assert e.value.code == 1
    with pytest.raises(tl.TlbError) as e:
        tl.QTensor.from_gguf_bytes(synth.Q4_K, 16, 128, np.zeros(16 * 72, dtype=np.uint8))     # K-quants need K % 256 == 0
    assert e.value.code == 1
    with pytest.raises(tl.TlbError) as e:
        tl.QTensor.from_gguf_bytes(5, 16, 256, np.zeros(16, dtype=np.uint8))  # type 5: a GGML id neither side knows
    assert e.value.code == 7
    q = tl.QTensor.from_gguf_bytes(synth.Q4_K, 0, 256, np.zeros(0, dtype=np.uint8))  # empty tensor
    assert q.dequantize().numpy().shape == (0, 256)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("n,k,m", [(16, 256, 1), (48, 1024, 1), (33, 512, 2), (256, 2048, 4), (64, 512, 6), (40, 768, 3)])
def test_qmatvec_matches_oracle(orc, t, n, k, m):
    rng = np.random.default_rng(2000 + t + n + m)
    w = synth.random_quant(t, n, k, rng)
    x = rng.standard_normal((m, k), dtype=np.float32)
    q = tl.QTensor.from_gguf_bytes(t, n, k, w)
    got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
    ref = orc.qmatmul(t, w.reshape(-1), n, k, x)
    assert got.shape == (m, n)
    # up to 4 rows: the matvec (two int8 levels per activation); 5 to 16: the few-rows kernel (f16 activations)
    assert relerr(got, ref) < (MATVEC_TOL if m <= 4 else GEMM_TOL)


@pytest.mark.parametrize("t,n,k", [(synth.Q4_K, 4096, 4096), (synth.Q4_K, 4096, 14336), (synth.Q6_K, 8192, 4096),
                                   (synth.Q8_0, 2048, 2048), (synth.Q4_0, 5632, 2048)])
def test_qmatvec_model_shapes(orc, t, n, k):
    rng = np.random.default_rng(3000 + t + n)
    w = synth.random_quant(t, n, k, rng)
    x = rng.standard_normal(k, dtype=np.float32)
    q = tl.QTensor.from_gguf_bytes(t, n, k, w)
    xt = tl.Tensor.from_numpy(x)
    got = xt.matmul_quantized(q).numpy()
    rows = np.unique(np.concatenate([np.arange(0, n, 61), [n - 1]]))
    wrows = w[rows]
    ref = orc.qmatmul(t, wrows.reshape(-1), len(rows), k, x)[0]
    assert got.shape == (n,)
    assert relerr(got[rows], ref) < MATVEC_TOL
    again = xt.matmul_quantized(q).numpy()      # scheduling-independent: bitwise repeatable
    np.testing.assert_array_equal(got.view(np.uint32), again.view(np.uint32))


def test_qmatvec_linearity_and_scale_invariance():
    """Size-independent properties on a full-size shape: W(a x + b y) = a Wx + b Wy, and the internal
    power-of-two activation scaling is invisible (W(2^20 x) = 2^20 Wx exactly)."""
    rng = np.random.default_rng(11)
    n, k = 4096, 4096
    q = tl.QTensor.from_gguf_bytes(synth.Q4_K, n, k, synth.random_quant(synth.Q4_K, n, k, rng))
    x = rng.standard_normal(k, dtype=np.float32)
    y = rng.standard_normal(k, dtype=np.float32)
    f = lambda v: tl.Tensor.from_numpy(v).matmul_quantized(q).numpy()
    wx, wy = f(x), f(y)
    assert relerr(f(np.float32(0.5) * x + np.float32(2) * y), np.float32(0.5) * wx + np.float32(2) * wy) < 1e-5
    np.testing.assert_array_equal(f(x * np.float32(2 ** 20)), wx * np.float32(2 ** 20))
    z = f(np.zeros(k, dtype=np.float32))
    assert not z.any()


def test_qmatvec_wide_dynamic_range(orc):
    """Activations spanning 12 orders of magnitude and huge values (no f16 overflow inside)."""
    rng = np.random.default_rng(12)
    n, k = 64, 1024
    w = synth.random_quant(synth.Q4_K, n, k, rng)
    x = (rng.standard_normal(k) * 10.0 ** rng.uniform(-6, 6, k)).astype(np.float32)
    q = tl.QTensor.from_gguf_bytes(synth.Q4_K, n, k, w)
    got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
    ref = orc.qmatmul(synth.Q4_K, w.reshape(-1), n, k, x)[0]
    assert relerr(got, ref) < MATVEC_TOL
    big = (x * np.float32(1e20)).astype(np.float32)
    got = tl.Tensor.from_numpy(big).matmul_quantized(q).numpy()
    assert np.isfinite(got).all()


def test_qmatvec_shape_errors():
    q = tl.QTensor.from_gguf_bytes(synth.Q4_K, 16, 256, np.zeros(16 * 144, dtype=np.uint8))
    with pytest.raises(tl.TlbError) as e:
        tl.Tensor.from_numpy(np.zeros(128, dtype=np.float32)).matmul_quantized(q)
    assert e.value.code == 1
    out = tl.Tensor.from_numpy(np.zeros((0, 256), dtype=np.float32)).matmul_quantized(q)  # empty batch
    assert out.shape == (0, 16)


# ---- many activation rows: the tensor-core GEMM behind the same entry point (rows > 16) ----------------
GEMM_TOL = 2e-3      # f16 operands (2^-12 relative rounding each), f32 accumulation; the required gate is 2e-2
GEMM_EMU_TOL = 2e-5  # against the same arithmetic done in numpy: only the summation order differs


def _f16_emulation(x, wd):
    amax = np.abs(x).max(axis=1)
    e = np.frexp(amax)[1]
    sc = np.where((amax > 0) & np.isfinite(amax), np.ldexp(1.0, 14 - e), 1.0).astype(np.float32)
    xs = (x * sc[:, None]).astype(np.float16).astype(np.float64)
    return (xs @ wd.astype(np.float16).astype(np.float64).T) / sc[:, None]


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("n,k,m", [(128, 256, 17), (33, 512, 40), (256, 1024, 100), (384, 2048, 300), (1024, 1024, 520)])
def test_qgemm_matches_oracle(orc, t, n, k, m):
    rng = np.random.default_rng(5000 + t + n + m)
    w = synth.random_quant(t, n, k, rng)
    x = rng.standard_normal((m, k), dtype=np.float32)
    x[0] *= 1000.0       # rows of very different magnitude: each row carries its own power-of-two scale
    x[-1] *= 1e-3
    x[1] = 0.0           # an all-zero row
    q = tl.QTensor.from_gguf_bytes(t, n, k, w)
    got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
    ref = orc.qmatmul(t, w.reshape(-1), n, k, x)
    assert got.shape == (m, n)
    assert np.all(got[1] == 0.0)
    for i in range(m):
        if i != 1:
            assert relerr(got[i], ref[i]) < GEMM_TOL, i
    if t in (synth.Q4_0, synth.Q8_0):
        # these weights are one f16 rounding of the f32 value, so numpy can redo the arithmetic
        # (the K formats round d * sc and dmin * m to f16 before the last multiply-add)
        emu = _f16_emulation(x, q.dequantize().numpy())
        assert relerr(got, emu) < GEMM_EMU_TOL


@pytest.mark.parametrize("t,n,k", [(synth.Q4_K, 4096, 4096), (synth.Q6_K, 16384, 4096), (synth.Q4_0, 2048, 5632), (synth.Q8_0, 2048, 2048)])
def test_qgemm_full_size_agrees_with_matvec(t, n, k):
    """Model-sized weights, 512 rows: sampled rows of the GEMM against the streaming matvec on the same rows."""
    rng = np.random.default_rng(77 + t)
    q = tl.QTensor.from_gguf_bytes(t, n, k, synth.random_quant(t, n, k, rng))
    x = rng.standard_normal((512, k), dtype=np.float32)
    got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
    again = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
    np.testing.assert_array_equal(got.view(np.uint32), again.view(np.uint32))   # bitwise repeatable
    for i in (0, 1, 255, 256, 300, 511):
        one = tl.Tensor.from_numpy(x[i]).matmul_quantized(q).numpy()
        assert relerr(got[i], one) < GEMM_TOL, i


def test_qgemm_rank3_input_and_shape_error():
    rng = np.random.default_rng(78)
    q = tl.QTensor.from_gguf_bytes(synth.Q8_0, 64, 256, synth.random_quant(synth.Q8_0, 64, 256, rng))
    x = rng.standard_normal((2, 20, 256), dtype=np.float32)
    got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
    assert got.shape == (2, 20, 64)
    flat = tl.Tensor.from_numpy(x.reshape(40, 256)).matmul_quantized(q).numpy()
    np.testing.assert_array_equal(got.reshape(40, 64), flat)
    with pytest.raises(tl.TlbError) as e:
        tl.Tensor.from_numpy(np.zeros((40, 512), dtype=np.float32)).matmul_quantized(q)
    assert e.value.code == 1


def test_mid_row_counts_on_a_wide_weight(orc):
    """5 to 16 rows on 14336 x 4096 (gate / up shape) run through the few-rows kernel: sampled output rows against the oracle."""
    n, k = 14336, 4096
    rng = np.random.default_rng(79)
    w = synth.random_quant(synth.Q4_K, n, k, rng)
    q = tl.QTensor.from_gguf_bytes(synth.Q4_K, n, k, w)
    rows = np.unique(np.concatenate([np.arange(0, n, 257), [n - 1]]))
    for m in (5, 8, 16):
        x = rng.standard_normal((m, k), dtype=np.float32)
        got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
        ref = orc.qmatmul(synth.Q4_K, w[rows].reshape(-1), len(rows), k, x)
        assert got.shape == (m, n)
        for i in range(m):
            assert relerr(got[i][rows], ref[i]) < GEMM_TOL, (m, i)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("n,k", [(1000, 512), (4100, 1024), (272, 2304)])
def test_few_rows_kernel_shapes(orc, t, n, k):
    """5 to 16 rows stream through the few-rows kernel: the unit steps (16-tile group x 256-wide unit) are cut evenly over
    the CTAs, so tile groups are split between CTAs at arbitrary units and summed by a second launch.  1000 rows: a last
    tile of 8 rows; 4100: a last tile group of one tile; 272 x 2304: 9 units over two tile groups.  Whole result against
    the oracle, one row 50 times larger than the rest (per-row activation scale)."""
    rng = np.random.default_rng(7000 + t + n)
    w = synth.random_quant(t, n, k, rng)
    q = tl.QTensor.from_gguf_bytes(t, n, k, w)
    for m in (5, 8, 9, 16):
        x = rng.standard_normal((m, k), dtype=np.float32)
        x[m - 1] *= 50.0
        got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
        ref = orc.qmatmul(t, w.reshape(-1), n, k, x)
        assert got.shape == (m, n)
        for i in range(m):
            assert relerr(got[i], ref[i]) < GEMM_TOL, (m, i)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("m", [777, 1100])
def test_qgemm_two_accumulators_ragged_rows(orc, t, m):
    """148 row tiles x more than 512 activation rows: the GEMM gives each CTA 512 rows as two accumulators.  777 rows leave
    the last CTA 9 rows in its second accumulator, 1100 rows leave the last CTA no second accumulator at all.  Sampled
    weight rows against the oracle, every activation row."""
    n, k = 148 * 128, 512
    rng = np.random.default_rng(6000 + t + m)
    w = synth.random_quant(t, n, k, rng)
    q = tl.QTensor.from_gguf_bytes(t, n, k, w)
    x = rng.standard_normal((m, k), dtype=np.float32)
    x[511] *= 300.0
    x[512] *= 1e-2
    got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
    rows = np.unique(np.concatenate([np.arange(0, n, 199), [127, 128, n - 1]]))
    ref = orc.qmatmul(t, w[rows].reshape(-1), len(rows), k, x)
    assert got.shape == (m, n)
    for i in range(m):
        assert relerr(got[i][rows], ref[i]) < GEMM_TOL, i


# ---- dense QTensors: every other tensor type the reference's loader wraps in a QTensor ---------------------
DENSE = [(synth.F32, 24, 80), (synth.F16, 24, 80), (synth.Q4_1, 24, 96), (synth.Q5_0, 24, 96), (synth.Q5_1, 40, 320),
         (synth.Q8_1, 24, 64), (synth.Q4_0, 24, 96), (synth.Q8_0, 33, 160)]


@pytest.mark.parametrize("t,n,k", DENSE)
def test_dense_qtensor_dequant_bit_exact_and_matmul(orc, t, n, k):
    """F32 / F16 / Q4_1 / Q5_0 / Q5_1 / Q8_1, and Q4_0 / Q8_0 rows that are not a multiple of 256 long: dequantised once,
    bit-exact against the oracle, and multiplied through the f32 matmul (the reference's route for types without a
    fused kernel, crates/tl_runtime/src/system.rs:236-264)."""
    rng = np.random.default_rng(4000 + t + n)
    w = synth.random_quant(t, n, k, rng)
    q = tl.QTensor.from_gguf_bytes(t, n, k, w)
    info = q.info()
    assert (info["type"], info["n"], info["k"]) == (t, n, k)
    ref = orc.dequantize(t, w.reshape(-1), n * k).reshape(n, k)
    np.testing.assert_array_equal(q.dequantize().numpy().view(np.uint32), ref.view(np.uint32))
    for m in (1, 3, 20):
        x = rng.standard_normal((m, k), dtype=np.float32)
        got = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
        want = orc.qmatmul(t, w.reshape(-1), n, k, x)
        assert got.shape == (m, n) and relerr(got, want) < 1e-5


def test_f16_and_f32_tensors_through_the_map(orc):
    """An F16 tensor through tlb_map_add / tlb_map_get is widened exactly (all 63488 finite bit patterns and both zeros,
    crates/tl_runtime/src/quantized.rs:167-180); tlb_map_get_quantized wraps F32 / F16 tensors too
    (crates/tl_runtime/src/tensor_map.rs:279)."""
    bits = np.array([b for b in range(65536) if (b & 0x7C00) != 0x7C00], dtype=np.uint16)
    bits = np.concatenate([bits, bits[:(-len(bits)) % 64]]).reshape(-1, 64)
    m = tl.TensorMap.new()
    m.add("h.weight", synth.F16, bits.shape, bits)
    got = m.get("h.weight").numpy()
    want = orc.dequantize(synth.F16, bits.view(np.uint8).reshape(-1), bits.size).reshape(bits.shape)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    np.testing.assert_array_equal(got, bits.view(np.float16).astype(np.float32))
    rng = np.random.default_rng(5)
    emb = (rng.standard_normal((50, 64), dtype=np.float32) * 0.02)
    m.add("token_embd.weight", synth.F32, emb.shape, emb)
    x = rng.standard_normal((2, 64), dtype=np.float32)
    tied = tl.Tensor.from_numpy(x).matmul_quantized(m.get_quantized("token_embd.weight")).numpy()   # a tied output head
    assert relerr(tied, orc.qmatmul(synth.F32, emb.view(np.uint8).reshape(-1), 50, 64, x)) < 1e-5
    hq = m.get_quantized("h.weight")
    assert hq.info()["type"] == synth.F16
    np.testing.assert_array_equal(hq.dequantize().numpy().view(np.uint32), want.view(np.uint32))
    xh = rng.standard_normal((1, 64), dtype=np.float32)
    finite = np.abs(want).max(axis=1) < 1e3            # rows without huge f16 values: a well-conditioned product
    gh = tl.Tensor.from_numpy(xh).matmul_quantized(hq).numpy()[0][finite]
    wh = orc.qmatmul(synth.F16, bits.view(np.uint8).reshape(-1), bits.shape[0], 64, xh)[0][finite]
    np.testing.assert_allclose(gh, wh, rtol=1e-4, atol=1e-3)


def test_misaligned_activation_view(orc):
    """A zero-copy view that starts at an odd element (tlb_narrow) is not 16-byte aligned: the matmul copies it first."""
    rng = np.random.default_rng(6)
    n, k = 64, 512
    w = synth.random_quant(synth.Q4_K, n, k, rng)
    q = tl.QTensor.from_gguf_bytes(synth.Q4_K, n, k, w)
    buf = rng.standard_normal(k + 3, dtype=np.float32)
    view = tl.Tensor.from_numpy(buf).narrow(0, 1, k)            # starts 4 bytes into the buffer
    got = view.matmul_quantized(q).numpy()
    assert relerr(got, orc.qmatmul(synth.Q4_K, w.reshape(-1), n, k, buf[1:k + 1])[0]) < MATVEC_TOL
    many = rng.standard_normal((40, k + 1), dtype=np.float32)   # the tensor-core route, rows at odd offsets
    v2 = tl.Tensor.from_numpy(many.reshape(-1)).narrow(0, 1, 40 * k).reshape([40, k])
    got2 = v2.matmul_quantized(q).numpy()
    want2 = orc.qmatmul(synth.Q4_K, w.reshape(-1), n, k, many.reshape(-1)[1:40 * k + 1].reshape(40, k))
    assert relerr(got2, want2) < 5e-3
