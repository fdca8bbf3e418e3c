"""GPU parity of the per-op tensor API against the CPU oracle, through the C ABI.  The first block
replays the known-answer tests of the reference (crates/tl_cuda/tests/nn_llm_test.rs,
matmul_special_test.rs, new_ops_comprehensive_test.rs; crates/tl_cpu/tests/cpu_tensor_tests.rs)."""
import math

import numpy as np
import pytest

import tl_b200 as tl

pytestmark = pytest.mark.gpu
T = tl.Tensor.from_numpy
F = lambda a: np.asarray(a, dtype=np.float32)


def close(a, b, tol=1e-5):
    np.testing.assert_allclose(a, b, rtol=tol, atol=tol)


def test_reference_kats():
    rms = math.sqrt(14.0 / 3.0)
    close(T(F([[1, 2, 3]])).rms_norm(None, 1e-5).numpy()[0], [1 / rms, 2 / rms, 3 / rms], 1e-4)
    close(T(F([[1, 2, 3]])).rms_norm(T(F([2, 3, 0.5])), 1e-5).numpy()[0], [2 / rms, 6 / rms, 1.5 / rms], 1e-4)
    m = tl.Tensor.new_causal_mask(3).numpy()
    assert m.shape == (3, 3) and m[0, 0] == 0 and np.isneginf(m[0, 1]) and m[1, 0] == 0 and m[1, 1] == 0 and np.isneginf(m[1, 2])
    c = tl.Tensor.rope_new_cos(8, 4, 10000.0, tl.ROPE_HALF).numpy()
    s = tl.Tensor.rope_new_sin(8, 4, 10000.0, tl.ROPE_HALF).numpy()
    assert c.shape == (4, 4)
    close(c[0], 1.0); close(s[0], 0.0)
    close(T(F([[1, 2], [3, 4]])).matmul(T(F([[5, 6], [7, 8]]))).numpy(), [[19, 22], [43, 50]], 1e-4)
    close(T(F([[1, 2, 3], [4, 5, 6]])).matmul(T(F([[7, 8], [9, 10], [11, 12]]))).numpy(), [[58, 64], [139, 154]], 1e-4)
    sm = T(F([[1, 2, 3]])).softmax(-1).numpy()[0]
    assert abs(sm.sum() - 1) < 1e-5 and sm[0] < sm[1] < sm[2]
    e = T(F([0, 2])).embedding(T(F([[10, 20], [30, 40], [50, 60]]))).numpy()
    np.testing.assert_array_equal(e, [[10, 20], [50, 60]])
    assert T(F([1, 5, 2, 3, 4])).sample(0.7, 0.9).item_i64() == 1
    assert T(F([1, 100, 2])).argmax().item_i64() == 1
    close(T(F([1, 2, 3, 4, 5])).repetition_penalty(T(F([1, 3])), 2.0).numpy(), [1, 1, 3, 2, 5], 1e-4)
    v = T(F([0, 1, -1, 2])).fused_silu_mul(T(F([1, 1, 1, 1]))).numpy()
    assert abs(v[0]) < 1e-5 and abs(v[1] - 0.7311) < 1e-3
    r4 = math.sqrt(30 / 4)
    close(T(F([[1, 2, 3, 4]])).fused_rms_norm(T(F([1, 1, 1, 1])), 1e-5).numpy()[0], [(i + 1) / r4 for i in range(4)], 1e-3)
    close(T(F([[1, 2]])).fused_add_rms_norm(T(F([[1, 0]])), T(F([1, 1])), 1e-5).numpy()[0], [1, 1], 1e-3)
    np.testing.assert_array_equal(T(F([1, 2, 3])).repeat_interleave(2, 0).numpy(), [1, 1, 2, 2, 3, 3])
    np.testing.assert_array_equal(T(F([1, 2, 3, 4, 5])).narrow(0, 1, 3).numpy(), [2, 3, 4])
    np.testing.assert_array_equal(T(F([1, 2])).cat(T(F([3, 4, 5])), 0).numpy(), [1, 2, 3, 4, 5])
    np.testing.assert_array_equal(T(F([[1, 2], [3, 4]])).cat(T(F([[5, 6], [7, 8]])), 0).numpy(), [[1, 2], [3, 4], [5, 6], [7, 8]])
    q = T(F([[[1, 0, 0, 0], [0, 1, 0, 0]]]))
    o = q.sdpa(q, T(np.arange(1, 9, dtype=np.float32).reshape(1, 2, 4))).numpy()
    assert o.shape == (1, 2, 4) and np.isfinite(o).all()


def test_argmax_tie_rules():
    x = T(F([7, 1, 7, 3]))
    assert x.argmax(tl.TIE_LAST).item_i64() == 2 and x.argmax(tl.TIE_FIRST).item_i64() == 0
    big = np.zeros(128256, dtype=np.float32)
    big[[5, 70000, 128255]] = 3.0
    assert T(big).argmax(tl.TIE_LAST).item_i64() == 128255 and T(big).argmax(tl.TIE_FIRST).item_i64() == 5


def test_elementwise_and_shape_ops_match_oracle(orc):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((2, 3, 5, 8), dtype=np.float32)
    b = rng.standard_normal((2, 3, 5, 8), dtype=np.float32)
    np.testing.assert_array_equal(T(a).add(T(b)).numpy(), orc.add(a, b))
    np.testing.assert_array_equal(T(a).mul(T(b)).numpy(), orc.mul(a, b))
    w = rng.standard_normal(8, dtype=np.float32)
    np.testing.assert_array_equal(T(a).mul(T(w)).numpy(), a * w)                       # trailing broadcast
    np.testing.assert_array_equal(T(a).add(T(b[:, :1, :, :1].copy())).numpy(), a + b[:, :1, :, :1])
    np.testing.assert_array_equal(T(a).scale(0.08839).numpy(), orc.scale(a, 0.08839))
    close(T(a).silu().numpy(), orc.silu(a), 2e-6)
    close(T(a).softmax(3).numpy(), orc.softmax(a, 3), 2e-6)
    close(T(a).softmax(1).numpy(), orc.softmax(a, 1), 2e-6)
    np.testing.assert_array_equal(T(a).transpose(1, 2).numpy(), a.transpose(0, 2, 1, 3))
    np.testing.assert_array_equal(T(a).transpose(2, 3).numpy(), a.transpose(0, 1, 3, 2))
    np.testing.assert_array_equal(T(a).reshape([6, 40]).numpy(), a.reshape(6, 40))
    np.testing.assert_array_equal(T(a).reshape([-1, 8]).numpy(), a.reshape(-1, 8))
    np.testing.assert_array_equal(T(a).narrow(2, 1, 3).numpy(), a[:, :, 1:4])
    np.testing.assert_array_equal(T(a).narrow(0, 1, 1).numpy(), a[1:2])
    np.testing.assert_array_equal(T(a).cat(T(b), 2).numpy(), np.concatenate([a, b], 2))
    np.testing.assert_array_equal(T(a).repeat_interleave(4, 1).numpy(), orc.repeat_interleave(a, 4, 1))
    np.testing.assert_array_equal(tl.Tensor.new_causal_mask(7).numpy(), orc.causal_mask(7))
    x = rng.standard_normal((5, 512), dtype=np.float32)
    close(T(x).rms_norm(T(F(np.ones(512) * 1.5)), 1e-5).numpy(), orc.rms_norm(x, np.ones(512) * 1.5, 1e-5), 2e-6)
    big = rng.standard_normal((3, 70, 33), dtype=np.float32)
    rhs = rng.standard_normal((33, 129), dtype=np.float32)
    close(T(big).matmul(T(rhs)).numpy(), orc.matmul(big, rhs), 1e-4)
    rhs3 = rng.standard_normal((3, 33, 20), dtype=np.float32)
    close(T(big).matmul_4d(T(rhs3)).numpy(), orc.matmul(big, rhs3), 1e-4)


def test_rope_both_conventions(orc):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 6, 4, 64), dtype=np.float32)
    cos, sin = orc.rope_table_cpu(32, 64, 10000.0)
    np.testing.assert_array_equal(tl.Tensor.rope_new_cos(64, 32, 10000.0).numpy(), cos)   # host libm tables: bit-identical
    np.testing.assert_array_equal(tl.Tensor.rope_new_sin(64, 32, 10000.0).numpy(), sin)
    got = T(x).apply_rope(T(cos[5:11]), T(sin[5:11])).numpy()
    np.testing.assert_array_equal(got, orc.apply_rope_cpu(x, cos[5:11], sin[5:11]))      # row 0 (= position 5) for all
    ch, sh = orc.rope_table_half(32, 64, 500000.0)
    np.testing.assert_array_equal(tl.Tensor.rope_new_cos(64, 32, 500000.0, tl.ROPE_HALF).numpy(), ch)
    got = T(x).apply_rope(T(ch[3:9]), T(sh[3:9]), tl.ROPE_HALF).numpy()
    np.testing.assert_array_equal(got[0], orc.apply_rope_rotate_half(x[0], ch[3:9], sh[3:9]))


def test_sdpa_mask_conventions(orc):
    rng = np.random.default_rng(2)
    q = rng.standard_normal((2, 4, 5, 64), dtype=np.float32)
    k = rng.standard_normal((2, 4, 9, 64), dtype=np.float32)
    v = rng.standard_normal((2, 4, 9, 64), dtype=np.float32)
    close(T(q).sdpa(T(k), T(v)).numpy(), orc.sdpa_cpu(q, k, v), 1e-5)
    keep = (rng.random((5, 9)) > 0.3).astype(np.float32)
    keep[:, 0] = 1
    close(T(q).sdpa(T(k), T(v), T(keep), 2).numpy(), orc.sdpa_cpu(q, k, v, keep), 1e-5)   # CPU: 0 -> -1e9
    addm = np.where(keep > 0, 0.0, -np.inf).astype(np.float32)
    close(T(q).sdpa(T(k), T(v), T(addm), 1).numpy(), orc.sdpa_cpu(q, k, v, keep), 1e-5)   # CUDA: additive


def test_errors_and_refcounts():
    a = T(F(np.zeros((2, 3))))
    with pytest.raises(tl.TlbError) as e:
        a.add(T(F(np.zeros((2, 4)))))
    assert e.value.code == 1
    with pytest.raises(tl.TlbError) as e:
        a.matmul(T(F(np.zeros((4, 2)))))
    assert e.value.code == 1
    with pytest.raises(tl.TlbError) as e:
        T(F([3])).embedding(T(F(np.zeros((3, 2)))))
    assert e.value.code == 6
    with pytest.raises(tl.TlbError) as e:
        a.narrow(1, 2, 5)
    assert e.value.code == 6
    v = a.reshape([3, 2])
    assert a.refcount() == 1 and v.refcount() == 1    # a view is a new handle on shared storage
    assert T(F(np.zeros((0, 4)))).add(T(F(np.zeros((0, 4))))).shape == (0, 4)   # empty tensors


def test_kvcache_handle_table():
    kv = tl.KVCache(2)
    k = T(F(np.ones((1, 2, 3, 4))))
    v = T(F(np.zeros((1, 2, 3, 4))))
    kv.update(0, k, v)
    assert k.refcount() == 2                                      # the cache keeps its own reference
    g = kv.get_k(0)
    assert k.refcount() == 3 and g.shape == (1, 2, 3, 4)
    k2 = g.cat_4d(T(F(np.full((1, 2, 1, 4), 2.0))), 2)           # the TL program's append (chatbot_llama3.tl:84-88)
    kv.update(0, k2, v)
    assert kv.get_k(0).shape == (1, 2, 4, 4) and k.refcount() == 2  # old K released by the cache, g still holds one
    with pytest.raises(tl.TlbError):
        kv.get_v(1)
    kv.clear()
    assert k2.refcount() == 1
    kv.free()


def test_stream_capture_and_graph_replay():
    a = T(F(np.arange(8)))
    out = a.scale(1.0)   # warm the pool so the capture holds no first-time allocation
    out.release()
    with tl.Graph() as g:
        b = a.scale(2.0)
        # entry points that wait for the device refuse cleanly during a capture and leave it usable
        for blocked in (lambda: a.item_i64(), lambda: a.numpy(), lambda: T(F([1, 2])), lambda: T(F([0])).embedding(T(F([[1, 2]])))):
            with pytest.raises(tl.TlbError) as e:
                blocked()
            assert e.value.code == 8
        c = b.add(a)
    assert g.node_count() >= 2
    for _ in range(3):       # a graph is there to be replayed: the allocations of one replay are freed by the next
        g.replay()
        np.testing.assert_array_equal(c.numpy(), np.arange(8) * 3)
        np.testing.assert_array_equal(b.numpy(), np.arange(8) * 2)
    g.destroy()


@pytest.mark.parametrize("n,temp,top_p", [(5, 1.0, 0.9), (1000, 0.7, 0.9), (1000, 1.3, 1.0), (32000, 0.8, 0.5),
                                          (128256, 1.0, 0.95), (128256, 0.6, 0.1)])
def test_sample_top_p_matches_oracle(orc, n, temp, top_p):
    """Device sampler against the restated CPU sampler for the same random numbers.  The device sums the
    exponentials in parallel, so its running sums differ from the sequential ones in the last bits: the token must
    be the oracle's, or one whose interval of the running sum (in the oracle's order) holds the drawn point within
    3e-6 (in the far tail of a flat distribution, tokens are narrower than that)."""
    rng = np.random.default_rng(100 + n)
    logits = (rng.standard_normal(n) * 3.0).astype(np.float32)
    t = tl.Tensor.from_numpy(logits)
    z = logits.astype(np.float64) / temp
    p = np.exp(z - z.max()); p /= p.sum()
    order = np.argsort(-p.astype(np.float32), kind="stable")
    cum = np.cumsum(p[order])
    above = np.nonzero(cum.astype(np.float32) > np.float32(top_p))[0]
    cutoff = int(above[0]) if len(above) else n - 1
    pos_of = np.empty(n, dtype=np.int64); pos_of[order] = np.arange(n)
    for u in list(rng.random(12)) + [0.0, 0.999999]:
        got = int(t.sample_top_p(temp, top_p, float(u)).numpy()[0])
        want = orc.sample_top_p(logits, temp, top_p, float(u))
        if got != want:
            r, pos = u * cum[cutoff], int(pos_of[got])
            assert pos <= cutoff + 1, (u, got, want)
            lo = cum[pos - 1] if pos else 0.0
            assert lo - 3e-6 <= r <= cum[pos] + 3e-6, (u, got, want, lo, r, cum[pos])
    assert int(t.sample_top_p(0.0, top_p, 0.5).numpy()[0]) == orc.argmax_last(logits)      # greedy branch
    with pytest.raises(tl.TlbError) as e:
        t.sample_top_p(1.0, top_p, 1.0)
    assert e.value.code == 8
