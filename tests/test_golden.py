"""The committed fixtures of tests/golden (made by tests/golden/make_golden.py): the oracle must keep
reproducing them on CPU, and the CUDA library must match them on a GPU - dequantisation bit for
bit, the fused matvec within 1e-4, decoder logits within the 2e-2 gate with identical greedy tokens."""
import os

import numpy as np
import pytest

from tl_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TYPES = [synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K]
DECODER_CFG = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=320,
                   eps=1e-5, rope_base=10000.0, attn_scale=0.125)


def relerr(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


@pytest.fixture(scope="module")
def qv():
    return np.load(os.path.join(GOLD, "quant_vectors.npz"))


@pytest.fixture(scope="module")
def dv():
    return np.load(os.path.join(GOLD, "decoder_vectors.npz"))


@pytest.fixture(scope="module")
def pv():
    return np.load(os.path.join(GOLD, "prompt_vectors.npz"))


@pytest.mark.parametrize("t", TYPES)
def test_oracle_reproduces_quant_fixtures(orc, qv, t):
    w, x = qv["w_%d" % t], qv["x_%d" % t]
    n, k = 16, 512
    deq = orc.dequantize(t, w.reshape(-1), n * k)
    np.testing.assert_array_equal(deq.view(np.uint32), qv["deq_%d" % t])
    y = orc.qmatmul(t, w.reshape(-1), n, k, x.reshape(1, k)).reshape(n)
    np.testing.assert_array_equal(y.view(np.uint32), qv["y_%d" % t].view(np.uint32))
    # and the product is what float64 numpy gives on the dequantised values, to f32 accumulation error
    ref = deq.reshape(n, k).astype(np.float64) @ x.astype(np.float64)
    assert relerr(y, ref) < 1e-5


def test_oracle_reproduces_decoder_fixture(orc, dv):
    tens = synth.llama_tensors(DECODER_CFG, int(dv["seed"][0]), synth.Q4_K, synth.Q6_K)
    ref = orc.Llama(dict(DECODER_CFG, kv_f16=1, max_seq=64), {k: (t, d) for k, (t, d, s) in tens.items()})
    prompt = [int(v) for v in dv["prompt"]]
    logits = ref.forward(prompt, 0)
    np.testing.assert_array_equal(logits.view(np.uint32), dv["prompt_logits"].view(np.uint32))
    tok, pos = orc.argmax_last(logits), len(prompt)
    assert tok == int(dv["first_token"][0])
    for want in dv["tokens"]:
        logits = ref.forward([tok], pos)
        tok = orc.argmax_last(logits)
        assert tok == int(want)
        pos += 1
    np.testing.assert_array_equal(logits.view(np.uint32), dv["last_logits"].view(np.uint32))
    ref.close()


@pytest.mark.gpu
@pytest.mark.parametrize("t", TYPES)
def test_gpu_matches_quant_fixtures(qv, t):
    import tl_b200 as tl
    w, x = qv["w_%d" % t], qv["x_%d" % t]
    q = tl.QTensor.from_gguf_bytes(t, 16, 512, w)
    np.testing.assert_array_equal(q.dequantize().numpy().view(np.uint32).reshape(-1), qv["deq_%d" % t])
    y = tl.Tensor.from_numpy(x).matmul_quantized(q).numpy()
    assert relerr(y, qv["y_%d" % t]) < 1e-4


@pytest.mark.gpu
def test_gpu_matches_decoder_fixture(dv):
    import tl_b200 as tl
    tens = synth.llama_tensors(DECODER_CFG, int(dv["seed"][0]), synth.Q4_K, synth.Q6_K)
    dec = tl.Decoder(DECODER_CFG, tl.map_from_tensors(tens), kv_f16=True, max_seq=64)
    prompt = [int(v) for v in dv["prompt"]]
    for i, t in enumerate(prompt):
        nxt = dec.step(t, i, rope_pos=0)     # the reference rotates a whole prompt at its first position
    assert relerr(dec.logits(), dv["prompt_logits"]) < 2e-2
    assert nxt == int(dv["first_token"][0])
    tok, pos = nxt, len(prompt)
    for want in dv["tokens"]:
        tok = dec.step(tok, pos)
        assert tok == int(want)
        pos += 1
    assert relerr(dec.logits(), dv["last_logits"]) < 2e-2


def test_oracle_reproduces_prompt_fixture(orc, qv, pv):
    tens = synth.llama_tensors(DECODER_CFG, int(pv["seed"][0]), synth.Q4_K, synth.Q6_K)
    ref = orc.Llama(dict(DECODER_CFG, kv_f16=1, max_seq=64), {k: (t, d) for k, (t, d, s) in tens.items()})
    logits = ref.forward([int(t) for t in pv["prompt"]], 0)
    ref.close()
    np.testing.assert_array_equal(logits.view(np.uint32), pv["prompt_logits"].view(np.uint32))
    assert orc.argmax_last(logits) == int(pv["first_token"][0])
    for t in TYPES:
        y = orc.qmatmul(t, qv["w_%d" % t].reshape(-1), 16, 512, pv["xrows_%d" % t])
        np.testing.assert_array_equal(y.view(np.uint32), pv["yrows_%d" % t].view(np.uint32))


@pytest.mark.gpu
def test_gpu_matches_prompt_fixture(qv, pv):
    """The many-row paths: 24 activation rows through the tensor-core GEMM (2e-3 per row: f16 operands), the
    40-token prompt through tlb_decoder_prefill (logits within the 2e-2 gate, the same greedy token)."""
    import tl_b200 as tl
    for t in TYPES:
        q = tl.QTensor.from_gguf_bytes(t, 16, 512, qv["w_%d" % t])
        y = tl.Tensor.from_numpy(pv["xrows_%d" % t]).matmul_quantized(q).numpy()
        for i in range(y.shape[0]):
            assert relerr(y[i], pv["yrows_%d" % t][i]) < 2e-3, (t, i)
    tens = synth.llama_tensors(DECODER_CFG, int(pv["seed"][0]), synth.Q4_K, synth.Q6_K)
    dec = tl.Decoder(DECODER_CFG, tl.map_from_tensors(tens), kv_f16=True, max_seq=64)
    nxt = dec.prefill([int(t) for t in pv["prompt"]], 0, rope_pos0=0, rope_step=0)
    assert relerr(dec.logits(), pv["prompt_logits"]) < 2e-2
    assert nxt == int(pv["first_token"][0])
