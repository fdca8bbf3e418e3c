"""The route an unmodified TL program takes: the chatbot's forward pass issued op by op through the per-op C ABI
(tl_b200.chatbot.PerOpLlama mirrors examples/apps/llama3/chatbot_llama3.tl:48-125,220-236), against the oracle's
driver of the same op sequence and against the fused session."""
import numpy as np
import pytest

import tl_b200 as tl
from tl_b200 import synth
from tl_b200.chatbot import PerOpLlama

pytestmark = pytest.mark.gpu
SMALL = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=320,
             eps=1e-5, rope_base=10000.0, attn_scale=0.125)


def relerr(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


@pytest.mark.parametrize("linear,head", [(synth.Q4_K, synth.Q6_K), (synth.Q4_0, synth.Q4_0), (synth.Q8_0, synth.F16)])
def test_per_op_route_matches_oracle_and_fused_session(orc, linear, head):
    # Q8_0 block scales at a trained model's magnitude (see test_gpu_decoder.test_prefill_matches_oracle_and_continues)
    tens = synth.llama_tensors(SMALL, 51, linear, head, scale_sigma=0.002 if linear == synth.Q8_0 else None)
    wmap = tl.map_from_tensors(tens)
    ref = orc.Llama(dict(SMALL, kv_f16=0, max_seq=64), {k: (t, d) for k, (t, d, s) in tens.items()})
    bot = PerOpLlama(SMALL, wmap, max_seq=64)
    prompt = [5, 17, 300, 9, 41, 77, 2]
    rl = ref.forward(prompt, 0)
    tok = bot.step(prompt, 0)                       # the whole prompt in one pass: causal mask, rotation at row 0
    # seven rows: the quantized matmuls run on the few-rows kernel (f16 activations); the single-token steps below on the matvec
    assert relerr(bot.last_logits.numpy()[0], rl) < 5e-3
    assert tok == orc.argmax_last(rl)
    fused = None
    if head != synth.F16:                           # the fused session takes tiled weights only; the per-op route any QTensor
        fused = tl.Decoder(SMALL, wmap, kv_f16=False, max_seq=64)
        for i, t in enumerate(prompt):
            ftok = fused.step(t, i, rope_pos=0)
        assert ftok == tok
    pos = len(prompt)
    for _ in range(10):
        rl = ref.forward([tok], pos)
        nxt = bot.step([tok], pos)
        # the prompt's cache rows came from the few-rows kernel (f16 activations): 5e-3 here as well, the gate is 2e-2
        assert relerr(bot.last_logits.numpy()[0], rl) < 5e-3
        assert nxt == orc.argmax_last(rl)
        if fused is not None:
            assert fused.step(tok, pos) == nxt
            assert relerr(fused.logits(), bot.last_logits.numpy()[0]) < 5e-3
        tok, pos = nxt, pos + 1
    # the cache the program holds grew by concatenation: [1, KVH, T, D]
    assert bot.cache.get_k(0).shape == (1, SMALL["n_kv_heads"], pos, SMALL["head_dim"])
    # the same op sequence issued by the library's native driver: the prompt, then steps, bit for bit the same logits
    nat = PerOpLlama(SMALL, wmap, max_seq=64)
    py = PerOpLlama(SMALL, wmap, max_seq=64)
    t_n, t_p = nat.step_native(prompt, 0), py.step(prompt, 0)
    assert t_n == t_p
    np.testing.assert_array_equal(nat.last_logits.numpy().view(np.uint32), py.last_logits.numpy().view(np.uint32))
    for i in range(4):
        t_n, t_p = nat.step_native([t_n], len(prompt) + i), py.step([t_p], len(prompt) + i)
        assert t_n == t_p
        np.testing.assert_array_equal(nat.last_logits.numpy().view(np.uint32), py.last_logits.numpy().view(np.uint32))
    assert nat.cache.get_k(0).shape == py.cache.get_k(0).shape
