"""Writes the golden fixtures of this folder.  Run from the repository root:

    python tests/golden/make_golden.py

quant_vectors.npz - per GGUF format a seeded [16, 512] tensor in GGUF block bytes, its
dequantised values computed TWICE - by the independent numpy statement of the block formats
(tests/npref.py, written from the format definition) and by the C oracle (oracle/tl_oracle.c,
restating crates/tl_runtime/src/quantized.rs:167-415) - which must agree bit for bit before the
file is written, and the oracle's dequantise-then-matmul product with a seeded activation
(crates/tl_runtime/src/system.rs:193-222 + crates/tl_cpu/src/tensor.rs:1284-1306).

decoder_vectors.npz - a 2-layer Llama-shaped model from tl_b200.synth (seed in the file): logits
after a 3-token prompt and the next 8 greedy tokens with their logits' checksums, from the oracle's
op-by-op driver (the op sequence of examples/apps/llama3/chatbot_llama3.tl:66-125,220-236).

prompt_vectors.npz - the same model, a 40-token seeded prompt in one oracle pass (logits of the last token, the
greedy token after it) and, per GGUF format, the oracle's product of the quant_vectors tensor with 24 seeded
activation rows: what the many-row (tensor-core) paths must reproduce within their f16 operand rounding.

The reference itself (Rust + LLVM JIT) cannot run here, so these pin this repository's restatement
against itself over time and against the independent numpy statement; the reference's own
known-answer values are asserted separately in tests/test_oracle_kat.py.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import npref  # noqa: E402
from oracle import oracle  # noqa: E402
from tl_b200 import synth  # noqa: E402

DECODER_CFG = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=320,
                   eps=1e-5, rope_base=10000.0, attn_scale=0.125)
DECODER_SEED = 77
PROMPT = [5, 17, 300]
STEPS = 8


def quant_vectors():
    out = {}
    npdeq = {synth.Q4_0: npref.deq_q4_0, synth.Q8_0: npref.deq_q8_0, synth.Q4_K: npref.deq_q4_k, synth.Q6_K: npref.deq_q6_k}
    for t in (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K):
        n, k = 16, 512
        rng = np.random.default_rng(4242 + t)
        w = synth.random_quant(t, n, k, rng)
        x = rng.standard_normal(k).astype(np.float32)
        deq_c = oracle.dequantize(t, w.reshape(-1), n * k)
        deq_np = npdeq[t](w.reshape(-1)).astype(np.float32)
        assert np.array_equal(deq_c.view(np.uint32), deq_np.view(np.uint32)), "oracle and numpy statement disagree for type %d" % t
        y = oracle.qmatmul(t, w.reshape(-1), n, k, x.reshape(1, k)).reshape(n)
        out["w_%d" % t] = w
        out["x_%d" % t] = x
        out["deq_%d" % t] = deq_c.view(np.uint32)
        out["y_%d" % t] = y
    return out


def decoder_vectors():
    tens = synth.llama_tensors(DECODER_CFG, DECODER_SEED, synth.Q4_K, synth.Q6_K)
    ref = oracle.Llama(dict(DECODER_CFG, kv_f16=1, max_seq=64), {k: (t, d) for k, (t, d, s) in tens.items()})
    logits = ref.forward(PROMPT, 0)
    out = {"prompt": np.array(PROMPT, np.int32), "seed": np.array([DECODER_SEED], np.int32),
           "prompt_logits": logits.astype(np.float32)}
    toks, sums = [], []
    tok, pos = oracle.argmax_last(logits), len(PROMPT)
    first = tok
    for _ in range(STEPS):
        logits = ref.forward([tok], pos)
        tok = oracle.argmax_last(logits)
        toks.append(tok)
        sums.append(float(np.sum(logits.astype(np.float64))))
        pos += 1
    out["first_token"] = np.array([first], np.int32)
    out["tokens"] = np.array(toks, np.int32)
    out["logit_sums"] = np.array(sums, np.float64)
    out["last_logits"] = logits.astype(np.float32)
    ref.close()
    return out


LONG_PROMPT = 40
ROWS = 24


def prompt_vectors(qv):
    tens = synth.llama_tensors(DECODER_CFG, DECODER_SEED, synth.Q4_K, synth.Q6_K)
    ref = oracle.Llama(dict(DECODER_CFG, kv_f16=1, max_seq=64), {k: (t, d) for k, (t, d, s) in tens.items()})
    prompt = np.random.default_rng(DECODER_SEED).integers(0, DECODER_CFG["vocab"], LONG_PROMPT).astype(np.int32)
    logits = ref.forward([int(t) for t in prompt], 0)
    out = {"prompt": prompt, "seed": np.array([DECODER_SEED], np.int32), "prompt_logits": logits.astype(np.float32),
           "first_token": np.array([oracle.argmax_last(logits)], np.int32)}
    ref.close()
    for t in (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K):
        x = np.random.default_rng(777 + t).standard_normal((ROWS, 512)).astype(np.float32)
        out["xrows_%d" % t] = x
        out["yrows_%d" % t] = oracle.qmatmul(t, qv["w_%d" % t].reshape(-1), 16, 512, x)
    return out


if __name__ == "__main__":
    qv = quant_vectors()
    np.savez_compressed(os.path.join(HERE, "quant_vectors.npz"), **qv)
    np.savez_compressed(os.path.join(HERE, "decoder_vectors.npz"), **decoder_vectors())
    np.savez_compressed(os.path.join(HERE, "prompt_vectors.npz"), **prompt_vectors(qv))
    for f in ("quant_vectors.npz", "decoder_vectors.npz", "prompt_vectors.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
