"""Small, self-contained cases to run under a profiler (one kernel family each, a few GB at most).

    python -m tl_b200.profile_cases qgemm [rows]      # Q4_K 4096 x 4096 weight, `rows` activation rows (default 1184)
    python -m tl_b200.profile_cases prefill [tokens]  # two Llama-3-8B-shaped layers + head, one prompt (default 2048)

Each case runs its work three times (two warm-ups and the launch to capture) and prints timings of its own,
taken without a profiler attached, for orientation only.
"""
import sys
import time

import numpy as np

import tl_b200 as tl
from tl_b200 import synth


def qgemm(rows=1184, n=4096, k=4096):
    rng = np.random.default_rng(1)
    q = tl.QTensor.from_gguf_bytes(synth.Q4_K, n, k, synth.random_quant(synth.Q4_K, n, k, rng))
    x = tl.Tensor.from_numpy(rng.standard_normal((rows, k), dtype=np.float32))
    for _ in range(2):
        x.matmul_quantized(q)
    tl.sync()
    t0 = time.perf_counter()
    x.matmul_quantized(q)
    tl.sync()
    dt = time.perf_counter() - t0
    print("qgemm %dx%d rows=%d: %.1f us, %.0f TFLOP/s (with the f16 conversion)" % (n, k, rows, dt * 1e6, 2.0 * rows * n * k / dt / 1e12))


def prefill(tokens=2048, layers=2):
    cfg = dict(synth.LLAMA3_8B, n_layers=layers)
    wmap = tl.map_from_tensors(synth.llama_tensors(cfg, 1, synth.Q4_K, synth.Q6_K))
    dec = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=tokens + 256)
    rng = np.random.default_rng(6)
    prompt = [int(t) for t in rng.integers(0, cfg["vocab"], tokens)]
    for _ in range(2):
        dec.prefill(prompt, 0)
    tl.sync()
    t0 = time.perf_counter()
    dec.prefill(prompt, 0)
    tl.sync()
    dt = time.perf_counter() - t0
    print("prefill %d tokens, %d layers + head: %.2f ms" % (tokens, layers, dt * 1e3))


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "qgemm"
    arg = [int(a) for a in sys.argv[2:3]]
    {"qgemm": qgemm, "prefill": prefill}[which](*arg)
