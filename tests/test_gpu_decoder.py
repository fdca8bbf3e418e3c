"""GPU parity of the fused decode session against the oracle's Llama driver: logits within
max-abs-rel 2e-2 (the stated gate) and identical greedy tokens over the first 32 steps."""
import numpy as np
import pytest

import tl_b200 as tl
from tl_b200 import synth

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-2


def relerr(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def build(orc, cfg, seed, linear_type, head_type, kv_f16, max_seq, sigma=None):
    tens = synth.llama_tensors(cfg, seed, linear_type, head_type, scale_sigma=sigma)
    ref = orc.Llama(dict(cfg, kv_f16=int(kv_f16), max_seq=max_seq), {k: (t, d) for k, (t, d, s) in tens.items()})
    wmap = tl.map_from_tensors(tens)
    dec = tl.Decoder(cfg, wmap, kv_f16=kv_f16, max_seq=max_seq)
    return ref, dec, wmap


def run_parity(orc, ref, dec, prompt, steps, ctx0=0):
    # prompt: the reference CPU path rotates every prompt token at the position of the first one and
    # masks causally; fed token by token that is rope_pos = ctx0 for all of them
    if ctx0 == 0:
        ref_logits = ref.forward(prompt, 0)
        for i, t in enumerate(prompt):
            nxt = dec.step(t, i, rope_pos=0)
        pos = len(prompt)
    else:
        assert len(prompt) == 1
        ref_logits = ref.forward(prompt, ctx0)
        nxt = dec.step(prompt[0], ctx0)
        pos = ctx0 + 1
    worst = relerr(dec.logits(), ref_logits)
    toks_ref, toks = [], []
    tok = orc.argmax_last(ref_logits)
    assert nxt == tok
    for s in range(steps):
        ref_logits = ref.forward([tok], pos)
        nxt = dec.step(tok, pos)
        worst = max(worst, relerr(dec.logits(), ref_logits))
        tok = orc.argmax_last(ref_logits)
        toks_ref.append(tok)
        toks.append(nxt)
        pos += 1
    assert toks == toks_ref
    assert worst < LOGIT_TOL, worst
    return toks, worst


SMALL = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=320,
             eps=1e-5, rope_base=10000.0, attn_scale=0.125)


@pytest.mark.parametrize("linear,head,kv_f16", [(synth.Q4_K, synth.Q6_K, True), (synth.Q4_K, synth.Q6_K, False),
                                                 (synth.Q4_0, synth.Q4_0, False), (synth.Q8_0, synth.Q8_0, True)])
def test_small_model_logits_and_tokens(orc, linear, head, kv_f16):
    ref, dec, wmap = build(orc, SMALL, 21, linear, head, kv_f16, 64)
    toks, worst = run_parity(orc, ref, dec, [5, 17, 300, 9, 41], 32)
    # device-side feedback loop reproduces the host-driven one
    ref2, dec2, wmap2 = build(orc, SMALL, 21, linear, head, kv_f16, 64)
    for i, t in enumerate([5, 17, 300, 9, 41]):
        first = dec2.step(t, i, rope_pos=0)
    gen = dec2.generate(first, 5, 32)
    assert gen == toks
    st = dec.stats(16)
    assert st["kernels_per_step"] == 5 * 2 + 2


def test_tinyllama_shaped_two_layers(orc):
    """Config C0's shapes (d 2048, 32 heads / 4 KV heads of 64, FFN 5632, vocab 32000, Q4_0, f32 KV), 2 layers."""
    cfg = dict(synth.TINYLLAMA, n_layers=2)
    ref, dec, wmap = build(orc, cfg, 3, synth.Q4_0, synth.Q4_0, False, 64)
    rng = np.random.default_rng(0)
    run_parity(orc, ref, dec, [int(t) for t in rng.integers(0, cfg["vocab"], 6)], 32)


def test_llama3_shaped_one_layer_long_context(orc):
    """Config C2's shapes (d 4096, 32 / 8 heads of 128, FFN 14336, vocab 128256, Q4_K + Q6_K head, f16 KV),
    one layer, with a random 300-token context already in the cache (three attention splits)."""
    cfg = dict(synth.LLAMA3_8B, n_layers=1)
    ref, dec, wmap = build(orc, cfg, 4, synth.Q4_K, synth.Q6_K, True, 384)
    rng = np.random.default_rng(1)
    kvd = cfg["n_kv_heads"] * cfg["head_dim"]
    k = rng.standard_normal((300, kvd)).astype(np.float16).astype(np.float32)
    v = rng.standard_normal((300, kvd)).astype(np.float16).astype(np.float32)
    dec.kv_write(0, 0, k, v)
    for p in range(300):
        ref.kv_write(0, p, k[p], v[p])
    run_parity(orc, ref, dec, [12345], 8, ctx0=300)


def test_decoder_argument_errors(orc):
    ref, dec, wmap = build(orc, SMALL, 5, synth.Q4_K, synth.Q6_K, True, 32)
    with pytest.raises(tl.TlbError) as e:
        dec.step(320, 0)
    assert e.value.code == 6
    with pytest.raises(tl.TlbError) as e:
        dec.step(1, 32)
    assert e.value.code == 6
    bad = dict(SMALL, d_model=512)
    with pytest.raises(tl.TlbError):
        tl.Decoder(bad, wmap, kv_f16=True, max_seq=32)


def test_gguf_file_round_trip(orc, tmp_path):
    """Weights written as a GGUF v3 file and loaded through tlb_gguf_load give the same session."""
    tens = synth.llama_tensors(SMALL, 9, synth.Q4_K, synth.Q6_K)
    path = tmp_path / "small.gguf"
    synth.write_gguf(path, tens, metadata={"general.architecture": "llama", "general.alignment": 32,
                                           "tokenizer.ggml.tokens": [1, 2, 3]})
    m = tl.TensorMap.load(path)
    assert sorted(m.names()) == sorted(tens.keys())
    t, d, s = tens["blk.1.ffn_down.weight"]
    got = m.get("blk.1.ffn_down.weight").numpy()
    np.testing.assert_array_equal(got.view(np.uint32), orc.dequantize(t, d, got.size).reshape(s).view(np.uint32))
    np.testing.assert_array_equal(m.get("token_embd.weight").numpy().reshape(-1), tens["token_embd.weight"][1].view(np.float32))
    dec = tl.Decoder(SMALL, m, kv_f16=True, max_seq=32)
    dec2 = tl.Decoder(SMALL, tl.map_from_tensors(tens), kv_f16=True, max_seq=32)
    assert dec.step(7, 0) == dec2.step(7, 0)
    np.testing.assert_array_equal(dec.logits(), dec2.logits())
    emb_q = m.get_quantized("token_embd.weight")   # an F32 tensor as a (dense) QTensor: a tied output head
    assert emb_q.info()["type"] == synth.F32
    with pytest.raises(tl.TlbError) as e:          # the fused session itself takes tiled weights only
        tl.Decoder(SMALL, tl.map_from_tensors(synth.llama_tensors(SMALL, 9, synth.Q4_K, synth.F16)), kv_f16=True, max_seq=32)
    assert e.value.code == 7
    with pytest.raises(tl.TlbError):
        m.get("missing.weight")


# ---- whole prompts at once (tensor-core GEMMs + prompt attention) ---------------------------------------
PROMPT = 70   # > 64: two query tiles of the prompt attention, ragged second tile


@pytest.mark.parametrize("linear,head,kv_f16", [(synth.Q4_K, synth.Q6_K, True), (synth.Q4_K, synth.Q6_K, False),
                                                 (synth.Q4_0, synth.Q4_0, False), (synth.Q8_0, synth.Q8_0, True)])
def test_prefill_matches_oracle_and_continues(orc, linear, head, kv_f16):
    """The prompt in one call (reference CPU rotation: every prompt token at row 0), then greedy decoding.
    Q8_0 block scales are drawn as |N(0, 0.002)| here: with the operator sweep's |N(0, 0.01)| and uniform int8 quants a
    weight is ~0.7 in magnitude (a trained model's is ~0.02), attention scores reach the hundreds, and the f16 operand
    rounding of the prompt GEMMs (4e-4 of a row's maximum, carried by the residual stream into every later layer's cache
    rows) moves logits by the same 5-7e-2 as the model's own f16 rounding of cached K/V does.  At a trained model's
    magnitudes every format stays inside the 2e-2 gate, prompt rows in the cache included."""
    ref, dec, wmap = build(orc, SMALL, 11, linear, head, kv_f16, 128, sigma=0.002 if linear == synth.Q8_0 else None)
    rng = np.random.default_rng(5)
    prompt = [int(t) for t in rng.integers(0, SMALL["vocab"], PROMPT)]
    ref_logits = ref.forward(prompt, 0)
    nxt = dec.prefill(prompt, 0, rope_pos0=0, rope_step=0)
    assert relerr(dec.logits(), ref_logits) < LOGIT_TOL
    tok = orc.argmax_last(ref_logits)
    assert nxt == tok
    pos, worst = PROMPT, 0.0
    for s in range(16):
        ref_logits = ref.forward([tok], pos)
        nxt = dec.step(tok, pos)
        worst = max(worst, relerr(dec.logits(), ref_logits))
        tok = orc.argmax_last(ref_logits)
        assert nxt == tok
        pos += 1
    assert worst < LOGIT_TOL, worst


def test_prefill_in_chunks_equals_token_by_token(orc):
    """Per-position rotation; a prompt given as two calls at consecutive cache rows against single-token steps."""
    ref, dec, wmap = build(orc, SMALL, 12, synth.Q4_K, synth.Q6_K, True, 128)
    rng = np.random.default_rng(6)
    prompt = [int(t) for t in rng.integers(0, SMALL["vocab"], PROMPT)]
    dec.prefill(prompt[:30], 0)
    a = dec.prefill(prompt[30:], 30)
    la, ha = dec.logits(), dec.hidden()
    dec2 = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=128)
    for i, t in enumerate(prompt):
        b = dec2.step(t, i)
    assert a == b
    assert relerr(la, dec2.logits()) < 2e-3
    assert relerr(ha, dec2.hidden()) < 2e-3
    # both sessions go on identically
    assert dec.generate(a, PROMPT, 8) == dec2.generate(b, PROMPT, 8)


def test_prefill_short_prompt_and_errors(orc):
    ref, dec, wmap = build(orc, SMALL, 13, synth.Q4_K, synth.Q6_K, True, 64)
    dec2 = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=64)
    dec3 = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=64)
    short = [3, 1, 4, 1]
    a = dec3.prefill(short, 0)             # 4 tokens or fewer: the single-token chain, bit for bit
    for i, t in enumerate(short):
        b = dec2.step(t, i)
    assert a == b
    np.testing.assert_array_equal(dec3.logits().view(np.uint32), dec2.logits().view(np.uint32))
    prompt = [3, 1, 4, 1, 5]               # from 5 tokens on: all rows at once (the few-rows kernel up to 16)
    ref_logits = ref.forward(prompt, 0)
    nxt = dec.prefill(prompt, 0)
    assert relerr(dec.logits(), ref_logits) < LOGIT_TOL
    assert nxt == orc.argmax_last(ref_logits)
    with pytest.raises(tl.TlbError) as e:
        dec.prefill([SMALL["vocab"]] * 20, 0)          # token out of range
    assert e.value.code == 6
    with pytest.raises(tl.TlbError) as e:
        dec.prefill([1] * 40, 30)                      # rows 30..69 do not fit a cache of 64
    assert e.value.code == 6
    with pytest.raises(tl.TlbError) as e:
        dec.prefill([], 0)
    assert e.value.code == 8


def test_prefill_llama3_shaped_one_layer(orc):
    """Llama-3-8B layer shapes (head_dim 128, GQA 4, Q4_K + Q6_K head): a 72-token prompt (two attention tiles)
    against the oracle."""
    cfg = dict(synth.LLAMA3_8B, n_layers=1)
    ref, dec, wmap = build(orc, cfg, 4, synth.Q4_K, synth.Q6_K, True, 384)
    rng = np.random.default_rng(7)
    prompt = [int(t) for t in rng.integers(0, cfg["vocab"], 72)]
    ref_logits = ref.forward(prompt, 0)
    nxt = dec.prefill(prompt, 0, rope_pos0=0, rope_step=0)
    assert relerr(dec.logits(), ref_logits) < LOGIT_TOL
    assert nxt == orc.argmax_last(ref_logits)
    # a long prompt on the same weights: chunked at 2048 tokens, against itself token by token at the end
    long_prompt = [int(t) for t in rng.integers(0, cfg["vocab"], 2100)]
    dec3 = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=2176)
    a = dec3.prefill(long_prompt, 0)
    la = dec3.logits()
    b = dec3.step(long_prompt[-1], 2099)     # the same last token again over the cache the prompt left
    assert a == b
    assert relerr(la, dec3.logits()) < 2e-3


def test_prefill_tensor_core_attention_chunks_and_offsets():
    """head_dim 128 over an f16 cache takes the tcgen05 attention kernel from 64 tokens on.  A 300-token prompt given as 100 +
    200 tokens (the second call starts at cache row 100: three key tiles, the last one ragged, queries offset against keys)
    against the same session fed token by token; then 70 more tokens at row 300 (one ragged query tile over four key tiles)."""
    cfg = dict(synth.LLAMA3_8B, n_layers=2, vocab=1024)
    wmap = tl.map_from_tensors(synth.llama_tensors(cfg, 9, synth.Q4_K, synth.Q6_K))
    rng = np.random.default_rng(10)
    prompt = [int(t) for t in rng.integers(0, cfg["vocab"], 370)]
    dec = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=512)
    dec.prefill(prompt[:100], 0)
    a = dec.prefill(prompt[100:300], 100)
    la = dec.logits()
    dec2 = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=512)
    for i, t in enumerate(prompt[:300]):
        b = dec2.step(t, i)
    assert a == b
    assert relerr(la, dec2.logits()) < 2e-3
    a = dec.prefill(prompt[300:], 300)
    la = dec.logits()
    for i, t in enumerate(prompt[300:]):
        b = dec2.step(t, 300 + i)
    assert a == b
    assert relerr(la, dec2.logits()) < 2e-3
    assert dec.generate(a, 370, 8) == dec2.generate(b, 370, 8)


def test_prefill_f32_cache_head_dim_128():
    """f32 KV cache with head_dim 128 (the tile conversion path of the prompt attention): prompt in one call against
    the same session fed token by token."""
    cfg = dict(synth.LLAMA3_8B, n_layers=1, vocab=1024)
    wmap = tl.map_from_tensors(synth.llama_tensors(cfg, 8, synth.Q4_K, synth.Q6_K))
    rng = np.random.default_rng(9)
    prompt = [int(t) for t in rng.integers(0, cfg["vocab"], 150)]
    a_dec = tl.Decoder(cfg, wmap, kv_f16=False, max_seq=192)
    b_dec = tl.Decoder(cfg, wmap, kv_f16=False, max_seq=192)
    a = a_dec.prefill(prompt, 0)
    for i, t in enumerate(prompt):
        b = b_dec.step(t, i)
    assert a == b
    assert relerr(a_dec.logits(), b_dec.logits()) < 2e-3
    assert a_dec.generate(a, 150, 6) == b_dec.generate(b, 150, 6)


def test_decoder_sampling_on_device(orc):
    """tlb_decoder_sample_top_p on the session's logits = the tensor-level sampler on the same logits = the oracle."""
    ref, dec, wmap = build(orc, SMALL, 21, synth.Q4_K, synth.Q6_K, True, 32)
    greedy = dec.step(7, 0)
    lg = dec.logits()
    assert dec.sample_top_p(0.0, 0.9, 0.3) == greedy
    for u in (0.0, 0.11, 0.5, 0.83, 0.97):
        tok = dec.sample_top_p(0.8, 0.9, u)
        assert tok == int(tl.Tensor.from_numpy(lg).sample_top_p(0.8, 0.9, u).numpy()[0])
        assert tok == orc.sample_top_p(lg, 0.8, 0.9, u)
    with pytest.raises(tl.TlbError) as e:
        dec.sample_top_p(1.0, 0.9, 1.5)
    assert e.value.code == 8


def test_mixed_weight_types_per_tensor_and_layer(orc):
    """A Q4_K_M-like file: attn_v and ffn_down of layer 0 in Q6_K, attn_k of layer 1 in Q8_0, the rest Q4_K.
    Decode steps and a whole prompt against the oracle."""
    mixed = {"blk.0.attn_v.weight": synth.Q6_K, "blk.0.ffn_down.weight": synth.Q6_K, "blk.1.attn_k.weight": synth.Q8_0}
    tens = synth.llama_tensors(SMALL, 31, synth.Q4_K, synth.Q6_K, overrides=mixed)
    ref = orc.Llama(dict(SMALL, kv_f16=1, max_seq=128), {k: (t, d) for k, (t, d, s) in tens.items()})
    wmap = tl.map_from_tensors(tens)
    dec = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=128)
    run_parity(orc, ref, dec, [3, 200, 41], 12)
    ref2 = orc.Llama(dict(SMALL, kv_f16=1, max_seq=128), {k: (t, d) for k, (t, d, s) in tens.items()})
    dec2 = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=128)
    prompt = [int(t) for t in np.random.default_rng(32).integers(0, SMALL["vocab"], 50)]
    ref_logits = ref2.forward(prompt, 0)
    nxt = dec2.prefill(prompt, 0, rope_pos0=0, rope_step=0)
    assert relerr(dec2.logits(), ref_logits) < LOGIT_TOL
    assert nxt == orc.argmax_last(ref_logits)


def test_decoder_sizes_from_gguf_metadata(tmp_path):
    """Model sizes read from the file's metadata give the session the hard-coded sizes give."""
    tens = synth.llama_tensors(SMALL, 10, synth.Q4_K, synth.Q6_K)
    path = tmp_path / "meta.gguf"
    synth.write_gguf(path, tens, metadata={
        "general.architecture": "llama", "general.alignment": 32, "llama.block_count": SMALL["n_layers"],
        "llama.embedding_length": SMALL["d_model"], "llama.attention.head_count": SMALL["n_heads"],
        "llama.attention.head_count_kv": SMALL["n_kv_heads"], "llama.feed_forward_length": SMALL["ffn"],
        "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.rope.freq_base": 10000.0,
        "llama.rope.dimension_count": SMALL["head_dim"]})
    m = tl.TensorMap.load(path)
    assert m.meta_string("general.architecture") == "llama"
    assert m.meta_number("llama.block_count") == SMALL["n_layers"]
    assert m.meta_string("llama.block_count") is None
    with pytest.raises(tl.TlbError) as e:
        m.meta_number("llama.no_such_key")
    assert e.value.code == 6
    cfg = m.decoder_cfg()
    for k, v in SMALL.items():
        assert cfg[k] == pytest.approx(v, rel=1e-6), k      # attn_scale: the literal 0.125 for head_dim 64
    dec = tl.Decoder(cfg, m, kv_f16=True, max_seq=32)
    dec2 = tl.Decoder(SMALL, tl.map_from_tensors(tens), kv_f16=True, max_seq=32)
    assert dec.step(7, 0) == dec2.step(7, 0)
    np.testing.assert_array_equal(dec.logits(), dec2.logits())
    with pytest.raises(tl.TlbError) as e:
        tl.map_from_tensors(tens).decoder_cfg()        # no metadata in a map built tensor by tensor
    assert e.value.code == 8


def test_sampled_generation_on_device(orc):
    """tlb_decoder_generate_sampled: temperature / top-k / top-p with the draws made on the device from (seed, step).  The same
    session driven from the host - logits read back, the oracle's sampler, the draw of tlb_rng_uniform(seed, step) - gives the
    same tokens; the same seed repeats them, another seed does not."""
    ref, dec, wmap = build(orc, SMALL, 61, synth.Q4_K, synth.Q6_K, True, 64, sigma=0.001)
    temp, top_k, top_p, seed = 25.0, 12, 0.95, 1234      # the synthetic model's logits span ~80: a temperature that leaves a choice
    gen = dec.generate_sampled(7, 0, 20, temp, top_k, top_p, seed)
    host = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=64)
    tok, toks = 7, []
    for i in range(20):
        host.step(tok, i)
        lg = host.logits()
        u = tl.rng_uniform(seed, i)
        assert u == orc.rng_uniform(seed, i)
        tok = orc.sample_top_k_top_p(lg, temp, top_k, top_p, u)
        dev_tok = int(tl.Tensor.from_numpy(lg).sample_top_k_top_p(temp, top_k, top_p, u).numpy()[0])
        assert dev_tok == tok
        toks.append(tok)
    assert gen == toks
    assert len(set(gen)) > 3                                                         # a real draw, not an argmax in disguise
    assert dec.generate_sampled(7, 0, 20, temp, top_k, top_p, seed) == gen           # repeatable
    assert dec.generate_sampled(7, 0, 20, temp, top_k, top_p, seed + 1) != gen       # a different stream of draws
    assert dec.generate_sampled(7, 0, 8, 0.0, top_k, top_p, seed) == dec.generate(7, 0, 8)   # temp <= 0: greedy
    assert dec.generate_sampled(7, 0, 8, temp, 1, top_p, seed) == dec.generate(7, 0, 8)     # top_k 1: greedy
