"""Batch sessions: several sequences share one pass over the weights per step (the few-rows kernel) and keep their own
caches and positions.  Every sequence is checked against its own instance of the oracle: logits within the 2e-2 gate,
greedy tokens identical (where the oracle's two best logits are closer than the measured error, either may come out)."""
import numpy as np
import pytest

import tl_b200 as tl
from tl_b200 import synth

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-2
SMALL = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=320,
             eps=1e-5, rope_base=10000.0, attn_scale=0.125)


def relerr(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def same_or_tie(got, ref_logits, err):
    want = int(np.flatnonzero(ref_logits == ref_logits.max())[-1])
    if got == want:
        return True
    top2 = np.sort(ref_logits)[-2:]
    return (top2[1] - top2[0]) < 2 * err * np.max(np.abs(ref_logits))


@pytest.mark.parametrize("linear,head,kv_f16,batch", [(synth.Q4_K, synth.Q6_K, True, 2), (synth.Q4_0, synth.Q4_0, False, 3), (synth.Q8_0, synth.Q8_0, True, 5)])
def test_batch_decode_matches_per_sequence_oracles(orc, linear, head, kv_f16, batch):
    sigma = 0.002 if linear == synth.Q8_0 else None      # weights of a trained model's magnitude (see test_gpu_decoder)
    tens = synth.llama_tensors(SMALL, 41, linear, head, scale_sigma=sigma)
    wmap = tl.map_from_tensors(tens)
    dec = tl.Decoder(SMALL, wmap, kv_f16=kv_f16, max_seq=96, batch=batch)
    rng = np.random.default_rng(batch)
    lens = [20, 37, 5, 18, 29][:batch]
    prompts = [[int(t) for t in rng.integers(0, SMALL["vocab"], n)] for n in lens]
    refs = [orc.Llama(dict(SMALL, kv_f16=int(kv_f16), max_seq=96), {k: (t, d) for k, (t, d, s) in tens.items()}) for _ in range(batch)]
    toks, pos = [], []
    for b in range(batch):
        rl = refs[b].forward(prompts[b], 0)                       # reference CPU rotation: the whole prompt at row 0
        nxt = dec.prefill_seq(b, prompts[b], 0, rope_pos0=0, rope_step=0)
        lg = dec.logits_batch()[b]
        err = relerr(lg, rl)
        assert err < LOGIT_TOL, (b, err)
        assert same_or_tie(nxt, rl, err)
        toks.append(orc.argmax_last(rl))
        pos.append(lens[b])
    worst = 0.0
    hist = []
    for step in range(12):
        nxt = dec.step_batch(toks, pos)
        lgs = dec.logits_batch()
        new = []
        for b in range(batch):
            rl = refs[b].forward([toks[b]], pos[b])
            err = relerr(lgs[b], rl)
            worst = max(worst, err)
            assert same_or_tie(nxt[b], rl, err), (step, b)
            new.append(orc.argmax_last(rl))
        hist.append(list(nxt))
        toks, pos = new, [p + 1 for p in pos]
    assert worst < LOGIT_TOL, worst
    assert len(hist) == 12


WIDE = dict(n_layers=1, d_model=1024, n_heads=8, n_kv_heads=2, head_dim=128, ffn=1024, vocab=512,
            eps=1e-5, rope_base=500000.0, attn_scale=0.08839)


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 128), (8, 1, 128), (8, 8, 128), (16, 4, 64)])
def test_batch_attention_key_ranges_and_head_groups(orc, heads, kv_heads, head_dim):
    """head_dim 128 with 4, 8 and 1 query heads per KV head, head_dim 64 with 4, and a cache long enough that the batch attention cuts a
    sequence's rows into several key ranges (several CTAs per sequence and KV head, merged by the last one): contexts of
    300, 3 and 131 rows in one batch - sixteen-key blocks spread over many warps, warps and whole CTAs without a block,
    a last block with one row.  Every sequence against its own oracle, as above."""
    cfg = dict(WIDE, n_heads=heads, n_kv_heads=kv_heads, head_dim=head_dim, attn_scale=float(head_dim) ** -0.5)
    tens = synth.llama_tensors(cfg, 61 + kv_heads, synth.Q4_K, synth.Q6_K)
    wmap = tl.map_from_tensors(tens)
    batch, lens = 3, [300, 3, 131]
    dec = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=640, batch=batch)
    rng = np.random.default_rng(17 + kv_heads)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in lens]
    refs = [orc.Llama(dict(cfg, kv_f16=1, max_seq=640), {k: (t, d) for k, (t, d, s) in tens.items()}) for _ in range(batch)]
    toks, pos = [], []
    for b in range(batch):
        rl = refs[b].forward(prompts[b], 0)
        nxt = dec.prefill_seq(b, prompts[b], 0, rope_pos0=0, rope_step=0)
        err = relerr(dec.logits_batch()[b], rl)
        assert err < LOGIT_TOL, (b, err)
        assert same_or_tie(nxt, rl, err)
        toks.append(orc.argmax_last(rl))
        pos.append(lens[b])
    worst = 0.0
    for step in range(20):                                   # the 3-row sequence crosses its first block border at row 16
        nxt = dec.step_batch(toks, pos)
        lgs = dec.logits_batch()
        new = []
        for b in range(batch):
            rl = refs[b].forward([toks[b]], pos[b])
            err = relerr(lgs[b], rl)
            worst = max(worst, err)
            assert same_or_tie(nxt[b], rl, err), (step, b)
            new.append(orc.argmax_last(rl))
        toks, pos = new, [p + 1 for p in pos]
    assert worst < LOGIT_TOL, worst


def test_generate_batch_feeds_tokens_back_on_the_device(orc):
    tens = synth.llama_tensors(SMALL, 42, synth.Q4_K, synth.Q6_K)
    wmap = tl.map_from_tensors(tens)
    a = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=64, batch=4)
    b = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=64, batch=4)
    rng = np.random.default_rng(7)
    kvd = SMALL["n_kv_heads"] * SMALL["head_dim"]
    starts = [3, 9, 0, 6]
    for seq in range(4):
        for layer in range(SMALL["n_layers"]):
            k = rng.standard_normal((max(1, starts[seq]), kvd), dtype=np.float32)
            v = rng.standard_normal((max(1, starts[seq]), kvd), dtype=np.float32)
            if starts[seq]:
                a.kv_write_seq(seq, layer, 0, k, v)
                b.kv_write_seq(seq, layer, 0, k, v)
    first = [11, 22, 33, 44]
    gen = a.generate_batch(first, starts, 10)
    assert gen.shape == (10, 4)
    toks, pos = first, list(starts)
    for i in range(10):
        toks = b.step_batch(toks, pos)
        assert toks == [int(t) for t in gen[i]], i
        pos = [p + 1 for p in pos]
    np.testing.assert_array_equal(a.logits_batch().view(np.uint32), b.logits_batch().view(np.uint32))
    # sequence 0 of a batch session is the sequence the single-sequence calls see
    c = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=64, batch=2)
    d = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=64)
    assert c.step(5, 0) == d.step(5, 0)
    np.testing.assert_array_equal(c.logits().view(np.uint32), d.logits().view(np.uint32))


def test_batch_argument_errors():
    tens = synth.llama_tensors(SMALL, 43, synth.Q4_K, synth.Q6_K)
    wmap = tl.map_from_tensors(tens)
    single = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=32)
    with pytest.raises(tl.TlbError) as e:
        single.step_batch([1], [0])
    assert e.value.code == 8
    dec = tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=32, batch=2)
    with pytest.raises(tl.TlbError) as e:
        dec.step_batch([1, SMALL["vocab"]], [0, 0])
    assert e.value.code == 6
    with pytest.raises(tl.TlbError) as e:
        dec.step_batch([1, 2], [0, 32])
    assert e.value.code == 6
    with pytest.raises(tl.TlbError) as e:
        dec.prefill_seq(2, [1, 2, 3], 0)
    assert e.value.code == 6
    with pytest.raises(tl.TlbError) as e:
        tl.Decoder(SMALL, wmap, kv_f16=True, max_seq=32, batch=65)
    assert e.value.code == 8
    odd = dict(SMALL, ffn=384)          # not a multiple of 256: the GEMM path does not take it
    with pytest.raises(tl.TlbError) as e:
        tl.Decoder(odd, tl.map_from_tensors(synth.llama_tensors(dict(odd, ffn=512), 43, synth.Q4_K, synth.Q6_K)), kv_f16=True, max_seq=32, batch=2)
    assert e.value.code in (1, 8)
