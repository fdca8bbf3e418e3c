"""The TL chatbot's forward pass, op by op, over the per-op C ABI.

Mirrors examples/apps/llama3/chatbot_llama3.tl:48-125,220-236 (and examples/apps/tinyllama/chatbot.tl:33-113): the
same calls in the same order - embedding, rms_norm + mul, tl_qtensor_matmul, reshape, narrow, apply_rope, transpose,
kv cache get / cat_4d / update, repeat_interleave, matmul_4d, scale, causal mask, softmax, silu, mul, add, sample,
item_i64 - each one a call through libtlb200's mirror of the runtime symbol.  This is the route an UNMODIFIED TL program
takes behind TL_DEVICE=cuda: one kernel (or more) per op, a cache that grows by concatenation.  The fused session
(tl_b200.Decoder) computes the same tokens in 5 launches per layer; this module exists to measure the difference and to
check that both routes agree.
"""
import ctypes as C

import numpy as np

from . import KVCache, Tensor, ROPE_CPU, TIE_LAST, check, lib
from ._lib import DecoderCfg


class PerOpLlama:
    def __init__(self, cfg, weights, max_seq=8192, tie=TIE_LAST):
        self.cfg = cfg
        self.w = weights
        self.tie = tie
        self.H, self.KVH, self.D = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
        # Tensor::rope_new_cos(128, 8192, 500000.0) once per program (chatbot_llama3.tl:196-197)
        self.cos = Tensor.rope_new_cos(self.D, max_seq, cfg["rope_base"], ROPE_CPU)
        self.sin = Tensor.rope_new_sin(self.D, max_seq, cfg["rope_base"], ROPE_CPU)
        self.emb = weights.get("token_embd.weight")
        self.on = weights.get_1d("output_norm.weight")
        self.oh = weights.get_quantized("output.weight")
        self.cache = KVCache(cfg["n_layers"])
        # Block::from_map looks the tensors up again for every token (chatbot_llama3.tl:229); the handles are the same
        # objects each time, so they are looked up once here
        self.blocks = []
        for li in range(cfg["n_layers"]):
            p = "blk.%d." % li
            self.blocks.append(dict(
                an=weights.get_1d(p + "attn_norm.weight"), ffn=weights.get_1d(p + "ffn_norm.weight"),
                q=weights.get_quantized(p + "attn_q.weight"), k=weights.get_quantized(p + "attn_k.weight"),
                v=weights.get_quantized(p + "attn_v.weight"), o=weights.get_quantized(p + "attn_output.weight"),
                g=weights.get_quantized(p + "ffn_gate.weight"), u=weights.get_quantized(p + "ffn_up.weight"),
                d=weights.get_quantized(p + "ffn_down.weight")))

    def seed_cache(self, layer, k, v):
        """Cache rows from outside (a synthetic context): k, v [T, KVH * D] -> tensors [1, KVH, T, D] as the program holds them."""
        T = k.shape[0]
        k4 = np.ascontiguousarray(k.reshape(T, self.KVH, self.D).transpose(1, 0, 2)[None], dtype=np.float32)
        v4 = np.ascontiguousarray(v.reshape(T, self.KVH, self.D).transpose(1, 0, 2)[None], dtype=np.float32)
        self.cache.update(layer, Tensor.from_numpy(k4), Tensor.from_numpy(v4))

    def _norm(self, x, w):
        return x.rms_norm(None, self.cfg["eps"]).mul(w)          # RMSNorm::forward: rms_norm then mul by the weight

    def _attention(self, b, x, sl, li, sp):
        H, KVH, D = self.H, self.KVH, self.D
        q4 = x.matmul_quantized(b["q"]).reshape([1, sl, H, D])
        k4 = x.matmul_quantized(b["k"]).reshape([1, sl, KVH, D])
        v4 = x.matmul_quantized(b["v"]).reshape([1, sl, KVH, D])
        cs = self.cos.narrow(0, sp, sl)
        ss = self.sin.narrow(0, sp, sl)
        qr = q4.apply_rope(cs, ss, ROPE_CPU)
        kr = k4.apply_rope(cs, ss, ROPE_CPU)
        kt = kr.transpose(1, 2)
        vt = v4.transpose(1, 2)
        k_tot = kt if sp == 0 else self.cache.get_k(li).cat_4d(kt, 2)
        v_tot = vt if sp == 0 else self.cache.get_v(li).cat_4d(vt, 2)
        self.cache.update(li, k_tot, v_tot)
        qt = qr.transpose(1, 2)
        rep = H // KVH
        kw = k_tot.repeat_interleave(rep, 1)
        vw = v_tot.repeat_interleave(rep, 1)
        sm = qt.matmul_4d(kw.transpose(2, 3)).scale(self.cfg["attn_scale"])
        if sl > 1:
            sm = sm.add_4d(Tensor.new_causal_mask(sl).reshape([1, 1, sl, sl]))
        ao = sm.softmax(3).matmul_4d(vw).transpose(1, 2)
        return ao.reshape([sl, H * D]).matmul_quantized(b["o"])

    def forward(self, tokens, start_pos):
        """One pass over `tokens` (f32-encoded ids, as TL holds them) from cache row start_pos; returns the logits tensor [sl, vocab]."""
        sl = len(tokens)
        x = Tensor.from_numpy(np.asarray(tokens, dtype=np.float32)).embedding(self.emb)
        for li, b in enumerate(self.blocks):
            attn_out = self._attention(b, self._norm(x, b["an"]), sl, li, start_pos)
            h = x.add(attn_out)
            y = self._norm(h, b["ffn"])
            mu = y.matmul_quantized(b["g"]).silu().mul(y.matmul_quantized(b["u"]))
            x = h.add(mu.matmul_quantized(b["d"]))
        return self._norm(x, self.on).matmul_quantized(self.oh)

    def step_native(self, tokens, start_pos):
        """The same step issued by the library's own native driver (tlb_chatbot_step_per_op): the same per-op entry points
        in the same order, without this interpreter's time per call.  Returns the token id; last_logits as in step()."""
        c = self.cfg
        dc = DecoderCfg(n_layers=c["n_layers"], d_model=c["d_model"], n_heads=c["n_heads"], n_kv_heads=c["n_kv_heads"],
                        head_dim=c["head_dim"], ffn=c["ffn"], vocab=c["vocab"], eps=c["eps"], rope_base=c["rope_base"],
                        attn_scale=c["attn_scale"], kv_f16=0, max_seq=0, tie_rule=self.tie, tp_size=1, tp_rank=0, batch=1)
        ids = np.ascontiguousarray(np.asarray(tokens, dtype=np.float32))
        nxt, lg = C.c_int64(), C.c_void_p()
        check(lib().tlb_chatbot_step_per_op(self.w.h, self.cache.h, self.cos.h, self.sin.h, C.byref(dc), ids.ctypes.data_as(C.c_void_p),
                                            len(ids), start_pos, C.byref(nxt), C.byref(lg)))
        self.last_logits = Tensor(lg)
        return int(nxt.value)

    def step(self, tokens, start_pos):
        """forward + lo.narrow(0, batch_len - 1, 1).sample(...).item_i64(): the token id on the host."""
        lo = self.forward(tokens, start_pos)
        self.last_logits = lo.narrow(0, len(tokens) - 1, 1)
        return self.last_logits.sample(0.0, 0.9, self.tie).item_i64()
