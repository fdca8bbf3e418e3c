"""Benchmark of the quantized Llama decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c0|c1|c3|small|...]

A step is one decoded token (batch 1).  Default workload c2: Llama-3-8B-shaped decoder, Q4_K linear
layers + Q6_K output head, f16 KV cache holding a 2048-token random context, greedy decoding; weights
are seeded synthetic GGUF blocks (no model file is needed or read).  Prints ONE JSON line (rank 0).

  value     tokens/s with everything resident in HBM: K graph replays with the token fed back on the
            device, CUDA events on the library's stream, max over ranks.
  e2e       tokens/s through tlb_decoder_step with HOST token in / HOST token out every step.
  roofline  the Q4_K streaming matvec, timed live over weight sets rotated through > 2x L2.
  cpu_baseline / --impl reference: the reference CPU path's per-token linear algebra (cached f32
            transposed weights, one thread, strided inner loop) on a bounded sample of output columns.
  sweep     (N = 1) the operator sweep of config C1: Q8_0 and Q4_K on the five weight shapes with 1 / 4 / 16 / 512
            activation rows through tlb_qtensor_matmul, weights rotated through > 2x L2.
  per_op    one decode step issued op by op through the per-op C ABI in the TL program's order: what an unmodified
            chatbot gets, beside the fused session's number.
  prefill   config C3: 8 sequences x 2048 prompt tokens through a batch session.
With N > 1 every rank decodes its own replica of the 8B model (no exchange step on this path): weak scaling; the
headline stays that.  A `tp` object is added: the 70B-shaped model of config C4 split over the N ranks (tensor
parallel, one process per GPU), its per-token all-reduce cost, and the same model on one GPU.
--workload c1 / c3 / qgemm / qrows / prefill-2layer run only that part (small cases for profiler captures among them).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (config, linear type, head type, kv_f16, context, description)
    "c2": ("LLAMA3_8B", 12, 14, True, 2048, "Llama-3-8B-shaped decode, Q4_K + Q6_K head, f16 KV, ctx 2048, batch 1"),
    "c0": ("TINYLLAMA", 2, 2, False, 128, "TinyLlama-1.1B-shaped decode, Q4_0, f32 KV, ctx 128, batch 1"),
    # the c2 shapes with 4 layers instead of 32: about 1.3 GB on the device, for profiler captures
    "c2-4layer": ("LLAMA3_8B:4", 12, 14, True, 2048, "Llama-3-8B-shaped decode cut to 4 layers, Q4_K + Q6_K head, f16 KV, ctx 2048, batch 1"),
    "small": (None, 12, 14, True, 64, "2-layer d512 test model, Q4_K + Q6_K head, f16 KV, ctx 64, batch 1"),
}
SMALL_CFG = dict(n_layers=2, d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=1000,
                 eps=1e-5, rope_base=10000.0, attn_scale=0.125)


def workload_cfg(name):
    from tl_b200 import synth
    cfg_name, lt, ht, kv16, ctx, desc = WORKLOADS[name]
    if cfg_name is None:
        cfg = SMALL_CFG
    elif ":" in cfg_name:
        base, layers = cfg_name.split(":")
        cfg = dict(getattr(synth, base), n_layers=int(layers))
    else:
        cfg = getattr(synth, cfg_name)
    return cfg, lt, ht, kv16, ctx, desc


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        clocks, reasons = [], set()
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                out["sm_max_mhz"] = float(parts[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        self.f.close()
        os.unlink(self.f.name)
        if clocks:
            out["sm_mhz"] = statistics.median(clocks)
            out["samples"] = len(clocks)
        out["reasons"] = sorted(reasons)
        return out


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return None, 0, 1
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", "0"))
    backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    dist.init_process_group(backend, init_method="env://")
    return dist, dist.get_rank(), dist.get_world_size()


def reduce_max(dist, value):
    if dist is None:
        return value
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(dist):
    if dist is not None:
        dist.barrier()


def whole_job_rate(world, steps, ms_max):
    """Tokens per second of the whole job: every rank decodes `steps` tokens of its own replica in the
    same (slowest rank's) time."""
    return world * steps / (ms_max / 1e3)


def profile_traffic_ratio():
    """DRAM bytes per algorithmic byte of the streaming matvec, read from the committed ncu summary of the 4-layer case
    (rows `algorithmic bytes`, `dram__bytes_read.sum`, `dram__bytes_write.sum` of its table, summed over the captured
    launches).  None when the summary is missing or has no such rows."""
    path = os.path.join(ROOT, "profiles", "qmatvec_q4k_llama3-8b-shapes_4layer_ncu-full.md")
    try:
        rows = {}
        for line in open(path):
            cells = [c.strip() for c in line.strip().strip("|").split("|")]
            if len(cells) >= 2:
                rows[cells[0]] = cells[1:]

        def mb(cells):
            out = []
            for c in cells:
                c = c.replace(",", "")
                num = float(c.split()[0])
                out.append(num * 1e6 if "MB" in c else num)
            return out
        algo = [k for k in rows if k.startswith("algorithmic bytes")]
        if not algo or "dram__bytes_read.sum" not in rows or "dram__bytes_write.sum" not in rows:
            return None
        a, r, w = mb(rows[algo[0]]), mb(rows["dram__bytes_read.sum"]), mb(rows["dram__bytes_write.sum"])
        return (sum(r) + sum(w)) / sum(a)
    except Exception:
        return None


# ---------------------------------------------------------------- CPU baseline (oracle port of the reference CPU path)

def cpu_token_time(cfg, frac, rng, cache):
    """Seconds the reference's CPU matmuls (crates/tl_cpu/src/tensor.rs:1284-1306 over the cached transposed
    f32 weights, crates/tl_runtime/src/system.rs:193-222) take for a fraction `frac` of the output columns
    of one layer's seven matvecs and of the head, one thread.  Returns (t_layer_sample, t_head_sample)."""
    from oracle import oracle
    d, qd = cfg["d_model"], cfg["n_heads"] * cfg["head_dim"]
    kvd, f, v = cfg["n_kv_heads"] * cfg["head_dim"], cfg["ffn"], cfg["vocab"]
    shapes = [(qd, d, 1), (kvd, d, 2), (d, qd, 1), (f, d, 2), (d, f, 1)]   # (n_out, k_in, count per layer)
    t_layer = 0.0
    for n, k, cnt in shapes + [(v, d, 0)]:
        cols = max(1, int(round(n * frac)))
        key = (n, k, cols)
        if key not in cache:
            w = np.zeros((k, n), dtype=np.float32)
            w[:, :cols] = rng.standard_normal((k, cols), dtype=np.float32)   # touch only the sampled columns
            cache[key] = (w, rng.standard_normal(k, dtype=np.float32))
        w, x = cache[key]
        t0 = time.perf_counter()
        oracle.matmul_cached_t_cols(w, x, 0, cols)
        dt = (time.perf_counter() - t0) * (n * frac / cols)
        if cnt:
            t_layer += dt * cnt
        else:
            t_head = dt
    return t_layer, t_head


def cpu_baseline(cfg, budget_s, steps=1):
    from oracle import oracle
    oracle.lib()
    rng = np.random.default_rng(0)
    cache = {}
    frac = 1.0 / 512
    t0 = time.perf_counter()
    tl_, th_ = cpu_token_time(cfg, frac, rng, cache)          # calibration (also pages the sample in)
    per_unit = (tl_ + th_) / frac
    target = max(budget_s / max(1, steps), 0.05)
    frac2 = min(1.0, max(frac, target / max(per_unit, 1e-9)))
    cache.clear()
    vals = []
    for _ in range(steps):
        tl_, th_ = cpu_token_time(cfg, frac2, rng, cache)
        tok_time = (cfg["n_layers"] * tl_ + th_) / frac2
        vals.append(1.0 / tok_time)
    return {"value": statistics.mean(vals), "unit": "tokens/s", "cores": 1, "kind": "port",
            "sample": "one thread (the reference CPU back end has no threading or SIMD); %.4f of the output columns of one "
                      "layer's 7 matvecs and of the head, f32 transposed weights, scaled to %d layers + head; attention, "
                      "norms and dequantisation (cached by the reference) excluded; %.1f s of CPU work"
                      % (frac2, cfg["n_layers"], time.perf_counter() - t0)}, vals


# ---------------------------------------------------------------- our arm

def build_session(name, seed=1234):
    import tl_b200 as tl
    from tl_b200 import synth
    cfg, lt, ht, kv16, ctx, desc = workload_cfg(name)
    m = tl.TensorMap.new()
    for tname, t, shape in synth.llama_tensor_specs(cfg, lt, ht):
        m.add(tname, t, shape, synth.make_tensor(tname, t, shape, seed))
    return tl, cfg, m, kv16, ctx, desc


def fill_context(dec, cfg, ctx, seed=99):
    rng = np.random.default_rng(seed)
    kvd = cfg["n_kv_heads"] * cfg["head_dim"]
    for layer in range(cfg["n_layers"]):
        k = rng.standard_normal((ctx, kvd), dtype=np.float32)
        v = rng.standard_normal((ctx, kvd), dtype=np.float32)
        dec.kv_write(layer, 0, k, v)


def _elapsed_ms(tl, ev0, ev1):
    import ctypes as C
    ms = C.c_float()
    tl.check(tl.lib().tlb_event_elapsed_ms(ev0, ev1, C.byref(ms)))
    return float(ms.value)


def measure_prefill(tl, cfg, wmap, kv16, ev, peaks, batch=8, tokens=2048):
    """Config C3: `batch` sequences x `tokens` prompt ids through a batch session (tlb_decoder_prefill_seq per sequence:
    tensor-core GEMMs over each prompt, causal attention with the f16 KV-cache write), timed with CUDA events after one
    warm-up prompt; arithmetic = linear layers + causal attention of all sequences (the head runs on the last token)."""
    if tokens <= 0:
        return None
    L = tl.lib()
    dec = tl.Decoder(cfg, wmap, kv_f16=kv16, max_seq=tokens + 16, batch=max(2, batch))
    rng = np.random.default_rng(4321)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], tokens)] for _ in range(batch)]
    dec.prefill_seq(0, prompts[0], 0, read=False)
    tl.sync()
    tl.check(L.tlb_event_record(ev[0]))
    for b in range(batch):
        dec.prefill_seq(b, prompts[b], 0, read=False)
    tl.check(L.tlb_event_record(ev[1]))
    tl.sync()
    ms = _elapsed_ms(tl, ev[0], ev[1])
    dec.destroy()
    dm, qd, kvd, F = cfg["d_model"], cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["ffn"]
    lin = 2.0 * batch * tokens * cfg["n_layers"] * (dm * (qd + 2 * kvd) + qd * dm + 3 * dm * F)
    att = 4.0 * batch * cfg["n_layers"] * cfg["n_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2
    tf = (lin + att) / (ms * 1e-3) / 1e12
    peak = peaks.get("bf16_tflops", 1590.0)
    return {"workload": "c3: %d x %d prompt tokens, all %d layers" % (batch, tokens, cfg["n_layers"]), "tokens": batch * tokens, "ms": round(ms, 2),
            "tokens_per_s": round(batch * tokens / (ms * 1e-3), 0), "tflops": round(tf, 1), "bound": "tensor", "peak_tflops": peak,
            "frac": round(tf / peak, 4),
            "note": "f16 tcgen05 GEMMs with on-the-fly dequantisation (weights in tensor memory) + tcgen05 attention (scores, probabilities and output in tensor memory); head on each sequence's last token"}


SWEEP_SHAPES = [(2048, 2048), (4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]   # (N out, K in): the config's K x N


def measure_sweep(tl, ev, peaks, types=(8, 12), rows=(1, 4, 16, 512), shapes=SWEEP_SHAPES, iters=None):
    """Config C1: y = x . W^T through tlb_qtensor_matmul for every format x shape x row count.  Each shape keeps enough
    distinct device copies of its weight to exceed 2x L2 (256 MB) and the timed calls rotate through them, so every
    call streams its weight from HBM.  Bytes = N K bpw + 4 M K + 4 M N; flops = 2 M N K."""
    from tl_b200 import synth
    L = tl.lib()
    hbm, tens = peaks["hbm_gbs"], peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", 1590.0))
    out = []
    rng = np.random.default_rng(7)
    for t in types:
        for n, k in shapes:
            w = synth.random_quant(t, n, k, rng)
            wbytes = w.size
            copies = max(2, int(np.ceil((256 << 20) / wbytes)))
            qs = [tl.QTensor.from_gguf_bytes(t, n, k, w) for _ in range(copies)]
            del w
            for m in rows:
                x = tl.Tensor.from_numpy(rng.standard_normal((m, k), dtype=np.float32))
                reps = iters or max(copies, min(200, int(2e9 / (wbytes + 1)) + 8))
                for i in range(min(3, copies) + 2):
                    x.matmul_quantized(qs[i % copies]).release()
                tl.sync()
                tl.check(L.tlb_event_record(ev[0]))
                for i in range(reps):
                    x.matmul_quantized(qs[i % copies]).release()
                tl.check(L.tlb_event_record(ev[1]))
                tl.sync()
                us = _elapsed_ms(tl, ev[0], ev[1]) * 1e3 / reps
                nbytes = wbytes + 4 * m * k + 4 * m * n
                e = {"type": synth.TYPE_NAMES[t], "n": n, "k": k, "m": m, "us": round(us, 2), "GBs": round(nbytes / us / 1e3, 1),
                     "frac_hbm": round(nbytes / us / 1e3 / hbm, 4), "copies": copies}
                if m >= 512:
                    tf = 2.0 * m * n * k / us / 1e6
                    e.update({"tflops": round(tf, 1), "frac_tensor_sustained": round(tf / tens, 4)})
                out.append(e)
                x.release()
            for q in qs:
                q.release()
    return out


def measure_per_op(tl, cfg, wmap, ctx, steps, ev):
    """One decode step issued op by op through the per-op C ABI in the TL program's order
    (examples/apps/llama3/chatbot_llama3.tl:66-125,220-236), with a context of `ctx` rows already in the program's cache:
    what an unmodified chatbot gets behind this library.  Host token in, host token out (item_i64), wall clock."""
    from tl_b200.chatbot import PerOpLlama
    bot = PerOpLlama(cfg, wmap, max_seq=ctx + 2 * steps + 16)
    rng = np.random.default_rng(99)
    kvd = cfg["n_kv_heads"] * cfg["head_dim"]
    for layer in range(cfg["n_layers"]):
        bot.seed_cache(layer, rng.standard_normal((ctx, kvd), dtype=np.float32), rng.standard_normal((ctx, kvd), dtype=np.float32))
    tok, pos = 1 % cfg["vocab"], ctx
    for _ in range(2):
        tok = bot.step([tok], pos)
        pos += 1
    tl.sync()
    l0 = tl.kernel_launches()
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = bot.step([tok], pos)
        pos += 1
    dt = (time.perf_counter() - t0) / steps
    launches = (tl.kernel_launches() - l0) // steps
    # the same calls from native code (tlb_chatbot_step_per_op), as the compiled TL program issues them
    for _ in range(2):
        tok = bot.step_native([tok], pos)
        pos += 1
    tl.sync()
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = bot.step_native([tok], pos)
        pos += 1
    dn = (time.perf_counter() - t0) / steps
    return {"tokens_per_s": round(1.0 / dn, 2), "ms_per_step": round(dn * 1e3, 3), "steps": steps, "kernel_launches_per_step": int(launches),
            "through_python": {"tokens_per_s": round(1.0 / dt, 2), "ms_per_step": round(dt * 1e3, 3)},
            "note": "one tlb_* call per TL op in the program's order, issued from native code (the ctypes route, with the "
                    "interpreter's time per call, beside it); f32 KV cache grown by cat_4d (the whole cache is copied every step, "
                    "as the program writes it), GQA expansion materialised; the fused session is the `value` / `e2e` of this line"}


# ---------------------------------------------------------------- tensor parallelism (config C4)

def build_tp_map(tl, cfg, rank, world, seed=4321):
    """70B-shaped weights for one rank.  Every layer holds the same seeded random tensors (generated once, uploaded per
    layer into device tensors of their own, so nothing is shared in HBM or L2); the embedding repeats 4096 random rows."""
    from tl_b200 import synth
    m = tl.TensorMap.new()
    layer = {}
    for name, t, shape in synth.llama_tensor_specs(dict(cfg, n_layers=1), 12, 14):
        if name == "token_embd.weight":
            rows = (synth.make_tensor("token_embd.weight", 0, (4096, shape[1]), seed)).view(np.float32).reshape(4096, shape[1])
            data = np.concatenate([rows] * ((shape[0] + 4095) // 4096))[:shape[0]]
            m.add_tp(name, t, shape, data, rank, world)
        elif name.startswith("blk.0."):
            layer[name[6:]] = (t, synth.make_tensor(name, t, shape, seed), shape)
        else:
            m.add_tp(name, t, shape, synth.make_tensor(name, t, shape, seed), rank, world)
    for li in range(cfg["n_layers"]):
        for suffix, (t, data, shape) in layer.items():
            m.add_tp("blk.%d.%s" % (li, suffix), t, shape, data, rank, world)
    return m


def time_generate(tl, dec, ev, first, ctx, warm, steps, batch=None):
    L = tl.lib()
    if batch:
        dec.generate_batch([first] * batch, [ctx] * batch, warm, read=False)
    else:
        dec.generate(first, ctx, warm, read=False)
    tl.sync()
    tl.check(L.tlb_event_record(ev[0]))
    if batch:
        dec.generate_batch([first] * batch, [ctx + warm] * batch, steps, read=False)
    else:
        dec.generate(first, ctx + warm, steps, read=False)
    tl.check(L.tlb_event_record(ev[1]))
    tl.sync()
    return _elapsed_ms(tl, ev[0], ev[1]) / steps


def measure_tp(tl, dist, rank, world, ev, steps=32, ctx=4096, with_single=True, batch=16):
    """Config C4: the Llama-3-70B-shaped model (80 layers, d 8192, 64 / 8 heads of 128, FFN 28672, Q4_K + Q6_K head, f16 KV
    with a 4096-row context) split over `world` ranks, batch 1 (fused chain) and batch 16 (few-rows kernel), greedy decoding;
    the all-reduce of one 32 KB residual timed alone over both transports; and the whole model on rank 0 alone."""
    from tl_b200 import synth
    cfg = dict(synth.LLAMA3_70B)
    box = [tl.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    tl.tp_init(box[0], rank, world, join_timeout_s=300.0)
    handles = [None] * world
    dist.all_gather_object(handles, tl.tp_p2p_export())
    tl.tp_p2p_attach(handles)
    dist.barrier()
    out = {"workload": "c4: Llama-3-70B-shaped decode, Q4_K + Q6_K head, f16 KV, ctx %d, tensor parallel x%d" % (ctx, world), "tp": world}
    L = tl.lib()

    def reduce_ms(v):
        return reduce_max(dist, v)

    # the collective alone: 160 sums of one residual row per token
    x = tl.Tensor.zeros([cfg["d_model"]])
    ar = {}
    for name in ("p2p", "nccl"):
        if name == "nccl":
            tl.tp_p2p_disable()
        for _ in range(20):
            tl.check(L.tlb_allreduce(x.h))
        tl.sync()
        dist.barrier()
        tl.check(L.tlb_event_record(ev[0]))
        for _ in range(320):
            tl.check(L.tlb_allreduce(x.h))
        tl.check(L.tlb_event_record(ev[1]))
        tl.sync()
        ar[name] = reduce_ms(_elapsed_ms(tl, ev[0], ev[1])) * 1e3 / 320
    tl.tp_p2p_enable()                   # back to the peer-memory transport
    out["allreduce_us"] = {k: round(v, 2) for k, v in ar.items()}
    out["allreduce_bytes"] = 4 * cfg["d_model"]
    out["allreduce_per_token_us"] = {k: round(160 * v, 1) for k, v in ar.items()}

    wmap = build_tp_map(tl, cfg, rank, world)
    dec = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=ctx + 2 * steps + 16, tp_size=world, tp_rank=rank)
    dist.barrier()       # the ranks enter a step together: waits on another rank's partial sums are bounded (about a second)
    ms = reduce_ms(time_generate(tl, dec, ev, 1, ctx, 4, steps))
    st = dec.stats(ctx)
    out["bs1"] = {"tokens_per_s": round(1e3 / ms, 2), "ms_per_token": round(ms, 3), "transport": "o_proj / ffn_down add their partial sums over the ranks inside the launch (tile-wise peer stores over NVLink)",
                  "weight_bytes_per_rank": st["weight_bytes"], "kv_bytes_per_rank": st["kv_bytes"],
                  "GBs_per_rank": round((st["weight_bytes"] + st["kv_bytes"]) / ms / 1e6, 1)}
    tl.tp_exchange_in_launch(False)
    dec_k = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=ctx + 2 * steps + 16, tp_size=world, tp_rank=rank)
    dist.barrier()
    ms_k = reduce_ms(time_generate(tl, dec_k, ev, 1, ctx, 4, steps))
    out["bs1_allreduce_launch"] = {"tokens_per_s": round(1e3 / ms_k, 2), "ms_per_token": round(ms_k, 3),
                                   "transport": "one-shot peer-memory all-reduce launch between the matvecs"}
    dec_k.destroy()
    tl.tp_exchange_in_launch(True)
    tl.tp_p2p_disable()
    dec_n = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=ctx + 2 * steps + 16, tp_size=world, tp_rank=rank)
    dist.barrier()
    ms_n = reduce_ms(time_generate(tl, dec_n, ev, 1, ctx, 4, steps))
    out["bs1_nccl"] = {"tokens_per_s": round(1e3 / ms_n, 2), "ms_per_token": round(ms_n, 3), "transport": "ncclAllReduce"}
    dec_n.destroy()
    tl.tp_p2p_enable()
    dec.destroy()
    if batch:
        decb = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=ctx + 2 * steps + 16, tp_size=world, tp_rank=rank, batch=batch)
        dist.barrier()
        msb = reduce_ms(time_generate(tl, decb, ev, 1, ctx, 2, max(4, steps // 4), batch=batch))
        out["bs%d" % batch] = {"tokens_per_s": round(batch * 1e3 / msb, 2), "ms_per_step": round(msb, 3)}
        decb.destroy()
    wmap.free()
    dist.barrier()
    if with_single:
        if rank == 0:
            tl.tp_shutdown()
            wm1 = build_tp_map(tl, cfg, 0, 1)
            d1 = tl.Decoder(cfg, wm1, kv_f16=True, max_seq=ctx + 2 * steps + 16)
            ms1 = time_generate(tl, d1, ev, 1, ctx, 4, steps)
            s1 = d1.stats(ctx)
            out["tp1"] = {"tokens_per_s": round(1e3 / ms1, 2), "ms_per_token": round(ms1, 3),
                          "GBs": round((s1["weight_bytes"] + s1["kv_bytes"]) / ms1 / 1e6, 1)}
            out["speedup_vs_tp1"] = round(ms1 / ms, 3)
            # what keeps a shard from 1 / world of the single-GPU time: the exchange (2 per layer) and the fixed cost of
            # every launch, which does not shrink with the shard
            out["limiting"] = ("per-launch latency and the %d exchanges: %.2f ms of the %.2f ms token are above the %.2f ms a rank "
                               "needs for its share of the weights at the single-GPU rate" % (2 * cfg["n_layers"], ms - ms1 / world, ms, ms1 / world))
            d1.destroy()
            wm1.free()
        else:
            tl.tp_shutdown()
        dist.barrier()
    else:
        tl.tp_shutdown()
    return out


def measure_c4_single(tl, ev, peaks, ctx=4096, steps=16):
    """Config C4's model (Llama-3-70B shapes, all 80 layers, Q4_K + Q6_K head, 40 GB) on ONE GPU: batch 1 through the fused
    matvec chain and batch 16 through the few-rows streaming kernel; f16 KV with a 4096-row context per sequence."""
    from tl_b200 import synth
    cfg = dict(synth.LLAMA3_70B)
    wmap = build_tp_map(tl, cfg, 0, 1)
    out = {"workload": "c4 on one GPU: Llama-3-70B-shaped decode, Q4_K + Q6_K head, f16 KV, ctx %d" % ctx}
    for b in (1, 16):
        dec = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=ctx + 64, batch=b)
        ms = time_generate(tl, dec, ev, 1, ctx, 3, steps if b == 1 else 6, batch=b if b > 1 else None)
        st = dec.stats(ctx)
        nbytes = st["weight_bytes"] + st["kv_bytes"] * b
        out["bs%d" % b] = {"ms_per_step": round(ms, 3), "tokens_per_s": round(b * 1e3 / ms, 1), "GBs": round(nbytes / ms / 1e6, 1),
                           "frac_hbm": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4)}
        dec.destroy()
    wmap.free()
    return out


def run_ours(args, dist, rank, world):
    import ctypes as C
    t_start = time.time()
    tl, cfg, wmap, kv16, ctx, desc = build_session(args.workload)
    K, W = args.steps, args.warmup
    max_seq = ctx + 2 * (K + W) + 16
    dec = tl.Decoder(cfg, wmap, kv_f16=kv16, max_seq=max_seq)
    fill_context(dec, cfg, ctx)
    L = tl.lib()
    ev = [C.c_void_p() for _ in range(4)]
    for e in ev:
        tl.check(L.tlb_event_create(C.byref(e)))
    first_tok = 1 % cfg["vocab"]
    gpu_index = tl.lib().tlb_device_id()

    # ---- device-resident timing: W warm-up tokens, then exactly K tokens
    dec.generate(first_tok, ctx, W)
    tl.sync()
    barrier(dist)
    sampler = ClockSampler(gpu_index) if rank == 0 else None
    launches0 = tl.kernel_launches()
    tl.check(L.tlb_event_record(ev[0]))
    toks = dec.generate(first_tok, ctx + W, K)
    tl.check(L.tlb_event_record(ev[1]))
    ms = C.c_float()
    tl.check(L.tlb_event_elapsed_ms(ev[0], ev[1], C.byref(ms)))
    tl.sync()
    launches = tl.kernel_launches() - launches0
    barrier(dist)
    ms_max = reduce_max(dist, float(ms.value))

    # ---- end to end: host token in, host token out, every step
    tok, pos = first_tok, ctx
    for _ in range(W):
        tok = dec.step(tok, pos)
        pos += 1
    tl.sync()
    barrier(dist)
    tl.check(L.tlb_event_record(ev[2]))
    t0 = time.perf_counter()
    for _ in range(K):
        tok = dec.step(tok, pos)
        pos += 1
    wall = time.perf_counter() - t0
    tl.check(L.tlb_event_record(ev[3]))
    ms2 = C.c_float()
    tl.check(L.tlb_event_elapsed_ms(ev[2], ev[3], C.byref(ms2)))
    e2e_ms = reduce_max(dist, max(float(ms2.value), wall * 1e3))
    clocks = sampler.stop() if sampler else None
    tp = None
    if world > 1 and not args.no_extras and args.workload == "c2":
        # the tensor-parallel figure needs every rank; the 8B replicas' sessions make room first
        try:
            tp = measure_tp(tl, dist, rank, world, ev)
        except Exception as e:      # the headline stands without it
            tp = {"error": str(e)[:300]}
    if rank != 0:
        return None

    # ---- roofline of the dominant kernel (Q4_K / linear-type streaming matvec), timed live
    peaks, peak_kind = measured_peaks()
    kern = {}
    tot_b, tot_us = 0, 0.0
    for which in ("qkv", "o", "gate_up", "down", "head"):
        us, b = dec.time_kernel(which, cfg["n_layers"], 64 if which != "head" else 16)
        kern[which] = {"us": round(us, 2), "GBs": round(b / us / 1e3, 1), "bytes": b}
        if which != "head":
            tot_b += b
            tot_us += us
    achieved = tot_b / tot_us / 1e3
    ratio = profile_traffic_ratio()
    st = dec.stats(ctx + W + K // 2)
    tok_s = whole_job_rate(world, K, ms_max)
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": int(tot_b * ratio) if ratio else None, "peak_kind": peak_kind,
                "traffic_note": "dram bytes of the same four launches: the committed ncu capture of the 4-layer case gives %s DRAM bytes "
                                "per algorithmic byte, scaled by the bytes of these launches" % (round(ratio, 4) if ratio else "no"),
                "kernel": "qmatvec_kernel over one layer's four launches (qkv, o, gate|up, down), weights of %d layers rotated"
                          % cfg["n_layers"],
                "per_launch": kern,
                "frac_of_8TBs_nominal": round(achieved / 8000.0, 4),
                "whole_step_GBs": round((st["weight_bytes"] + st["kv_bytes"]) * (tok_s / world) / 1e9, 1)}
    dec.destroy()
    extras = {}
    if not args.no_extras:
        big = args.workload == "c2"
        extras["prefill"] = measure_prefill(tl, cfg, wmap, kv16, ev, peaks, batch=8 if big else 2, tokens=min(ctx, 2048) if ctx >= 32 else 0)
        extras["per_op"] = measure_per_op(tl, cfg, wmap, ctx, 4, ev)
        if world == 1:
            wmap.free()
            extras["sweep"] = measure_sweep(tl, ev, peaks) if big else measure_sweep(tl, ev, peaks, shapes=SWEEP_SHAPES[:2])
            if big:
                extras["c4_single_gpu"] = measure_c4_single(tl, ev, peaks)
    cpu, _ = cpu_baseline(cfg, args.cpu_budget)
    line = {"metric": "Q4_K Llama-3-8B decode tok/s @bs1" if args.workload == "c2" else "decode tok/s @bs1",
            "value": round(tok_s, 2), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(ms_max / K, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 MMA (s32 sums) + f32", "data": "synthetic",
            "config": {"workload": args.workload + ": " + desc, "l2": "inputs larger than L2: %.2f GB of weights streamed per step"
                       % (st["weight_bytes"] / 1e9), "parallelism": "replicas x%d" % world if world > 1 else "single GPU",
                       "weight_bytes_per_token": st["weight_bytes"], "kv_bytes_per_token": st["kv_bytes"],
                       "greedy_tokens_head": toks[:8], "setup_s": round(time.time() - t_start, 1)},
            "clocks": clocks,
            "e2e": {"value": round(whole_job_rate(world, K, e2e_ms), 2), "unit": "tokens/s", "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "roofline": roofline, "cpu_baseline": cpu}
    if tp:
        line["tp"] = tp
    for key, val in extras.items():
        if val:
            line[key] = val
    return line


def run_reference(args, dist, rank, world):
    if rank != 0:
        return None
    cfg, lt, ht, kv16, ctx, desc = workload_cfg(args.workload)
    K, W = args.steps, args.warmup
    cpu_baseline(cfg, 2.0, 1)                       # warm-up of caches / page faults
    per_step_budget = max(0.05, min(20.0, 150.0 / max(1, K + W)))
    t0 = time.perf_counter()
    cpu, vals = cpu_baseline(cfg, per_step_budget * (K + W), K + W)
    vals = vals[W:] if len(vals) > W else vals
    v = statistics.mean(vals)
    cpu["value"] = v
    return {"impl": "reference", "metric": "Q4_K Llama-3-8B decode tok/s @bs1" if args.workload == "c2" else "decode tok/s @bs1",
            "value": round(v, 5), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(1e3 / v, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload + ": " + desc, "note": "reference CPU path (TL_DEVICE=cpu) restated in C; the Rust "
                       "reference cannot be built here (no cargo/rustc/LLVM)", "wall_s": round(time.perf_counter() - t0, 1)},
            "cpu_baseline": cpu,
            "e2e": {"value": round(v, 5), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


PARTS = {
    "c1": "operator sweep of config C1 (Q8_0 / Q4_K x 5 shapes x 1 / 4 / 16 / 512 rows)",
    "c3": "batched prompt processing of config C3 (8 x 2048 tokens, Llama-3-8B shapes)",
    "qgemm": "one Q4_K 4096 x 4096 weight with 1184 activation rows, three calls (small case for a profiler capture)",
    "qrows": "one Q4_K 57344 x 8192 weight (gate | up of the 70B shapes, 264 MB) with 16 activation rows, four calls (small case for a profiler capture)",
    "c4-4layer": "Llama-3-70B-shaped decode on one GPU, 4 layers + head, 4096-row f16 context: batch 1 (fused matvec chain) and batch 16 (few-rows streaming kernel)",
    "per-op-4layer": "the TL chatbot's op sequence through the per-op entry points (native driver), Llama-3-8B shapes cut to 4 layers, 2048 cached rows, 3 steps",
    "prefill-2layer": "one 2048-token prompt through two Llama-3-8B-shaped layers + head, three times (small case for a profiler capture)",
}


def run_part(args):
    """The stand-alone parts: one JSON line of their own."""
    import ctypes as C
    import tl_b200 as tl
    from tl_b200 import synth
    tl.init(-1)
    L = tl.lib()
    ev = [C.c_void_p() for _ in range(2)]
    for e in ev:
        tl.check(L.tlb_event_create(C.byref(e)))
    peaks, peak_kind = measured_peaks()
    name = args.workload
    line = {"metric": PARTS[name], "n_gpus": 1, "data": "synthetic", "config": {"workload": name + ": " + PARTS[name]}, "peak_kind": peak_kind}
    if name == "c1":
        sweep = measure_sweep(tl, ev, peaks)
        big = [e for e in sweep if e["m"] <= 16 and e["n"] * e["k"] >= 4096 * 14336]
        line.update({"sweep": sweep, "value": round(float(np.median([e["GBs"] for e in big])), 1), "unit": "GB/s (median of the >= 33 MB shapes, rows <= 16)",
                     "higher_is_better": True})
    elif name == "c3":
        cfg = synth.LLAMA3_8B
        wmap = tl.TensorMap.new()
        for tname, t, shape in synth.llama_tensor_specs(cfg, 12, 14):
            wmap.add(tname, t, shape, synth.make_tensor(tname, t, shape, 1234))
        pf = measure_prefill(tl, cfg, wmap, True, ev, peaks, batch=8, tokens=2048)
        line.update({"prefill": pf, "value": pf["tokens_per_s"], "unit": "prompt tokens/s", "higher_is_better": True})
    elif name == "qgemm":
        rng = np.random.default_rng(1)
        q = tl.QTensor.from_gguf_bytes(12, 4096, 4096, synth.random_quant(12, 4096, 4096, rng))
        x = tl.Tensor.from_numpy(rng.standard_normal((1184, 4096), dtype=np.float32))
        for _ in range(2):
            x.matmul_quantized(q).release()
        tl.sync()
        tl.check(L.tlb_event_record(ev[0]))
        x.matmul_quantized(q).release()
        tl.check(L.tlb_event_record(ev[1]))
        tl.sync()
        ms = _elapsed_ms(tl, ev[0], ev[1])
        line.update({"value": round(2.0 * 1184 * 4096 * 4096 / ms / 1e9, 1), "unit": "TFLOP/s (with the f16 conversion)", "ms": round(ms, 4), "higher_is_better": True})
    elif name == "qrows":
        rng = np.random.default_rng(1)
        n, k, m = 57344, 8192, 16
        q = tl.QTensor.from_gguf_bytes(12, n, k, synth.random_quant(12, n, k, rng))
        x = tl.Tensor.from_numpy(rng.standard_normal((m, k), dtype=np.float32))
        for _ in range(3):
            x.matmul_quantized(q).release()
        tl.sync()
        tl.check(L.tlb_event_record(ev[0]))
        x.matmul_quantized(q).release()
        tl.check(L.tlb_event_record(ev[1]))
        tl.sync()
        ms = _elapsed_ms(tl, ev[0], ev[1])
        nbytes = n * k // 256 * 144
        line.update({"value": round(nbytes / ms / 1e6, 1), "unit": "GB/s of weight bytes (with the f16 conversion of the activations)", "ms": round(ms, 4),
                     "frac_hbm": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4), "higher_is_better": True})
    elif name == "per-op-4layer":
        cfg = dict(synth.LLAMA3_8B, n_layers=4)
        wmap = tl.map_from_tensors(synth.llama_tensors(cfg, 1, 12, 14))
        po = measure_per_op(tl, cfg, wmap, 2048, 3, ev)
        line.update({"value": po["tokens_per_s"], "unit": "tokens/s (4 layers + head)", "higher_is_better": True, "per_op": po})
    elif name == "c4-4layer":
        cfg = dict(synth.LLAMA3_70B, n_layers=4)
        wmap = build_tp_map(tl, cfg, 0, 1)
        ctx, steps = 4096, 16
        res = {}
        for b in (1, 16):
            dec = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=ctx + 64, batch=b)
            ms = time_generate(tl, dec, ev, 1, ctx, 3, steps, batch=b if b > 1 else None)
            st = dec.stats(ctx)
            nbytes = st["weight_bytes"] + st["kv_bytes"] * b
            res["bs%d" % b] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(b * 1e3 / ms, 1), "GBs": round(nbytes / ms / 1e6, 1),
                               "frac_hbm": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4)}
            dec.destroy()
        line.update({"value": res["bs16"]["tokens_per_s"], "unit": "tokens/s at batch 16 (4 layers + head)", "higher_is_better": True, "c4": res})
    else:
        cfg = dict(synth.LLAMA3_8B, n_layers=2)
        wmap = tl.map_from_tensors(synth.llama_tensors(cfg, 1, 12, 14))
        dec = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=2048 + 256)
        prompt = [int(t) for t in np.random.default_rng(6).integers(0, cfg["vocab"], 2048)]
        for _ in range(2):
            dec.prefill(prompt, 0, read=False)
        tl.sync()
        tl.check(L.tlb_event_record(ev[0]))
        dec.prefill(prompt, 0, read=False)
        tl.check(L.tlb_event_record(ev[1]))
        tl.sync()
        ms = _elapsed_ms(tl, ev[0], ev[1])
        line.update({"value": round(2048 / ms * 1e3, 0), "unit": "prompt tokens/s (2 layers + head)", "ms": round(ms, 3), "higher_is_better": True})
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(PARTS))
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU work for the cpu_baseline sample")
    ap.add_argument("--no-extras", action="store_true", help="headline, e2e, roofline and cpu_baseline only (no sweep / per_op / prefill / tp)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    # stdout carries the one JSON line: whatever NCCL is asked to log (NCCL_DEBUG in the environment) goes to stderr
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    if args.workload in PARTS:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(run_part(args)), flush=True)
        return
    if args.impl == "reference":
        # CPU arm: rank 0 alone measures; the other ranks of a torchrun launch leave at once
        rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        line = run_reference(args, None, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    dist, rank, world = dist_setup(args.gpus)
    try:
        line = run_reference(args, dist, rank, world) if args.impl == "reference" else run_ours(args, dist, rank, world)
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if dist is not None:
            try:
                dist.barrier()
                dist.destroy_process_group()
            except Exception:
                pass


if __name__ == "__main__":
    main()
