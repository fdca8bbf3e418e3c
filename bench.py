"""Benchmark of the quantized Llama decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c0|small]

A step is one decoded token (batch 1).  Default workload c2: Llama-3-8B-shaped decoder, Q4_K linear
layers + Q6_K output head, f16 KV cache holding a 2048-token random context, greedy decoding; weights
are seeded synthetic GGUF blocks (no model file is needed or read).  Prints ONE JSON line (rank 0).

  value     tokens/s with everything resident in HBM: K graph replays with the token fed back on the
            device, CUDA events on the library's stream, max over ranks.
  e2e       tokens/s through tlb_decoder_step with HOST token in / HOST token out every step.
  roofline  the Q4_K streaming matvec, timed live over weight sets rotated through > 2x L2.
  cpu_baseline / --impl reference: the reference CPU path's per-token linear algebra (cached f32
            transposed weights, one thread, strided inner loop) on a bounded sample of output columns.
With N > 1 every rank decodes its own replica of the model (no exchange step on this path): weak scaling.
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


# DRAM bytes moved per algorithmic byte by the streaming matvec, from the ncu capture summarised in
# profiles/qmatvec_q4k_llama3-8b-shapes_4layer_ncu-full.md (dram__bytes_read + dram__bytes_write over the weight bytes)
NCU_TRAFFIC_RATIO = 1.003


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


def measure_prefill(tl, dec, cfg, tokens, ev, peaks):
    """Secondary figure: one prompt of `tokens` random ids through tlb_decoder_prefill (tensor-core GEMMs),
    timed with CUDA events after one warm-up run; arithmetic = linear layers + causal attention."""
    import ctypes as C
    if tokens <= 0:
        return None
    L = tl.lib()
    rng = np.random.default_rng(4321)
    prompt = [int(t) for t in rng.integers(0, cfg["vocab"], tokens)]
    dec.prefill(prompt, 0, read=False)
    tl.sync()
    tl.check(L.tlb_event_record(ev[0]))
    dec.prefill(prompt, 0, read=False)
    tl.check(L.tlb_event_record(ev[1]))
    tl.sync()
    ms = C.c_float()
    tl.check(L.tlb_event_elapsed_ms(ev[0], ev[1], C.byref(ms)))
    dm, qd, kvd, F = cfg["d_model"], cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["ffn"]
    lin = 2.0 * tokens * cfg["n_layers"] * (dm * (qd + 2 * kvd) + qd * dm + 3 * dm * F)
    att = 4.0 * cfg["n_layers"] * cfg["n_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2
    tf = (lin + att) / (ms.value * 1e-3) / 1e12
    peak = peaks.get("bf16_tflops", 1590.0)
    return {"tokens": tokens, "ms": round(float(ms.value), 2), "tokens_per_s": round(tokens / (ms.value * 1e-3), 0),
            "tflops": round(tf, 1), "bound": "tensor", "peak_tflops": peak, "frac": round(tf / peak, 4),
            "note": "f16 tcgen05 GEMMs with on-the-fly dequantisation + mma.sync attention; all layers, head on the last token"}


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
    st = dec.stats(ctx + W + K // 2)
    tok_s = whole_job_rate(world, K, ms_max)
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": int(tot_b * NCU_TRAFFIC_RATIO), "peak_kind": peak_kind,
                "traffic_note": "bytes of the same four launches; ncu capture of a 4-layer case, scaled by the weight bytes",
                "kernel": "qmatvec_kernel over one layer's four launches (qkv, o, gate|up, down), weights of %d layers rotated"
                          % cfg["n_layers"],
                "per_launch": kern,
                "frac_of_8TBs_nominal": round(achieved / 8000.0, 4),
                "whole_step_GBs": round((st["weight_bytes"] + st["kv_bytes"]) * (tok_s / world) / 1e9, 1)}
    prefill = measure_prefill(tl, dec, cfg, min(ctx, 2048) if ctx >= 32 else 0, ev, peaks)
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
    if prefill:
        line["prefill"] = prefill
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU work for the cpu_baseline sample")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
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
