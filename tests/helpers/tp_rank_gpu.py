"""One rank of the 2-GPU tensor-parallel parity test (started by tests/test_gpu_tp.py, one process per GPU).

A Llama-3-70B-shaped model cut to 2 layers and a 32k vocabulary (d 8192, 64 / 8 heads of 128, FFN 28672, Q4_K + Q6_K
head, f16 KV with 300 cached rows), sharded over the ranks; rank 0 compares every step's gathered logits and greedy
token with the oracle's unsharded model.  First over NCCL, then again over the peer-memory all-reduce.
"""
import faulthandler
import os
import pickle
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import tl_b200 as tl  # noqa: E402
from oracle import oracle  # noqa: E402
from tl_b200 import synth  # noqa: E402


def relerr(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


class FileExchange:
    """The host-side channel between the ranks of this test: files in a shared directory (no network set-up involved).
    Every wait has a deadline."""

    def __init__(self, folder, rank, world, timeout=120.0):
        self.folder, self.rank, self.world, self.timeout, self.n = folder, rank, world, timeout, 0

    def _wait(self, path):
        t0 = time.time()
        while not os.path.exists(path):
            if time.time() - t0 > self.timeout:
                raise TimeoutError("no answer from the other rank: " + path)
            time.sleep(0.005)

    def all_gather_object(self, obj):
        self.n += 1
        mine = os.path.join(self.folder, "x%d.%d" % (self.n, self.rank))
        with open(mine + ".tmp", "wb") as f:
            pickle.dump(obj, f)
        os.replace(mine + ".tmp", mine)
        out = []
        for r in range(self.world):
            path = os.path.join(self.folder, "x%d.%d" % (self.n, r))
            self._wait(path)
            with open(path, "rb") as f:
                out.append(pickle.load(f))
        return out

    def broadcast(self, obj, src=0):
        return self.all_gather_object(obj if self.rank == src else None)[src]

    def barrier(self):
        self.all_gather_object(None)


def log(rank, *a):
    print("[rank %d %.1fs]" % (rank, time.time() - T0), *a, flush=True)


T0 = time.time()


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "parity"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    faulthandler.dump_traceback_later(int(os.environ.get("TP_TEST_DEADLINE", "240")), exit=True)   # a stuck rank ends with its stack
    dist = FileExchange(os.environ["TP_TEST_DIR"], rank, world)
    tl.init(rank)
    log(rank, "device bound")
    if mode == "absent":
        # rank 1 leaves before joining: rank 0's join must give up at its deadline
        if rank == 1:
            dist.barrier()
            print("rank 1 left without joining")
            return
        uid = tl.tp_unique_id()
        t0 = time.time()
        try:
            tl.tp_init(uid, 0, world, join_timeout_s=4.0)
            print("FAIL: joined alone")
            sys.exit(1)
        except tl.TlbError as e:
            assert e.code == 2 and "did not answer" in str(e), e
        assert time.time() - t0 < 60
        # the device is still usable afterwards
        x = tl.Tensor.from_numpy(np.arange(8, dtype=np.float32))
        assert x.scale(2.0).numpy()[7] == 14.0
        dist.barrier()
        print("rank 0: bounded join ok")
        return

    uid = dist.broadcast(tl.tp_unique_id() if rank == 0 else None)
    tl.tp_init(uid, rank, world, join_timeout_s=60.0)
    log(rank, "communicator joined")

    cfg = dict(synth.LLAMA3_70B, n_layers=2, vocab=32064)
    tens = synth.llama_tensors(cfg, 5, synth.Q4_K, synth.Q6_K)
    wmap = tl.map_from_tensors(tens, rank, world)
    log(rank, "weights sharded and uploaded")
    ctx = 300
    rng = np.random.default_rng(9)
    kvd = cfg["n_kv_heads"] * cfg["head_dim"]
    kv = [(rng.standard_normal((ctx, kvd)).astype(np.float16).astype(np.float32),
           rng.standard_normal((ctx, kvd)).astype(np.float16).astype(np.float32)) for _ in range(cfg["n_layers"])]

    def session():
        d = tl.Decoder(cfg, wmap, kv_f16=True, max_seq=ctx + 64, tp_size=world, tp_rank=rank)
        for layer, (k, v) in enumerate(kv):
            d.kv_write(layer, 0, k, v)
        return d

    ref = None
    if rank == 0:
        ref = oracle.Llama(dict(cfg, kv_f16=1, max_seq=ctx + 64), {k: (t, d) for k, (t, d, s) in tens.items()})
        for layer, (k, v) in enumerate(kv):
            for p in range(ctx):
                ref.kv_write(layer, p, k[p], v[p])

    steps = 8
    dec = session()
    tok, pos, worst, want, got, logits_nccl = 777, ctx, 0.0, [], [], []
    for _ in range(steps):
        nxt = dec.step(tok, pos)
        lg = dec.logits()                      # gathers the shards' rows: every rank calls it
        logits_nccl.append(lg)
        if rank == 0:
            rl = ref.forward([tok], pos)
            worst = max(worst, relerr(lg, rl))
            want.append(oracle.argmax_last(rl))
        got.append(nxt)
        ref_tok = dist.broadcast(want[-1] if rank == 0 else None)
        assert nxt == ref_tok, (rank, nxt, ref_tok)    # every rank picked the oracle's token
        tok, pos = ref_tok, pos + 1
        log(rank, "step", len(got), "token", nxt)
    if rank == 0:
        assert worst < 2e-2, worst
        print("nccl: worst logit error %.2e, tokens %s" % (worst, got))
    st = dec.stats(ctx)
    assert st["kernels_per_step"] == 5 * 2 + 3

    # the same steps over the peer-memory all-reduce
    handles = dist.all_gather_object(tl.tp_p2p_export())
    tl.tp_p2p_attach(handles)
    dist.barrier()
    log(rank, "peer memory attached")
    dec2 = session()
    tok, pos = 777, ctx
    for i in range(steps):
        nxt = dec2.step(tok, pos)
        lg = dec2.logits()
        assert nxt == got[i], (rank, i, nxt, got[i])
        assert relerr(lg, logits_nccl[i]) < 1e-4       # only the order of the cross-rank sum differs
        tok, pos = nxt, pos + 1
    log(rank, "peer-memory steps agree")
    # generate: device-side feedback, one graph replay per token, every rank the same tokens
    dec3 = session()
    gen = dec3.generate(777, ctx, steps)
    assert gen == got, (rank, gen, got)
    # timing, for the record: the collective alone, then graph replays, over both transports
    x = tl.Tensor.zeros([cfg["d_model"]])
    for name, use_p2p in (("p2p", True), ("nccl", False)):
        if not use_p2p:
            tl.tp_p2p_disable()
        for _ in range(20):
            tl.check(tl.lib().tlb_allreduce(x.h))
        tl.sync()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(500):
            tl.check(tl.lib().tlb_allreduce(x.h))
        tl.sync()
        if rank == 0:
            print("%s: all-reduce of %d floats alone, %.2f us per call (launched back to back)" % (name, cfg["d_model"], (time.perf_counter() - t0) / 500 * 1e6))
        d4 = session()
        d4.generate(777, ctx, 4)
        tl.sync()
        dist.barrier()
        t0 = time.perf_counter()
        d4.generate(777, ctx + 4, 32)
        tl.sync()
        dt = (time.perf_counter() - t0) / 32
        if rank == 0:
            print("%s: %.1f us per token (2 layers + head, %d ranks)" % (name, dt * 1e6, world))
        d4.destroy()
    tl.tp_poll()
    dist.barrier()
    try:
        tl.tp_shutdown()
        raise SystemExit("shut down with sessions alive")
    except tl.TlbError as e:
        assert e.code == 8 and "still alive" in str(e)
    for d in (dec, dec2, dec3):
        d.destroy()                # their graphs hold the communicator's kernels
    tl.tp_shutdown()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
