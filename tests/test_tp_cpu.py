"""Host side of the tensor-parallel path, on CPU.

* Two gloo ranks shard every tensor of a small Llama-shaped model with the library's byte-slice sharding
  (tlb_tp_shard_bytes, no device needed) and run the oracle on their shards: rows concatenated over the ranks
  (attn_q/k/v, ffn_gate/up, head) and partial products summed over the ranks (attn_output, ffn_down) must give the
  unsharded oracle's result.
* A rank that never joins: with a stand-in for libnccl whose peers never arrive, tlb_tp_init gives up after its
  deadline with TLB_ERR_DEVICE and aborts the communicator (no GPU, no hang).
"""
import ctypes as C
import os
import subprocess
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HERE = os.path.dirname(os.path.abspath(__file__))

RANK_SCRIPT = r"""
import os, sys
sys.path.insert(0, %r)
import numpy as np
import torch
import torch.distributed as dist
import tl_b200 as tl
from tl_b200 import synth
from oracle import oracle

dist.init_process_group("gloo", init_method="env://")
rank, world = dist.get_rank(), dist.get_world_size()
cfg = dict(n_layers=1, d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=96, eps=1e-5, rope_base=10000.0, attn_scale=0.125)
rng = np.random.default_rng(3)
for linear in (synth.Q4_K, synth.Q8_0, synth.Q6_K, synth.Q4_0):
    tens = synth.llama_tensors(cfg, 11, linear, linear)
    for name, (t, data, shape) in tens.items():
        kind = tl.tp_split_kind(name)
        if len(shape) != 2 or t == synth.F32:
            assert kind == 0, name
            continue
        assert kind in (1, 2), name
        n, k = shape
        x = rng.standard_normal((2, k), dtype=np.float32)              # the same draw on both ranks (same seed)
        full = oracle.qmatmul(t, data, n, k, x)
        sb, (sn, sk) = tl.tp_shard_bytes(kind, t, n, k, data, rank, world)
        assert sb.size == synth.type_nbytes(t, sn * sk)
        if kind == 1:                                                   # rows: every rank's output columns, concatenated
            assert (sn, sk) == (n // world, k)
            mine = oracle.qmatmul(t, sb, sn, sk, x)
            parts = [torch.zeros(2, sn) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(mine))
            got = torch.cat(parts, dim=1).numpy()
            np.testing.assert_array_equal(got.view(np.uint32), full.view(np.uint32))     # the same dot products, bit for bit
        else:                                                           # columns: partial sums over this rank's slice of K
            assert (sn, sk) == (n, k // world)
            mine = torch.from_numpy(oracle.qmatmul(t, sb, sn, sk, x[:, rank * sk:(rank + 1) * sk]))
            dist.all_reduce(mine)
            err = float(np.max(np.abs(mine.numpy() - full)) / np.max(np.abs(full)))
            assert err < 2e-6, (name, err)
        # the shard dequantises to the matching block of the full tensor
        deq = oracle.dequantize(t, data, n * k).reshape(n, k)
        want = deq[rank * sn:(rank + 1) * sn] if kind == 1 else deq[:, rank * sk:(rank + 1) * sk]
        np.testing.assert_array_equal(oracle.dequantize(t, sb, sn * sk).reshape(sn, sk).view(np.uint32), np.ascontiguousarray(want).view(np.uint32))
# shapes that do not divide are refused
try:
    tl.tp_shard_bytes(2, synth.Q4_K, 16, 256, np.zeros(16 * 144, dtype=np.uint8), 0, 2)
    raise SystemExit("a 256-wide Q4_K row was split in two")
except tl.TlbError as e:
    assert e.code == 1
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_sharding_reassembles_to_the_unsharded_oracle(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT % ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29617", WORLD_SIZE="2", CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o
        assert "rank %d ok" % r in o


def test_split_kinds_by_name():
    import tl_b200 as tl
    assert tl.tp_split_kind("blk.7.attn_q.weight") == 1 and tl.tp_split_kind("blk.0.ffn_up.weight") == 1
    assert tl.tp_split_kind("output.weight") == 1
    assert tl.tp_split_kind("blk.3.attn_output.weight") == 2 and tl.tp_split_kind("blk.3.ffn_down.weight") == 2
    assert tl.tp_split_kind("token_embd.weight") == 0 and tl.tp_split_kind("blk.3.attn_norm.weight") == 0
    assert tl.tp_split_kind("output_norm.weight") == 0


FAIL_SCRIPT = r"""
import ctypes, os, sys, time
sys.path.insert(0, %r)
import tl_b200 as tl
uid = tl.tp_unique_id()
assert uid == b"\x5a" * 128
t0 = time.time()
try:
    tl.tp_init(uid, 0, 2, join_timeout_s=0.5)
    raise SystemExit("joined a communicator whose peer never arrived")
except tl.TlbError as e:
    assert e.code == 2, e
    assert "did not answer" in str(e) and "aborted" in str(e), e
dt = time.time() - t0
assert 0.4 < dt < 10.0, dt
fake = ctypes.CDLL(os.environ["TLB_NCCL_LIB"])
assert ctypes.c_int.in_dll(fake, "fake_nccl_aborts").value == 1
assert tl.lib().tlb_tp_size() == 1          # no communicator was kept
tl.tp_poll()                                 # nothing to report without a communicator
print("bounded join ok")
"""


def test_rank_that_never_joins_is_a_bounded_error(tmp_path):
    """The failure is made on the host (a peer that never arrives, through a stand-in for the NCCL library): joining
    gives up at its deadline, aborts the communicator and returns TLB_ERR_DEVICE; nothing waits for ever."""
    so = tmp_path / "libfakenccl.so"
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    subprocess.check_call([cc, "-shared", "-fPIC", "-O1", "-o", str(so), os.path.join(HERE, "helpers", "fake_nccl.c")])
    script = tmp_path / "fail.py"
    script.write_text(FAIL_SCRIPT % ROOT)
    env = dict(os.environ, TLB_NCCL_LIB=str(so), CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=120)
    assert p.returncode == 0, p.stdout
    assert "bounded join ok" in p.stdout
