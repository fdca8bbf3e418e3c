"""The multi-GPU leg of bench.py is N independent replicas (the decode path of one sequence does not
shard): ranks only meet at a barrier and a max-reduction of their step time.  Exercised here with two
gloo ranks on CPU."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_SCRIPT = r"""
import os, sys
sys.path.insert(0, %r)
import bench
dist, rank, world = bench.dist_setup(2)
assert world == 2 and dist is not None and dist.get_backend() == "gloo"
bench.barrier(dist)
ms = bench.reduce_max(dist, 10.0 * (rank + 1))      # rank 0 took 10 ms, rank 1 took 20 ms
assert ms == 20.0, ms
rate = bench.whole_job_rate(world, 64, ms)          # 2 replicas x 64 tokens in 20 ms
assert abs(rate - 6400.0) < 1e-9, rate
bench.barrier(dist)
print("rank", rank, "ok")
"""


def test_two_gloo_ranks_aggregate(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT % ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29613", WORLD_SIZE="2", CUDA_VISIBLE_DEVICES="")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o
        assert "rank %d ok" % r in o


def test_single_process_has_no_collective():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.reduce_max(None, 3.5) == 3.5
    bench.barrier(None)
    assert bench.whole_job_rate(1, 256, 512.0) == 500.0
