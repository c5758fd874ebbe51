"""World-size-2 gloo test of the expert-parallel protocol on CPU: split sizes, arrival order,
stable regrouping by local expert and the reverse path must reproduce the single-process MoE
layer bit for bit."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ep_splits():
    from gem16_b200.ep import ep_splits
    counts = np.arange(2 * 8).reshape(2, 8)            # 2 ranks, 8 experts, 4 per rank
    send, recv = ep_splits(counts, 0, 4)
    assert send == [0 + 1 + 2 + 3, 4 + 5 + 6 + 7] and recv == [6, 8 + 9 + 10 + 11]
    send, recv = ep_splits(counts, 1, 4)
    assert send == [38, 54] and recv == [22, 54]


def test_expert_parallel_protocol_two_ranks():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(ROOT, "tests", "ep_cpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


def test_tensor_parallel_mlp_two_ranks():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29633", os.path.join(ROOT, "tests", "tp_cpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
