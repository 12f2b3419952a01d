"""The data-parallel training step on real peer memory: two (or more) processes, one per GPU.

Skipped on a box with a single GPU.  Each rank runs the benchmark's own multi-GPU path
(``bench.py`` under ``torch.distributed.run``): CUDA IPC handles, NVLink loads and stores and both
flag barriers of the peer-memory update kernel.  The run ends with ``data_parallel_check``: every
rank's master parameters and compute copy hash to the same SHA-256 digest, and three steps through
the peer-memory kernel equal three steps through NCCL all-reduce + SGD up to the order of the fp32
sums (relative to the update itself).  The benchmark exits non-zero if that check fails; this test
also reads the figures from its JSON line.  No rank is made to fail here.
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(n, workload, batch, port):
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n),
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "bench.py"),
           "--gpus", str(n), "--steps", "3", "--warmup", "3", "--workload", workload, "--batch", str(batch),
           "--no-sweep", "--no-cpu-baseline"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert lines, res.stdout[-2000:]
    return json.loads(lines[-1])


@pytest.mark.parametrize("workload,batch", [("holdem_train", 16384), ("leduc_train", 8192)])
def test_two_ranks_end_bit_identical_and_agree_with_nccl(gpu, workload, batch):
    if gpu.device_count() < 2:
        pytest.skip("needs two GPUs")
    line = run_bench(2, workload, batch, 29541 if workload == "holdem_train" else 29542)
    check = line["extra"]["dp_check"]
    assert check["replicas_identical"] is True
    assert check["peer_vs_nccl_rel_diff_of_update"] <= 1e-4
    assert line["n_gpus"] == 2 and line["config"]["gradient_exchange"].startswith("peer-memory")
