"""Two-GPU data parallelism on real devices: two ranks, each on its own shard, with one NCCL all-reduce after the backward
pass or with the overlapped exchange (ready gradients leave on a side stream during the backward pass), must end with the
parameters one GPU reaches on the concatenated batch.  Skipped on machines with a single GPU."""
import os
import subprocess
import sys

import numpy as np
import pytest

import rusttensor_b200
from helpers import assert_close, workload_data

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpu_count():
    import torch

    return torch.cuda.device_count()


@pytest.mark.parametrize("exchange", ["nccl", "nccl-overlap", "peer-fused"])
@pytest.mark.parametrize("mode", ["graph", "eager"])
def test_two_ranks_match_one_gpu_on_the_joint_batch(gpu_engine, tmp_path, mode, exchange):
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "dp2.npz")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(HERE, "dp_worker.py"), out, mode]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", RT_B200_DP_OVERLAP="1" if exchange == "nccl-overlap" else "0",
               RT_B200_DP_FUSED="1" if exchange == "peer-fused" else "0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    got = np.load(out)
    dims = [4, 8, 4, 6, 16, 5]
    joint = [8] + dims[1:]
    params, _ = workload_data(3, dims, seed=0)
    one = rusttensor_b200.DataParallelTrainer(3, joint)
    for t, p in zip(one.params, params):
        t.update_from_host(p)
    losses = []
    for step in range(3):
        shards = [workload_data(3, dims, seed=100 + step, rank=r)[1] for r in range(2)]
        inputs = [np.concatenate([shards[0][i], shards[1][i]], axis=0) for i in range(len(shards[0]))]
        one.step(inputs)
        losses.append(one.last_loss())
    for i, t in enumerate(one.params):
        assert_close(got[f"arr_{i}"], t.numpy(), 1e-4, f"{mode}: parameter {i} after 3 data-parallel steps", abs_floor=5e-4 * 1e-3)
    # rank 0 reports the loss of its own shard; the joint loss is the mean over both shards, so only the trend is comparable
    assert np.all(np.isfinite(got["losses"]))
