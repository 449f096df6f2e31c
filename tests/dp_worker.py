"""One rank of the two-GPU data-parallel check (launched by test_gpu_multi.py through torch.distributed.run).
Trains the small CNN for a few steps on this rank's shard and lets rank 0 save the parameters."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    import torch
    import torch.distributed as dist

    import rusttensor_b200 as rt
    from helpers import workload_data

    out_path, mode = sys.argv[1], sys.argv[2]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        idt = torch.tensor(list(rt.DataParallelTrainer.unique_id()), dtype=torch.uint8, device="cuda")
    dist.broadcast(idt, 0)
    dims = [4, 8, 4, 6, 16, 5]
    tr = rt.DataParallelTrainer(3, dims, rank=rank, world=world, nccl_id=idt.cpu().tolist(), device=local)
    if os.environ.get("RT_B200_DP_FUSED", "0") == "1":
        assert tr.connect_peers(dist), getattr(tr, "peer_error", "peer set-up failed on another rank")
    params, _ = workload_data(3, dims, seed=0)
    for t, p in zip(tr.params, params):
        t.update_from_host(p)
    losses = []
    for step in range(3):
        _, inputs = workload_data(3, dims, seed=100 + step, rank=rank)
        if mode == "eager":
            losses.append(tr.step_eager(inputs))
        else:
            tr.step(inputs)
            losses.append(tr.last_loss())
    if rank == 0:
        np.savez(out_path, *[t.numpy() for t in tr.params], losses=np.array(losses, np.float64))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
