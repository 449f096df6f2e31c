"""Host-side set-up of a data-parallel job: rendezvous with a deadline and agreement checks.

The reference has no distributed code; these helpers are what keeps a job from hanging on the host when a rank is
missing or was started with another model: every failure ends in an exception on every rank that is still there,
before any kernel or collective of the step has been launched.
"""
import datetime

import numpy as np


class RendezvousError(RuntimeError):
    """Not every rank joined the process group within the deadline."""


class LayoutMismatch(RuntimeError):
    """The ranks do not agree on a quantity that must be equal on all of them (e.g. the flat gradient length)."""


def rendezvous(backend, rank, world, addr="127.0.0.1", port=29500, timeout_s=60.0, **kwargs):
    """``torch.distributed.init_process_group`` over TCP with a deadline.  A rank that never starts makes the others
    raise RendezvousError after ``timeout_s`` instead of waiting for ever.  Returns the ``torch.distributed`` module."""
    import torch.distributed as dist

    try:
        dist.init_process_group(backend, init_method=f"tcp://{addr}:{port}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        # the store-based barrier names the ranks that are missing; plain init only connects to the store
        if backend == "gloo":
            dist.monitored_barrier(timeout=datetime.timedelta(seconds=timeout_s))
        else:
            dist.barrier()
    except Exception as e:  # noqa: BLE001 - torch raises several types here (DistStoreError, DistNetworkError, RuntimeError)
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass
        raise RendezvousError(f"rank {rank} of {world}: the other ranks did not join within {timeout_s:g} s ({type(e).__name__}: "
                              f"{str(e).splitlines()[0] if str(e) else ''})") from e
    return dist


def agree(dist, what, values, device="cpu"):
    """Every rank passes its own ``values`` (a list of ints); raises LayoutMismatch on EVERY rank when they differ on any
    rank, naming each rank's values.  Costs one all-gather; call it before the first gradient exchange."""
    import torch

    mine = torch.tensor([int(v) for v in values], dtype=torch.int64, device=device)
    world = dist.get_world_size()
    # ranks may even disagree on how many values they pass: gather the counts first
    count = torch.tensor([mine.numel()], dtype=torch.int64, device=device)
    counts = [torch.zeros_like(count) for _ in range(world)]
    dist.all_gather(counts, count)
    counts = [int(c.item()) for c in counts]
    if len(set(counts)) == 1:
        rows = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(rows, mine)
        rows = [r.cpu().numpy().tolist() for r in rows]
    else:
        rows = [f"{c} values" for c in counts]
    if any(r != rows[0] for r in rows):
        raise LayoutMismatch(f"the ranks disagree on {what}: " + ", ".join(f"rank {i}: {r}" for i, r in enumerate(rows)))
    return rows[0]


def share_unique_id(dist, make_id, rank, device="cpu"):
    """Rank 0 creates the 128-byte communicator id with ``make_id()`` and every rank receives it."""
    import torch

    buf = torch.zeros(128, dtype=torch.uint8, device=device)
    if rank == 0:
        buf = torch.tensor(np.frombuffer(bytes(make_id()), dtype=np.uint8).copy(), dtype=torch.uint8, device=device)
    dist.broadcast(buf, 0)
    return buf.cpu().numpy().tolist()
