"""Process-group plumbing: one process per GPU, torch.distributed (NCCL on GPUs, Gloo on CPUs)."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from .. import _C


def init_distributed(device: str = "cuda", timeout_s: float = 600.0):
    """Initialises torch.distributed from the torchrun environment and returns (comm, rank, world, local_rank).

    With WORLD_SIZE unset or 1 no process group is created and a size-1 communicator is returned.
    """
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world <= 1:
        return _C.get_comm_self(), 0, 1, local_rank
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if not dist.is_initialized():
        if device == "cuda":
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s),
                                    device_id=torch.device("cuda", local_rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    pg = dist.distributed_c10d._get_default_group()
    comm = _C.comm_from_process_group(pg.group_name, device)
    return comm, rank, world, local_rank
