"""Process-group bootstrap: one process per GPU, NCCL for the device group, gloo for control traffic.

Reads the ``torchrun`` environment (``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` / ``MASTER_PORT``).
The control group (gloo, CPU) carries heartbeats and scheduling decisions so that a stuck device never blocks the
detection of the failure.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional


@dataclass
class DistEnv:
    rank: int
    local_rank: int
    world: int
    device: str
    group: object = None           # device group (NCCL) or None
    control: object = None         # gloo group or None
    store: object = None


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def init_distributed(backend: Optional[str] = None, timeout_s: float = 120.0, control_group: bool = True) -> DistEnv:
    import torch

    rank, local, world = env_rank_world()
    cuda = torch.cuda.is_available()
    dev = f"cuda:{local}" if cuda else "cpu"
    if cuda:
        torch.cuda.set_device(local)
    if world == 1:
        from .health import DictStore

        return DistEnv(rank, local, world, dev, store=DictStore())
    import torch.distributed as dist

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    backend = backend or ("nccl" if cuda else "gloo")
    kw = {"device_id": torch.device(dev)} if (backend == "nccl") else {}
    dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    control = None
    if control_group:
        control = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s)) if backend != "gloo" else dist.group.WORLD
    store = dist.distributed_c10d._get_default_store()
    return DistEnv(rank, local, world, dev, dist.group.WORLD, control, store)


def shutdown() -> None:
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
