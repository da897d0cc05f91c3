"""Process-group plumbing for runs with one process per GPU.

The 0.6B / 8B paths do not shard: every rank runs an independent replica and no tensor crosses
ranks on the data path. What the ranks share is only the timing protocol: a barrier on both sides
of the timed region and the maximum of the per-rank device times, from which the whole-job
throughput is computed (units of all ranks / slowest rank's time)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def world() -> tuple[int, int, int]:
    """(rank, local_rank, world_size) from the launcher's environment (1 process = rank 0 of 1)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def init(backend: str, device: torch.device | None = None) -> None:
    if world()[2] > 1 and not dist.is_initialized():
        if device is not None and backend == "nccl":
            dist.init_process_group(backend, device_id=device)
        else:
            dist.init_process_group(backend)


def barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def max_over_ranks(values: list[float], device: str = "cpu") -> list[float]:
    """Element-wise maximum of `values` over all ranks (identity without a process group)."""
    if not (dist.is_available() and dist.is_initialized()):
        return [float(v) for v in values]
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def whole_job_rate(units_per_rank: float, ms_slowest: float, world_size: int) -> float:
    """Units per second of the whole job: every rank processed `units_per_rank` in at most
    `ms_slowest` milliseconds (weak scaling: per-rank work is fixed)."""
    return world_size * units_per_rank / (ms_slowest * 1e-3)


def shutdown() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
