"""Replica bookkeeping for multi-GPU runs: co-location is per GPU, so N GPUs are N independent replicas of
the same job with no collective on the data path.  The only communication is the timing protocol of the
benchmark: a barrier around the timed region, the maximum of the per-rank times, and the sum of the per-rank
work.  Works with any torch.distributed backend (NCCL on GPUs, gloo in the CPU tests)."""
from __future__ import annotations

import os
from typing import Optional


class Replicas:
    def __init__(self, backend: Optional[str] = None, device=None):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        self.device = device
        if self.world > 1:
            import torch.distributed as dist

            if not dist.is_initialized():
                kw = {}
                if backend == "nccl" and device is not None:
                    kw["device_id"] = device
                dist.init_process_group(backend or "gloo", **kw)
            self.dist = dist

    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.barrier()

    def _tensor(self, v: float):
        import torch

        return torch.tensor([v], dtype=torch.float64, device=self.device if self.device is not None else "cpu")

    def max(self, v: float) -> float:
        """The slowest rank defines the time of the whole job."""
        if self.dist is None:
            return v
        t = self._tensor(v)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, v: float) -> float:
        if self.dist is None:
            return v
        t = self._tensor(v)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def gather(self, obj) -> list:
        if self.dist is None:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out

    def throughput(self, units_this_rank: float, seconds_this_rank: float) -> float:
        """Whole-job throughput: all ranks' units over the slowest rank's time (weak scaling)."""
        return self.sum(units_this_rank) / self.max(seconds_this_rank)

    def close(self) -> None:
        if self.dist is not None and self.dist.is_initialized():
            self.dist.destroy_process_group()
            self.dist = None
