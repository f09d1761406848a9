"""Data-parallel replicas: one process per GPU, full weights on each, no collective on the token path.

The reference serves one model per process (crates/daemon/src/engine.rs:1-3: a single model thread); scaling out is
running more of them. What the ranks share is bookkeeping only: which sessions a rank serves, a barrier around timed
regions, and the reduction of per-rank timings and counters (maximum for times, sum for token counts). NCCL carries
those few scalars when the ranks own GPUs, gloo when they run on CPU (tests).
"""
from __future__ import annotations

import os


class Replicas:
    def __init__(self, backend: str | None = None):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        self.device = "cpu"
        if self.world > 1:
            import torch
            import torch.distributed as dist
            if backend is None:
                backend = "nccl" if torch.cuda.is_available() else "gloo"
            if backend == "nccl":
                torch.cuda.set_device(self.local_rank)
                self.device = f"cuda:{self.local_rank}"
                dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            else:
                dist.init_process_group(backend)
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def _reduce(self, value: float, op_name: str) -> float:
        if not self.dist:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device)
        self.dist.all_reduce(t, op=getattr(self.dist.ReduceOp, op_name))
        return float(t.item())

    def max(self, value: float) -> float:
        """Largest value over the ranks (timings: the job is as slow as its slowest replica)."""
        return self._reduce(value, "MAX")

    def sum(self, value: float) -> float:
        """Sum over the ranks (tokens, sessions, per-replica rates)."""
        return self._reduce(value, "SUM")

    def sessions_of_rank(self, n_sessions: int) -> list[int]:
        """Round-robin assignment of independent sessions to replicas."""
        return list(range(self.rank, n_sessions, self.world))

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()
            self.dist = None


def whole_job_rate(units_per_rank: float, seconds: float, r: Replicas) -> float:
    """Aggregate throughput of replicas that each processed units_per_rank in their own `seconds`: all units over the
    slowest replica's time."""
    total_units = r.sum(units_per_rank)
    slowest = r.max(seconds)
    return total_units / slowest
