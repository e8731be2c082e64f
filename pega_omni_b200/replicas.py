"""Scale-out by sessions: independent per-GPU replicas, no collective on the data path.

Sessions are independent (own KV pages, state slot and random stream), so a box of G GPUs runs G full
replicas and session i lives on replica i mod G. The reference runs one device per process
(crates/omni-server/src/main.rs:172-173); this is the partitioning a front end would apply above it.
"""
from __future__ import annotations

from typing import Sequence


def owner(session: int, world_size: int) -> int:
    return session % world_size


def partition(n_sessions: int, world_size: int) -> list[list[int]]:
    """Round-robin: global session ids owned by each rank."""
    return [list(range(r, n_sessions, world_size)) for r in range(world_size)]


def local_sessions(n_sessions: int, rank: int, world_size: int) -> list[int]:
    return partition(n_sessions, world_size)[rank]


def aggregate_frames_per_second(frames_per_rank: Sequence[int], seconds_per_rank: Sequence[float]) -> float:
    """Whole-job throughput: all frames over the slowest rank's time."""
    return float(sum(frames_per_rank)) / max(seconds_per_rank)
