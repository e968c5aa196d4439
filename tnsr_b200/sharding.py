"""Session sharding over the GPUs of one host.

Sessions are independent (no term of the decode graph couples two rows of the
batch, src/nn/kv_cache/graph.rs:15-167), so N processes each own a contiguous
block of sessions with their own handle, stream and K/V cache, and nothing is
exchanged on the data path.  Token ids are gathered on the host when a caller
wants the whole batch back.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_sessions(total: int, world: int, rank: int) -> Tuple[int, int]:
    """(first session, count) of `rank`: contiguous blocks, sizes differing by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank must lie in [0, world)")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def gather_token_rows(local_rows: Sequence[Sequence[int]], group=None) -> List[List[int]]:
    """All ranks' token rows in session order (host-side concatenation; rank r's rows come r-th).
    Uses torch.distributed's object gather on whatever backend the group has; with no
    initialised process group it returns the local rows."""
    import torch.distributed as dist
    rows = [list(map(int, r)) for r in local_rows]
    if not dist.is_available() or not dist.is_initialized():
        return rows
    gathered = [None] * dist.get_world_size(group)
    dist.all_gather_object(gathered, rows, group=group)
    return [row for part in gathered for row in part]
