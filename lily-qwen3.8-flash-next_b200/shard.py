"""Row partition of a sampling batch over ranks.

Rows never depend on one another (the reference: "a row never depends on the
rows beside it", src/qwen4exp/batch.rs:43-44), so a batch shards by row with no
collective on the data path: rank r draws rows row_range(B, world, r) and the
host concatenates the ids. The rows of ONE speculative verify step share their
penalty state (src/qwen4exp/model.rs:3008-3012) and stay on one rank.
"""
from __future__ import annotations


def row_range(rows: int, world: int, rank: int) -> range:
    """Contiguous, balanced (sizes differ by at most one), in rank order."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    base, extra = divmod(rows, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def owner_of(row: int, rows: int, world: int) -> int:
    """The rank that draws `row`."""
    if not 0 <= row < rows:
        raise ValueError("row outside the batch")
    base, extra = divmod(rows, world)
    edge = extra * (base + 1)
    if row < edge:
        return row // (base + 1)
    return extra + (row - edge) // base


def gather_tokens(local_tokens, rows: int, world: int, rank: int, group=None):
    """All ranks' token ids in row order (torch.distributed, any backend):
    the only exchange a row-partitioned step needs, and it is on the host side
    of the boundary (B ids), not on the data path."""
    import torch
    import torch.distributed as dist

    counts = [len(row_range(rows, world, r)) for r in range(world)]
    width = max(counts)
    mine = torch.full((width,), -1, dtype=torch.int64)
    mine[:len(local_tokens)] = torch.as_tensor(list(local_tokens), dtype=torch.int64)
    out = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(out, mine, group=group)
    return [int(v) for r in range(world) for v in out[r][:counts[r]]]
