"""Partitions of the sampling path over ranks: by row (no collective), and
by vocabulary for the 8-bit LM head (one small all-gather of candidate records).

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


# ---------------------------------------------------------------- vocabulary --

RECORD_BYTES = 520  # lily_sampler.h: LILY_SHARD_RECORD_BYTES


def vocab_range(vocab: int, world: int, rank: int) -> range:
    """The vocabulary ids whose LM-head rows rank `rank` holds: equal
    contiguous shards (the vocabulary must divide evenly so that every rank
    runs the same launch geometry)."""
    if vocab % world != 0:
        raise ValueError("the vocabulary must be a multiple of the number of shards")
    per = vocab // world
    return range(rank * per, (rank + 1) * per)


def gather_records(local_records, group=None):
    """[rows, 520] uint8 on every rank -> [world, rows, 520] on every rank,
    shard-major, the layout lily_merge_draw reads. One all-gather of
    rows * 520 bytes per rank (NCCL for CUDA tensors, gloo for CPU ones)."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local_records.unsqueeze(0)
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(local_records.shape), dtype=local_records.dtype,
                      device=local_records.device)
    if local_records.is_cuda:
        dist.all_gather_into_tensor(out, local_records, group=group)
    else:
        parts = [out[r] for r in range(world)]
        dist.all_gather(parts, local_records, group=group)
    return out


def sharded_lmhead_draw(scratch, weights, scales, hidden, params, out_ids, first_id: int, *,
                        uniforms=None, steps=None, records=None, want_sums: bool = False,
                        out_lse=None, group=None, stream=None, **kept):
    """One vocab-sharded step on this rank: the 8-bit head over this rank's
    rows and its candidate records (lily_lmhead_shard_candidates), the
    all-gather of the records, the merged draw (lily_merge_draw). Every rank
    ends with the same token ids in `out_ids`. `scratch` was created with
    lmhead=True for this rank's shard size."""
    import contextlib

    import torch

    rows = hidden.shape[0]
    if records is None:
        records = torch.empty((rows, RECORD_BYTES), dtype=torch.uint8, device=hidden.device)
    # The collective is ordered against torch's CURRENT stream only: a stream
    # that is given is made current for the whole step, so that the records are
    # written before the all-gather reads them and gathered before the merge.
    current = torch.cuda.stream(stream) if (stream is not None and hidden.is_cuda) else contextlib.nullcontext()
    with current:
        scratch.lmhead_shard_candidates(weights, scales, hidden, params, records, first_id=first_id,
                                        want_sums=want_sums, stream=stream)
        gathered = gather_records(records, group=group)
        scratch.merge_draw(gathered, params, out_ids, uniforms=uniforms, steps=steps, out_lse=out_lse,
                           stream=stream, **kept)
    return gathered
