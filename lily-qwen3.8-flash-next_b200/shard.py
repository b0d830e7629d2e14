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
                        out_lse=None, group=None, stream=None, exchange=None, **kept):
    """One vocab-sharded step on this rank: the 8-bit head over this rank's
    rows and its candidate records (lily_lmhead_shard_candidates), the
    all-gather of the records, the merged draw (lily_merge_draw). Every rank
    ends with the same token ids in `out_ids`. `scratch` was created with
    lmhead=True for this rank's shard size. With `exchange` (a PeerExchange) the
    all-gather is the ranks' own stores into each other's memory instead."""
    import contextlib

    import torch

    rows = hidden.shape[0]
    if records is None:
        records = torch.empty((rows, RECORD_BYTES), dtype=torch.uint8, device=hidden.device)
    if exchange is not None:
        # No collective library on the data path: the records go straight into the
        # other ranks' memory, and the merge waits for their flags.
        scratch.lmhead_shard_candidates(weights, scales, hidden, params, records, first_id=first_id,
                                        want_sums=want_sums, stream=stream)
        exchange.publish_and_merge(scratch, records, params, out_ids, uniforms=uniforms, steps=steps,
                                   out_lse=out_lse, stream=stream, **kept)
        return None
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


class PeerExchange:
    """The exchange of the shards' records over peer memory (lily_shard_publish /
    lily_merge_draw_peer): one buffer per rank, opened by every other rank through
    its inter-process handle, which travels once through torch.distributed (any
    backend) when the exchange is set up. One process per GPU, all on one node.

    `emulate` > 0: no process group; this process plays that many ranks on one GPU
    with one buffer (for tests: the ranks publish one after the other, then merge)."""

    def __init__(self, device: int, max_rows: int, group=None, emulate: int = 0):
        import ctypes as C

        import lily_b200 as lily

        self._lily, self._C, self.device, self.max_rows, self.step = lily, C, device, max_rows, 0
        self._opened = []
        L = lily.lib()
        if emulate:
            self.world, self.rank = emulate, 0
        else:
            import torch.distributed as dist

            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > lily.PEER_MAX:
            raise ValueError("at most 16 ranks")
        own = C.c_void_p()
        handle = (C.c_ubyte * lily.IPC_HANDLE_BYTES)()
        st = L.lily_peer_buffer_create(device, self.world, max_rows, C.byref(own), handle)
        if st != lily.OK:
            raise lily.LilyError(st, "lily_peer_buffer_create failed")
        self._own = own
        x = lily.PeerExchangeStruct()
        x.struct_size = C.sizeof(lily.PeerExchangeStruct)
        x.n_shards, x.rank, x.max_rows = self.world, self.rank, max_rows
        if emulate:
            for r in range(self.world):
                x.buffers[r] = own.value
        else:
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            failed = None
            for r in range(self.world):
                if r == self.rank:
                    x.buffers[r] = own.value
                    continue
                theirs = C.c_void_p()
                raw = (C.c_ubyte * lily.IPC_HANDLE_BYTES).from_buffer_copy(handles[r])
                st = L.lily_peer_buffer_open(device, raw, C.byref(theirs))
                if st != lily.OK:
                    failed = f"rank {self.rank} cannot open rank {r}'s buffer (no peer access?)"
                    break
                self._opened.append(theirs)
                x.buffers[r] = theirs.value
            # Every rank learns of a failure anywhere before any of them goes on
            # (this also keeps a buffer alive until everybody has opened it).
            verdicts = [None] * self.world
            dist.all_gather_object(verdicts, failed, group=group)
            if any(v is not None for v in verdicts):
                for p in self._opened:
                    L.lily_peer_buffer_close(device, p)
                self._opened = []
                dist.barrier(group=group)
                L.lily_peer_buffer_destroy(device, own)
                self._own = None
                raise lily.LilyError(lily.ERR_CUDA, "; ".join(v for v in verdicts if v is not None))
        self.x = x
        self._group = group

    def as_rank(self, rank: int):
        """(emulation) the exchange as rank `rank` sees it."""
        self.x.rank = rank
        return self.x

    def publish_and_merge(self, scratch, records, params, out_ids, *, stream=None, **kw):
        self.step += 1
        scratch.merge_draw_peer(self.x, self.step, params, out_ids, records=records, stream=stream, **kw)

    def close(self):
        L = self._lily.lib()
        if self._own is None:
            return
        if self._opened:
            import torch
            import torch.distributed as dist

            torch.cuda.synchronize(self.device)
            dist.barrier(group=self._group)  # nobody writes into a buffer that is going away
            for p in self._opened:
                L.lily_peer_buffer_close(self.device, p)
            dist.barrier(group=self._group)
        L.lily_peer_buffer_destroy(self.device, self._own)
        self._own = None
