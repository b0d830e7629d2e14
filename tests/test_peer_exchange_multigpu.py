"""The shards' records over peer memory between real ranks: one process per GPU,
the exchange buffers opened through their inter-process handles (which travel
over a gloo group: no NCCL anywhere in this test), lily_merge_draw_peer on every
rank. Needs two GPUs with peer access; skipped otherwise.

Every rank holds one vocabulary shard of the same seeded logits, runs
lily_shard_candidates on it and merges through the exchange; rank 0 also
computes every shard's records itself and merges them with lily_merge_draw.
All ranks have to end with rank 0's tokens and log-sum-exps, step after step
(three steps: both slots of the exchange and the step counter are used)."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ROWS, VOCAB, STEPS = 24, 262_144, 3


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, result):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    import lily_b200 as lily
    import oracle
    import workloads as wl
    from lily_b200.shard import PeerExchange

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    per = VOCAB // world
    shard = lily.SamplerScratch(per, max_rows=ROWS, device=rank)
    ex = PeerExchange(rank, max_rows=ROWS)
    plist = [dict(temperature=[0.7, 1.0, 0.0, 0.9][r % 4], top_k=[40, 64, 1, 7][r % 4],
                  top_p=[0.95, 1.0, 1.0, 0.8][r % 4], seed=r) for r in range(ROWS)]
    params = [lily.SamplingParams(**p) for p in plist]
    ok = True
    for step in range(STEPS):
        rng = np.random.default_rng([91, step])  # the same logits on every rank
        x = wl.zipf_logits(rng, ROWS, VOCAB)
        u = torch.from_numpy(np.array([oracle.uniform_for(300 + r, step) for r in range(ROWS)],
                                      dtype=np.float32)).cuda()
        mine = torch.from_numpy(np.ascontiguousarray(x[:, rank * per:(rank + 1) * per])).cuda()
        rec = torch.zeros((ROWS, 520), dtype=torch.uint8, device="cuda")
        shard.shard_candidates(mine, params, rec, first_id=rank * per, want_sums=True)
        out = torch.full((ROWS,), -1, dtype=torch.int32, device="cuda")
        lse = torch.zeros(ROWS, dtype=torch.float32, device="cuda")
        ex.publish_and_merge(shard, rec, params, out, uniforms=u, out_lse=lse)
        torch.cuda.synchronize()
        ok = ok and shard.status() == lily.OK
        # Rank 0's own account of the step: all shards on its GPU, no exchange.
        want, want_lse = out.cpu().clone(), lse.cpu().clone()
        if rank == 0:
            every = torch.zeros((world, ROWS, 520), dtype=torch.uint8, device="cuda")
            for s in range(world):
                part = torch.from_numpy(np.ascontiguousarray(x[:, s * per:(s + 1) * per])).cuda()
                shard.shard_candidates(part, params, every[s], first_id=s * per, want_sums=True)
            alone = torch.full((ROWS,), -1, dtype=torch.int32, device="cuda")
            alone_lse = torch.zeros(ROWS, dtype=torch.float32, device="cuda")
            shard.merge_draw(every, params, alone, uniforms=u, out_lse=alone_lse)
            torch.cuda.synchronize()
            want, want_lse = alone.cpu(), alone_lse.cpu()
        dist.broadcast(want, src=0)
        dist.broadcast(want_lse, src=0)
        ok = ok and bool(torch.equal(out.cpu(), want)) and bool(torch.equal(lse.cpu(), want_lse))
    ex.close()
    shard.close()
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        result.put(all(flags))
    dist.destroy_process_group()


def test_two_ranks_exchange_their_records_without_a_collective(cuda):
    torch = cuda
    if torch.cuda.device_count() < 2 or not torch.cuda.can_device_access_peer(0, 1):
        pytest.skip("needs two GPUs with peer access")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():  # (its waits are bounded: this is for a rank stuck on the host side)
            p.terminate()
            p.join(timeout=10)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert result.get(timeout=10) is True
