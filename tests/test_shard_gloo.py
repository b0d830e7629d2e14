"""Row-partitioned sampling over two ranks (gloo, CPU): the partition covers
every row once, and the tokens gathered from the ranks equal a single
process's. The draws themselves are the CPU oracle's here (no GPU in this
test); the GPU path runs the same partition in bench.py under torchrun."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_range_is_a_balanced_cover(lily):
    import lily_b200.shard as sh

    for rows in (1, 4, 7, 256, 257):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                rr = sh.row_range(rows, world, r)
                seen += list(rr)
                for row in rr:
                    assert sh.owner_of(row, rows, world) == r
            assert seen == list(range(rows))
            sizes = [len(sh.row_range(rows, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sh.row_range(4, 2, 2)


def _worker(rank, world, port, rows, vocab, out):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    import lily_b200  # noqa: F401
    import lily_b200.shard as sh
    import workloads as w
    import oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    batch = w.config2_step(0, vocab=vocab, rows=rows, history=256)
    lf = batch.logits_f32()
    mine = []
    for r in sh.row_range(rows, world, rank):
        if batch.forced[r] >= 0:
            mine.append(int(batch.forced[r]))
            continue
        d = oracle.sample(lf[r], oracle.params(**batch.params[r]), float(batch.uniforms[r]),
                          history=batch.history[r], bias_ids=batch.bias_ids[r],
                          bias_vals=batch.bias_vals[r], ban_ids=batch.ban_ids[r])
        mine.append(d.token)
    tokens = sh.gather_tokens(mine, rows, world, rank)
    if rank == 0:
        np.save(out, np.array(tokens, dtype=np.int64))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_draw_the_same_tokens_as_one(lily, tmp_path):
    import torch.multiprocessing as mp

    import workloads as w
    import oracle

    rows, vocab = 7, 4099
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "tokens.npy")
    mp.spawn(_worker, args=(2, port, rows, vocab, out), nprocs=2, join=True)
    got = np.load(out).tolist()
    batch = w.config2_step(0, vocab=vocab, rows=rows, history=256)
    lf = batch.logits_f32()
    want = []
    for r in range(rows):
        if batch.forced[r] >= 0:
            want.append(int(batch.forced[r]))
            continue
        want.append(oracle.sample(lf[r], oracle.params(**batch.params[r]), float(batch.uniforms[r]),
                                  history=batch.history[r], bias_ids=batch.bias_ids[r],
                                  bias_vals=batch.bias_vals[r], ban_ids=batch.ban_ids[r]).token)
    assert got == want


# ---------------------------------------------------------------- vocabulary --

def _top_record(adj, first_id, keep=64):
    """What a shard's record holds for one row: its best `keep` adjusted
    logits as (monotone key, vocabulary id), best first, ties by lower id."""
    bits = adj.view(np.uint32)
    key = np.where(bits >> 31, ~bits, bits | np.uint32(0x80000000)).astype(np.uint32)
    order = np.lexsort((np.arange(adj.size), -key.astype(np.int64)))[:keep]
    rec = np.zeros(520, dtype=np.uint8)
    pairs = rec[:512].view(np.uint32).reshape(64, 2)
    pairs[:, 1] = 0xFFFFFFFF
    pairs[:len(order), 0] = key[order]
    pairs[:len(order), 1] = order + first_id
    rec[512:516].view(np.float32)[0] = adj[order[0]]
    return rec


def _vocab_worker(rank, world, port, rows, vocab, out):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import lily_b200  # noqa: F401
    import lily_b200.shard as sh
    import workloads as w

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = w.zipf_logits(np.random.default_rng(91), rows, vocab)
    mine = sh.vocab_range(vocab, world, rank)
    local = np.stack([_top_record(np.ascontiguousarray(x[r, mine.start:mine.stop]), mine.start)
                      for r in range(rows)])
    gathered = sh.gather_records(torch.from_numpy(local))
    assert tuple(gathered.shape) == (world, rows, 520)
    if rank == 0:
        np.save(out, gathered.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_vocab_shards_gather_records_that_hold_the_global_top_k(lily, tmp_path):
    """Two gloo ranks build their shards' records on the CPU and all-gather
    them: the result is shard-major on every rank, and the best 40 of the
    union are the best 40 of the whole row (the property lily_merge_draw
    relies on)."""
    import torch.multiprocessing as mp

    import lily_b200.shard as sh
    import workloads as w

    rows, vocab, world = 3, 8192, 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "records.npy")
    mp.spawn(_vocab_worker, args=(world, port, rows, vocab, out), nprocs=world, join=True)
    g = np.load(out)
    x = w.zipf_logits(np.random.default_rng(91), rows, vocab)
    for r in range(rows):
        whole = _top_record(np.ascontiguousarray(x[r]), 0)[:512].view(np.uint32).reshape(64, 2)
        union = np.concatenate([g[s, r, :512].view(np.uint32).reshape(64, 2) for s in range(world)])
        for s in range(world):  # each shard's ids lie in its own range
            ids = g[s, r, :512].view(np.uint32).reshape(64, 2)[:, 1]
            rng_s = sh.vocab_range(vocab, world, s)
            assert ((ids >= rng_s.start) & (ids < rng_s.stop)).all()
        order = np.lexsort((union[:, 1], -union[:, 0].astype(np.int64)))[:40]
        assert np.array_equal(union[order], whole[:40])
    with pytest.raises(ValueError):
        sh.vocab_range(10, 3, 0)
