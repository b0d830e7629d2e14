"""The 8-bit LM head and the vocabulary-sharded draw, on the GPU through the
C ABI, against the oracle.

The head's group sums run on the tensor cores, whose order of additions is
not the oracle's sequential one: logits are compared by tolerance (and bit for
bit on inputs whose sums are exact in binary32 in any order). The sharded
draw is then checked bit for bit: the oracle samples the very logits the GPU
produced, one pass over the whole row, and the shards' merged draw has to
give the same token, kept set and probabilities."""
from __future__ import annotations

import numpy as np
import pytest

import oracle
from gpu_util import np_u32, t_f32

pytestmark = pytest.mark.gpu


def _bf16(torch, bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).cuda()


def _to_bf16_bits(x):
    import workloads as wl

    return wl.to_bf16_bits(np.asarray(x, dtype=np.float32))


def _head_inputs(torch, rng, tokens, hidden, rows, exact=False):
    if exact:
        # Small integers times powers of two: every partial sum is exact.
        h = _to_bf16_bits(rng.integers(-4, 5, size=(tokens, hidden)).astype(np.float32))
        s = _to_bf16_bits(2.0 ** rng.integers(-6, -2, size=(rows, hidden // 64)).astype(np.float32))
        w = rng.integers(-128, 128, size=(rows, hidden), dtype=np.int8)
    else:
        h = _to_bf16_bits(rng.standard_normal((tokens, hidden), dtype=np.float32))
        s = _to_bf16_bits(rng.uniform(0.002, 0.02, size=(rows, hidden // 64)).astype(np.float32))
        w = rng.integers(-127, 128, size=(rows, hidden), dtype=np.int8)
    return h, w, s


def _gpu_logits(torch, lily, scratch, h, w, s):
    rows, tokens = w.shape[0], h.shape[0]
    out = torch.full((tokens, rows), float("nan"), dtype=torch.float32, device="cuda")
    scratch.lmhead_logits(torch.from_numpy(w).cuda(), _bf16(torch, s), _bf16(torch, h), out)
    torch.cuda.synchronize()
    assert scratch.status() == 0
    return out


@pytest.mark.parametrize("tokens,hidden,rows", [(64, 512, 256), (64, 1024, 1000), (5, 512, 257),
                                                (1, 2048, 4096), (33, 512, 40_000)])
def test_head_is_exact_where_the_sums_are(cuda, lily, tokens, hidden, rows):
    torch = cuda
    rng = np.random.default_rng([71, tokens, hidden, rows])
    h, w, s = _head_inputs(torch, rng, tokens, hidden, rows, exact=True)
    scratch = lily.SamplerScratch(rows, max_rows=64)
    got = _gpu_logits(cuda, lily, scratch, h, w, s).cpu().numpy()
    want = oracle.lmhead_int8(h, w, s, 64, 0, rows)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("tokens,hidden,rows", [(64, 1024, 2048), (17, 4096, 777)])
def test_head_matches_the_oracle_within_rounding(cuda, lily, tokens, hidden, rows):
    torch = cuda
    rng = np.random.default_rng([72, tokens, hidden, rows])
    h, w, s = _head_inputs(torch, rng, tokens, hidden, rows)
    scratch = lily.SamplerScratch(rows, max_rows=64)
    got = _gpu_logits(cuda, lily, scratch, h, w, s).cpu().numpy()
    want = oracle.lmhead_int8(h, w, s, 64, 0, rows)
    # Same products, same group order; only the order of the 64 adds inside a
    # group differs: a few ulp of the group sums.
    tol = 4e-6 * np.abs(want).max()
    assert np.abs(got - want).max() <= tol, (np.abs(got - want).max(), tol)


def _records(torch, n_shards, rows):
    return torch.zeros((n_shards, rows, 520), dtype=torch.uint8, device="cuda")


def _sharded_draw(torch, lily, logits, params, uniforms, n_shards, want_sums=True):
    """Shards run one after the other on this GPU: none waits for another."""
    rows, vocab = logits.shape
    assert vocab % n_shards == 0
    per = vocab // n_shards
    rec = _records(torch, n_shards, rows)
    shard = lily.SamplerScratch(per, max_rows=rows)
    for s in range(n_shards):
        part = logits[:, s * per:(s + 1) * per].contiguous()
        shard.shard_candidates(part, params, rec[s], first_id=s * per, want_sums=want_sums)
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    status = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    kept_n = torch.zeros(rows, dtype=torch.int32, device="cuda")
    kept_ids = torch.zeros((rows, 64), dtype=torch.int32, device="cuda")
    kept_probs = torch.zeros((rows, 64), dtype=torch.float32, device="cuda")
    lse = torch.zeros(rows, dtype=torch.float32, device="cuda")
    shard.merge_draw(rec, params, out, uniforms=t_f32(torch, uniforms), out_status=status,
                     kept_n=kept_n, kept_ids=kept_ids, kept_probs=kept_probs, out_lse=lse)
    torch.cuda.synchronize()
    assert shard.status() == 0
    return (np_u32(out), np_u32(status), np_u32(kept_n), np_u32(kept_ids), kept_probs.cpu().numpy(),
            lse.cpu().numpy())


def _check_against_oracle(lf, plist, uniforms, got):
    ids, status, kept_n, kept_ids, kept_probs, lse = got
    for r in range(lf.shape[0]):
        d = oracle.sample(lf[r], oracle.params(**plist[r]), float(uniforms[r]), mode=1)
        assert status[r] == 0
        assert ids[r] == d.token, f"row {r}"
        n = len(d.kept_ids)
        assert kept_n[r] == n, f"row {r}: kept {kept_n[r]} vs {n}"
        assert np.array_equal(kept_ids[r, :n], d.kept_ids), f"row {r}: kept ids"
        assert np.abs(kept_probs[r, :n] - d.kept_prob).max() <= 1e-5
        p = plist[r]
        greedy = p.get("temperature", 0.0) <= 0.0 or p.get("top_k", 1) == 1
        adj = lf[r].astype(np.float64) / (1.0 if greedy else np.float32(p["temperature"]))
        want_lse = adj.max() + np.log(np.exp(adj - adj.max()).sum())
        assert abs(lse[r] - want_lse) <= 1e-3 * max(1.0, abs(want_lse)), (r, lse[r], want_lse)


@pytest.mark.parametrize("n_shards", [1, 2, 8])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_sharded_draw_equals_the_whole_row_draw(cuda, lily, n_shards, dtype):
    torch = cuda
    import workloads as wl

    rows, vocab = 12, 65_536
    rng = np.random.default_rng([73, n_shards])
    x = wl.zipf_logits(rng, rows, vocab)
    plist = [dict(temperature=[0.7, 1.0, 0.0, 0.9][r % 4], top_k=[40, 64, 1, 7][r % 4],
                  top_p=[0.95, 1.0, 1.0, 0.8][r % 4], min_p=[0.0, 0.02, 0.0, 0.0][r % 4], seed=r)
             for r in range(rows)]
    u = np.array([oracle.uniform_for(500 + r, 3) for r in range(rows)], dtype=np.float32)
    if dtype == "bf16":
        bits = wl.to_bf16_bits(x)
        logits = _bf16(torch, bits)
        lf = oracle.widen_bf16(bits)
    else:
        logits = t_f32(torch, x)
        lf = x
    params = [lily.SamplingParams(**p) for p in plist]
    got = _sharded_draw(cuda, lily, logits, params, u, n_shards)
    _check_against_oracle(lf, plist, u, got)


@pytest.mark.parametrize("n_shards", [2, 4])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_sharded_draw_of_a_batch_the_one_block_per_row_kernel_takes(cuda, lily, n_shards, dtype):
    """From 16 rows on, with shards of eight rounds and more, the candidate launch is
    the kernel of one block per row, which ends in the rows' records; greedy rows,
    a top-k of 64 and equal logits across the shards' borders included."""
    torch = cuda
    import workloads as wl

    rows, vocab = 24, 262_144
    rng = np.random.default_rng([74, n_shards])
    x = wl.zipf_logits(rng, rows, vocab)
    per = vocab // n_shards
    for r in range(0, rows, 3):  # the row's largest value again, just across a border
        x[r, per + (r % 5)] = x[r].max()
    plist = [dict(temperature=[0.7, 1.0, 0.0, 0.9][r % 4], top_k=[40, 64, 1, 7][r % 4],
                  top_p=[0.95, 1.0, 1.0, 0.8][r % 4], min_p=[0.0, 0.02, 0.0, 0.0][r % 4], seed=r)
             for r in range(rows)]
    u = np.array([oracle.uniform_for(700 + r, 5) for r in range(rows)], dtype=np.float32)
    if dtype == "bf16":
        bits = wl.to_bf16_bits(x)
        logits = _bf16(torch, bits)
        lf = oracle.widen_bf16(bits)
    else:
        logits = t_f32(torch, x)
        lf = x
    params = [lily.SamplingParams(**p) for p in plist]
    got = _sharded_draw(cuda, lily, logits, params, u, n_shards)
    _check_against_oracle(lf, plist, u, got)


def test_sharded_draw_with_ties_across_shards(cuda, lily):
    """Equal logits in different shards: the lower id wins, as in one pass."""
    torch = cuda
    rows, vocab = 4, 32_768
    x = np.full((rows, vocab), -3.0, dtype=np.float32)
    x[:, 100::4096] = 2.0  # the same value once per 4096 ids
    x[1, 20_000] = 2.0
    plist = [dict(temperature=1.0, top_k=k, top_p=1.0, seed=1) for k in (3, 5, 8, 64)]
    u = np.array([0.1, 0.5, 0.9, 0.999], dtype=np.float32)
    params = [lily.SamplingParams(**p) for p in plist]
    got = _sharded_draw(cuda, lily, t_f32(torch, x), params, u, 8)
    _check_against_oracle(x, plist, u, got)


def test_sharded_calls_refuse_what_they_cannot_do(cuda, lily):
    torch = cuda
    scratch = lily.SamplerScratch(4096, max_rows=4)
    logits = torch.zeros((1, 4096), dtype=torch.float32, device="cuda")
    rec = _records(torch, 1, 1)
    with pytest.raises(lily.LilyError):
        scratch.shard_candidates(logits, [lily.SamplingParams(temperature=1.0, top_k=0)], rec[0])
    with pytest.raises(lily.LilyError):
        scratch.shard_candidates(logits, [lily.SamplingParams(temperature=1.0, top_k=65)], rec[0])
    with pytest.raises(lily.LilyError):
        scratch.shard_candidates(logits, [lily.SamplingParams(temperature=1.0, top_k=8,
                                                              repetition_penalty=1.2)], rec[0])
    with pytest.raises(lily.LilyError):  # no LM head scratch on this handle
        scratch.lmhead_shard_candidates(torch.zeros((4096, 512), dtype=torch.int8, device="cuda"),
                                        torch.zeros((4096, 8), dtype=torch.bfloat16, device="cuda"),
                                        torch.zeros((1, 512), dtype=torch.bfloat16, device="cuda"),
                                        [lily.SamplingParams(temperature=1.0, top_k=8)], rec[0])


@pytest.mark.parametrize("n_shards", [1, 4])
def test_head_then_sharded_draw_small(cuda, lily, n_shards):
    """The fused call of each shard (head into the handle's logits, then the
    records), merged; the oracle draws from the logits the GPU head produced."""
    torch = cuda
    import workloads as wl

    cfg = wl.config5(tokens=64, hidden=1024, vocab=16_384, seed=77)
    rows, vocab = 64, 16_384
    per = vocab // n_shards
    w = torch.from_numpy(cfg.weight).cuda()
    s = _bf16(torch, cfg.scales)
    h = _bf16(torch, cfg.hidden)
    plist = [dict(cfg.params, seed=cfg.params["seed"] + t) for t in range(rows)]
    params = [lily.SamplingParams(**p) for p in plist]
    rec = _records(torch, n_shards, rows)
    shard = lily.SamplerScratch(per, max_rows=rows, lmhead=True)
    for i in range(n_shards):
        shard.lmhead_shard_candidates(w[i * per:(i + 1) * per], s[i * per:(i + 1) * per], h, params,
                                      rec[i], first_id=i * per, want_sums=True)
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    status = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    kept_n = torch.zeros(rows, dtype=torch.int32, device="cuda")
    kept_ids = torch.zeros((rows, 64), dtype=torch.int32, device="cuda")
    kept_probs = torch.zeros((rows, 64), dtype=torch.float32, device="cuda")
    lse = torch.zeros(rows, dtype=torch.float32, device="cuda")
    shard.merge_draw(rec, params, out, uniforms=t_f32(torch, cfg.uniforms), out_status=status,
                     kept_n=kept_n, kept_ids=kept_ids, kept_probs=kept_probs, out_lse=lse)
    torch.cuda.synchronize()
    assert shard.status() == 0
    whole = lily.SamplerScratch(vocab, max_rows=rows)
    lf = _gpu_logits(cuda, lily, whole, cfg.hidden, cfg.weight, cfg.scales).cpu().numpy()
    ref = oracle.lmhead_int8(cfg.hidden, cfg.weight, cfg.scales, 64, 0, vocab)
    assert np.abs(lf - ref).max() <= 4e-6 * np.abs(ref).max()
    got = (np_u32(out), np_u32(status), np_u32(kept_n), np_u32(kept_ids), kept_probs.cpu().numpy(),
           lse.cpu().numpy())
    _check_against_oracle(lf, plist, cfg.uniforms, got)


def test_config5_full_size(cuda, lily):
    """hidden [64, 4096] x int8 [262144, 4096], 8 shards run in turn on this
    GPU. The head is checked on three bands of rows against the oracle; the
    sharded draw against the oracle's draw from the GPU's own logits."""
    torch = cuda
    import workloads as wl

    cfg = wl.config5()
    rows, vocab, n_shards = 64, 262_144, 8
    per = vocab // n_shards
    w = torch.from_numpy(cfg.weight).cuda()
    s = _bf16(torch, cfg.scales)
    h = _bf16(torch, cfg.hidden)
    plist = [dict(cfg.params, seed=cfg.params["seed"] + t) for t in range(rows)]
    params = [lily.SamplingParams(**p) for p in plist]
    rec = _records(torch, n_shards, rows)
    shard = lily.SamplerScratch(per, max_rows=rows, lmhead=True)
    for i in range(n_shards):
        shard.lmhead_shard_candidates(w[i * per:(i + 1) * per], s[i * per:(i + 1) * per], h, params,
                                      rec[i], first_id=i * per, want_sums=True)
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    status = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    kept_n = torch.zeros(rows, dtype=torch.int32, device="cuda")
    kept_ids = torch.zeros((rows, 64), dtype=torch.int32, device="cuda")
    kept_probs = torch.zeros((rows, 64), dtype=torch.float32, device="cuda")
    lse = torch.zeros(rows, dtype=torch.float32, device="cuda")
    shard.merge_draw(rec, params, out, uniforms=t_f32(torch, cfg.uniforms), out_status=status,
                     kept_n=kept_n, kept_ids=kept_ids, kept_probs=kept_probs, out_lse=lse)
    torch.cuda.synchronize()
    assert shard.status() == 0
    whole = lily.SamplerScratch(vocab, max_rows=rows)
    lf_t = torch.empty((rows, vocab), dtype=torch.float32, device="cuda")
    whole.lmhead_logits(w, s, h, lf_t)
    torch.cuda.synchronize()
    assert whole.status() == 0
    lf = lf_t.cpu().numpy()
    # The whole head against the oracle's fp32 product (all host threads).
    ref = oracle.lmhead_int8_all(cfg.hidden, cfg.weight, cfg.scales, 64)
    assert np.abs(lf - ref).max() <= 4e-6 * np.abs(ref).max()
    got = (np_u32(out), np_u32(status), np_u32(kept_n), np_u32(kept_ids), kept_probs.cpu().numpy(),
           lse.cpu().numpy())
    _check_against_oracle(lf, plist, cfg.uniforms, got)
    # End to end: the oracle's product, then the oracle's draw, against the GPU
    # head and its sharded draw. The two products differ in the order of a
    # group's 64 adds (a few 1e-6 relative), so a token may differ only where
    # the draw sits that close to a boundary: such rows are listed and checked.
    differ = []
    for r in range(rows):
        d = oracle.sample(ref[r], oracle.params(**plist[r]), float(cfg.uniforms[r]), mode=1)
        n = len(d.kept_ids)
        # The global top-k lies inside the union of the shards' best 64.
        sent = set(np_u32(rec[:, r, :512].contiguous().view(torch.int32)).reshape(n_shards, 64, 2)[:, :, 1]
                   .ravel().tolist())
        assert set(d.kept_ids.tolist()) <= sent, f"row {r}: a kept id is in no shard's record"
        if got[0][r] != d.token:
            cum = np.cumsum(d.kept_prob.astype(np.float64))
            gap = np.abs(cum - float(cfg.uniforms[r]) * cum[-1]).min()
            differ.append((r, int(got[0][r]), int(d.token), int(d.near_tie), float(gap)))
    print(f"config 5 end to end: {rows - len(differ)} of {rows} tokens equal the oracle's; others "
          f"(row, gpu, oracle, near-tie flag, distance of the draw to a boundary): {differ}")
    assert len(differ) <= 2
    for r, g, o, near, gap in differ:
        assert near or gap < 1e-5, f"row {r}: token {g} vs {o} with no boundary near"


def test_a_wait_that_runs_out_returns_with_a_named_status(cuda, lily):
    """Failure detection without a fault. The head kernel's roles wait on one
    another through barriers in shared memory, every wait bounded on the device
    (the reference bounds its waits on the host: src/metal.rs:856-861,
    1276-1279). The test hook leaves out one weight copy of the first block, so
    the wait of that stage's consumers runs out at a 2 ms limit: the launch has
    to complete, the handle has to report LILY_ERR_TIMEOUT once and stay
    usable, and the next launch (which needs the tensor memory the block that
    gave up held) has to be bit-exact."""
    torch = cuda
    tokens, hidden, rows = 64, 1024, 16_384
    rng = np.random.default_rng([73, tokens, hidden, rows])
    h, w, s = _head_inputs(torch, rng, tokens, hidden, rows, exact=True)
    want = oracle.lmhead_int8(h, w, s, 64, 0, rows)
    scratch = lily.SamplerScratch(rows, max_rows=64)
    wd, sd, hd = torch.from_numpy(w).cuda(), _bf16(torch, s), _bf16(torch, h)
    out = torch.zeros((tokens, rows), dtype=torch.float32, device="cuda")

    scratch.set_wait_limit(2_000_000)
    scratch.inject_lost_copy(3)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    scratch.lmhead_logits(wd, sd, hd, out)
    t1.record()
    torch.cuda.synchronize()
    assert 1.5 < t0.elapsed_time(t1) < 200.0, "the block gives up after its limit, not after a second"
    assert scratch.status() == lily.ERR_TIMEOUT
    assert scratch.status() == lily.OK, "reading the status clears it"
    # The other blocks were not disturbed: their tiles of 256 rows are exact.
    got = out.cpu().numpy()
    assert np.array_equal(got[:, 256:].view(np.uint32), want[:, 256:].view(np.uint32))

    # The hook was for one launch; the default limit is back with 0.
    scratch.set_wait_limit(0)
    out.zero_()
    scratch.lmhead_logits(wd, sd, hd, out)
    torch.cuda.synchronize()
    assert scratch.status() == lily.OK
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    scratch.close()


@pytest.mark.parametrize("n_shards", [2, 8])
def test_records_through_peer_memory_one_gpu_playing_every_rank(cuda, lily, n_shards):
    """lily_shard_publish / lily_merge_draw_peer with one GPU in the part of every
    rank (one exchange buffer, the ranks publish one after the other): three steps,
    so that both slots and the step counter are used; each has to give what
    lily_merge_draw gives on the same records handed over as one tensor."""
    torch = cuda
    import workloads as wl
    from lily_b200.shard import PeerExchange

    rows, vocab = 12, 65_536
    per = vocab // n_shards
    rng = np.random.default_rng([75, n_shards])
    plist = [dict(temperature=[0.7, 1.0, 0.0, 0.9][r % 4], top_k=[40, 64, 1, 7][r % 4],
                  top_p=[0.95, 1.0, 1.0, 0.8][r % 4], seed=r) for r in range(rows)]
    params = [lily.SamplingParams(**p) for p in plist]
    shard = lily.SamplerScratch(per, max_rows=rows)
    ex = PeerExchange(torch.cuda.current_device(), max_rows=16, emulate=n_shards)
    for step in range(3):
        logits = t_f32(torch, wl.zipf_logits(rng, rows, vocab))
        u = t_f32(torch, np.array([oracle.uniform_for(800 + r, step) for r in range(rows)], dtype=np.float32))
        rec = _records(torch, n_shards, rows)
        for s in range(n_shards):
            shard.shard_candidates(logits[:, s * per:(s + 1) * per].contiguous(), params, rec[s],
                                   first_id=s * per, want_sums=True)
        want, want_lse = (torch.zeros(rows, dtype=torch.int32, device="cuda"),
                          torch.zeros(rows, dtype=torch.float32, device="cuda"))
        shard.merge_draw(rec, params, want, uniforms=u, out_lse=want_lse)
        got, got_lse = torch.full_like(want, -1), torch.zeros_like(want_lse)
        # The other ranks publish apart from their merge; the last one in one call.
        ex.step += 1
        last = n_shards - 1
        for s in range(last):
            shard.shard_publish(ex.as_rank(s), rec[s], ex.step)
        shard.merge_draw_peer(ex.as_rank(last), ex.step, params, got, records=rec[last], uniforms=u,
                              out_lse=got_lse)
        torch.cuda.synchronize()
        assert shard.status() == lily.OK
        assert torch.equal(got, want) and torch.equal(got_lse, want_lse), f"step {step}"
    # A rank that never publishes: the wait runs out at its limit, the call returns,
    # and the status says so (failure detection without a fault).
    shard.set_wait_limit(2_000_000)
    ex.step += 1
    for s in range(1, last):
        shard.shard_publish(ex.as_rank(s), rec[s], ex.step)
    shard.merge_draw_peer(ex.as_rank(last), ex.step, params, got, records=rec[last], uniforms=u)
    torch.cuda.synchronize()
    assert shard.status() == lily.ERR_TIMEOUT
    shard.set_wait_limit(0)
    shard.shard_publish(ex.as_rank(0), rec[0], ex.step)
    shard.merge_draw_peer(ex.as_rank(last), ex.step, params, got, uniforms=u, out_lse=got_lse)
    torch.cuda.synchronize()
    assert shard.status() == lily.OK and torch.equal(got, want)
    ex.close()
    shard.close()
