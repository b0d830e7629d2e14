"""GPU parity: lily_sample_batch (through the C ABI) against the CPU oracle
on identical seeded logits, histories, lists and uniforms. Token ids and the
kept sets are compared bit-exact; kept probabilities within 1e-5 absolute."""
import numpy as np
import pytest

import oracle
from gpu_util import assert_parity, np_u32, oracle_rows, run_batch, t_logits

pytestmark = pytest.mark.gpu


def make_batch(w, rng, rows, vocab, k, bf16, *, temperature=0.8, top_p=0.9, min_p=0.02,
               history=0, rep=1.0, presence=0.0, frequency=0.0, n_bias=0, n_ban=0,
               quantise=None, kind="uniform"):
    if kind == "uniform":
        x = rng.uniform(-8, 8, (rows, vocab)).astype(np.float32)
    elif kind == "zipf":
        x = w.zipf_logits(rng, rows, vocab)
    elif kind == "ascending":
        x = np.tile(np.linspace(-10, 10, vocab, dtype=np.float32), (rows, 1))
    elif kind == "descending":
        x = np.tile(np.linspace(10, -10, vocab, dtype=np.float32), (rows, 1))
    elif kind == "constant":
        x = np.full((rows, vocab), 0.25, dtype=np.float32)
    else:
        raise ValueError(kind)
    if quantise:
        x = np.round(x * quantise) / quantise
        x = x.astype(np.float32)
    logits = w.to_bf16_bits(x) if bf16 else x
    params = [dict(temperature=temperature, top_k=k, top_p=top_p, min_p=min_p,
                   repetition_penalty=rep, presence_penalty=presence,
                   frequency_penalty=frequency, seed=1000 + r) for r in range(rows)]
    u = rng.random(rows, dtype=np.float32)
    b = w.Batch(logits, bf16, params, u)
    if history:
        b.history = (rng.zipf(1.2, size=(rows, history)) % vocab).astype(np.uint32)
        b.history_len = rng.integers(history // 2, history + 1, rows).astype(np.uint32)
    ld = max(n_bias, n_ban)
    if n_bias:
        b.bias_ids = rng.integers(0, vocab, (rows, ld)).astype(np.uint32)
        b.bias_vals = rng.choice(np.array([-5.0, 5.0], dtype=np.float32), (rows, ld))
        b.bias_len = np.full(rows, n_bias, dtype=np.uint32)
        if n_bias > 2:
            b.bias_ids[:, 1] = b.bias_ids[:, 0]  # a duplicate: entries add
    if n_ban:
        b.ban_ids = rng.integers(0, vocab, (rows, ld)).astype(np.uint32)
        b.ban_len = np.full(rows, n_ban, dtype=np.uint32)
        if n_bias > 2:
            b.ban_ids[:, 0] = b.bias_ids[:, 2]  # banned and biased at once
    return b


@pytest.fixture(scope="module")
def W(lily):
    import workloads as w
    return w


def check(cuda, lily, W, batch, vocab, label, **kw):
    rows = batch.logits.shape[0]
    s = lily.SamplerScratch(vocab, max_rows=max(rows, 1), max_list=256)
    try:
        res = run_batch(cuda, lily, s, batch, **kw)
        again = run_batch(cuda, lily, s, batch, **kw)
        assert np.array_equal(res.ids, again.ids), f"{label}: not deterministic"
        want = oracle_rows(batch)
        return assert_parity(batch, res, want, label=label)
    finally:
        s.close()


def test_greedy_tie_takes_the_lowest_id(cuda, lily, W):
    # tests/unit/kernels/sample.rs:74-83
    for bf16 in (False, True):
        x = np.zeros((1, 5000), dtype=np.float32)
        x[0, 1234] = 7.5
        x[0, 4321] = 7.5
        b = W.Batch(W.to_bf16_bits(x) if bf16 else x, bf16, [dict()], np.array([0.5], np.float32))
        s = lily.SamplerScratch(5000)
        res = run_batch(cuda, lily, s, b)
        assert res.ids[0] == 1234 and res.status[0] == 0
        out = cuda.zeros(1, dtype=cuda.int32, device="cuda")
        s.argmax_batch(t_logits(cuda, b), out)
        cuda.cuda.synchronize()
        assert np_u32(out)[0] == 1234
        s.close()


def test_argmax_route_ignores_nan_and_ties_zeros(cuda, lily, W):
    # src/kernels/metal/elementwise.metal:145-150: NaN never wins; -0 == +0.
    x = np.full((3, 777), -1.0, dtype=np.float32)
    x[0, 5] = np.nan
    x[0, 9] = 2.0
    x[1, 100] = -0.0
    x[1, 200] = 0.0
    x[2, :] = np.nan
    b = W.Batch(x, False, [dict()] * 3, np.zeros(3, np.float32))
    s = lily.SamplerScratch(777, max_rows=3)
    res = run_batch(cuda, lily, s, b)
    assert list(res.ids) == [9, 100, 0]
    assert [oracle.argmax(x[r]) for r in range(3)] == [9, 100, 0]
    s.close()
    # The same with several rounds and several slices per row, the NaN in the
    # first round, in a later one, and at the very end.
    for vocab in (4096, 5000, 40_000):
        for at in (5, vocab // 2, vocab - 1):
            y = np.full((1, vocab), -1.0, dtype=np.float32)
            y[0, at] = np.nan
            want = 9 if at != 9 else 10
            y[0, want] = 2.0
            for bf16 in (False, True):
                b = W.Batch(W.to_bf16_bits(y) if bf16 else y, bf16, [dict()], np.zeros(1, np.float32))
                s = lily.SamplerScratch(vocab)
                res = run_batch(cuda, lily, s, b)
                assert res.ids[0] == want and res.status[0] == 0, (vocab, at, bf16)
                s.close()


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("vocab", [1, 31, 32, 33, 700, 4099, 6007])
def test_small_vocabularies(cuda, lily, W, vocab, bf16):
    rng = np.random.default_rng(vocab * 2 + bf16)
    near = 0
    for k in (0, 1, 2, 20, 64, 65, 1024):
        for rows in (1, 3, 4):
            b = make_batch(W, rng, rows, vocab, k, bf16, history=64, rep=1.2, presence=0.3,
                           frequency=0.1)
            near += check(cuda, lily, W, b, vocab, f"V={vocab} k={k} B={rows}")
    print(f"near-tie rows (reported, all matched): {near}")


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("rows", [1, 4, 37, 200])
def test_full_vocabulary(cuda, lily, W, rows, bf16):
    rng = np.random.default_rng(rows * 2 + bf16)
    vocab = W.VOCAB
    for k, kw in ((50, dict(history=4096, rep=1.1)),
                  (0, dict(top_p=0.95, min_p=0.0)),
                  (20, dict(history=2048, presence=0.5, frequency=0.2)),
                  (40, dict(history=1024, rep=0.8, presence=-0.2)),  # penalties that raise logits
                  (1, dict(history=512, rep=1.3)),                   # greedy with penalties
                  (1, dict())):                                       # exact argmax
        b = make_batch(W, rng, rows, vocab, k, bf16, kind="zipf", **kw)
        check(cuda, lily, W, b, vocab, f"V={vocab} k={k} B={rows} {kw}")


def test_bias_ban_and_forced_rows(cuda, lily, W):
    rng = np.random.default_rng(77)
    for vocab, rows in ((6007, 4), (W.VOCAB, 4), (W.VOCAB, 64)):
        b = make_batch(W, rng, rows, vocab, 20, True, kind="zipf", history=1024, presence=0.5,
                       frequency=0.2, n_bias=64, n_ban=8)
        b.forced = np.full(rows, -1, dtype=np.int32)
        b.forced[2] = 4242
        check(cuda, lily, W, b, vocab, f"lists V={vocab} B={rows}")
    # A banned top token must not win a greedy row.
    x = np.zeros((1, 4099), dtype=np.float32)
    x[0, 17], x[0, 99] = 9.0, 8.0
    b = W.Batch(x, False, [dict()], np.zeros(1, np.float32))
    b.ban_ids = np.array([[17]], dtype=np.uint32)
    b.ban_len = np.array([1], dtype=np.uint32)
    s = lily.SamplerScratch(4099)
    res = run_batch(cuda, lily, s, b)
    assert res.ids[0] == 99
    s.close()


@pytest.mark.parametrize("kind", ["ascending", "descending", "constant"])
def test_adversarial_orders_and_ties(cuda, lily, W, kind):
    rng = np.random.default_rng(5)
    for vocab, rows in ((40000, 2), (W.VOCAB, 1), (W.VOCAB, 150)):
        for k in (0, 50):
            b = make_batch(W, rng, rows, vocab, k, kind != "constant", kind=kind, top_p=0.99,
                           min_p=0.0)
            check(cuda, lily, W, b, vocab, f"{kind} V={vocab} k={k} B={rows}")


def test_heavy_ties_at_the_top_k_boundary(cuda, lily, W):
    # Logits on a coarse grid: hundreds of exact ties straddle the k-th value,
    # which the oracle resolves by lowest id (tests/unit/kernels/sample.rs:32-34).
    rng = np.random.default_rng(9)
    for vocab, rows in ((6007, 3), (W.VOCAB, 1), (W.VOCAB, 160)):
        for k in (20, 64, 1024):
            b = make_batch(W, rng, rows, vocab, k, False, quantise=4, top_p=1.0, min_p=0.0)
            check(cuda, lily, W, b, vocab, f"ties V={vocab} k={k} B={rows}")


def test_a_row_does_not_depend_on_its_batch(cuda, lily, W):
    # src/qwen4exp/batch.rs:43-44; also: many slices per row == one slice per row.
    rng = np.random.default_rng(21)
    vocab = W.VOCAB
    big = make_batch(W, rng, 160, vocab, 50, True, kind="zipf", history=2048, rep=1.1)
    s = lily.SamplerScratch(vocab, max_rows=160)
    whole = run_batch(cuda, lily, s, big)
    for r in (0, 7, 159):
        one = W.Batch(big.logits[r:r + 1], True, [big.params[r]], big.uniforms[r:r + 1],
                      big.history[r:r + 1], big.history_len[r:r + 1])
        alone = run_batch(cuda, lily, s, one)
        assert alone.ids[0] == whole.ids[r]
        assert alone.kept_n[0] == whole.kept_n[r]
        n = alone.kept_n[0]
        assert np.array_equal(alone.kept_ids[0, :n], whole.kept_ids[r, :n])
        assert np.array_equal(alone.kept_probs[0, :n], whole.kept_probs[r, :n])
    s.close()


def test_error_rows(cuda, lily, W):
    vocab = 6007
    x = np.random.default_rng(1).uniform(-4, 4, (3, vocab)).astype(np.float32)
    x[0, 100] = np.nan
    b = W.Batch(x, False, [dict(temperature=1.0, top_k=20)] * 3, np.full(3, 0.5, np.float32))
    b.ban_ids = np.zeros((3, 1), dtype=np.uint32)
    b.ban_len = np.zeros(3, dtype=np.uint32)
    s = lily.SamplerScratch(vocab, max_rows=3)
    res = run_batch(cuda, lily, s, b)
    want = oracle_rows(b)
    assert res.status[0] == lily.ROW_NAN == want[0].status and res.ids[0] == 0xFFFFFFFF
    assert res.status[1] == 0 and res.ids[1] == want[1].token
    assert s.status() == lily.ERR_DEVICE_ROW
    assert s.status() == lily.OK
    # Every id banned: the row has no finite logit.
    small = 64
    y = np.zeros((1, small), dtype=np.float32)
    b2 = W.Batch(y, False, [dict(temperature=1.0, top_k=8)], np.zeros(1, np.float32))
    b2.ban_ids = np.arange(small, dtype=np.uint32)[None, :]
    b2.ban_len = np.array([small], dtype=np.uint32)
    s2 = lily.SamplerScratch(small)
    r2 = run_batch(cuda, lily, s2, b2)
    assert r2.status[0] == lily.ROW_NONFINITE and oracle_rows(b2)[0].status == oracle.ERR_NONFINITE
    s.close()
    s2.close()


@pytest.mark.parametrize("vocab, rows", [(6007, 3), (151_936, 150)])
def test_a_list_length_beyond_its_bound_refuses_the_row(cuda, lily, W, vocab, rows):
    # The lengths are device values. One beyond max_history / max_list (or beyond
    # the row pitch) would walk into the next row or past the buffer: the row is
    # refused instead. The lists here are longer than the bound, so nothing is
    # read out of bounds whatever the kernel does with the length.
    rng = np.random.default_rng(3)
    b = make_batch(W, rng, rows, vocab, 20, True, kind="zipf", history=256, rep=1.2, n_bias=8, n_ban=8)
    b.history_len[:] = 100
    b.history_len[0] = 200               # > max_history = 128, inside the 256-id row
    b.bias_len[1] = 7                    # > max_list = 6, inside the 8-entry row
    b.bias_len[2:] = 5
    b.bias_len[0] = 5
    b.ban_len[:] = 5
    s = lily.SamplerScratch(vocab, max_rows=rows, max_history=128, max_list=6)
    res = run_batch(cuda, lily, s, b)
    want = oracle_rows(b)
    for r in (0, 1):
        assert res.status[r] == lily.ROW_LIST and res.ids[r] == 0xFFFFFFFF and res.kept_n[r] == 0
    for r in range(2, rows):
        assert res.status[r] == 0 and res.ids[r] == want[r].token, f"row {r}"
    assert s.status() == lily.ERR_DEVICE_ROW
    s.close()


def test_host_side_argument_errors(cuda, lily, W):
    vocab = 1000
    s = lily.SamplerScratch(vocab, max_rows=2)
    logits = cuda.zeros((2, vocab), dtype=cuda.float32, device="cuda")
    out = cuda.zeros(2, dtype=cuda.int32, device="cuda")
    u = cuda.zeros(2, dtype=cuda.float32, device="cuda")
    bad = [lily.SamplingParams(temperature=1.0, top_k=5), lily.SamplingParams(top_p=0.0)]
    with pytest.raises(lily.LilyError) as e:
        s.sample_batch(logits, bad, out, uniforms=u)
    assert e.value.code == lily.ERR_PARAMS
    three = cuda.zeros((3, vocab), dtype=cuda.float32, device="cuda")
    with pytest.raises(lily.LilyError) as e:
        s.sample_batch(three, [lily.SamplingParams()] * 3, out, uniforms=u)
    assert e.value.code == lily.ERR_CAPACITY
    with pytest.raises(lily.LilyError) as e:
        s.sample_batch(logits, [lily.SamplingParams()] * 2, out)
    assert e.value.code == lily.ERR_ARG
    # Fault latch (src/metal.rs:681-696): host-side only, nothing reaches the GPU.
    s.inject_fault(7)
    with pytest.raises(lily.LilyError) as e:
        s.sample_batch(logits, [lily.SamplingParams()] * 2, out, uniforms=u)
    assert e.value.code == lily.ERR_FAULT
    assert s.status() == lily.ERR_FAULT
    s.clear_fault()
    s.sample_batch(logits, [lily.SamplingParams()] * 2, out, uniforms=u)
    cuda.cuda.synchronize()
    assert s.status() == lily.OK
    s.close()


def test_seed_and_step_replace_uniforms(cuda, lily, W):
    # src/kernels/sample.rs:435-441: the draw for (seed, step) replays.
    rng = np.random.default_rng(4)
    vocab = 6007
    b = make_batch(W, rng, 4, vocab, 40, False)
    steps = [3, 4, 5, 0x40000006]
    b.uniforms = np.array([oracle.uniform_for(p["seed"], st) for p, st in zip(b.params, steps)],
                          dtype=np.float32)
    s = lily.SamplerScratch(vocab, max_rows=4)
    a = run_batch(cuda, lily, s, b, use_steps=steps)
    c = run_batch(cuda, lily, s, b)
    d = run_batch(cuda, lily, s, b, use_steps=steps, params_on_device=True)
    assert np.array_equal(a.ids, c.ids) and np.array_equal(a.ids, d.ids)
    assert_parity(b, a, oracle_rows(b), label="steps")
    s.close()


def test_unaligned_rows_take_the_scalar_path(cuda, lily, W):
    rng = np.random.default_rng(8)
    vocab = 6007  # odd pitch: rows 1.. are not 16-byte aligned
    for bf16 in (False, True):
        b = make_batch(W, rng, 3, vocab, 40, bf16, history=128, rep=1.1)
        check(cuda, lily, W, b, vocab, f"unaligned bf16={bf16}")


def test_histogram_slots(cuda, lily, W):
    # tests/unit/kernels/sample.rs:142-197
    v = 3000
    s = lily.SamplerScratch(v, max_rows=2, counts_table=True)
    x = np.zeros((1, v), dtype=np.float32)
    x[0, 10], x[0, 20] = 5.0, 4.0
    counts = np.zeros(v, dtype=np.uint32)
    counts[10] = 3
    s.write_counts(counts, slot=1)
    p = dict(presence_penalty=0.5, frequency_penalty=0.5, repetition_penalty=1.5)
    b = W.Batch(x, False, [p], np.zeros(1, np.float32))
    res = run_batch(cuda, lily, s, b, count_slots=[1])
    assert res.ids[0] == 20  # 5.0/1.5 - 0.5 - 1.5 = 1.33 < 4.0
    after = s.read_counts(slot=1)
    assert after[20] == 1 and after[10] == 3
    # The draw is now seen: drawing again penalises id 20 as well.
    want = oracle.sample(x[0], oracle.params(**p), 0.0, counts=after)
    res = run_batch(cuda, lily, s, b, count_slots=[1])
    assert res.ids[0] == want.token
    # Counts move between samplers whole, as a copy.
    engine = lily.SamplerScratch(v, max_rows=1, counts_table=True)
    c2 = np.zeros(v, dtype=np.uint32)
    c2[7], c2[v - 1] = 2, 5
    engine.write_counts(c2)
    s.write_counts(np.full(v, 9, dtype=np.uint32), slot=0)
    s.copy_counts_from(engine, slot=0)
    assert np.array_equal(s.read_counts(0), c2)
    engine.reset_counts()
    assert s.read_counts(0)[v - 1] == 5 and engine.read_counts().sum() == 0
    s.uncount(7, slot=0)
    s.uncount(v + 5, slot=0)  # out of range: ignored
    engine.copy_counts_from(s, other_slot=0)
    assert engine.read_counts()[7] == 1
    s.uncount(7, slot=0)
    s.uncount(7, slot=0)  # saturates at zero
    assert s.read_counts(0)[7] == 0
    other = lily.SamplerScratch(v + 1, counts_table=True)
    with pytest.raises(lily.LilyError) as e:
        other.copy_counts_from(engine)
    assert e.value.code == lily.ERR_VOCAB
    for h in (s, engine, other):
        h.close()


def test_histogram_mode_equals_history_mode(cuda, lily, W):
    rng = np.random.default_rng(31)
    vocab = W.VOCAB
    b = make_batch(W, rng, 4, vocab, 20, True, kind="zipf", history=4096, rep=1.1, presence=0.5,
                   frequency=0.2)
    s = lily.SamplerScratch(vocab, max_rows=4, counts_table=True)
    for r in range(4):
        s.write_counts(oracle.counts_from_history(b.history[r, :b.history_len[r]], vocab), slot=r)
    with_hist = run_batch(cuda, lily, s, b)
    hist, hl = b.history, b.history_len
    b.history = b.history_len = None
    with_table = run_batch(cuda, lily, s, b, count_slots=[0, 1, 2, 3])
    assert np.array_equal(with_hist.ids, with_table.ids)
    b.history, b.history_len = hist, hl
    assert_parity(b, with_table, oracle_rows(b), label="table")
    s.close()


def test_exp_matches_the_oracle_bit_for_bit(cuda, lily, W):
    xs = np.concatenate([
        np.linspace(-104.5, 0.0, 400_001), np.linspace(0, 89, 20_001),
        -np.logspace(-30, 2, 50_001),
        np.array([-np.inf, np.inf, 0.0, -0.0, -87.33654, -87.33655, -103.9720840, -103.9720841]),
    ]).astype(np.float32)
    got = lily.debug_exp(cuda.from_numpy(xs).cuda()).cpu().numpy()
    want = oracle.expf(xs)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # Reported distance from the platform libm (what Rust's f32::exp calls).
    libm = np.exp(xs.astype(np.float64)).astype(np.float32)
    fin = np.isfinite(libm) & (libm > 0)
    ulp = np.abs(got.view(np.int32).astype(np.int64) - libm.view(np.int32).astype(np.int64))[fin]
    print(f"exp vs correctly rounded: max {ulp.max()} ulp, {100 * (ulp == 0).mean():.2f}% exact")
    assert ulp.max() <= 1
