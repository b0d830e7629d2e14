"""The benchmark's configurations at their full shapes, GPU against the CPU
oracle: token ids and accepted-draft counts bit-exact, kept probabilities
within 1e-5. Rows whose top-k / top-p cut lies within 1e-6 relative of a tie
are counted and printed (they are still required to match)."""
import numpy as np
import pytest

import oracle
from gpu_util import assert_parity, oracle_rows, run_batch
from test_spec_gpu import gpu_verify

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def W(lily):
    import workloads as w
    return w


def test_config1_single_row_1000_steps(cuda, lily, W):
    s = lily.SamplerScratch(W.VOCAB, max_rows=1)
    near = 0
    for greedy in (False, True):
        for step in range(1000):
            b = W.config1_step(step, greedy=greedy)
            res = run_batch(cuda, lily, s, b, want_kept=(step % 50 == 0))
            near += assert_parity(b, res, oracle_rows(b), label=f"config1 greedy={greedy} step {step}")
    print(f"config 1: 2000 draws bit-exact; near-tie rows among them: {near}")
    s.close()


def test_config2_server_batch(cuda, lily, W):
    s = lily.SamplerScratch(W.VOCAB, max_rows=4, max_list=64)
    near = 0
    for step in range(48):
        b = W.config2_step(step)
        res = run_batch(cuda, lily, s, b)
        near += assert_parity(b, res, oracle_rows(b), label=f"config2 step {step}")
        assert res.ids[2] == np.uint32(b.forced[2])
    print(f"config 2: 48 steps x 4 rows bit-exact; near-tie rows: {near}")
    s.close()


def test_config3_speculative_verification_10000_steps(cuda, lily, W):
    # The configuration's full length: 10 000 seeded steps in each acceptance
    # mode. Host threads make a step's inputs and run the CPU oracle on them
    # (numpy and the oracle both release the GIL); this thread runs the GPU.
    import os
    from concurrent.futures import ThreadPoolExecutor

    steps = 10_000
    s = lily.SamplerScratch(W.VOCAB, max_rows=3)
    hist = {False: np.zeros(3, dtype=np.int64), True: np.zeros(3, dtype=np.int64)}

    def host_side(args):
        step, greedy = args
        c = W.config3_step(step, greedy=greedy)
        st, want, want_acc = oracle.spec_verify(c.target_f32(), oracle.params(**c.params),
                                                c.draft_ids, c.u_accept, c.u_resid, q_dense=c.q)
        return step, greedy, c, st, want, want_acc

    work = [(step, greedy) for greedy in (False, True) for step in range(steps)]
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        chunk = 256  # bounds the inputs held in memory (2 MB a step)
        for at in range(0, len(work), chunk):
            for step, greedy, c, st, want, want_acc in pool.map(host_side, work[at:at + chunk]):
                assert st == 0
                got, acc, status = gpu_verify(cuda, lily, s, c.target, c.params, c.draft_ids, c.u_accept,
                                              c.u_resid, q_dense=c.q,
                                              mode=lily.SPEC_GREEDY_MATCH if greedy else lily.SPEC_REJECTION)
                assert np.array_equal(got, want), f"config3 greedy={greedy} step {step}"
                assert acc == want_acc and not status.any()
                hist[greedy][acc] += 1
    assert hist[False].sum() == steps and hist[True].sum() == steps
    print(f"config 3, {steps} steps per mode, accepted-draft histogram (0 / 1 / 2 drafts): rejection "
          f"sampling {hist[False].tolist()}, greedy match {hist[True].tolist()}")
    s.close()


def test_config4_large_batch(cuda, lily, W):
    b = W.config4_batch()
    s = lily.SamplerScratch(W.VOCAB, max_rows=256)
    res = run_batch(cuda, lily, s, b)
    near = assert_parity(b, res, oracle_rows(b), label="config4")
    print(f"config 4: 256 rows bit-exact; near-tie rows: {near}")
    # Size-independent properties: every token is in its kept set, the kept set
    # is sorted by adjusted logit, its probabilities sum to one, and a batch
    # of the same rows in another order draws the same tokens.
    lf = b.logits_f32()
    for r in range(256):
        n = res.kept_n[r]
        assert 1 <= n <= 50 and res.ids[r] in res.kept_ids[r, :n]
        assert abs(float(res.kept_probs[r, :n].sum()) - 1.0) < 1e-4
        assert np.all(np.diff(res.kept_probs[r, :n]) <= 0)
    perm = np.random.default_rng(0).permutation(256)
    shuffled = W.Batch(b.logits[perm], True, [b.params[i] for i in perm], b.uniforms[perm],
                       b.history[perm], b.history_len[perm])
    res2 = run_batch(cuda, lily, s, shuffled, want_kept=False)
    assert np.array_equal(res2.ids, res.ids[perm])
    # A rank's share of the 256 rows when they are split over 2, 4 or 8 GPUs (and a
    # ragged one): from 148 rows down a block has its SM to itself and streams
    # through the deep ring. Same rows, same tokens and kept sets.
    for lo, n in ((0, 128), (64, 64), (224, 32), (100, 17)):
        part = W.Batch(b.logits[lo:lo + n], True, b.params[lo:lo + n], b.uniforms[lo:lo + n],
                       b.history[lo:lo + n], b.history_len[lo:lo + n])
        res3 = run_batch(cuda, lily, s, part)
        assert np.array_equal(res3.ids, res.ids[lo:lo + n]), f"rows {lo}..{lo + n}"
        assert np.array_equal(res3.kept_n, res.kept_n[lo:lo + n])
        assert np.array_equal(res3.kept_ids, res.kept_ids[lo:lo + n])
    s.close()
