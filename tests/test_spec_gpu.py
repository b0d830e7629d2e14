"""GPU parity of the speculative verify step (lily_spec_verify) and of the
accept-count control block (lily_spec_accept) against the CPU oracle."""
import numpy as np
import pytest

import oracle
from gpu_util import np_u32, t_f32, t_u32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def W(lily):
    import workloads as w
    return w


def gpu_verify(torch, lily, scratch, target_bits, params, draft_ids, u_accept, u_resid, *,
               mode=0, q_dense=None, q_sparse=None, history=None, count_slot=None, step0=None):
    m = target_bits.shape[0]
    if target_bits.dtype == np.uint16:
        target = torch.from_numpy(target_bits.view(np.int16)).view(torch.bfloat16).cuda()
    else:
        target = t_f32(torch, target_bits)
    out = torch.full((m,), -1, dtype=torch.int32, device="cuda")
    acc = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    status = torch.full((m,), -1, dtype=torch.int32, device="cuda")
    kw = {}
    if q_dense is not None:
        kw["q_dense"] = t_f32(torch, q_dense)
    if q_sparse is not None:
        kw["q_ids"], kw["q_probs"], kw["q_n"] = (t_u32(torch, q_sparse[0]), t_f32(torch, q_sparse[1]),
                                                  t_u32(torch, q_sparse[2]))
    if history is not None:
        kw["history_ids"] = t_u32(torch, history)
    if step0 is None:
        kw["u_accept"], kw["u_resid"] = t_f32(torch, u_accept), t_f32(torch, u_resid)
    else:
        kw["step0"] = step0
    scratch.spec_verify(target, lily.SamplingParams(**params), t_u32(torch, draft_ids), out, acc,
                        mode=mode, count_slot=count_slot, out_status=status, **kw)
    torch.cuda.synchronize()
    return np_u32(out), int(np_u32(acc)[0]), np_u32(status)


def sparse_q(head, params, drafts):
    """The draft head's exported distributions (src/kernels/sample.rs:186-215)."""
    ids = np.zeros((drafts, 1024), dtype=np.uint32)
    probs = np.zeros((drafts, 1024), dtype=np.float32)
    n = np.zeros(drafts, dtype=np.uint32)
    for j in range(drafts):
        d = oracle.sample(head[j], oracle.params(**params), 0.0, mode=1)
        n[j] = len(d.kept_ids)
        ids[j, :n[j]] = d.kept_ids
        probs[j, :n[j]] = d.kept_prob
    return ids, probs, n


def test_spec_accept_control_block(cuda, lily):
    # tests/unit/kernels/spec.rs:14-48
    s = lily.SamplerScratch(1000)
    pos0, ratio, chain, stride = 13, 4, 3, 4
    cases = [
        ([5, 6, 7, 8], [1, 5, 6, 7], 3),
        ([5, 6, 9, 8], [1, 5, 6, 7], 2),
        ([5, 0, 7, 8], [1, 5, 6, 7], 1),
        ([4, 6, 7, 8], [1, 5, 6, 7], 0),
        ([5], [1], 0),
    ]
    for draws, ids, expected in cases:
        ctrl = cuda.zeros(lily.ctrl_words(chain, stride), dtype=cuda.int32, device="cuda")
        s.spec_accept(t_u32(cuda, draws), t_u32(cuda, ids), ctrl, pos0, ratio, chain, stride)
        cuda.cuda.synchronize()
        words = np_u32(ctrl)
        slot = lambda i: int(words[i * stride])
        assert slot(0) == expected == oracle.spec_accept(draws, ids)
        assert slot(1) == expected + 1
        for i in range(chain):
            p = pos0 + expected + 1 + i
            assert slot(2 + 3 * i) == p
            assert slot(3 + 3 * i) == p // ratio
            assert slot(4 + 3 * i) == int((p + 1) % ratio == 0)
    s.close()


@pytest.mark.parametrize("vocab", [4099, 151_936])
def test_rejection_sampling_matches_the_oracle(cuda, lily, W, vocab):
    # tests/unit/kernels/sample.rs:352-409 with own seeded inputs; exact here.
    rng = np.random.default_rng(23 + vocab)
    scratch = lily.SamplerScratch(vocab, max_rows=4)
    for name, params in (("server defaults", dict(temperature=1.0, top_k=20, top_p=0.95, seed=77)),
                         ("wide", dict(temperature=1.3, top_k=0, top_p=1.0, min_p=0.001, seed=78))):
        accepted_rows = rejected_rows = 0
        for step in range(24):
            drafts = 2 + step % 2
            m = drafts + 1
            head = rng.uniform(-6, 6, (drafts, vocab)).astype(np.float32)
            trunk = np.empty((m, vocab), dtype=np.float32)
            trunk[:drafts] = head + rng.uniform(-2.5, 2.5, (drafts, vocab)).astype(np.float32)
            trunk[drafts] = rng.uniform(-6, 6, vocab)
            trunk_bits = W.to_bf16_bits(trunk)
            trunk_w = W.bf16_bits_to_f32(trunk_bits)
            dp = {k: v for k, v in params.items()}
            q_ids, q_probs, q_n = sparse_q(head, dp, drafts)
            draft_ids = np.array([
                oracle.sample(head[j], oracle.params(**dp),
                              oracle.uniform_for(params["seed"], (step * m + j) | 0x40000000)).token
                for j in range(drafts)], dtype=np.uint32)
            ua = np.array([oracle.uniform_for(params["seed"], step * m + j) for j in range(m)], np.float32)
            ur = np.array([oracle.uniform_for(params["seed"], (step * m + j) | 0x80000000)
                           for j in range(drafts)], np.float32)
            st, want, want_acc = oracle.spec_verify(trunk_w, oracle.params(**params), draft_ids, ua, ur,
                                                    q_ids=q_ids, q_probs=q_probs, q_n=q_n)
            assert st == 0
            got, acc, status = gpu_verify(cuda, lily, scratch, trunk_bits, params, draft_ids, ua, ur,
                                          q_sparse=(q_ids, q_probs, q_n))
            assert np.array_equal(got, want), f"{name} step {step}: {got} vs {want}"
            assert acc == want_acc and not status.any()
            # The same step with the uniforms derived from (seed, step0 + j).
            got2, acc2, _ = gpu_verify(cuda, lily, scratch, trunk_bits, params, draft_ids, None, None,
                                       q_sparse=(q_ids, q_probs, q_n), step0=step * m)
            assert np.array_equal(got2, want) and acc2 == want_acc
            accepted_rows += int((got[:drafts] == draft_ids).sum())
            rejected_rows += int((got[:drafts] != draft_ids).sum())
        assert accepted_rows > 0 and rejected_rows > 0, f"{name}: both outcomes must occur"
    scratch.close()


def test_dense_draft_distribution_and_greedy_match(cuda, lily, W):
    vocab = W.VOCAB
    scratch = lily.SamplerScratch(vocab, max_rows=3)
    hist = np.zeros(3, dtype=np.int64)
    for step in range(40):
        s = W.config3_step(step, vocab=vocab)
        st, want, want_acc = oracle.spec_verify(s.target_f32(), oracle.params(**s.params), s.draft_ids,
                                                s.u_accept, s.u_resid, q_dense=s.q)
        assert st == 0
        got, acc, status = gpu_verify(cuda, lily, scratch, s.target, s.params, s.draft_ids, s.u_accept,
                                      s.u_resid, q_dense=s.q)
        assert np.array_equal(got, want) and acc == want_acc and not status.any()
        hist[acc] += 1
        g = W.config3_step(step, vocab=vocab, greedy=True)
        st, want, want_acc = oracle.spec_verify(g.target_f32(), oracle.params(**g.params), g.draft_ids,
                                                g.u_accept, g.u_resid, q_dense=g.q)
        got, acc, _ = gpu_verify(cuda, lily, scratch, g.target, g.params, g.draft_ids, g.u_accept,
                                 g.u_resid, q_dense=g.q, mode=lily.SPEC_GREEDY_MATCH)
        assert np.array_equal(got, want) and acc == want_acc
        assert np.array_equal(got, np.argmax(g.target_f32(), axis=1).astype(np.uint32))
    print("accepted-draft histogram over 40 sampled steps:", hist.tolist())
    scratch.close()


@pytest.mark.parametrize("table", [False, True])
def test_rows_of_a_step_share_the_penalty_state(cuda, lily, W, table):
    # src/qwen4exp/model.rs:3008-3012: row j's penalties see the draws of rows < j.
    vocab = 6007
    rng = np.random.default_rng(41)
    params = dict(temperature=0.9, top_k=8, top_p=1.0, presence_penalty=1.5, frequency_penalty=0.7,
                  repetition_penalty=1.3, seed=5)
    scratch = lily.SamplerScratch(vocab, max_rows=4, counts_table=True)
    for step in range(12):
        m = 4
        # Nearly identical rows so that an earlier draw matters to the next row.
        base = rng.uniform(-3, 3, vocab).astype(np.float32)
        trunk = np.tile(base, (m, 1)) + rng.uniform(-0.05, 0.05, (m, vocab)).astype(np.float32)
        head = trunk[:m - 1] + rng.uniform(-1, 1, (m - 1, vocab)).astype(np.float32)
        dp = dict(temperature=0.9, top_k=8, top_p=1.0, seed=5)
        q_ids, q_probs, q_n = sparse_q(head, dp, m - 1)
        draft_ids = np.array([oracle.sample(head[j], oracle.params(**dp), rng.random()).token
                              for j in range(m - 1)], dtype=np.uint32)
        ua = rng.random(m, dtype=np.float32)
        ur = rng.random(m - 1, dtype=np.float32)
        history = rng.integers(0, vocab, 200).astype(np.uint32)
        counts = oracle.counts_from_history(history, vocab)
        st, want, want_acc = oracle.spec_verify(trunk, oracle.params(**params), draft_ids, ua, ur,
                                                q_ids=q_ids, q_probs=q_probs, q_n=q_n,
                                                counts=counts.copy())
        assert st == 0
        if table:
            scratch.write_counts(counts, slot=2)
            got, acc, _ = gpu_verify(cuda, lily, scratch, trunk, params, draft_ids, ua, ur,
                                     q_sparse=(q_ids, q_probs, q_n), count_slot=2)
            after = scratch.read_counts(slot=2)
            expect = counts.copy()
            for t in want:
                expect[t] += 1
            assert np.array_equal(after, expect)
            # finish_speculation un-counts the rejected rows' draws
            # (src/qwen4exp/spec.rs:213-217).
            for t in want[want_acc + 1:]:
                scratch.uncount(int(t), slot=2)
                expect[t] -= 1
            assert np.array_equal(scratch.read_counts(slot=2), expect)
        else:
            got, acc, _ = gpu_verify(cuda, lily, scratch, trunk, params, draft_ids, ua, ur,
                                     q_sparse=(q_ids, q_probs, q_n), history=history)
        assert np.array_equal(got, want), f"step {step}: {got} vs {want}"
        assert acc == want_acc
    scratch.close()


def test_speculative_draw_is_distributed_as_the_trunk(cuda, lily, W):
    # tests/unit/kernels/sample.rs:414-487: chi-square < 82 (47 dof), every
    # frequency within 0.02, acceptance within 0.03 of sum(min(p, q)).
    rng = np.random.default_rng(25)
    v = 48
    head = rng.uniform(-2, 2, v).astype(np.float32)
    trunk = (head + rng.uniform(-1.5, 1.5, v)).astype(np.float32)
    params = dict(temperature=1.0, top_k=0, top_p=1.0, seed=31)
    pd = oracle.sample(trunk, oracle.params(**params), 0.0)
    qd = oracle.sample(head, oracle.params(**params), 0.0)
    q_of = dict(zip(qd.kept_ids.tolist(), qd.kept_prob.tolist()))
    overlap = sum(min(x, q_of.get(i, 0.0)) for i, x in zip(pd.kept_ids.tolist(), pd.kept_prob.tolist()))
    n = 2048
    scratch = lily.SamplerScratch(v, max_rows=8)
    q_ids, q_probs, q_n = sparse_q(np.tile(head, (7, 1)), params, 7)
    target = np.tile(trunk, (8, 1))
    hist = np.zeros(v)
    accepted = total = 0
    # Batches of 7 independent speculative rows (+ 1 plain row) per call.
    for it in range(n // 7):
        steps = np.arange(it * 8, it * 8 + 8)
        drafts = np.array([oracle.sample(head, oracle.params(**params),
                                         oracle.uniform_for(31, int(st) | 0x40000000)).token
                           for st in steps[:7]], dtype=np.uint32)
        got, _, _ = gpu_verify(cuda, lily, scratch, target, params, drafts, None, None,
                               q_sparse=(q_ids, q_probs, q_n), step0=int(steps[0]))
        for j in range(7):
            hist[got[j]] += 1
            accepted += got[j] == drafts[j]
            total += 1
    chi2 = 0.0
    for i, x in zip(pd.kept_ids.tolist(), pd.kept_prob.tolist()):
        chi2 += (hist[i] - x * total) ** 2 / (x * total)
        assert abs(hist[i] / total - x) < 0.03
    assert chi2 < 82.0, chi2
    assert abs(accepted / total - overlap) < 0.04
    scratch.close()
