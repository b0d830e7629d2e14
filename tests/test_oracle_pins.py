"""Pins the CPU oracle to the reference's deterministic known-answer cases.

Each test replays a case of the reference's own tests (paths relative to the
reference project) with the inputs transcribed from it.
"""
import numpy as np
import pytest

import oracle


def py_uniform_for(seed, step):
    m = (1 << 64) - 1
    z = (seed + step * 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z ^= z >> 31
    return np.float32(z >> 40) * np.float32(1.0 / 16777216.0)


def test_uniform_for_matches_the_splitmix_definition():
    # src/kernels/sample.rs:435-441
    for seed in (0, 1, 99, 0xDEADBEEF, (1 << 64) - 1):
        for step in (0, 1, 3, 63, 0x40000004, 0x80000000):
            u = oracle.uniform_for(seed, step)
            assert u == py_uniform_for(seed, step)
            assert 0.0 <= u < 1.0


def test_draft_and_residual_domains():
    # src/kernels/sample.rs:220-222, src/kernels/metal/sample.metal:649
    L = oracle.lib()
    assert L.lo_draft_step(4) == 4 | 0x40000000
    assert L.lo_residual_step(4) == 4 | 0x80000000


def test_greedy_matches_argmax_with_lowest_id_on_ties():
    # tests/unit/kernels/sample.rs:74-83
    logits = np.zeros(5000, dtype=np.float32)
    logits[1234] = 7.5
    logits[4321] = 7.5
    for mode in (0, 1):
        d = oracle.sample(logits, oracle.params(), 0.5, mode=mode)
        assert d.status == oracle.OK and d.token == 1234
    assert oracle.argmax(logits) == 1234


def test_penalties_suppress_repeated_ids():
    # tests/unit/kernels/sample.rs:142-172: 5.0/1.5 - 0.5 - 0.5*3 = 1.33 < 4.0
    v = 3000
    logits = np.zeros(v, dtype=np.float32)
    logits[10], logits[20] = 5.0, 4.0
    counts = np.zeros(v, dtype=np.uint32)
    counts[10] = 3
    p = oracle.params(presence_penalty=0.5, frequency_penalty=0.5, repetition_penalty=1.5)
    d = oracle.sample(logits, p, 0.0, counts=counts, mode=0)
    assert d.token == 20
    st, adj = oracle.adjust(logits, p, counts=counts)
    assert st == oracle.OK
    assert abs(adj[10] - (5.0 / 1.5 - 0.5 - 1.5)) < 1e-5
    assert adj[20] == 4.0


def test_effective_params():
    # src/kernels/sample.rs:83-94
    import ctypes as C
    L = oracle.lib()
    t, k = C.c_float(), C.c_uint32()
    for p, want in [
        (oracle.params(), (1.0, 1)),
        (oracle.params(temperature=0.8, top_k=1), (1.0, 1)),
        (oracle.params(temperature=0.8, top_k=0), (np.float32(0.8), 1024)),
        (oracle.params(temperature=0.8, top_k=40), (np.float32(0.8), 40)),
        (oracle.params(temperature=0.8, top_k=5000), (np.float32(0.8), 1024)),
    ]:
        L.lo_effective(C.byref(p), C.byref(t), C.byref(k))
        assert (np.float32(t.value), k.value) == (np.float32(want[0]), want[1])


def test_validate():
    # src/kernels/sample.rs:57-79
    import ctypes as C
    L = oracle.lib()
    ok = oracle.params(temperature=0.7, top_k=20, top_p=0.95)
    assert L.lo_validate(C.byref(ok)) == oracle.OK
    for bad in (dict(temperature=-1.0), dict(temperature=float("nan")), dict(top_p=0.0),
                dict(top_p=1.5), dict(min_p=-0.1), dict(min_p=1.1), dict(repetition_penalty=0.0),
                dict(presence_penalty=float("inf")), dict(frequency_penalty=float("nan"))):
        p = oracle.params(**bad)
        assert L.lo_validate(C.byref(p)) == oracle.ERR_PARAMS, bad


def test_spec_accept_table():
    # tests/unit/kernels/spec.rs:19-25
    cases = [
        ([5, 6, 7, 8], [1, 5, 6, 7], 3),
        ([5, 6, 9, 8], [1, 5, 6, 7], 2),
        ([5, 0, 7, 8], [1, 5, 6, 7], 1),
        ([4, 6, 7, 8], [1, 5, 6, 7], 0),
        ([5], [1], 0),
    ]
    for draws, ids, want in cases:
        assert oracle.spec_accept(draws, ids) == want


def test_full_vocabulary_top_p_truncates_and_replays():
    # tests/unit/kernels/sample.rs:118-140 (own seeded inputs, same shape)
    rng = np.random.default_rng(11)
    v = 700
    logits = rng.uniform(-3, 3, v).astype(np.float32)
    p = oracle.params(temperature=1.0, top_k=0, top_p=0.5, seed=99)
    u = oracle.uniform_for(99, 3)
    a = oracle.sample(logits, p, u, mode=0)
    b = oracle.sample(logits, p, u, mode=0)
    assert a.token == b.token
    assert a.token in a.kept_ids
    assert len(a.kept_ids) < v


def test_selection_modes_agree():
    rng = np.random.default_rng(5)
    for v, k in ((6007, 40), (700, 0), (33, 20), (1, 5), (4099, 1000)):
        logits = rng.uniform(-8, 8, v).astype(np.float32)
        logits[rng.integers(0, v, 5)] = logits[0]  # some exact ties
        p = oracle.params(temperature=0.8, top_k=k, top_p=0.9, min_p=0.02)
        for step in range(8):
            u = oracle.uniform_for(7, step)
            a = oracle.sample(logits, p, u, mode=0)
            b = oracle.sample(logits, p, u, mode=1)
            assert a.token == b.token
            assert np.array_equal(a.kept_ids, b.kept_ids)
            assert np.array_equal(a.kept_cum, b.kept_cum)


def test_kept_probabilities_sum_to_one_and_top_p_is_over_the_top_k_mass():
    rng = np.random.default_rng(3)
    logits = rng.uniform(-8, 8, 6007).astype(np.float32)
    p = oracle.params(temperature=0.8, top_k=40, top_p=0.9, min_p=0.02)
    d = oracle.sample(logits, p, 0.25, mode=0)
    assert abs(float(d.kept_prob.sum()) - 1.0) < 1e-5
    # The kept set is a prefix of the 40 best by value.
    order = np.argsort(-logits, kind="stable")[:40]
    assert np.array_equal(d.kept_ids, order[:len(d.kept_ids)].astype(np.uint32))
    # The mass before the last kept candidate is below top_p * (mass of the 40).
    w = np.exp((logits[order] - logits[order[0]]) / np.float32(0.8)).astype(np.float64)
    assert w[:len(d.kept_ids) - 1].sum() < 0.9 * w.sum() + 1e-6


def test_spec_draw_statistics():
    # tests/unit/kernels/sample.rs:414-487 with own seeded inputs: the marginal
    # of the speculative draw is the trunk's distribution and the acceptance
    # rate is sum(min(p, q)).
    rng = np.random.default_rng(25)
    v = 48
    head = rng.uniform(-2, 2, v).astype(np.float32)
    trunk = (head + rng.uniform(-1.5, 1.5, v)).astype(np.float32)
    params = oracle.params(temperature=1.0, top_k=0, top_p=1.0, seed=31)
    pd = oracle.sample(trunk, params, 0.0, mode=0)
    qd = oracle.sample(head, params, 0.0, mode=0)
    q_of = dict(zip(qd.kept_ids.tolist(), qd.kept_prob.tolist()))
    overlap = sum(min(x, q_of.get(i, 0.0)) for i, x in zip(pd.kept_ids.tolist(), pd.kept_prob.tolist()))
    n = 8192
    hist = np.zeros(v)
    accepted = 0
    for step in range(n):
        ud = oracle.uniform_for(31, step | 0x40000000)
        d = oracle.sample(head, params, ud, mode=1).token
        out = oracle.spec_draw(pd, d, oracle.uniform_for(31, step),
                               oracle.uniform_for(31, step | 0x80000000),
                               q_ids=qd.kept_ids, q_probs=qd.kept_prob)
        hist[out] += 1
        accepted += out == d
    chi2 = 0.0
    for i, x in zip(pd.kept_ids.tolist(), pd.kept_prob.tolist()):
        chi2 += (hist[i] - x * n) ** 2 / (x * n)
        assert abs(hist[i] / n - x) < 0.02
    assert chi2 < 82.0
    assert abs(accepted / n - overlap) < 0.03


def test_exp_is_within_one_ulp_of_correct_rounding():
    xs = np.concatenate([np.linspace(-104, 0, 40001), np.linspace(0, 88.7, 5001),
                         [-np.inf, -200.0, -103.98, -87.4, -87.3, 0.0, 1e-8, -1e-8]]).astype(np.float32)
    got = oracle.expf(xs)
    want = np.exp(xs.astype(np.float64)).astype(np.float32)
    ulp = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
    assert ulp.max() <= 1
    assert oracle.expf([0.0])[0] == 1.0
    assert oracle.expf([-np.inf])[0] == 0.0


def test_nan_and_all_masked_rows_are_errors():
    logits = np.zeros(64, dtype=np.float32)
    logits[3] = np.nan
    p = oracle.params(temperature=1.0, top_k=8)
    assert oracle.sample(logits, p, 0.1).status == oracle.ERR_NAN
    logits[:] = 0
    d = oracle.sample(logits, p, 0.1, ban_ids=np.arange(64))
    assert d.status == oracle.ERR_NONFINITE


def test_bias_ban_order():
    # Extension semantics (no reference counterpart): bias, penalties, ban, /T.
    v = 100
    logits = np.zeros(v, dtype=np.float32)
    logits[5], logits[6], logits[7] = 3.0, 2.0, 2.5
    p = oracle.params(temperature=0.5, top_k=4, repetition_penalty=2.0)
    counts = np.zeros(v, dtype=np.uint32)
    counts[6] = 1
    st, adj = oracle.adjust(logits, p, counts=counts, bias_ids=[6, 6, 8], bias_vals=[1.0, 1.0, 5.0],
                            ban_ids=[5])
    assert st == oracle.OK
    assert adj[5] == -np.inf
    assert adj[6] == np.float32(((2.0 + 1.0 + 1.0) / 2.0) / 0.5)
    assert adj[8] == np.float32(5.0 / 0.5)
    assert adj[7] == np.float32(2.5 / 0.5)


def test_lmhead_matches_float64():
    rng = np.random.default_rng(1)
    import workloads as w
    cfg = w.config5(tokens=3, hidden=256, vocab=64, group=64, seed=9)
    got = oracle.lmhead_int8(cfg.hidden, cfg.weight, cfg.scales, 64, 0, 64)
    h = w.bf16_bits_to_f32(cfg.hidden).astype(np.float64)
    s = w.bf16_bits_to_f32(cfg.scales).astype(np.float64)
    wd = cfg.weight.astype(np.float64).reshape(64, 4, 64) * s[:, :, None]
    want = h @ wd.reshape(64, 256).T
    assert np.allclose(got, want, rtol=1e-5, atol=1e-4)


def test_dequant_affine_matches_the_reference_golden_bit_for_bit():
    # tests/unit/kernels/quant.rs:39-63 on tests/goldens/quant_fixture.json
    # (4- and 8-bit cases; re-emitted by tests/golden/make_quant_fixture.py).
    import json
    import os

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quant_fixture.json")
    with open(path) as f:
        cases = json.load(f)["cases"]
    assert {c["bits"] for c in cases} == {4, 8}
    for c in cases:
        f32 = lambda bits: np.array(bits, dtype=np.uint32).view(np.float32)
        got = oracle.dequant_affine(c["codes"], f32(c["scales_f32_bits"]), f32(c["biases_f32_bits"]),
                                    c["rows"], c["cols"], c["group_size"], c["bits"])
        want = np.array(c["expected_f32_bits"], dtype=np.uint32)
        assert np.array_equal(got.reshape(-1).view(np.uint32), want), c["name"]


def test_gemm_nt_sums_in_index_order():
    # tests/support/cpu_ref.rs:50-62: one fp32 accumulator, index order.
    a = np.array([[1e8, 1.0, -1e8, 1.0]], dtype=np.float32)
    b = np.ones((1, 4), dtype=np.float32)
    assert oracle.gemm_nt(a, b)[0, 0] == np.float32(1.0)  # (1e8 + 1) - 1e8 = 0, + 1
