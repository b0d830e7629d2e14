"""The CPU oracle held to the reference's shipped Metal sampler.

tests/golden/metal_draws.json records what src/kernels/metal/sample.metal
draws (run on the CPU through oracle/metal_shim) on seeded inputs of the shapes
the reference's own tests use, and lists every draw on which the oracle
answers differently, with its cause. These tests regenerate the inputs and
require of the oracle:

* the reference's own bars between its kernel and its CPU sampler: at least
  62 of 64 plain draws and 93 of 96 speculative draws equal
  (tests/unit/kernels/sample.rs:113-115, 402-403), every draw inside the kept
  set, exported probabilities within 1e-5 (:343-347);
* and, beyond them, that every draw equals the kernel's unless the fixture
  lists it, in which case the oracle gives exactly the listed answer and the
  listed cause can be checked (equal logits for the tie cases, the kept sets
  equal for the rounding cases).

Where a reference checkout is at hand the fixture is also checked against a
fresh build of the kernel's CPU library.
"""
import hashlib
import importlib.util
import json
import os

import numpy as np
import pytest

import oracle
from oracle import metal_ref

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURE = os.path.join(HERE, "golden", "metal_draws.json")
TIES = "equal logits: thread order against ascending id"

_spec = importlib.util.spec_from_file_location("make_metal_draws", os.path.join(HERE, "golden", "make_metal_draws.py"))
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)


@pytest.fixture(scope="module")
def doc():
    with open(FIXTURE) as f:
        return json.load(f)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def full_params(p):
    out = dict(temperature=0.0, top_k=1, top_p=1.0, min_p=0.0, seed=0)
    out.update(p)
    return out


def explained_for(doc, name):
    return {e["step"]: e for e in doc["explained"] if e["case"] == name}


def test_the_uniform_is_the_shaders(doc):
    """sample_uniform (sample.metal:93-101) against the oracle's, on the recorded steps."""
    if not metal_ref.available():
        pytest.skip("no reference checkout: the kernel's CPU library is not built")
    rng = np.random.default_rng(3)
    for seed in [0, 1, 0xDEADBEEF, 2**64 - 1] + [int(s) for s in rng.integers(0, 2**63, 28)]:
        for step in [0, 1, 63, 0x40000000, 0x80000005, 0xFFFFFFFF] + [int(s) for s in rng.integers(0, 2**32, 26)]:
            assert metal_ref.uniform_for(seed, step) == oracle.uniform_for(seed, step)


@pytest.mark.parametrize("index", range(len(gen.PLAIN_CASES)))
def test_plain_draws(doc, index):
    case = doc["plain"][index]
    assert case["name"] == gen.PLAIN_CASES[index]["name"]
    logits = gen.make_logits(case)
    assert sha(logits) == case["logits_sha256"], "the inputs must regenerate bit for bit"
    P = full_params(case["params"])
    op = oracle.params(**P)
    listed = explained_for(doc, case["name"])
    adj = oracle.adjust(logits, op)[1]
    kept_kernel = np.array(case["kept_ids"], dtype=np.uint32)
    probs_kernel = np.array(case["kept_prob_bits"], dtype=np.uint32).view(np.float32)
    agree = 0
    for step, token in zip(case["steps"], case["tokens"]):
        d = oracle.sample(logits, op, oracle.uniform_for(P["seed"], step))
        assert d.status == oracle.OK
        same = d.token == token and np.array_equal(d.kept_ids, kept_kernel)
        agree += d.token == token
        # the reference's first bar: the kernel's token lies in the CPU sampler's kept set,
        # or shares its logit with a member of it (a tie the two order differently)
        assert token in d.kept_ids or adj[token] in adj[d.kept_ids], f"step {step}"
        if step in listed:
            e = listed[step]
            assert not same and e["kernel"] == token and e["oracle"] == d.token
            assert e["kept_equal"] == bool(np.array_equal(d.kept_ids, kept_kernel))
            if e["causes"] == [TIES]:
                assert np.array_equal(adj[d.kept_ids], adj[kept_kernel]) and adj[token] == adj[d.token]
            else:
                assert e["kept_equal"] and set(e["causes"]) <= set(gen.SWITCHES)
        else:
            assert same, f"{case['name']} step {step}: kernel {token}, oracle {d.token}, and no listed cause"
    assert agree == case["agree"]
    if "marginal" not in gen.PLAIN_CASES[index] and not any(e["causes"] == [TIES] for e in listed.values()):
        assert agree >= len(case["steps"]) - 2, "the reference's bar between its kernel and its CPU sampler"
    # exported probabilities: the reference's tolerance, and how many are equal to the bit
    if d.kept_ids.size == kept_kernel.size:
        order = np.argsort(d.kept_ids, kind="stable"), np.argsort(kept_kernel, kind="stable")
        if np.array_equal(d.kept_ids[order[0]], kept_kernel[order[1]]):
            assert np.max(np.abs(d.kept_prob[order[0]] - probs_kernel[order[1]])) < 1e-5


def test_the_reference_shaped_cases_have_no_listed_difference(doc):
    """On the inputs shaped like the reference's own tests the oracle equals the
    kernel on every draw and every kept set: nothing to explain there."""
    quiet = {"draws_match_the_cpu_reference", "full_vocabulary_top_p", "wide_min_p", "server_defaults_two_phase"}
    assert not [e for e in doc["explained"] if e["case"] in quiet or e["case"].startswith("speculative")]
    assert {c["name"]: c["agree"] for c in doc["plain"] if c["name"] in quiet} == {
        "draws_match_the_cpu_reference": 64, "full_vocabulary_top_p": 32, "wide_min_p": 32,
        "server_defaults_two_phase": 6}
    assert next(c for c in doc["plain"] if c["name"] == "server_defaults_two_phase")["two_phase"]


def test_penalties_known_answer_and_growing_histogram(doc):
    """tests/unit/kernels/sample.rs:142-172 on the kernel and on the oracle, then
    96 draws whose histogram the kernel bumps itself (sample.metal:509-511)."""
    known = doc["penalties"]["known_answer"]
    assert (known["token"], known["counts_20"], known["counts_10"]) == (20, 1, 3)
    logits = gen.make_logits(dict(input="two_token_penalty", vocab=3000))
    counts = np.zeros(3000, dtype=np.uint32)
    counts[10] = 3
    p = oracle.params(presence_penalty=0.5, frequency_penalty=0.5, repetition_penalty=1.5)
    adj = oracle.adjust(logits, p, counts=counts)[1]
    assert int(adj[10:11].view(np.uint32)[0]) == known["adjusted_10_bits"]
    assert int(adj[20:21].view(np.uint32)[0]) == known["adjusted_20_bits"]
    assert oracle.sample(logits, p, 0.0, counts=counts).token == 20

    run = doc["penalties"]["run"]
    logits = gen.make_logits(run)
    assert sha(logits) == run["logits_sha256"]
    P = full_params(run["params"])
    op = oracle.params(**P)
    counts = np.zeros(logits.size, dtype=np.uint32)
    for step, token in enumerate(run["tokens"]):
        d = oracle.sample(logits, op, oracle.uniform_for(P["seed"], step), counts=counts)
        assert d.token == token, f"step {step}"
        counts[d.token] += 1
    assert sha(counts) == run["counts_sha256"]
    assert counts.max() >= 3 and int(counts.sum()) == len(run["tokens"]), "ids must repeat for the frequency term to count"


def test_speculative_draws(doc):
    """tests/unit/kernels/sample.rs:352-409: at least 93 of 96 equal, both outcomes occur."""
    spec = doc["speculative"]
    head, trunk = gen.spec_inputs()
    assert sha(head) == spec["head_sha256"] and sha(trunk) == spec["trunk_sha256"]
    for s in spec["sets"]:
        P = full_params(s["params"])
        op = oracle.params(**P)
        agree = accepted = 0
        for step, (d, token) in enumerate(zip(s["drafted"], s["tokens"])):
            oq = oracle.sample(head, op, oracle.uniform_for(P["seed"], step | 0x40000000))
            assert oq.token == d, "the draft head's own draw"
            ot = oracle.sample(trunk, op, oracle.uniform_for(P["seed"], step))
            want = oracle.spec_draw(ot, d, oracle.uniform_for(P["seed"], step),
                                    oracle.uniform_for(P["seed"], step | 0x80000000),
                                    q_ids=oq.kept_ids, q_probs=oq.kept_prob)
            assert token in ot.kept_ids, "inside p's support"
            agree += want == token
            accepted += token == d
        assert agree >= 93 and agree == s["agree"] == 96, s["name"]
        assert 0 < accepted < 96 and accepted == s["accepted"]


def test_the_fixture_is_what_the_kernel_draws_now(doc):
    """A fresh build of the kernel's CPU library redraws part of the fixture."""
    if not metal_ref.available():
        pytest.skip("no reference checkout: the kernel's CPU library is not built")
    for index in (0, 5, 7):
        case = doc["plain"][index]
        logits = gen.make_logits(case)
        P = full_params(case["params"])
        counts = np.zeros(logits.size, dtype=np.uint32)
        for step, token in list(zip(case["steps"], case["tokens"]))[:24]:
            dist = metal_ref.Dist()
            got, two_phase = metal_ref.draw(logits, counts, step=step, mode=metal_ref.DRAFT, dist=dist, **P)
            assert got == token and two_phase == case["two_phase"]
            assert dist.kept()[0].tolist() == case["kept_ids"]
        assert not counts.any(), "without penalties the histogram stays untouched"
    # the argmax route is another shader: refused, not emulated
    with pytest.raises(RuntimeError):
        metal_ref.draw(np.zeros(64, dtype=np.float32), np.zeros(64, dtype=np.uint32), temperature=0.0, top_k=1)
