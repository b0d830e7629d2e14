"""Writes tests/golden/metal_draws.json: what the reference's shipped Metal
sampler (src/kernels/metal/sample.metal, run on the CPU through
oracle/metal_ref.py) draws on seeded inputs of the shapes its own tests use
(tests/unit/kernels/sample.rs:85-116, 118-140, 142-172, 325-350, 352-409), and,
for every draw on which the CPU oracle answers differently, why.

    python tests/golden/make_metal_draws.py            (needs a reference checkout)

Inputs are not stored: a case names its numpy generator seed and carries a
SHA-256 of the logits it must regenerate. The reference's tests draw their
inputs from Rust's StdRng, which is not reproduced here; the shapes, value
ranges and parameters are theirs.

How a differing draw gets its cause. `variant()` below restates the kernel's
arithmetic in numpy with four switches, each naming one place where the kernel
and the reference's CPU sampler (tests/unit/kernels/sample.rs:8-54) differ:

    inv_t    `l *= 1/T` (sample.metal:123,137)        against `l / T` (sample.rs:28)
    exp      the C library's expf under the stand-in   against the oracle's own exp
    blocked  prefix sums per 32 lanes, then the         against one running sum
             groups' totals (sample.metal:158-174)
    c_minus  `(c - p) < top_p * total` on the           against the running sum before
             inclusive prefix (sample.metal:430-431)    the candidate (sample.rs:42-46)

With all four on it must reproduce the kernel's kept set and token on every
examined draw (asserted), with all four off the oracle's (asserted); a cause of a
difference is a switch that, turned off alone, moves the kernel's answer or,
turned on alone, moves the oracle's. Equal logits are their own cause: the kernel takes
boundary ties in thread order and its sort orders equal keys as the network
leaves them (sample.metal:292-296, 362-412), the CPU sampler by ascending id.
"""
import ctypes
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from oracle import metal_ref as M  # noqa: E402

F = np.float32
K_CAP = 1024
_libm = ctypes.CDLL("libm.so.6")
_libm.expf.restype = ctypes.c_float
_libm.expf.argtypes = [ctypes.c_float]


def libm_expf(x):
    return np.array([_libm.expf(float(v)) for v in x], dtype=F)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def make_logits(case):
    rng = np.random.default_rng(case.get("rng_seed", 0))
    kind = case["input"]
    v = case["vocab"]
    if kind == "uniform":
        x = rng.uniform(case["lo"], case["hi"], v).astype(F)
    elif kind == "bf16_normal":
        x = (rng.standard_normal(v) * case["scale"]).astype(F)
        x = ((x.view(np.uint32) + 0x8000) & 0xFFFF0000).astype(np.uint32).view(F)
    elif kind == "boundary_plateau":
        # Four equal values at ranks k-2 .. k+1: two of them fit under top-k.
        x = rng.uniform(case["lo"], case["hi"], v).astype(F)
        x[np.array(case["plateau_ids"])] = F(-100.0)
        order = np.argsort(-x, kind="stable")
        k = case["params"]["top_k"]
        x[np.array(case["plateau_ids"])] = F(0.5) * (x[order[k - 3]] + x[order[k - 2]])
    elif kind == "two_token_penalty":
        x = np.zeros(v, dtype=F)
        x[10], x[20] = 5.0, 4.0
    else:
        raise ValueError(kind)
    return x


def effective(P):
    greedy = P["temperature"] <= 0 or P["top_k"] == 1
    if greedy:
        return F(1.0), 1
    k = K_CAP if P["top_k"] == 0 else min(P["top_k"], K_CAP)
    return F(P["temperature"]), k


def variant(logits, P, u, inv_t, exp_libm, blocked, c_minus):
    """The draw without penalties, ties by ascending id, under the four switches."""
    t, k = effective(P)
    adj = logits * (F(1.0) / t) if inv_t else logits / t
    adj = adj.astype(F)
    k = min(k, adj.size)
    order = np.lexsort((np.arange(adj.size), -adj.astype(np.float64)))[:k]
    x = (adj[order] - adj[order[0]]).astype(F)
    p = libm_expf(x) if exp_libm else oracle.expf(x)
    if blocked:
        cum = np.zeros(k, dtype=F)
        before = F(0.0)
        for s in range(0, k, 32):
            local = np.cumsum(p[s:s + 32], dtype=F)
            cum[s:s + 32] = before + local
            # the group's total, the inclusive prefix of its 32nd lane; the lanes past k add zeros
            before = F(before + local[-1])
    else:
        cum = np.cumsum(p, dtype=F)
    total = cum[-1]
    bound = F(F(P.get("top_p", 1.0)) * total)
    min_p = F(P.get("min_p", 0.0))
    n_keep = 0
    for r in range(k):
        prev = F(cum[r] - p[r]) if c_minus else (F(0.0) if r == 0 else cum[r - 1])
        if r > 0 and not (prev < bound and p[r] >= min_p):
            break
        n_keep += 1
    target = F(F(u) * cum[n_keep - 1])
    pick = n_keep - 1
    for r in range(n_keep):
        if target < cum[r]:
            pick = r
            break
    return int(order[pick]), order[:n_keep].astype(np.uint32), adj


SWITCHES = ("inv_t", "exp", "blocked", "c_minus")


def explain(logits, P, u, shim_tok, shim_kept, orc):
    """Causes of a draw on which the kernel and the oracle differ."""
    adj = (logits * (F(1.0) / effective(P)[0])).astype(F)
    if (shim_kept.size == orc.kept_ids.size and np.array_equal(adj[shim_kept], adj[orc.kept_ids])
            and adj[shim_tok] == adj[orc.token]):
        return ["equal logits: thread order against ascending id"]
    tok_on, kept_on, _ = variant(logits, P, u, True, True, True, True)
    assert tok_on == shim_tok and np.array_equal(kept_on, shim_kept), "the restatement must reproduce the kernel"
    tok_off, kept_off, _ = variant(logits, P, u, False, False, False, False)
    assert tok_off == orc.token and np.array_equal(kept_off, orc.kept_ids), "and, switched off, the oracle"
    # A switch is a cause if turning it off alone moves the kernel's answer, or
    # turning it on alone moves the oracle's.
    causes = []
    for i, name in enumerate(SWITCHES):
        off = [True] * 4
        off[i] = False
        tok, kept, _ = variant(logits, P, u, *off)
        on = [False] * 4
        on[i] = True
        tok2, kept2, _ = variant(logits, P, u, *on)
        if (tok != shim_tok or not np.array_equal(kept, shim_kept)
                or tok2 != orc.token or not np.array_equal(kept2, orc.kept_ids)):
            causes.append(name)
    return causes or ["only jointly: no single switch moves either answer"]


def marginal_steps(orc, seed, search, take):
    """The steps of [0, search) whose target lies closest to an interval boundary."""
    steps = np.arange(search, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + steps * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z ^= z >> np.uint64(31)
    u = (z >> np.uint64(40)).astype(F) * F(1.0 / 16777216.0)
    inner = orc.kept_cum[:-1].astype(np.float64)  # the boundaries between two candidates
    target = (u * orc.kept_cum[-1]).astype(np.float64)
    at = np.clip(np.searchsorted(inner, target), 1, inner.size - 1)
    gap = np.minimum(np.abs(target - inner[at]), np.abs(target - inner[at - 1]))
    return [int(s) for s in np.argsort(gap, kind="stable")[:take]]


PLAIN_CASES = [
    dict(name="draws_match_the_cpu_reference", input="uniform", vocab=6007, lo=-8.0, hi=8.0, rng_seed=7,
         params=dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.02, seed=0xDEADBEEF), steps=64),
    dict(name="full_vocabulary_top_p", input="uniform", vocab=700, lo=-3.0, hi=3.0, rng_seed=11,
         params=dict(temperature=1.0, top_k=0, top_p=0.5, seed=99), steps=32),
    dict(name="wide_min_p", input="uniform", vocab=4099, lo=-6.0, hi=6.0, rng_seed=23,
         params=dict(temperature=1.3, top_k=0, top_p=1.0, min_p=0.001, seed=78), steps=32),
    dict(name="server_defaults_two_phase", input="uniform", vocab=32768, lo=-8.0, hi=8.0, rng_seed=31,
         params=dict(temperature=0.7, top_k=20, top_p=0.95, seed=5), steps=6),
    dict(name="reference_vocabulary", input="uniform", vocab=248320, lo=-10.0, hi=10.0, rng_seed=37,
         params=dict(temperature=0.6, top_k=100, top_p=0.95, seed=12), steps=4),
    dict(name="marginal_targets", input="uniform", vocab=6007, lo=-8.0, hi=8.0, rng_seed=7,
         params=dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.02, seed=0xDEADBEEF),
         marginal=dict(search=4_000_000, take=48)),
    dict(name="marginal_targets_wide", input="uniform", vocab=4099, lo=-1.0, hi=1.0, rng_seed=41,
         params=dict(temperature=1.1, top_k=200, top_p=0.97, seed=4),
         marginal=dict(search=4_000_000, take=48)),
    dict(name="bf16_logits_with_ties", input="bf16_normal", vocab=6007, scale=3.0, rng_seed=43,
         params=dict(temperature=1.0, top_k=50, top_p=0.98, seed=6), steps=64),
    dict(name="ties_at_the_top_k_boundary", input="boundary_plateau", vocab=6007, lo=-2.0, hi=2.0, rng_seed=47,
         plateau_ids=[5000, 1030, 2050, 300],
         params=dict(temperature=1.0, top_k=40, top_p=1.0, seed=8), steps=64),
]


def run_plain(case, explained):
    logits = make_logits(case)
    P = case["params"]
    full = dict(temperature=0.0, top_k=1, top_p=1.0, min_p=0.0, seed=0)
    full.update(P)
    counts = np.zeros(logits.size, dtype=np.uint32)
    op = oracle.params(**full)
    first = oracle.sample(logits, op, 0.0)
    steps = (marginal_steps(first, full["seed"], **case["marginal"]) if "marginal" in case
             else list(range(case["steps"])))
    tokens, kept0, probs0, two_phase, agree = [], None, None, False, 0
    for step in steps:
        dist = M.Dist()
        tok, two_phase = M.draw(logits, counts, step=step, mode=M.DRAFT, dist=dist, **full)
        ids, probs = dist.kept()
        u = oracle.uniform_for(full["seed"], step)
        assert u == M.uniform_for(full["seed"], step)
        orc = oracle.sample(logits, op, u)
        assert orc.status == oracle.OK
        tokens.append(tok)
        if kept0 is None:
            kept0, probs0 = ids, probs
        assert np.array_equal(ids, kept0), "the kept set does not depend on the step"
        same = tok == orc.token and np.array_equal(ids, orc.kept_ids)
        agree += tok == orc.token
        if not same:
            explained.append(dict(case=case["name"], step=step, kernel=tok, oracle=int(orc.token),
                                  kept_equal=bool(np.array_equal(ids, orc.kept_ids)),
                                  causes=explain(logits, full, u, tok, ids, orc)))
    out = {k: v for k, v in case.items() if k != "marginal"}
    out.update(logits_sha256=sha(logits), steps=steps, tokens=tokens, two_phase=bool(two_phase),
               kept_ids=[int(i) for i in kept0], kept_prob_bits=[int(b) for b in probs0.view(np.uint32)],
               agree=int(agree))
    print(case["name"], f"{agree}/{len(steps)} equal the oracle; kept {kept0.size}; two-phase {two_phase}", flush=True)
    return out


def run_penalties():
    """tests/unit/kernels/sample.rs:142-172, then a run whose histogram grows with the draws."""
    v = 3000
    logits = make_logits(dict(input="two_token_penalty", vocab=v))
    counts = np.zeros(v, dtype=np.uint32)
    counts[10] = 3
    P = dict(temperature=0.0, top_k=1, presence_penalty=0.5, frequency_penalty=0.5, repetition_penalty=1.5)
    tok, _, adjusted = M.draw(logits, counts, step=0, want_adjusted=True, **P)
    known = dict(token=tok, counts_20=int(counts[20]), counts_10=int(counts[10]),
                 adjusted_10_bits=int(adjusted[10:11].view(np.uint32)[0]),
                 adjusted_20_bits=int(adjusted[20:21].view(np.uint32)[0]))
    case = dict(name="histogram_grows_with_the_draws", input="uniform", vocab=700, lo=-4.0, hi=4.0, rng_seed=53,
                params=dict(temperature=0.9, top_k=0, top_p=0.9, presence_penalty=0.1, frequency_penalty=0.05,
                            repetition_penalty=1.05, seed=9), steps=96)
    logits = make_logits(case)
    counts = np.zeros(logits.size, dtype=np.uint32)
    tokens = [M.draw(logits, counts, step=s, **case["params"])[0] for s in range(case["steps"])]
    case.update(logits_sha256=sha(logits), tokens=tokens, counts_sha256=sha(counts))
    print("penalties", known, "distinct tokens", len(set(tokens)), "largest count", int(counts.max()), flush=True)
    return dict(known_answer=known, run=case)


SPEC_CASES = [
    dict(name="server defaults", params=dict(temperature=1.0, top_k=20, top_p=0.95, seed=77)),
    dict(name="wide", params=dict(temperature=1.3, top_k=0, top_p=1.0, min_p=0.001, seed=78)),
]


def spec_inputs():
    rng = np.random.default_rng(23)
    head = rng.uniform(-6.0, 6.0, 4099).astype(F)
    trunk = (head + rng.uniform(-2.5, 2.5, 4099).astype(F)).astype(F)
    return head, trunk


def run_spec(explained):
    """tests/unit/kernels/sample.rs:352-409: the draft head's draw on its own
    index (src/kernels/sample.rs:216-218), then the trunk's speculative draw."""
    head, trunk = spec_inputs()
    out = dict(vocab=4099, rng_seed=23, head_sha256=sha(head), trunk_sha256=sha(trunk), sets=[])
    for case in SPEC_CASES:
        P = dict(temperature=0.0, top_k=1, top_p=1.0, min_p=0.0, seed=0)
        P.update(case["params"])
        op = oracle.params(**P)
        counts = np.zeros(head.size, dtype=np.uint32)
        drafted, got, agree, accepted = [], [], 0, 0
        for step in range(96):
            dist = M.Dist()
            d, _ = M.draw(head, counts, step=step | 0x40000000, mode=M.DRAFT, dist=dist, **P)
            t, _ = M.draw(trunk, counts, step=step, mode=M.SPEC, dist=dist, draft=d, **P)
            q_ids, q_probs = dist.kept()
            # the oracle's side: its own draft distribution, the kernel's proposal
            oq = oracle.sample(head, op, oracle.uniform_for(P["seed"], step | 0x40000000))
            op_ = oracle.sample(trunk, op, oracle.uniform_for(P["seed"], step))
            want = oracle.spec_draw(op_, d, oracle.uniform_for(P["seed"], step),
                                    oracle.uniform_for(P["seed"], step | 0x80000000),
                                    q_ids=oq.kept_ids, q_probs=oq.kept_prob)
            drafted.append(d)
            got.append(t)
            agree += t == want
            accepted += t == d
            if t != want or d != oq.token:
                explained.append(dict(case="speculative: " + case["name"], step=step, kernel=t, oracle=int(want),
                                      kept_equal=bool(np.array_equal(q_ids, oq.kept_ids)),
                                      causes=["speculative draw: see the case's note"]))
        out["sets"].append(dict(name=case["name"], params=case["params"], steps=96, drafted=drafted, tokens=got,
                                agree=int(agree), accepted=int(accepted)))
        print("speculative", case["name"], f"{agree}/96 equal the oracle, {accepted}/96 accepted", flush=True)
    return out


def main():
    assert M.available(), "needs a reference checkout (LILY_REFERENCE) to build the kernel's CPU library"
    explained = []
    doc = dict(
        source="src/kernels/metal/sample.metal through oracle/metal_shim (CPU); inputs seeded numpy",
        plain=[run_plain(c, explained) for c in PLAIN_CASES],
        penalties=run_penalties(),
        speculative=run_spec(explained),
        explained=explained,
    )
    path = os.path.join(HERE, "metal_draws.json")
    with open(path, "w") as f:
        json.dump(doc, f, separators=(",", ":"))
    print(path, os.path.getsize(path), "bytes;", len(explained), "differing draws explained")


if __name__ == "__main__":
    main()
