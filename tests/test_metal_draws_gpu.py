"""The CUDA sampler against what the reference's shipped Metal kernel draws.

tests/golden/metal_draws.json holds the tokens and kept sets of
src/kernels/metal/sample.metal (run on the CPU by tests/golden/
make_metal_draws.py) on seeded inputs, and the list of draws on which the
reference's kernel and its CPU sampler (tests/unit/kernels/sample.rs:8-54, the
rule this library follows) differ, each with its cause. One launch per case, a
row per recorded step: every row has to give the kernel's token and kept set,
and on a listed draw the CPU sampler's answer recorded there.
"""
import importlib.util
import json
import os

import numpy as np
import pytest

from gpu_util import np_u32

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_metal_draws", os.path.join(HERE, "golden", "make_metal_draws.py"))
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)
TIES = "equal logits: thread order against ascending id"
K_CAP = 1024


@pytest.fixture(scope="module")
def doc():
    with open(os.path.join(HERE, "golden", "metal_draws.json")) as f:
        return json.load(f)


def draw_rows(torch, lily, logits, P, steps, counts_table=False):
    rows = len(steps)
    scratch = lily.SamplerScratch(logits.size, max_rows=rows, counts_table=counts_table)
    x = torch.from_numpy(np.ascontiguousarray(np.broadcast_to(logits, (rows, logits.size)))).cuda()
    params = [lily.SamplingParams(**P) for _ in range(rows)]
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    status = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    kept_n = torch.zeros(rows, dtype=torch.int32, device="cuda")
    kept_ids = torch.zeros((rows, K_CAP), dtype=torch.int32, device="cuda")
    kept_probs = torch.zeros((rows, K_CAP), dtype=torch.float32, device="cuda")
    scratch.sample_batch(x, params, out, steps=list(steps), out_status=status, kept_n=kept_n, kept_ids=kept_ids,
                         kept_probs=kept_probs)
    torch.cuda.synchronize()
    assert scratch.status() == lily.OK and not np_u32(status).any()
    scratch.close()
    n = np_u32(kept_n)
    return np_u32(out), [np_u32(kept_ids[r])[:n[r]] for r in range(rows)], kept_probs.cpu().numpy()


@pytest.mark.parametrize("index", range(len(gen.PLAIN_CASES)))
def test_plain_draws(cuda, lily, doc, index):
    case = doc["plain"][index]
    logits = gen.make_logits(case)
    P = dict(temperature=0.0, top_k=1, top_p=1.0, min_p=0.0, seed=0)
    P.update(case["params"])
    listed = {e["step"]: e for e in doc["explained"] if e["case"] == case["name"]}
    tokens, kept, probs = draw_rows(cuda, lily, logits, P, case["steps"])
    kernel_kept = np.array(case["kept_ids"], dtype=np.uint32)
    kernel_probs = np.array(case["kept_prob_bits"], dtype=np.uint32).view(np.float32)
    tied = any(e["causes"] == [TIES] for e in listed.values())
    for r, (step, token) in enumerate(zip(case["steps"], case["tokens"])):
        want = listed[step]["oracle"] if step in listed else token
        assert tokens[r] == want, f"{case['name']} step {step}"
        if not tied:
            assert np.array_equal(kept[r], kernel_kept), f"{case['name']} step {step}: kept set"
            assert np.max(np.abs(probs[r][:kernel_kept.size] - kernel_probs)) < 1e-5
        else:
            assert np.array_equal(logits[kept[r]], logits[kernel_kept]), "the same logits, tied ids in another order"


def test_a_histogram_that_grows_with_the_draws(cuda, lily, doc):
    """One row, 96 launches: the library's histogram slot against the kernel's
    own `counts[chosen] += 1` (sample.metal:509-511)."""
    torch = cuda
    run = doc["penalties"]["run"]
    logits = gen.make_logits(run)
    P = dict(temperature=0.0, top_k=1, top_p=1.0, min_p=0.0, seed=0)
    P.update(run["params"])
    scratch = lily.SamplerScratch(logits.size, max_rows=1, counts_table=True)
    x = torch.from_numpy(logits[None, :].copy()).cuda()
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = []
    for step in range(len(run["tokens"])):
        scratch.sample_batch(x, [lily.SamplingParams(**P)], out, steps=[step], count_slots=[0])
        got.append(int(np_u32(out)[0]))
    assert got == run["tokens"]
    counts = scratch.read_counts(0)
    assert gen.sha(counts.astype(np.uint32)) == run["counts_sha256"]
    assert scratch.status() == lily.OK
    scratch.close()
