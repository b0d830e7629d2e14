"""Helpers shared by the GPU parity tests: move a synthetic batch to the
device, run it through the C ABI, run the same rows through the CPU oracle."""
from __future__ import annotations

import numpy as np

import oracle

K_CAP = 1024
POISON = 0x5A5A5A5A


def t_u32(torch, a, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).to(device)


def t_f32(torch, a, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)


def t_logits(torch, batch, device="cuda"):
    if batch.bf16:
        return torch.from_numpy(np.ascontiguousarray(batch.logits).view(np.int16)).view(torch.bfloat16).to(device)
    return t_f32(torch, batch.logits, device)


def np_u32(t):
    return t.cpu().numpy().view(np.uint32)


def make_params(lily, batch):
    return [lily.SamplingParams(**p) for p in batch.params]


class Result:
    def __init__(self, ids, status, kept_n=None, kept_ids=None, kept_probs=None):
        self.ids, self.status = ids, status
        self.kept_n, self.kept_ids, self.kept_probs = kept_n, kept_ids, kept_probs


def run_batch(torch, lily, scratch, batch, want_kept=True, count_slots=None, use_steps=None,
              params_on_device=False):
    rows = batch.logits.shape[0]
    logits = t_logits(torch, batch)
    # Every output buffer sits between poisoned guard words (rows): the stand-in
    # for a memory checker, which this GPU pool does not offer.
    out = torch.full((rows + 2,), POISON, dtype=torch.int32, device="cuda")
    status_g = torch.full((rows + 2,), POISON, dtype=torch.int32, device="cuda")
    status = status_g[1:rows + 1]
    status.fill_(-1)
    kw = {}
    if batch.history is not None:
        kw["history_ids"] = t_u32(torch, batch.history)
        kw["history_len"] = t_u32(torch, batch.history_len)
    if batch.bias_ids is not None:
        kw["bias_ids"] = t_u32(torch, batch.bias_ids)
        kw["bias_vals"] = t_f32(torch, batch.bias_vals)
        kw["bias_len"] = t_u32(torch, batch.bias_len)
    if batch.ban_ids is not None:
        kw["ban_ids"] = t_u32(torch, batch.ban_ids)
        kw["ban_len"] = t_u32(torch, batch.ban_len)
    if batch.forced is not None:
        kw["forced_ids"] = torch.from_numpy(batch.forced).to("cuda")
    guards = [status_g]
    if want_kept:
        kept_n_g = torch.full((rows + 2,), POISON, dtype=torch.int32, device="cuda")
        kept_ids_g = torch.full((rows + 2, K_CAP), POISON, dtype=torch.int32, device="cuda")
        kept_probs_g = torch.full((rows + 2, K_CAP), POISON, dtype=torch.int32, device="cuda")
        for g in (kept_n_g, kept_ids_g, kept_probs_g):
            g[1:rows + 1].zero_()
        guards += [kept_n_g, kept_ids_g, kept_probs_g]
        kw["kept_n"] = kept_n_g[1:rows + 1]
        kw["kept_ids"] = kept_ids_g[1:rows + 1]
        kw["kept_probs"] = kept_probs_g[1:rows + 1].view(torch.float32)
    if count_slots is not None:
        kw["count_slots"] = count_slots
    params = make_params(lily, batch)
    if use_steps is not None:
        kw["steps"] = use_steps
    else:
        kw["uniforms"] = t_f32(torch, batch.uniforms)
    if params_on_device:
        raw = np.frombuffer(b"".join(bytes(p) for p in params), dtype=np.uint8).copy()
        params = torch.from_numpy(raw).to("cuda")
        if use_steps is not None:
            kw["steps"] = t_u32(torch, np.asarray(use_steps, dtype=np.uint32))
        kw["params_on_device"] = True
    scratch.sample_batch(logits, params, out[1:rows + 1], out_status=status, **kw)
    torch.cuda.synchronize()
    o = np_u32(out)
    assert o[0] == POISON and o[rows + 1] == POISON, "the kernel wrote outside out_ids"
    for g in guards:
        edge = np_u32(torch.stack([g[0].reshape(-1), g[rows + 1].reshape(-1)]))
        assert (edge == POISON).all(), "the kernel wrote outside an output buffer"
    res = Result(o[1:rows + 1].copy(), np_u32(status))
    if want_kept:
        res.kept_n = np_u32(kw["kept_n"])
        res.kept_ids = np_u32(kw["kept_ids"])
        res.kept_probs = kw["kept_probs"].cpu().numpy()
    return res


def oracle_rows(batch, counts=None, uniforms=None):
    """The oracle's draw for every row of the batch (None for forced rows)."""
    lf = batch.logits_f32()
    out = []
    for r in range(lf.shape[0]):
        if batch.forced is not None and batch.forced[r] >= 0:
            out.append(None)
            continue
        p = oracle.params(**batch.params[r])
        kw = {}
        if counts is not None:
            kw["counts"] = counts[r]
        elif batch.history is not None:
            kw["history"] = batch.history[r, :batch.history_len[r]]
        if batch.bias_ids is not None:
            n = batch.bias_len[r]
            kw["bias_ids"], kw["bias_vals"] = batch.bias_ids[r, :n], batch.bias_vals[r, :n]
        if batch.ban_ids is not None:
            kw["ban_ids"] = batch.ban_ids[r, :batch.ban_len[r]]
        u = float(batch.uniforms[r] if uniforms is None else uniforms[r])
        out.append(oracle.sample(lf[r], p, u, mode=1, **kw))
    return out


def assert_parity(batch, res, want, check_kept=True, label=""):
    """Token ids and kept ids bit-exact; kept probabilities within 1e-5
    absolute (they are in fact expected to be bit-equal)."""
    near = 0
    for r, d in enumerate(want):
        if d is None:
            assert res.ids[r] == np.uint32(batch.forced[r]), f"{label} row {r}: forced id"
            assert res.status[r] == 16
            continue
        if d.status != oracle.OK:
            assert res.status[r] == d.status, f"{label} row {r}: status {res.status[r]} vs oracle {d.status}"
            assert res.ids[r] == 0xFFFFFFFF
            continue
        near += d.near_tie != 0
        assert res.status[r] == 0, f"{label} row {r}: status {res.status[r]}"
        assert res.ids[r] == d.token, (
            f"{label} row {r}: token {res.ids[r]} vs oracle {d.token} (near_tie={d.near_tie})")
        if check_kept and res.kept_n is not None:
            n = len(d.kept_ids)
            assert res.kept_n[r] == n, f"{label} row {r}: kept {res.kept_n[r]} vs {n}"
            assert np.array_equal(res.kept_ids[r, :n], d.kept_ids), f"{label} row {r}: kept ids"
            err = np.abs(res.kept_probs[r, :n] - d.kept_prob).max()
            assert err <= 1e-5, f"{label} row {r}: kept probability error {err}"
    return near
