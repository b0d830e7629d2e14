"""The allocation-free draw (lily_sample_batch_noalloc) against the regular
one. Hosts that may not call cudaMalloc after start-up (a fixed memory plan, a
plugin in a process that forbids it, a capture in progress elsewhere) use the
entry point whose scratch is static device storage; it has to give the same
tokens, kept sets and statuses as lily_sample_batch, call after call, although
every call reuses the same array. Collected last on purpose."""
import numpy as np
import pytest

from gpu_util import K_CAP, Result, assert_parity, make_params, np_u32, oracle_rows, run_batch, t_f32, t_logits, t_u32

pytestmark = pytest.mark.gpu


def run_noalloc(torch, lily, vocab, batch):
    rows = batch.logits.shape[0]
    out = torch.full((rows + 2,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    status = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    kept_n = torch.zeros(rows, dtype=torch.int32, device="cuda")
    kept_ids = torch.zeros((rows, K_CAP), dtype=torch.int32, device="cuda")
    kept_probs = torch.zeros((rows, K_CAP), dtype=torch.float32, device="cuda")
    kw = {}
    if batch.history is not None:
        kw["history_ids"], kw["history_len"] = t_u32(torch, batch.history), t_u32(torch, batch.history_len)
    if batch.bias_ids is not None:
        kw["bias_ids"], kw["bias_vals"] = t_u32(torch, batch.bias_ids), t_f32(torch, batch.bias_vals)
        kw["bias_len"] = t_u32(torch, batch.bias_len)
    if batch.ban_ids is not None:
        kw["ban_ids"], kw["ban_len"] = t_u32(torch, batch.ban_ids), t_u32(torch, batch.ban_len)
    if batch.forced is not None:
        kw["forced_ids"] = torch.from_numpy(batch.forced).to("cuda")
    lily.sample_batch_noalloc(vocab, t_logits(torch, batch), make_params(lily, batch), out[1:rows + 1],
                              uniforms=t_f32(torch, batch.uniforms), out_status=status,
                              kept_n=kept_n, kept_ids=kept_ids, kept_probs=kept_probs, **kw)
    torch.cuda.synchronize()
    o = np_u32(out)
    assert o[0] == 0x5A5A5A5A and o[rows + 1] == 0x5A5A5A5A
    return o[1:rows + 1].copy(), np_u32(status), np_u32(kept_n), np_u32(kept_ids), kept_probs.cpu().numpy()


def test_the_allocation_free_draw_equals_the_regular_one_call_after_call(cuda, lily):
    import workloads as w

    vocab = 151_936
    scratch = lily.SamplerScratch(vocab, max_rows=8, max_list=64)
    for call in range(2):
        # Two different batches in a row over the one static array: mixed
        # params, histories, bias, bans, a forced row; several slices per row.
        batch = w.config2_step(call, vocab=vocab, rows=4 + 4 * call, history=2048)
        for p in batch.params:
            p["frequency_penalty"] = 0.0  # needs a count table the static scratch has no room for
        want = run_batch(cuda, lily, scratch, batch)
        ids, status, kept_n, kept_ids, kept_probs = run_noalloc(cuda, lily, vocab, batch)
        assert np.array_equal(ids, want.ids), f"call {call}"
        assert np.array_equal(status, want.status)
        assert np.array_equal(kept_n, want.kept_n)
        for r in range(len(ids)):
            n = kept_n[r]
            assert np.array_equal(kept_ids[r, :n], want.kept_ids[r, :n])
            assert np.abs(kept_probs[r, :n] - want.kept_probs[r, :n]).max(initial=0.0) <= 1e-5
        # And against the CPU oracle directly, not only against the other CUDA path.
        assert_parity(batch, Result(ids, status, kept_n, kept_ids, kept_probs), oracle_rows(batch),
                      label=f"allocation-free call {call}")
    scratch.close()


def test_the_allocation_free_draw_refuses_what_it_has_no_room_for(cuda, lily):
    import workloads as w

    vocab = 32_768
    batch = w.config2_step(0, vocab=vocab, rows=4, history=256)  # frequency penalty 0.2 + history
    with pytest.raises(lily.LilyError) as e:
        run_noalloc(cuda, lily, vocab, batch)
    assert e.value.code == lily.ERR_CAPACITY and "count table" in str(e.value)
    big = w.config2_step(0, vocab=vocab, rows=lily.NOALLOC_MAX_ROWS + 1, history=16)
    for p in big.params:
        p["frequency_penalty"] = 0.0
    with pytest.raises(lily.LilyError) as e:
        run_noalloc(cuda, lily, vocab, big)
    assert e.value.code == lily.ERR_CAPACITY
