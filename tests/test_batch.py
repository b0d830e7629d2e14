"""The bookkeeping around the sampler for rows of a batch, against the
reference's own cases (tests/unit/serve/batch.rs:5-135 slots, admission, the
next action, sharing statistics, parking the next step; src/serve/batch.rs
191-226 SoloStop; 421-438 the draw index). Host logic: no GPU, except the last
test, where a request's penalty counts follow it between the engine's sampler
and a batch slot (src/serve/batch.rs:762-829, 1117-1121)."""
import numpy as np
import pytest

import oracle


@pytest.fixture(scope="module")
def bt(lily):
    import lily_b200.batch as batch

    return batch


def test_slots_hand_out_the_lowest_free_one_and_take_them_back(lily, bt):
    slots = bt.Slots(3)
    assert (slots.take(), slots.take()) == (0, 1)
    slots.give(0)
    assert slots.in_use() == 1
    assert (slots.take(), slots.take()) == (0, 2)
    assert slots.take() is None
    assert slots.in_use() == 3 and len(slots) == 3
    slots.give(7)  # out of range: ignored, the table does not grow
    assert slots.in_use() == 3 and len(slots) == 3
    slots.give(1)
    with pytest.raises(lily.LilyError):
        slots.give(1)  # given back twice
    assert slots.in_use() == 2
    assert bt.Slots(0).take() is None


def test_admission(bt):
    assert bt.admits(0, 2, 0, 50, 10)  # alone, whatever its size
    assert bt.admits(1, 2, 4, 6, 10)
    assert not bt.admits(1, 2, 4, 7, 10)
    assert not bt.admits(2, 2, 0, 0, 10)
    assert bt.admits(2, 3, 3, 3, 10)
    big = 2 ** 64 - 1
    assert not bt.admits(1, 2, big, 1, big - 1)  # saturates, no overflow


def test_next_action(bt):
    assert bt.next_action(0, False) == (bt.DONE, None)
    assert bt.next_action(1, False) == (bt.SOLO, True)
    assert bt.next_action(1, True) == (bt.SOLO, False)
    assert bt.next_action(2, False) == (bt.STEP, None)
    assert bt.next_action(4, True) == (bt.STEP, None)


def test_sharing_statistics(lily, bt):
    stats = bt.BatchStats()
    assert stats.mean_rows() is None
    stats.record_step(1, [1, 2])
    stats.record_step(1, [1, 2, 3])
    stats.record_step(1, [2, 1])
    assert (stats.batched_tokens, stats.rows_sum, stats.max_rows) == (3, 7, 3)
    assert stats.peers == [2, 3]
    assert stats.mean_rows() == 7.0 / 3.0
    small = bt.BatchStats(max_peers=1)
    with pytest.raises(lily.LilyError):
        small.record_step(1, [1, 2, 3])
    assert small.peers == [2] and small.rows_sum == 3


def test_park_next(bt):
    on = lambda pos, **kw: bt.RowAhead(pos=pos, **kw)
    rows = [on(100), on(4000)]
    assert bt.park_next(rows, True, False, False)
    assert bt.park_next(rows[:1], True, False, False)
    assert not bt.park_next(rows, False, False, False)  # step budget spent
    assert not bt.park_next(rows, True, True, False)    # admission next
    assert not bt.park_next(rows, True, False, True)    # cancelled
    assert not bt.park_next([on(100), on(512, checkpoint_due=True)], True, False, False)
    assert not bt.park_next([on(100, ending=True), on(200)], True, False, False)
    assert not bt.park_next([on(100), on(300, may_insert=True)], True, False, False)
    at = lambda pos: on(pos, capacity=1024)
    assert bt.park_next([at(1022)], True, False, False)
    assert not bt.park_next([at(1023)], True, False, False)
    assert not bt.park_next([at(1024)], True, False, False)
    assert not bt.park_next([on(10), at(1023)], True, False, False)
    assert bt.park_next([], True, False, False)  # `all` over no rows


def test_solo_stop(bt):
    s = bt.SoloStop()
    assert s.observe(False, False) and not s.yielded_only()
    assert not s.observe(False, True) and s.yielded_only()
    # A terminal reason later in an inserted group wins over the yield.
    assert not s.observe(True, True) and not s.yielded_only()
    t = bt.SoloStop()
    assert not t.observe(True, False) and not t.yielded_only()


def test_draw_step(bt):
    # The step that feeds a row's last draw draws number generated.len(); the
    # one parked behind it the number after that.
    assert bt.draw_step(5) == 5 and bt.draw_step(5, 1) == 6
    assert oracle.uniform_for(9, bt.draw_step(5, 1)) == oracle.uniform_for(9, 6)


@pytest.mark.gpu
def test_counts_follow_a_request_between_engine_and_batch_slot(cuda, lily, bt):
    torch = cuda
    import workloads as W
    from gpu_util import run_batch

    v = 4096
    rng = np.random.default_rng(5)
    engine = lily.SamplerScratch(v, max_rows=1, counts_table=True)
    batch = lily.SamplerScratch(v, max_rows=3, counts_table=True)
    slots = bt.Slots(3)
    p = dict(temperature=0.8, top_k=50, presence_penalty=0.4, frequency_penalty=0.3,
             repetition_penalty=1.2, seed=3)
    x = rng.normal(0, 3, size=(1, v)).astype(np.float32)
    generated = []
    counts = np.zeros(v, dtype=np.uint32)  # the oracle's view of the request

    def draw(handle, slot, step):
        u = np.array([oracle.uniform_for(p["seed"], step)], dtype=np.float32)
        res = run_batch(torch, lily, handle, W.Batch(x, False, [p], u), count_slots=[slot])
        want = oracle.sample(x[0], oracle.params(**p), float(u[0]), counts=counts.copy())
        assert res.ids[0] == want.token
        counts[want.token] += 1
        generated.append(int(res.ids[0]))

    # Prefill draw and two single-session steps on the engine's sampler.
    for _ in range(3):
        draw(engine, 0, bt.draw_step(len(generated)))
    # Another request holds slot 0; this one enters the batch in slot 1.
    assert slots.take() == 0
    slot = slots.take()
    assert slot == 1
    batch.write_counts(np.full(v, 7, dtype=np.uint32), slot=slot)  # a previous owner's leftovers
    bt.move_sampler_counts(engine, batch, bt.ENGINE, slot)
    assert np.array_equal(batch.read_counts(slot), counts)
    for _ in range(3):
        draw(batch, slot, bt.draw_step(len(generated)))
    # The engine's copy went stale meanwhile; leaving the batch brings the counts back.
    assert not np.array_equal(engine.read_counts(), counts)
    bt.move_sampler_counts(engine, batch, slot, bt.ENGINE)
    slots.give(slot)
    assert np.array_equal(engine.read_counts(), counts)
    draw(engine, 0, bt.draw_step(len(generated)))
    # Same place: nothing moves. A slot the batch does not have is refused.
    bt.move_sampler_counts(engine, batch, bt.ENGINE, bt.ENGINE)
    bt.move_sampler_counts(engine, batch, 2, 2)
    with pytest.raises(lily.LilyError) as e:
        bt.move_sampler_counts(engine, batch, bt.ENGINE, 3)
    assert e.value.code == lily.ERR_ARG and "batch slot 3 of 3" in str(e.value)
    # Batch slot to batch slot (a row that changes slots).
    bt.move_sampler_counts(engine, batch, 1, 2)
    assert np.array_equal(batch.read_counts(2), batch.read_counts(1))
    assert len(set(generated)) > 1
    engine.close()
    batch.close()
