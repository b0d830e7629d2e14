"""ctypes mirror of include/lily_batch.h: the bookkeeping around the sampler
when requests decode as rows of a batch (the reference: src/serve/batch.rs:74-264,
421-438; src/engine.rs:588-596, 983-994; src/qwen4exp/batch.rs:137-162)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

from . import LilyError, SamplerScratch, _stream_ptr
from . import lib as _lib

ENGINE = 0xFFFFFFFF  # CountsSlot::Engine; any other value i is CountsSlot::Batch(i)
DONE, SOLO, STEP = 0, 1, 2


class _RowAhead(C.Structure):
    _fields_ = [("pos", C.c_uint64), ("capacity", C.c_uint64), ("checkpoint_due", C.c_uint8),
                ("ending", C.c_uint8), ("may_insert", C.c_uint8), ("reserved", C.c_uint8 * 5)]


class _SoloStop(C.Structure):
    _fields_ = [("yielded", C.c_uint8), ("terminal", C.c_uint8)]


class _Stats(C.Structure):
    _fields_ = [("batched_tokens", C.c_uint64), ("rows_sum", C.c_uint64), ("max_rows", C.c_uint64),
                ("peers", C.POINTER(C.c_uint64)), ("n_peers", C.c_uint32), ("peers_cap", C.c_uint32)]


_ready = False


def _bound():
    global _ready
    L = _lib()
    if not _ready:
        L.lily_slots_create.argtypes = [C.c_uint32, C.POINTER(C.c_void_p)]
        L.lily_slots_destroy.argtypes = [C.c_void_p]
        L.lily_slots_destroy.restype = None
        L.lily_slots_take.argtypes = [C.c_void_p]
        L.lily_slots_give.argtypes = [C.c_void_p, C.c_uint32]
        L.lily_slots_in_use.argtypes = [C.c_void_p]
        L.lily_slots_in_use.restype = C.c_uint32
        L.lily_slots_capacity.argtypes = [C.c_void_p]
        L.lily_slots_capacity.restype = C.c_uint32
        L.lily_move_counts.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32]
        L.lily_row_draw_step.argtypes = [C.c_uint64, C.c_uint32]
        L.lily_row_draw_step.restype = C.c_uint32
        L.lily_admits.argtypes = [C.c_uint64] * 5
        L.lily_next_action.argtypes = [C.c_uint64, C.c_int32, C.POINTER(C.c_int32)]
        L.lily_park_next.argtypes = [C.POINTER(_RowAhead), C.c_uint32, C.c_int32, C.c_int32, C.c_int32]
        L.lily_solo_stop_observe.argtypes = [C.POINTER(_SoloStop), C.c_int32, C.c_int32]
        L.lily_solo_stop_yielded_only.argtypes = [C.POINTER(_SoloStop)]
        L.lily_batch_stats_record_step.argtypes = [C.POINTER(_Stats), C.c_uint64,
                                                   C.POINTER(C.c_uint64), C.c_uint32]
        L.lily_batch_stats_mean_rows.argtypes = [C.POINTER(_Stats)]
        L.lily_batch_stats_mean_rows.restype = C.c_double
        _ready = True
    return L


class Slots:
    """src/serve/batch.rs:74-102: the batch slots, each owning one histogram
    slot of the batch sampler."""

    def __init__(self, n: int):
        h = C.c_void_p()
        if _bound().lily_slots_create(n, C.byref(h)) != 0:
            raise LilyError(-1, "slots")
        self._h = h

    def take(self) -> Optional[int]:
        slot = _bound().lily_slots_take(self._h)
        return None if slot < 0 else slot

    def give(self, slot: int) -> None:
        if _bound().lily_slots_give(self._h, slot) != 0:
            raise LilyError(-1, f"slot {slot} given back twice")

    def in_use(self) -> int:
        return _bound().lily_slots_in_use(self._h)

    def __len__(self) -> int:
        return _bound().lily_slots_capacity(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            _bound().lily_slots_destroy(self._h)
            self._h = None


def move_sampler_counts(engine: SamplerScratch, batch: SamplerScratch, src: int, dst: int,
                        stream=None) -> None:
    """src/engine.rs:983-994: `src` and `dst` are ENGINE or a batch slot."""
    st = _bound().lily_move_counts(engine._h, batch._h, _stream_ptr(stream), src, dst)
    if st != 0:
        raise LilyError(st, _lib().lily_sampler_last_error(batch._h).decode())


def draw_step(generated: int, ahead: int = 0) -> int:
    """src/serve/batch.rs:421-438: the draw index of a row in the step that
    feeds its last draw, or (`ahead` 1) in the step parked behind it."""
    return _bound().lily_row_draw_step(generated, ahead)


def admits(rows: int, max_rows: int, in_flight: int, estimate: int, budget: int) -> bool:
    return bool(_bound().lily_admits(rows, max_rows, in_flight, estimate, budget))


def next_action(rows: int, held: bool):
    """(DONE | SOLO | STEP, preempt) -- preempt is None unless SOLO."""
    pre = C.c_int32(-1)
    kind = _bound().lily_next_action(rows, int(held), C.byref(pre))
    return kind, (bool(pre.value) if kind == SOLO else None)


@dataclass
class RowAhead:
    pos: int
    capacity: int = 8192
    checkpoint_due: bool = False
    ending: bool = False
    may_insert: bool = False


def park_next(rows: Sequence[RowAhead], another_step: bool, admission: bool, cancel: bool) -> bool:
    arr = (_RowAhead * max(len(rows), 1))()
    for i, r in enumerate(rows):
        arr[i].pos, arr[i].capacity = r.pos, r.capacity
        arr[i].checkpoint_due, arr[i].ending, arr[i].may_insert = r.checkpoint_due, r.ending, r.may_insert
    return bool(_bound().lily_park_next(arr, len(rows), int(another_step), int(admission), int(cancel)))


class SoloStop:
    def __init__(self):
        self._s = _SoloStop()

    def observe(self, terminal: bool, waiting: bool) -> bool:
        return bool(_bound().lily_solo_stop_observe(C.byref(self._s), int(terminal), int(waiting)))

    def yielded_only(self) -> bool:
        return bool(_bound().lily_solo_stop_yielded_only(C.byref(self._s)))


class BatchStats:
    def __init__(self, max_peers: int = 64):
        self._peers = (C.c_uint64 * max_peers)()
        self._s = _Stats(0, 0, 0, C.cast(self._peers, C.POINTER(C.c_uint64)), 0, max_peers)

    def record_step(self, own: int, members: Sequence[int]) -> None:
        arr = (C.c_uint64 * max(len(members), 1))(*members)
        if _bound().lily_batch_stats_record_step(C.byref(self._s), own, arr, len(members)) != 0:
            raise LilyError(-1, "more peers than the statistics hold")

    batched_tokens = property(lambda self: self._s.batched_tokens)
    rows_sum = property(lambda self: self._s.rows_sum)
    max_rows = property(lambda self: self._s.max_rows)
    peers = property(lambda self: [self._peers[i] for i in range(self._s.n_peers)])

    def mean_rows(self) -> Optional[float]:
        v = _bound().lily_batch_stats_mean_rows(C.byref(self._s))
        return None if v < 0 else v
