"""Python binding of the thinking-budget control (include/lily_thinking.h).

Mirrors the reference's src/thinking.rs: `ThinkingTexts`, `ThinkingTokens`,
`ThinkingSettings`, `ThinkingControl` with `decide` / `decide_stop` /
`may_act_next`, the `Action` kinds, `opens_thinking`, and the emit helpers
`push_group` / `emit_acted` of src/generate.rs:121-169. All logic lives in
the C++ library; this file only marshals.
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass, field

from . import lib as _lib

DEFAULT_GRACE = 128

KEEP, BEFORE, AFTER, REPLACE = 0, 1, 2, 3
CLOSED_TOOL_CALL, CLOSED_BUDGET, CLOSED_END_OF_TURN = 0, 1, 2
FINISH_NONE, FINISH_CALLBACK, FINISH_LENGTH = 0, 1, 2

_ENCODE = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_char_p, C.c_uint32, C.POINTER(C.c_uint32),
                      C.c_uint32)
_IS_ADDED = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_uint32)
_ON_TOKEN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_uint32)


class _NudgeLevel(C.Structure):
    _fields_ = [("at", C.c_double), ("texts", C.POINTER(C.c_char_p)), ("n_texts", C.c_uint32)]


class _Texts(C.Structure):
    _fields_ = [("close", C.POINTER(C.c_char_p)), ("n_close", C.c_uint32),
                ("nudges", C.POINTER(_NudgeLevel)), ("n_nudges", C.c_uint32)]


class _Settings(C.Structure):
    _fields_ = [("budget", C.c_int64), ("grace", C.c_uint64), ("nudges", C.c_int32),
                ("tool_call_ends_thinking", C.c_int32), ("seed", C.c_uint64)]


_bound = False


def _L():
    global _bound
    L = _lib()
    if not _bound:
        L.lily_thinking_tokens_create.argtypes = [
            C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(_Texts), _ENCODE, _IS_ADDED, C.c_void_p,
            C.POINTER(C.c_void_p), C.c_char_p, C.c_uint32]
        L.lily_thinking_tokens_create_json.argtypes = [
            C.c_uint32, C.c_uint32, C.c_uint32, C.c_char_p, C.c_uint32, _ENCODE, _IS_ADDED,
            C.c_void_p, C.POINTER(C.c_void_p), C.c_char_p, C.c_uint32]
        L.lily_thinking_tokens_destroy.argtypes = [C.c_void_p]
        L.lily_thinking_tokens_destroy.restype = None
        L.lily_thinking_settings_any.argtypes = [C.POINTER(_Settings)]
        L.lily_thinking_control_create.argtypes = [C.c_void_p, C.POINTER(_Settings), C.c_int32]
        L.lily_thinking_control_create.restype = C.c_void_p
        L.lily_thinking_control_destroy.argtypes = [C.c_void_p]
        L.lily_thinking_control_destroy.restype = None
        L.lily_thinking_is_open.argtypes = [C.c_void_p]
        L.lily_thinking_closed.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_uint64)]
        L.lily_thinking_close_emitted.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_uint64]
        L.lily_thinking_nudged.argtypes = [C.c_void_p]
        L.lily_thinking_nudged.restype = C.c_uint64
        L.lily_thinking_tokens_counted.argtypes = [C.c_void_p]
        L.lily_thinking_tokens_counted.restype = C.c_uint64
        L.lily_thinking_may_act_next.argtypes = [C.c_void_p]
        L.lily_thinking_decide.argtypes = [C.c_void_p, C.c_uint32, C.c_char_p, C.c_uint32]
        L.lily_thinking_decide_stop.argtypes = [C.c_void_p]
        L.lily_thinking_action_ids.argtypes = [C.c_void_p, C.POINTER(C.POINTER(C.c_uint32)),
                                               C.POINTER(C.c_uint32)]
        L.lily_thinking_action_ids.restype = None
        L.lily_opens_thinking.argtypes = [C.c_char_p, C.c_uint32]
        L.lily_push_group.argtypes = [C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.c_uint64,
                                      C.POINTER(C.c_uint32), C.c_uint64, C.c_uint64, _ON_TOKEN,
                                      C.c_void_p, C.POINTER(C.c_int32)]
        L.lily_emit_acted.argtypes = [C.c_int32, C.POINTER(C.c_uint32), C.c_uint64, C.c_uint32,
                                      C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.c_uint64,
                                      C.c_uint64, _ON_TOKEN, C.c_void_p, C.POINTER(C.c_int32)]
        _bound = True
    return L


@dataclass
class NudgeLevel:
    at: float
    texts: list


@dataclass
class ThinkingTexts:
    """src/thinking.rs:124-131; `None` passed to ThinkingTokens means the built-in set."""

    close: list = field(default_factory=list)
    nudges: list = field(default_factory=list)

    @classmethod
    def from_json(cls, text: str) -> "ThinkingTexts":
        raw = json.loads(text)
        unknown = set(raw) - {"close", "nudges"}
        if unknown:
            raise ValueError(f"unknown field {sorted(unknown)[0]!r}")
        return cls(list(raw.get("close", [])),
                   [NudgeLevel(n["at"], list(n["texts"])) for n in raw.get("nudges", [])])


@dataclass
class Action:
    """src/thinking.rs:356-367."""

    kind: int = KEEP
    ids: list = field(default_factory=list)

    def __eq__(self, other):
        return isinstance(other, Action) and (self.kind, self.ids) == (other.kind, other.ids)


Keep = Action(KEEP, [])


@dataclass
class ThinkingSettings:
    """src/thinking.rs:329-352."""

    budget: int | None = None
    grace: int = 0
    nudges: bool = False
    tool_call_ends_thinking: bool = False
    seed: int = 0

    def _c(self) -> _Settings:
        return _Settings(-1 if self.budget is None else self.budget, self.grace, int(self.nudges),
                         int(self.tool_call_ends_thinking), self.seed & 0xFFFFFFFFFFFFFFFF)

    def any(self) -> bool:
        return bool(_L().lily_thinking_settings_any(C.byref(self._c())))


class ThinkingTokens:
    """src/thinking.rs:224-326: the markers and every sequence the controls insert,
    encoded once with the caller's tokenizer."""

    def __init__(self, think_end, tool_call, tool_call_end, texts, encode, is_added, *,
                 json_text: str | None = None):
        def _enc(_user, data, n, out, cap):
            try:
                ids = encode(C.string_at(data, n).decode("utf-8"))
            except Exception:
                return -1
            for i, v in enumerate(ids[:cap]):
                out[i] = v
            return len(ids)

        def _added(_user, tok):
            return 1 if is_added(tok) else 0

        self._enc, self._added = _ENCODE(_enc), _IS_ADDED(_added)  # keep the thunks alive
        self._h = C.c_void_p()
        err = C.create_string_buffer(512)
        if json_text is not None:
            raw = json_text.encode("utf-8")
            st = _L().lily_thinking_tokens_create_json(think_end, tool_call, tool_call_end, raw,
                                                       len(raw), self._enc, self._added, None,
                                                       C.byref(self._h), err, len(err))
        else:
            ct, keep = None, []
            if texts is not None:
                close = (C.c_char_p * max(len(texts.close), 1))(*[t.encode() for t in texts.close])
                levels = (_NudgeLevel * max(len(texts.nudges), 1))()
                for i, lv in enumerate(texts.nudges):
                    arr = (C.c_char_p * max(len(lv.texts), 1))(*[t.encode() for t in lv.texts])
                    keep.append(arr)
                    levels[i] = _NudgeLevel(lv.at, arr, len(lv.texts))
                ct = _Texts(close, len(texts.close), levels, len(texts.nudges))
                keep += [close, levels]
            st = _L().lily_thinking_tokens_create(think_end, tool_call, tool_call_end,
                                                  C.byref(ct) if ct is not None else None,
                                                  self._enc, self._added, None, C.byref(self._h),
                                                  err, len(err))
        if st != 0:
            raise ValueError(err.value.decode("utf-8", "replace"))
        self.think_end, self.tool_call, self.tool_call_end = think_end, tool_call, tool_call_end

    def __del__(self):
        if getattr(self, "_h", None):
            _L().lily_thinking_tokens_destroy(self._h)
            self._h = None


@dataclass
class Closed:
    by: int
    thinking_tokens: int


class ThinkingControl:
    """src/thinking.rs:397-646: one generation's thinking state."""

    def __init__(self, tokens: ThinkingTokens, settings: ThinkingSettings, opens_thinking: bool):
        self._tokens = tokens
        self._h = _L().lily_thinking_control_create(tokens._h, C.byref(settings._c()),
                                                    int(opens_thinking))
        if not self._h:
            raise ValueError("lily_thinking_control_create failed")

    def __del__(self):
        if getattr(self, "_h", None):
            _L().lily_thinking_control_destroy(self._h)
            self._h = None

    def _action(self, kind: int) -> Action:
        if kind == KEEP:
            return Action(KEEP, [])
        ids, n = C.POINTER(C.c_uint32)(), C.c_uint32()
        _L().lily_thinking_action_ids(self._h, C.byref(ids), C.byref(n))
        return Action(kind, [ids[i] for i in range(n.value)])

    def decide(self, token: int, text: str) -> Action:
        raw = text.encode("utf-8")
        return self._action(_L().lily_thinking_decide(self._h, token, raw, len(raw)))

    def decide_stop(self) -> Action:
        return self._action(_L().lily_thinking_decide_stop(self._h))

    def is_open(self) -> bool:
        return bool(_L().lily_thinking_is_open(self._h))

    def may_act_next(self) -> bool:
        return bool(_L().lily_thinking_may_act_next(self._h))

    def closed(self):
        by, n = C.c_int32(), C.c_uint64()
        if _L().lily_thinking_closed(self._h, C.byref(by), C.byref(n)):
            return Closed(by.value, n.value)
        return None

    def close_emitted(self, generated) -> bool:
        arr = (C.c_uint32 * max(len(generated), 1))(*generated)
        return bool(_L().lily_thinking_close_emitted(self._h, arr, len(generated)))

    def nudged(self) -> int:
        return int(_L().lily_thinking_nudged(self._h))

    def thinking_tokens(self) -> int:
        return int(_L().lily_thinking_tokens_counted(self._h))


def opens_thinking(prompt_tail: str) -> bool:
    """src/thinking.rs:848-850."""
    raw = prompt_tail.encode("utf-8")
    return bool(_L().lily_opens_thinking(raw, len(raw)))


def _run_emit(call, tokens: list, extra: int, on_token):
    cap = len(tokens) + extra + 1
    buf = (C.c_uint32 * cap)(*tokens)
    n = C.c_uint64(len(tokens))
    finish = C.c_int32(0)
    failure = []

    def _cb(_user, tok):
        try:
            return 1 if on_token(tok) else 0
        except Exception as exc:  # surfaced below, not thrown across the C frame
            failure.append(exc)
            return -1

    st = call(buf, C.byref(n), cap, _ON_TOKEN(_cb), C.byref(finish))
    if failure:
        raise failure[0]
    if st != 0:
        raise ValueError("emit_acted with nothing to insert" if st == 4 else f"emit failed ({st})")
    tokens[:] = [buf[i] for i in range(n.value)]
    return None if finish.value == FINISH_NONE else finish.value


def push_group(tokens: list, group, max_tokens: int, on_token):
    """src/generate.rs:121-142; returns None or FINISH_CALLBACK / FINISH_LENGTH."""
    g = (C.c_uint32 * max(len(group), 1))(*group)
    return _run_emit(lambda buf, n, cap, cb, fin: _L().lily_push_group(
        buf, n, cap, g, len(group), max_tokens, cb, None, fin), tokens, len(group), on_token)


def emit_acted(action: Action, drawn: int, tokens: list, max_tokens: int, on_token):
    """src/generate.rs:144-169."""
    g = (C.c_uint32 * max(len(action.ids), 1))(*action.ids)
    return _run_emit(lambda buf, n, cap, cb, fin: _L().lily_emit_acted(
        action.kind, g, len(action.ids), drawn, buf, n, cap, max_tokens, cb, None, fin),
        tokens, len(action.ids) + 1, on_token)
