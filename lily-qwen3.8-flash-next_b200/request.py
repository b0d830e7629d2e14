"""ctypes mirror of include/lily_request.h: an OpenAI-style request's sampling
and thinking fields resolved over the server's defaults (the reference:
src/serve/api.rs:436-457, 498-708, 798-888; src/serve.rs:1762-1835)."""
from __future__ import annotations

import ctypes as C

from . import LilyError, SamplingParams
from . import lib as _lib
from .thinking import _Settings as _ThinkingSettingsStruct  # lily_thinking_settings_t

HAS_TEMPERATURE, HAS_TOP_P, HAS_TOP_K, HAS_MIN_P, HAS_SEED = 1, 2, 4, 8, 16
HAS_PRESENCE, HAS_FREQUENCY, HAS_REPETITION = 32, 64, 128
HAS_THINKING_BUDGET, HAS_THINKING_NUDGES, HAS_TOOL_CALL_ENDS_THINKING = 256, 512, 1024
MAX_THINKING_TOKENS = 1 << 20


class Overrides(C.Structure):
    _fields_ = [("present", C.c_uint32), ("temperature", C.c_float), ("top_k", C.c_uint64),
                ("top_p", C.c_float), ("min_p", C.c_float), ("presence_penalty", C.c_float),
                ("frequency_penalty", C.c_float), ("repetition_penalty", C.c_float)]


class Fields(C.Structure):
    _fields_ = [("present", C.c_uint32), ("temperature", C.c_float), ("top_p", C.c_float),
                ("min_p", C.c_float), ("presence_penalty", C.c_float), ("frequency_penalty", C.c_float),
                ("repetition_penalty", C.c_float), ("top_k", C.c_int64), ("seed", C.c_int64),
                ("thinking_budget", C.c_int64), ("thinking_nudges", C.c_int32),
                ("tool_call_ends_thinking", C.c_int32)]

    def has(self, bit: int) -> bool:
        return bool(self.present & bit)


class Budgets(C.Structure):
    _fields_ = [("low", C.c_int64), ("medium", C.c_int64), ("xhigh", C.c_int64)]

    def as_tuple(self):
        none = lambda v: None if v < 0 else int(v)
        return none(self.low), none(self.medium), none(self.xhigh)


class ThinkingDefaults(C.Structure):
    _fields_ = [("budgets", Budgets), ("tool_turn_factor", C.c_double), ("nudges", C.c_int32),
                ("tool_call_ends_thinking", C.c_int32), ("grace", C.c_uint64)]

    def __init__(self, **kw):
        super().__init__()
        _bound().lily_thinking_defaults_init(C.byref(self))
        for k, v in kw.items():
            setattr(self, k, v)


_ready = False


def _bound():
    global _ready
    L = _lib()
    if not _ready:
        err = [C.c_char_p, C.c_uint32]
        L.lily_sampling_defaults.argtypes = [C.c_char_p, C.c_uint32, C.POINTER(Overrides), C.c_int32,
                                             C.POINTER(SamplingParams)] + err
        L.lily_request_fields_from_json.argtypes = [C.c_char_p, C.c_uint32, C.POINTER(Fields)] + err
        L.lily_resolve_sampling.argtypes = [C.POINTER(Fields), C.POINTER(SamplingParams), C.c_uint64,
                                            C.POINTER(SamplingParams)] + err
        L.lily_thinking_budgets_parse.argtypes = [C.c_char_p, C.POINTER(Budgets)] + err
        L.lily_thinking_budgets_at.argtypes = [C.POINTER(Budgets), C.c_char_p]
        L.lily_thinking_budgets_at.restype = C.c_int64
        L.lily_template_effort.argtypes = [C.c_char_p]
        L.lily_template_effort.restype = C.c_char_p
        L.lily_thinking_defaults_init.argtypes = [C.POINTER(ThinkingDefaults)]
        L.lily_thinking_defaults_init.restype = None
        L.lily_thinking_defaults_validate.argtypes = [C.POINTER(ThinkingDefaults)] + err
        L.lily_thinking_defaults_budget.argtypes = [C.POINTER(ThinkingDefaults), C.c_char_p, C.c_int32]
        L.lily_thinking_defaults_budget.restype = C.c_int64
        L.lily_thinking_resolve.argtypes = [C.POINTER(Fields), C.POINTER(ThinkingDefaults), C.c_int64,
                                            C.c_uint64, C.POINTER(_ThinkingSettingsStruct)]
        L.lily_thinking_resolve.restype = None
        _ready = True
    return L


def _call(fn, *args):
    buf = C.create_string_buffer(256)
    st = fn(*args, buf, 256)
    if st != 0:
        raise LilyError(st, buf.value.decode())


def sampling_defaults(generation_config: bytes | None = None, overrides: Overrides | None = None,
                      validate: bool = True) -> SamplingParams:
    """src/serve.rs:1762-1835 sampling_defaults / sampling_unvalidated."""
    out = SamplingParams()
    _call(_bound().lily_sampling_defaults, generation_config,
          len(generation_config) if generation_config else 0,
          C.byref(overrides) if overrides is not None else None, int(validate), C.byref(out))
    return out


def fields_from_json(body: bytes) -> Fields:
    """The request's flattened SamplingFields and ThinkingFields (chat_template_kwargs win)."""
    out = Fields()
    _call(_bound().lily_request_fields_from_json, body, len(body), C.byref(out))
    return out


def resolve_sampling(fields: Fields, defaults: SamplingParams, entropy: int = 0) -> SamplingParams:
    """src/serve/api.rs:798-834 resolve_sampling."""
    out = SamplingParams()
    _call(_bound().lily_resolve_sampling, C.byref(fields), C.byref(defaults), entropy & (2**64 - 1),
          C.byref(out))
    return out


def thinking_budgets(text: str) -> Budgets:
    """src/serve/api.rs:608-650 ThinkingBudgets::parse."""
    out = Budgets()
    _call(_bound().lily_thinking_budgets_parse, text.encode(), C.byref(out))
    return out


def budget_at(b: Budgets, effort: str | None):
    v = _bound().lily_thinking_budgets_at(C.byref(b), effort.encode() if effort is not None else None)
    return None if v < 0 else int(v)


def template_effort(value: str):
    v = _bound().lily_template_effort(value.encode())
    return v.decode() if v is not None else None


def validate_thinking_defaults(d: ThinkingDefaults) -> None:
    _call(_bound().lily_thinking_defaults_validate, C.byref(d))


def default_budget(d: ThinkingDefaults, effort: str | None, tool_turn: bool):
    v = _bound().lily_thinking_defaults_budget(C.byref(d), effort.encode() if effort is not None else None,
                                               int(tool_turn))
    return None if v < 0 else int(v)


def resolve_thinking(fields: Fields, defaults: ThinkingDefaults, budget, seed: int):
    """src/serve/api.rs:568-589 ThinkingFields::resolve -> lily_thinking_settings_t."""
    out = _ThinkingSettingsStruct()
    _bound().lily_thinking_resolve(C.byref(fields), C.byref(defaults), -1 if budget is None else int(budget),
                                   seed & (2**64 - 1), C.byref(out))
    return out
