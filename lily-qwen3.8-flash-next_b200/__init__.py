"""Python binding of the B200 token sampler's C ABI (include/lily_sampler.h).

The names mirror the reference's sampler interface (paths relative to the
reference project): `SamplingParams` (src/kernels/sample.rs:19-95),
`SamplerScratch` (:115-179), `sample_f32` / `sample_draft_f32` /
`sample_spec_f32` (:373-432), `uniform_for` (:435-441), `draft_step`,
`draft_params` (:217-234), `spec_accept` (src/kernels/spec.rs:52-91).

torch is used for device memory and streams only; every computation happens
in liblily_sampler.so. There is no CPU fallback: importing works anywhere,
calling a device entry point without the library or without a GPU raises.
"""
from __future__ import annotations

import ctypes as C
import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblily_sampler.so")

K_CAP = 1024
F32, BF16 = 0, 1
SPEC_REJECTION, SPEC_GREEDY_MATCH = 0, 1
FLAG_COUNTS_TABLE = 1
FLAG_PHASE_CLOCKS = 2
MAX_SLICES, PHASES = 128, 20

OK = 0
ERR_ARG, ERR_PARAMS, ERR_CAPACITY, ERR_FAULT, ERR_VOCAB = -1, -2, -3, -4, -5
ERR_CUDA, ERR_DEVICE_ROW, ERR_TIMEOUT = 1, 2, 3
ROW_OK, ROW_NAN, ROW_NONFINITE, ROW_PARAMS, ROW_LIST, ROW_FORCED = 0, 1, 2, 3, 4, 16


class LilyError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"lily sampler error {code}: {message}")
        self.code = code


class SamplingParams(C.Structure):
    """src/kernels/sample.rs:19-31; defaults are SamplingParams::greedy()."""

    _fields_ = [
        ("temperature", C.c_float),
        ("top_k", C.c_uint32),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("presence_penalty", C.c_float),
        ("frequency_penalty", C.c_float),
        ("repetition_penalty", C.c_float),
        ("reserved", C.c_uint32),
        ("seed", C.c_uint64),
    ]

    def __init__(self, temperature=0.0, top_k=1, top_p=1.0, min_p=0.0, presence_penalty=0.0,
                 frequency_penalty=0.0, repetition_penalty=1.0, seed=0):
        super().__init__(temperature, max(int(top_k), 0), top_p, min_p, presence_penalty,
                         frequency_penalty, repetition_penalty, 0, seed & 0xFFFFFFFFFFFFFFFF)

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls()

    def is_greedy(self) -> bool:
        return bool(lib().lily_params_is_greedy(C.byref(self)))

    def uses_penalties(self) -> bool:
        return bool(lib().lily_params_uses_penalties(C.byref(self)))

    def validate(self) -> None:
        st = lib().lily_params_validate(C.byref(self))
        if st != OK:
            raise LilyError(st, "invalid sampling parameters")

    def effective(self):
        t, k = C.c_float(), C.c_uint32()
        lib().lily_params_effective(C.byref(self), C.byref(t), C.byref(k))
        return t.value, k.value


_vp, _u32p, _f32p, _i32p = C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p


class SampleArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("rows", C.c_uint32),
        ("logits", _vp), ("logits_dtype", C.c_uint32), ("params_on_device", C.c_uint32),
        ("logits_ld", C.c_uint64),
        ("params", _vp), ("uniforms", _f32p), ("steps", _u32p),
        ("history_ids", _u32p), ("history_len", _u32p), ("history_ld", C.c_uint64),
        ("bias_ids", _u32p), ("bias_vals", _f32p), ("bias_len", _u32p), ("bias_ld", C.c_uint64),
        ("ban_ids", _u32p), ("ban_len", _u32p), ("ban_ld", C.c_uint64),
        ("forced_ids", _i32p), ("count_slots", _u32p),
        ("out_ids", _u32p), ("out_status", _u32p),
        ("kept_n", _u32p), ("kept_ids", _u32p), ("kept_probs", _f32p), ("kept_ld", C.c_uint64),
    ]


class LmHead(C.Structure):
    """lily_lmhead_t: an 8-bit head (or one vocabulary shard of it) on the device."""

    _fields_ = [("struct_size", C.c_uint32), ("rows", C.c_uint32), ("hidden", C.c_uint32),
                ("group", C.c_uint32), ("weights", C.c_void_p), ("scales_bf16", C.c_void_p),
                ("biases_bf16", C.c_void_p), ("code_bits", C.c_uint32), ("reserved", C.c_uint32)]


class PeerExchangeStruct(C.Structure):
    """lily_peer_exchange_t: every rank's exchange buffer as this process sees it."""

    _fields_ = [("struct_size", C.c_uint32), ("n_shards", C.c_uint32), ("rank", C.c_uint32),
                ("max_rows", C.c_uint32), ("buffers", C.c_void_p * 16)]


PEER_MAX = 16
IPC_HANDLE_BYTES = 64
SHARD_CANDIDATES = 64
SHARD_RECORD_BYTES = 520
FLAG_LMHEAD = 4


class SpecArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("m", C.c_uint32),
        ("target_logits", _vp), ("logits_dtype", C.c_uint32), ("mode", C.c_uint32),
        ("logits_ld", C.c_uint64),
        ("params", _vp), ("draft_ids", _u32p),
        ("q_dense", _f32p), ("q_ld", C.c_uint64),
        ("q_ids", _u32p), ("q_probs", _f32p), ("q_n", _u32p),
        ("u_accept", _f32p), ("u_resid", _f32p),
        ("step0", C.c_uint32), ("history_len", C.c_uint32),
        ("history_ids", _u32p), ("count_slot", _u32p),
        ("out_ids", _u32p), ("out_accepted", _u32p), ("out_status", _u32p),
    ]


_lib = None


def lib():
    """The loaded C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LilyError(ERR_CUDA, f"{LIB_PATH} is missing: run build.py (there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        L.lily_abi_version.restype = C.c_uint32
        L.lily_uniform_for.restype = C.c_float
        L.lily_uniform_for.argtypes = [C.c_uint64, C.c_uint32]
        L.lily_draft_step.restype = C.c_uint32
        L.lily_draft_step.argtypes = [C.c_uint32]
        L.lily_residual_step.restype = C.c_uint32
        L.lily_residual_step.argtypes = [C.c_uint32]
        L.lily_params_validate.argtypes = [C.POINTER(SamplingParams)]
        L.lily_params_is_greedy.argtypes = [C.POINTER(SamplingParams)]
        L.lily_params_uses_penalties.argtypes = [C.POINTER(SamplingParams)]
        L.lily_params_effective.argtypes = [C.POINTER(SamplingParams), C.POINTER(C.c_float),
                                            C.POINTER(C.c_uint32)]
        L.lily_params_effective.restype = None
        L.lily_draft_params.argtypes = [C.POINTER(SamplingParams), C.POINTER(SamplingParams)]
        L.lily_draft_params.restype = None
        L.lily_sampler_create.argtypes = [C.c_int32, C.c_uint32, C.c_uint32, C.c_uint32,
                                          C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p)]
        L.lily_sampler_destroy.argtypes = [C.c_void_p]
        L.lily_sampler_destroy.restype = None
        L.lily_sampler_vocab.argtypes = [C.c_void_p]
        L.lily_sampler_vocab.restype = C.c_uint32
        L.lily_sampler_last_error.argtypes = [C.c_void_p]
        L.lily_sampler_last_error.restype = C.c_char_p
        L.lily_sampler_inject_fault.argtypes = [C.c_void_p, C.c_int32]
        L.lily_sampler_inject_fault.restype = None
        L.lily_sampler_set_wait_limit.argtypes = [C.c_void_p, C.c_uint64]
        L.lily_sampler_set_wait_limit.restype = C.c_int32
        L.lily_sampler_inject_lost_copy.argtypes = [C.c_void_p, C.c_uint32]
        L.lily_sampler_inject_lost_copy.restype = None
        L.lily_sampler_clear_fault.argtypes = [C.c_void_p]
        L.lily_sampler_clear_fault.restype = None
        L.lily_sampler_status.argtypes = [C.c_void_p, C.c_void_p]
        L.lily_sampler_reset_counts.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32]
        L.lily_sampler_uncount.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32]
        L.lily_sampler_copy_counts.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32,
                                               C.c_void_p]
        L.lily_sampler_read_counts.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]
        L.lily_sampler_write_counts.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]
        L.lily_sample_batch.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(SampleArgs)]
        L.lily_argmax_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32,
                                        C.c_uint64, C.c_uint32, C.c_void_p]
        L.lily_spec_verify.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(SpecArgs)]
        L.lily_spec_accept.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32,
                                       C.c_uint32, C.c_uint32]
        L.lily_debug_exp.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64]
        L.lily_sample_batch_noalloc.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(SampleArgs),
                                                C.c_char_p, C.c_uint32]
        L.lily_sampler_read_phase_clocks.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.lily_lmhead_logits.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(LmHead), C.c_void_p,
                                         C.c_uint64, C.c_uint32, C.c_void_p, C.c_uint64]
        L.lily_shard_candidates.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(SampleArgs),
                                            C.c_uint32, C.c_int32, C.c_void_p]
        L.lily_lmhead_shard_candidates.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(LmHead),
                                                   C.c_void_p, C.c_uint64, C.POINTER(SampleArgs),
                                                   C.c_uint32, C.c_int32, C.c_void_p]
        L.lily_merge_draw.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64,
                                      C.POINTER(SampleArgs), C.c_void_p]
        L.lily_peer_buffer_bytes.restype = C.c_uint64
        L.lily_peer_buffer_bytes.argtypes = [C.c_uint32, C.c_uint32]
        L.lily_peer_buffer_create.argtypes = [C.c_int32, C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p),
                                              C.c_void_p]
        L.lily_peer_buffer_open.argtypes = [C.c_int32, C.c_void_p, C.POINTER(C.c_void_p)]
        L.lily_peer_buffer_close.argtypes = [C.c_int32, C.c_void_p]
        L.lily_peer_buffer_destroy.argtypes = [C.c_int32, C.c_void_p]
        L.lily_shard_publish.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(PeerExchangeStruct), C.c_void_p,
                                         C.c_uint32, C.c_uint32]
        L.lily_merge_draw_peer.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(PeerExchangeStruct), C.c_void_p,
                                           C.c_uint32, C.POINTER(SampleArgs), C.c_void_p]
        _lib = L
    return _lib


def debug_exp(x, stream=None):
    """The kernels' exp on a float32 CUDA tensor (lily_debug_exp)."""
    import torch

    out = torch.empty_like(x)
    st = lib().lily_debug_exp(_stream_ptr(stream), _ptr(x), _ptr(out), x.numel())
    if st != OK:
        raise LilyError(st, "lily_debug_exp failed")
    return out


def uniform_for(seed: int, step: int) -> float:
    """src/kernels/sample.rs:435-441."""
    return float(lib().lily_uniform_for(seed & 0xFFFFFFFFFFFFFFFF, step & 0xFFFFFFFF))


def draft_step(step: int) -> int:
    """src/kernels/sample.rs:220-222."""
    return int(lib().lily_draft_step(step))


def residual_step(step: int) -> int:
    return int(lib().lily_residual_step(step))


def draft_params(p: SamplingParams) -> SamplingParams:
    """src/kernels/sample.rs:227-234."""
    out = SamplingParams()
    lib().lily_draft_params(C.byref(p), C.byref(out))
    return out


def _ptr(t):
    """Device (or pinned host) address of a torch tensor, or None."""
    if t is None:
        return None
    assert t.is_contiguous(), "tensors passed to the sampler must be contiguous"
    return t.data_ptr()


def _ld(t) -> int:
    """Row pitch in elements of a [rows, n] (or [n]) tensor."""
    if t.dim() == 2 and t.shape[0] > 1:
        return t.stride(0)
    return t.shape[-1]


def _dtype_code(t) -> int:
    import torch

    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise LilyError(ERR_ARG, "logits must be F32 or BF16")


def _stream_ptr(stream) -> int:
    import torch

    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream


class SamplerScratch:
    """Per-engine sampler state for one vocabulary (src/kernels/sample.rs:115-179),
    for up to `max_rows` rows per call."""

    def __init__(self, vocab: int, max_rows: int = 1, max_history: int = 1 << 16,
                 max_list: int = 256, counts_table: bool = False, device: int | None = None,
                 phase_clocks: bool = False, lmhead: bool = False):
        import torch

        if device is None:
            device = torch.cuda.current_device()
        self._h = C.c_void_p()
        self.device = device
        self.max_rows = max_rows
        st = lib().lily_sampler_create(device, vocab, max_rows, max_history, max_list,
                                       (FLAG_COUNTS_TABLE if counts_table else 0)
                                       | (FLAG_PHASE_CLOCKS if phase_clocks else 0)
                                       | (FLAG_LMHEAD if lmhead else 0),
                                       C.byref(self._h))
        if st != OK:
            raise LilyError(st, "lily_sampler_create failed (is a CUDA device present?)")

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            lib().lily_sampler_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st: int):
        if st != OK:
            raise LilyError(st, lib().lily_sampler_last_error(self._h).decode())

    def vocab(self) -> int:
        return int(lib().lily_sampler_vocab(self._h))

    # -- fault latch (src/metal.rs:681-696)
    def inject_fault(self, code: int = 1):
        lib().lily_sampler_inject_fault(self._h, code)

    def clear_fault(self):
        lib().lily_sampler_clear_fault(self._h)

    def status(self, stream=None) -> int:
        return int(lib().lily_sampler_status(self._h, _stream_ptr(stream)))

    # -- bounded waits of the LM-head kernel (src/metal.rs:856-861, 1276-1279)
    def set_wait_limit(self, nanoseconds: int):
        self._check(lib().lily_sampler_set_wait_limit(self._h, nanoseconds))

    def inject_lost_copy(self, stage: int):
        """Test hook: the next LM-head launch leaves out one weight copy of its first block."""
        lib().lily_sampler_inject_lost_copy(self._h, stage)

    # -- histogram slots (src/kernels/sample.rs:145-174)
    def reset_counts(self, slot: int = 0, stream=None):
        self._check(lib().lily_sampler_reset_counts(self._h, _stream_ptr(stream), slot))

    def uncount(self, token: int, slot: int = 0, stream=None):
        self._check(lib().lily_sampler_uncount(self._h, _stream_ptr(stream), slot, token))

    def copy_counts_from(self, other: "SamplerScratch", slot: int = 0, other_slot: int = 0,
                         stream=None):
        self._check(lib().lily_sampler_copy_counts(self._h, slot, other._h, other_slot,
                                                   _stream_ptr(stream)))

    def read_counts(self, slot: int = 0, stream=None):
        import numpy as np

        out = np.zeros(self.vocab(), dtype=np.uint32)
        self._check(lib().lily_sampler_read_counts(self._h, _stream_ptr(stream), slot,
                                                   out.ctypes.data))
        return out

    def write_counts(self, counts, slot: int = 0, stream=None):
        import numpy as np

        counts = np.ascontiguousarray(counts, dtype=np.uint32)
        assert counts.size == self.vocab()
        self._check(lib().lily_sampler_write_counts(self._h, _stream_ptr(stream), slot,
                                                    counts.ctypes.data))

    def read_phase_clocks(self, stream=None):
        """SM clock stamps [max_rows, MAX_SLICES, PHASES] of the last launch
        (needs phase_clocks=True); see lily_sampler_read_phase_clocks."""
        import numpy as np

        out = np.zeros((self.max_rows, MAX_SLICES, PHASES), dtype=np.int64)
        self._check(lib().lily_sampler_read_phase_clocks(self._h, _stream_ptr(stream),
                                                         out.ctypes.data))
        return out

    # -- draws
    def sample_batch(self, logits, params, out_ids, *, stream=None, **kw):
        """lily_sample_batch: `params` is a list of SamplingParams (host), or with
        params_on_device a uint8 tensor holding the 40-byte structs."""
        a, keep = self._sample_args(logits, params, out_ids, **kw)
        self._check(lib().lily_sample_batch(self._h, _stream_ptr(stream), C.byref(a)))

    def prepare_sample_batch(self, logits, params, out_ids, **kw):
        """The argument block of a sample_batch call, built once: a decode loop
        that draws from the same buffers every step passes it to
        sample_prepared() and pays no per-step marshalling."""
        return self._sample_args(logits, params, out_ids, **kw)

    def sample_prepared(self, prepared, stream=None):
        self._check(lib().lily_sample_batch(self._h, _stream_ptr(stream), C.byref(prepared[0])))

    def _sample_args(self, logits, params, out_ids, *, uniforms=None, steps=None,
                     history_ids=None, history_len=None, bias_ids=None, bias_vals=None,
                     bias_len=None, ban_ids=None, ban_len=None, forced_ids=None,
                     count_slots=None, out_status=None, kept_n=None, kept_ids=None,
                     kept_probs=None, params_on_device=False):
        rows = logits.shape[0] if logits.dim() == 2 else 1
        a = SampleArgs()
        a.struct_size = C.sizeof(SampleArgs)
        a.rows = rows
        a.logits = _ptr(logits)
        a.logits_dtype = _dtype_code(logits)
        a.logits_ld = _ld(logits)
        keep = []
        if params_on_device:
            a.params_on_device = 1
            a.params = _ptr(params)
            a.steps = _ptr(steps)
        else:
            arr = (SamplingParams * rows)(*params)
            keep.append(arr)
            a.params = C.cast(arr, C.c_void_p)
            if steps is not None:
                sarr = (C.c_uint32 * rows)(*[int(s) for s in steps])
                keep.append(sarr)
                a.steps = C.cast(sarr, C.c_void_p)
        a.uniforms = _ptr(uniforms)
        if history_ids is not None:
            a.history_ids = _ptr(history_ids)
            a.history_len = _ptr(history_len)
            a.history_ld = _ld(history_ids)
        if bias_ids is not None:
            a.bias_ids, a.bias_vals, a.bias_len = _ptr(bias_ids), _ptr(bias_vals), _ptr(bias_len)
            a.bias_ld = _ld(bias_ids)
        if ban_ids is not None:
            a.ban_ids, a.ban_len = _ptr(ban_ids), _ptr(ban_len)
            a.ban_ld = _ld(ban_ids)
        a.forced_ids = _ptr(forced_ids)
        if count_slots is not None:
            carr = (C.c_uint32 * rows)(*[int(s) for s in count_slots])
            keep.append(carr)
            a.count_slots = C.cast(carr, C.c_void_p)
        a.out_ids = _ptr(out_ids)
        a.out_status = _ptr(out_status)
        if kept_n is not None:
            a.kept_n, a.kept_ids, a.kept_probs = _ptr(kept_n), _ptr(kept_ids), _ptr(kept_probs)
            a.kept_ld = _ld(kept_ids)
        return a, keep

    # -- 8-bit LM head and vocabulary shards
    @staticmethod
    def _head(weights, scales, biases=None, group: int = 64, code_bits: int = 8) -> LmHead:
        hd = LmHead()
        hd.struct_size = C.sizeof(LmHead)
        # (`weights` as bytes: a row of 4-bit codes is hidden / 2 bytes long)
        hd.rows, hd.hidden = int(weights.shape[0]), int(weights.shape[1]) * (2 if code_bits == 4 else 1)
        hd.code_bits = code_bits
        hd.group = group
        hd.weights = _ptr(weights)
        hd.scales_bf16 = _ptr(scales)
        hd.biases_bf16 = _ptr(biases) if biases is not None else None
        return hd

    def _shard_args(self, rows, params, steps, keep):
        a = SampleArgs()
        a.struct_size = C.sizeof(SampleArgs)
        a.rows = rows
        arr = (SamplingParams * rows)(*params)
        keep.append(arr)
        a.params = C.cast(arr, C.c_void_p)
        if steps is not None:
            sarr = (C.c_uint32 * rows)(*[int(s) for s in steps])
            keep.append(sarr)
            a.steps = C.cast(sarr, C.c_void_p)
        return a

    def lmhead_logits(self, weights, scales, hidden, out_logits, stream=None, biases=None, code_bits: int = 8):
        """lily_lmhead_logits: int8 `weights` [rows, hidden], bf16 `scales`
        [rows, hidden/64], bf16 `hidden` [tokens, hidden] -> F32 out [tokens, >= rows].
        With bf16 `biases` [rows, hidden/64] the head is in MLX affine 8-bit
        storage: `weights` are unsigned bytes, w = scale * q + bias; with
        code_bits=4 they are the 4-bit codes as bytes [rows, hidden/2]."""
        hd = self._head(weights, scales, biases, code_bits=code_bits)
        self._check(lib().lily_lmhead_logits(self._h, _stream_ptr(stream), C.byref(hd), _ptr(hidden),
                                             _ld(hidden), int(hidden.shape[0]), _ptr(out_logits),
                                             _ld(out_logits)))

    def shard_candidates(self, logits, params, records, first_id: int = 0, want_sums: bool = False,
                         stream=None):
        """lily_shard_candidates: this shard's records (uint8 [rows, 520]) of `logits`."""
        rows = logits.shape[0]
        keep = []
        a = self._shard_args(rows, params, None, keep)
        a.logits, a.logits_dtype, a.logits_ld = _ptr(logits), _dtype_code(logits), _ld(logits)
        self._check(lib().lily_shard_candidates(self._h, _stream_ptr(stream), C.byref(a), first_id,
                                                int(want_sums), _ptr(records)))

    def lmhead_shard_candidates(self, weights, scales, hidden, params, records, first_id: int = 0,
                                want_sums: bool = False, stream=None, biases=None, code_bits: int = 8):
        """lily_lmhead_shard_candidates: head projection into the handle's own
        logits, then this shard's records (needs lmhead=True at creation)."""
        rows = int(hidden.shape[0])
        keep = []
        a = self._shard_args(rows, params, None, keep)
        hd = self._head(weights, scales, biases, code_bits=code_bits)
        self._check(lib().lily_lmhead_shard_candidates(self._h, _stream_ptr(stream), C.byref(hd),
                                                       _ptr(hidden), _ld(hidden), C.byref(a),
                                                       first_id, int(want_sums), _ptr(records)))

    def merge_draw(self, gathered, params, out_ids, *, uniforms=None, steps=None, out_status=None,
                   kept_n=None, kept_ids=None, kept_probs=None, out_lse=None, stream=None):
        """lily_merge_draw over `gathered` (uint8 [n_shards, rows, 520])."""
        n_shards, rows = int(gathered.shape[0]), int(gathered.shape[1])
        keep = []
        a = self._shard_args(rows, params, steps, keep)
        a.uniforms = _ptr(uniforms)
        a.out_ids = _ptr(out_ids)
        a.out_status = _ptr(out_status)
        if kept_n is not None:
            a.kept_n, a.kept_ids, a.kept_probs = _ptr(kept_n), _ptr(kept_ids), _ptr(kept_probs)
            a.kept_ld = _ld(kept_ids)
        self._check(lib().lily_merge_draw(self._h, _stream_ptr(stream), _ptr(gathered), n_shards,
                                          rows, C.byref(a), _ptr(out_lse)))

    def shard_publish(self, exchange: "PeerExchangeStruct", records, step: int, stream=None):
        """lily_shard_publish: this rank's records (uint8 [rows, 520]) into every rank's buffer."""
        self._check(lib().lily_shard_publish(self._h, _stream_ptr(stream), C.byref(exchange), _ptr(records),
                                             int(records.shape[0]), step))

    def merge_draw_peer(self, exchange: "PeerExchangeStruct", step: int, params, out_ids, *, records=None,
                        uniforms=None, steps=None, out_status=None, kept_n=None, kept_ids=None, kept_probs=None,
                        out_lse=None, stream=None):
        """lily_merge_draw_peer: a row's block publishes this rank's record of the row
        (`records`, uint8 [rows, 520]; None: published already), waits for every
        rank's flag of the row, then merges."""
        rows = len(params)
        keep = []
        a = self._shard_args(rows, params, steps, keep)
        a.uniforms = _ptr(uniforms)
        a.out_ids = _ptr(out_ids)
        a.out_status = _ptr(out_status)
        if kept_n is not None:
            a.kept_n, a.kept_ids, a.kept_probs = _ptr(kept_n), _ptr(kept_ids), _ptr(kept_probs)
            a.kept_ld = _ld(kept_ids)
        self._check(lib().lily_merge_draw_peer(self._h, _stream_ptr(stream), C.byref(exchange), _ptr(records),
                                               step, C.byref(a), _ptr(out_lse)))

    def argmax_batch(self, logits, out_ids, stream=None):
        """src/kernels/elementwise.rs:297-308 argmax_f32 for each row."""
        rows = logits.shape[0] if logits.dim() == 2 else 1
        ld = _ld(logits)
        self._check(lib().lily_argmax_batch(self._h, _stream_ptr(stream), _ptr(logits),
                                            _dtype_code(logits), ld, rows, _ptr(out_ids)))

    def spec_verify(self, target_logits, params: SamplingParams, draft_ids, out_ids,
                    out_accepted, *, mode=SPEC_REJECTION, q_dense=None, q_ids=None,
                    q_probs=None, q_n=None, u_accept=None, u_resid=None, step0=0,
                    history_ids=None, count_slot=None, out_status=None, stream=None):
        a = SpecArgs()
        a.struct_size = C.sizeof(SpecArgs)
        a.m = target_logits.shape[0]
        a.target_logits = _ptr(target_logits)
        a.logits_dtype = _dtype_code(target_logits)
        a.mode = mode
        a.logits_ld = _ld(target_logits)
        a.params = C.cast(C.pointer(params), C.c_void_p)
        a.draft_ids = _ptr(draft_ids)
        if q_dense is not None:
            a.q_dense = _ptr(q_dense)
            a.q_ld = _ld(q_dense)
        a.q_ids, a.q_probs, a.q_n = _ptr(q_ids), _ptr(q_probs), _ptr(q_n)
        a.u_accept, a.u_resid = _ptr(u_accept), _ptr(u_resid)
        a.step0 = step0
        if history_ids is not None:
            a.history_ids = _ptr(history_ids)
            a.history_len = history_ids.numel()
        slot = None
        if count_slot is not None:
            slot = C.c_uint32(count_slot)
            a.count_slot = C.cast(C.pointer(slot), C.c_void_p)
        a.out_ids, a.out_accepted, a.out_status = _ptr(out_ids), _ptr(out_accepted), _ptr(out_status)
        self._check(lib().lily_spec_verify(self._h, _stream_ptr(stream), C.byref(a)))

    def spec_accept(self, draws, ids, ctrl, pos0: int, ratio: int, chain: int, stride: int = 4,
                    stream=None):
        """src/kernels/spec.rs:52-91."""
        self._check(lib().lily_spec_accept(self._h, _stream_ptr(stream), _ptr(draws), _ptr(ids),
                                           draws.numel(), _ptr(ctrl), pos0, ratio, chain, stride))


NOALLOC_MAX_ROWS = 8


def sample_batch_noalloc(vocab, logits, params, out_ids, *, uniforms=None, steps=None,
                         history_ids=None, history_len=None, bias_ids=None, bias_vals=None,
                         bias_len=None, ban_ids=None, ban_len=None, forced_ids=None,
                         out_status=None, kept_n=None, kept_ids=None, kept_probs=None,
                         stream=None):
    """lily_sample_batch_noalloc: the draw of `SamplerScratch.sample_batch` for hosts
    that may not allocate device memory. No handle: the kernel's scratch is static
    device storage inside the library, shared by all calls (calls that overlap on
    the GPU race on it). `params` is a list of at most NOALLOC_MAX_ROWS
    SamplingParams; histogram slots and a frequency penalty over a history list
    are not available here."""
    rows = logits.shape[0] if logits.dim() == 2 else 1
    a = SampleArgs()
    a.struct_size = C.sizeof(SampleArgs)
    a.rows = rows
    a.logits = _ptr(logits)
    a.logits_dtype = _dtype_code(logits)
    a.logits_ld = _ld(logits)
    arr = (SamplingParams * rows)(*params)
    a.params = C.cast(arr, C.c_void_p)
    sarr = None
    if steps is not None:
        sarr = (C.c_uint32 * rows)(*[int(s) for s in steps])
        a.steps = C.cast(sarr, C.c_void_p)
    a.uniforms = _ptr(uniforms)
    if history_ids is not None:
        a.history_ids, a.history_len = _ptr(history_ids), _ptr(history_len)
        a.history_ld = _ld(history_ids)
    if bias_ids is not None:
        a.bias_ids, a.bias_vals, a.bias_len = _ptr(bias_ids), _ptr(bias_vals), _ptr(bias_len)
        a.bias_ld = _ld(bias_ids)
    if ban_ids is not None:
        a.ban_ids, a.ban_len = _ptr(ban_ids), _ptr(ban_len)
        a.ban_ld = _ld(ban_ids)
    a.forced_ids = _ptr(forced_ids)
    a.out_ids, a.out_status = _ptr(out_ids), _ptr(out_status)
    if kept_n is not None:
        a.kept_n, a.kept_ids, a.kept_probs = _ptr(kept_n), _ptr(kept_ids), _ptr(kept_probs)
        a.kept_ld = _ld(kept_ids)
    err = C.create_string_buffer(256)
    st = lib().lily_sample_batch_noalloc(_stream_ptr(stream), vocab, C.byref(a), err, len(err))
    if st != OK:
        raise LilyError(st, err.value.decode("utf-8", "replace"))


# -- single-row conveniences with the reference's call shapes ------------------

def sample_f32(logits, scratch: SamplerScratch, params: SamplingParams, step: int, out,
               history_ids=None, stream=None):
    """src/kernels/sample.rs:373-387: one draw from `logits` [V] into `out` [1]."""
    import torch

    hl = None
    if history_ids is not None:
        hl = torch.tensor([history_ids.numel()], dtype=torch.int32, device=logits.device)
    scratch.sample_batch(logits.view(1, -1), [params], out, steps=[step],
                         history_ids=None if history_ids is None else history_ids.view(1, -1),
                         history_len=hl, stream=stream)


def ctrl_words(chain: int, stride: int = 4) -> int:
    """src/kernels/spec.rs:37-39."""
    return (2 + 3 * chain) * stride


def _load_sibling(name: str):
    spec = importlib.util.spec_from_file_location(f"{__name__}.{name}",
                                                  os.path.join(_HERE, f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
