"""ctypes binding of the CPU oracle (oracle/lily_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg, never by the shipped sampler.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liblily_oracle.so")

K_CAP = 1024
OK, ERR_NAN, ERR_NONFINITE, ERR_PARAMS, ERR_ARG = 0, 1, 2, -1, -2


class Params(C.Structure):
    """src/kernels/sample.rs:19-31 as a 40-byte POD."""

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


def params(temperature=0.0, top_k=1, top_p=1.0, min_p=0.0, presence_penalty=0.0,
           frequency_penalty=0.0, repetition_penalty=1.0, seed=0) -> Params:
    """Defaults are SamplingParams::greedy() (src/kernels/sample.rs:34-45)."""
    return Params(temperature, top_k, top_p, min_p, presence_penalty,
                  frequency_penalty, repetition_penalty, 0, seed)


def build(force: bool = False) -> str:
    """Compiles the oracle with gcc (oracle/Makefile)."""
    src = os.path.join(_HERE, "lily_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "lily_oracle.h")))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None

_u32p = C.POINTER(C.c_uint32)
_f32p = C.POINTER(C.c_float)


def _ptr(a, typ):
    if a is None:
        return None
    return a.ctypes.data_as(typ)


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.lo_expf.restype = C.c_float
        L.lo_expf.argtypes = [C.c_float]
        L.lo_uniform_for.restype = C.c_float
        L.lo_uniform_for.argtypes = [C.c_uint64, C.c_uint32]
        L.lo_draft_step.restype = C.c_uint32
        L.lo_draft_step.argtypes = [C.c_uint32]
        L.lo_residual_step.restype = C.c_uint32
        L.lo_residual_step.argtypes = [C.c_uint32]
        L.lo_validate.argtypes = [C.POINTER(Params)]
        L.lo_is_greedy.argtypes = [C.POINTER(Params)]
        L.lo_uses_penalties.argtypes = [C.POINTER(Params)]
        L.lo_effective.argtypes = [C.POINTER(Params), _f32p, _u32p]
        L.lo_counts_from_history.argtypes = [_u32p, C.c_uint32, C.c_uint32, _u32p]
        L.lo_widen_bf16.argtypes = [C.POINTER(C.c_uint16), C.c_uint64, _f32p]
        L.lo_adjust.argtypes = [_f32p, C.c_uint32, C.POINTER(Params), _u32p, _u32p, _f32p,
                                C.c_uint32, _u32p, C.c_uint32, _f32p]
        L.lo_sample.argtypes = [_f32p, C.c_uint32, C.POINTER(Params), _u32p, _u32p, _f32p,
                                C.c_uint32, _u32p, C.c_uint32, C.c_float, C.c_int, _u32p,
                                _u32p, _f32p, _f32p, _f32p, _u32p, _u32p]
        L.lo_argmax.restype = C.c_uint32
        L.lo_argmax.argtypes = [_f32p, C.c_uint32]
        L.lo_spec_draw.restype = C.c_uint32
        L.lo_spec_draw.argtypes = [_u32p, _f32p, _f32p, C.c_uint32, _f32p, _u32p, _f32p,
                                   C.c_uint32, C.c_uint32, C.c_float, C.c_float]
        L.lo_spec_verify.argtypes = [_f32p, C.c_uint32, C.c_uint64, C.c_uint32,
                                     C.POINTER(Params), _u32p, _u32p, _f32p, C.c_uint64,
                                     _u32p, _f32p, _u32p, _f32p, _f32p, _u32p, _u32p]
        L.lo_spec_accept.restype = C.c_uint32
        L.lo_spec_accept.argtypes = [_u32p, _u32p, C.c_uint32]
        L.lo_lmhead_int8.argtypes = [C.POINTER(C.c_uint16), C.c_uint32, C.c_uint32,
                                     C.POINTER(C.c_int8), C.POINTER(C.c_uint16), C.c_uint32,
                                     C.c_uint32, C.c_uint32, _f32p, C.c_uint64]
        _lib = L
    return _lib


# ---------------------------------------------------------------- helpers --

def expf(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    f = lib().lo_expf
    return np.array([f(float(v)) for v in x], dtype=np.float32)


def uniform_for(seed: int, step: int) -> float:
    return float(lib().lo_uniform_for(seed & 0xFFFFFFFFFFFFFFFF, step & 0xFFFFFFFF))


def widen_bf16(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 (exact)."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def counts_from_history(history, vocab: int) -> np.ndarray:
    history = np.ascontiguousarray(history, dtype=np.uint32)
    counts = np.zeros(vocab, dtype=np.uint32)
    lib().lo_counts_from_history(_ptr(history, _u32p), history.size, vocab, _ptr(counts, _u32p))
    return counts


def adjust(logits, p: Params, counts=None, bias_ids=None, bias_vals=None, ban_ids=None):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    out = np.empty_like(logits)
    bi, bv, nb, ba, nn = _lists(bias_ids, bias_vals, ban_ids)
    if counts is not None:
        counts = np.ascontiguousarray(counts, dtype=np.uint32)
    st = lib().lo_adjust(_ptr(logits, _f32p), logits.size, C.byref(p), _ptr(counts, _u32p),
                         _ptr(bi, _u32p), _ptr(bv, _f32p), nb, _ptr(ba, _u32p), nn,
                         _ptr(out, _f32p))
    return st, out


def _lists(bias_ids, bias_vals, ban_ids):
    bi = bv = ba = None
    nb = nn = 0
    if bias_ids is not None and len(bias_ids):
        bi = np.ascontiguousarray(bias_ids, dtype=np.uint32)
        bv = np.ascontiguousarray(bias_vals, dtype=np.float32)
        nb = bi.size
    if ban_ids is not None and len(ban_ids):
        ba = np.ascontiguousarray(ban_ids, dtype=np.uint32)
        nn = ba.size
    return bi, bv, nb, ba, nn


class Draw:
    """Result of one oracle draw."""

    __slots__ = ("status", "token", "kept_ids", "kept_w", "kept_cum", "kept_prob", "near_tie")

    def __init__(self, status, token, ids, w, cum, prob, tie):
        self.status, self.token = status, token
        self.kept_ids, self.kept_w, self.kept_cum, self.kept_prob = ids, w, cum, prob
        self.near_tie = tie


def sample(logits, p: Params, uniform: float, counts=None, history=None, bias_ids=None,
           bias_vals=None, ban_ids=None, mode: int = 1) -> Draw:
    """One draw from f32 logits (bf16 inputs are widened by the caller)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    vocab = logits.size
    if counts is None and history is not None:
        counts = counts_from_history(history, vocab)
    if counts is not None:
        counts = np.ascontiguousarray(counts, dtype=np.uint32)
    bi, bv, nb, ba, nn = _lists(bias_ids, bias_vals, ban_ids)
    ids = np.zeros(K_CAP, dtype=np.uint32)
    w = np.zeros(K_CAP, dtype=np.float32)
    cum = np.zeros(K_CAP, dtype=np.float32)
    prob = np.zeros(K_CAP, dtype=np.float32)
    out = C.c_uint32(0xFFFFFFFF)
    n = C.c_uint32(0)
    tie = C.c_uint32(0)
    st = lib().lo_sample(_ptr(logits, _f32p), vocab, C.byref(p), _ptr(counts, _u32p),
                         _ptr(bi, _u32p), _ptr(bv, _f32p), nb, _ptr(ba, _u32p), nn,
                         C.c_float(uniform), mode, C.byref(out), _ptr(ids, _u32p),
                         _ptr(w, _f32p), _ptr(cum, _f32p), _ptr(prob, _f32p), C.byref(n),
                         C.byref(tie))
    k = n.value
    return Draw(st, out.value, ids[:k].copy(), w[:k].copy(), cum[:k].copy(), prob[:k].copy(),
                tie.value)


def argmax(x) -> int:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return int(lib().lo_argmax(_ptr(x, _f32p), x.size))


def spec_draw(d: Draw, draft: int, u_accept: float, u_resid: float, q_dense=None,
              q_ids=None, q_probs=None) -> int:
    qd = qi = qp = None
    nq = 0
    if q_dense is not None:
        qd = np.ascontiguousarray(q_dense, dtype=np.float32)
    else:
        qi = np.ascontiguousarray(q_ids, dtype=np.uint32)
        qp = np.ascontiguousarray(q_probs, dtype=np.float32)
        nq = qi.size
    return int(lib().lo_spec_draw(_ptr(d.kept_ids, _u32p), _ptr(d.kept_w, _f32p),
                                  _ptr(d.kept_cum, _f32p), d.kept_ids.size, _ptr(qd, _f32p),
                                  _ptr(qi, _u32p), _ptr(qp, _f32p), nq, draft,
                                  C.c_float(u_accept), C.c_float(u_resid)))


def spec_verify(target, p: Params, draft_ids, u_accept, u_resid, q_dense=None, q_ids=None,
                q_probs=None, q_n=None, counts=None):
    """One verify step over target f32 [m, V]; returns (status, ids[m], accepted)."""
    target = np.ascontiguousarray(target, dtype=np.float32)
    m, vocab = target.shape
    draft_ids = np.ascontiguousarray(draft_ids, dtype=np.uint32)
    ua = np.ascontiguousarray(u_accept, dtype=np.float32)
    ur = np.ascontiguousarray(u_resid, dtype=np.float32)
    qd = qi = qp = qn = None
    q_ld = 0
    if q_dense is not None:
        qd = np.ascontiguousarray(q_dense, dtype=np.float32)
        q_ld = qd.shape[1]
    elif q_ids is not None:
        qi = np.ascontiguousarray(q_ids, dtype=np.uint32)
        qp = np.ascontiguousarray(q_probs, dtype=np.float32)
        qn = np.ascontiguousarray(q_n, dtype=np.uint32)
        assert qi.shape[1] == K_CAP and qp.shape[1] == K_CAP
    if counts is not None:
        assert counts.dtype == np.uint32 and counts.flags.c_contiguous
    out = np.zeros(m, dtype=np.uint32)
    acc = C.c_uint32(0)
    st = lib().lo_spec_verify(_ptr(target, _f32p), m, vocab, vocab, C.byref(p),
                              _ptr(counts, _u32p), _ptr(draft_ids, _u32p), _ptr(qd, _f32p),
                              q_ld, _ptr(qi, _u32p), _ptr(qp, _f32p), _ptr(qn, _u32p),
                              _ptr(ua, _f32p), _ptr(ur, _f32p), _ptr(out, _u32p),
                              C.byref(acc))
    return st, out, acc.value


def spec_accept(draws, ids) -> int:
    draws = np.ascontiguousarray(draws, dtype=np.uint32)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    return int(lib().lo_spec_accept(_ptr(draws, _u32p), _ptr(ids, _u32p), draws.size))


def lmhead_int8(hidden_bf16, w, scales_bf16, group: int, n_begin: int, n_end: int) -> np.ndarray:
    hidden_bf16 = np.ascontiguousarray(hidden_bf16, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.int8)
    scales_bf16 = np.ascontiguousarray(scales_bf16, dtype=np.uint16)
    tokens, hidden = hidden_bf16.shape
    out = np.zeros((tokens, w.shape[0]), dtype=np.float32)
    lib().lo_lmhead_int8(hidden_bf16.ctypes.data_as(C.POINTER(C.c_uint16)), tokens, hidden,
                         w.ctypes.data_as(C.POINTER(C.c_int8)),
                         scales_bf16.ctypes.data_as(C.POINTER(C.c_uint16)), group, n_begin,
                         n_end, _ptr(out, _f32p), out.shape[1])
    return out


def lmhead_int8_all(hidden_bf16, w, scales_bf16, group: int, threads: int | None = None) -> np.ndarray:
    """lmhead_int8 over every row of the head, bands of rows on `threads` host
    threads (the C call releases the GIL); the sums of a logit do not depend on
    the band it falls in."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    hidden_bf16 = np.ascontiguousarray(hidden_bf16, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.int8)
    scales_bf16 = np.ascontiguousarray(scales_bf16, dtype=np.uint16)
    tokens, hidden = hidden_bf16.shape
    rows = w.shape[0]
    out = np.zeros((tokens, rows), dtype=np.float32)
    threads = threads or os.cpu_count() or 1
    band = max(256, -(-rows // (threads * 8)))
    f = lib().lo_lmhead_int8

    def one(lo):
        f(hidden_bf16.ctypes.data_as(C.POINTER(C.c_uint16)), tokens, hidden,
          w.ctypes.data_as(C.POINTER(C.c_int8)), scales_bf16.ctypes.data_as(C.POINTER(C.c_uint16)),
          group, lo, min(rows, lo + band), _ptr(out, _f32p), out.shape[1])

    with ThreadPoolExecutor(max_workers=threads) as pool:
        list(pool.map(one, range(0, rows, band)))
    return out


def dequant_affine(codes, scales, biases, rows: int, cols: int, group: int, bits: int) -> np.ndarray:
    """tests/support/cpu_ref.rs:402-430: MLX affine codes -> f32 [rows, cols]."""
    codes = np.ascontiguousarray(codes, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    biases = np.ascontiguousarray(biases, dtype=np.float32)
    assert codes.size == rows * cols * bits // 32 and scales.size == biases.size == rows * cols // group
    out = np.zeros((rows, cols), dtype=np.float32)
    f = lib().lo_dequant_affine
    f.argtypes = [_u32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _f32p]
    f.restype = None
    f(_ptr(codes, _u32p), _ptr(scales, _f32p), _ptr(biases, _f32p), rows, cols, group, bits,
      _ptr(out, _f32p))
    return out


def gemm_nt(a, b) -> np.ndarray:
    """tests/support/cpu_ref.rs:50-62: a [m, k] times b [n, k] transposed, fp32 in index order."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    m, k = a.shape
    n = b.shape[0]
    assert b.shape[1] == k
    out = np.zeros((m, n), dtype=np.float32)
    f = lib().lo_gemm_nt
    f.argtypes = [_f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p]
    f.restype = None
    f(_ptr(a, _f32p), _ptr(b, _f32p), m, k, n, _ptr(out, _f32p))
    return out


def lmhead_affine(hidden_bf16, codes, scales_bf16, biases_bf16, group: int, bits: int) -> np.ndarray:
    """The head in MLX affine storage as the reference's tests state it
    (tests/unit/kernels/quant.rs:418-434): bf16 hidden states times the
    dequantised weights. codes uint32 [rows, hidden * bits / 32], scales and
    biases bf16 bits [rows, hidden / group]. Returns f32 [tokens, rows]."""
    hidden_bf16 = np.ascontiguousarray(hidden_bf16, dtype=np.uint16)
    codes = np.ascontiguousarray(codes, dtype=np.uint32)
    rows = codes.shape[0]
    hidden = hidden_bf16.shape[1]
    widen = lambda bits16: (np.ascontiguousarray(bits16, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
    w = dequant_affine(codes, widen(scales_bf16), widen(biases_bf16), rows, hidden, group, bits)
    return gemm_nt(widen(hidden_bf16), w)
