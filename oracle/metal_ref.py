"""ctypes binding of the reference's Metal sampler run on the CPU.

The shader (src/kernels/metal/sample.metal of the reference checkout) is
compiled as C++ under the stand-in headers of oracle/metal_shim/ by
oracle/Makefile's `_ref/liblily_metal_shim.so` target, straight from where the
checkout lies: none of its text enters this repository. The library only
exists where a checkout was present at build time; `available()` says so.

TEST INFRASTRUCTURE ONLY: it pins the CPU oracle (oracle/lily_oracle.c) to the
kernel the reference ships, within the tolerance the reference's own tests
give that kernel against its CPU sampler (tests/unit/kernels/sample.rs:113-115,
402-403).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_ref", "liblily_metal_shim.so")
_SHADER = os.path.join("src", "kernels", "metal", "sample.metal")

K_CAP = 1024
PLAIN, DRAFT, SPEC = 0, 1, 2
OK, ERR_ARG, ERR_ARGMAX_ROUTE, ERR_DEADLOCK = 0, 1, 2, 3

_u32p = C.POINTER(C.c_uint32)
_f32p = C.POINTER(C.c_float)
_lib = None


def reference_dir() -> str:
    """Where the reference checkout lies (LILY_REFERENCE overrides the default)."""
    return os.environ.get("LILY_REFERENCE", "/root/reference")


def build(force: bool = False) -> str | None:
    """Builds the library if a reference checkout is at hand; returns its path,
    or None where there is neither a checkout nor a library built earlier."""
    shader = os.path.join(reference_dir(), _SHADER)
    if os.path.exists(shader):
        sources = [shader] + [os.path.join(_HERE, "metal_shim", f) for f in ("metal_stdlib", "shim_driver.h")]
        stale = (not os.path.exists(_LIB_PATH)
                 or any(os.path.getmtime(_LIB_PATH) < os.path.getmtime(s) for s in sources))
        if force or stale:
            subprocess.run(["make", "-C", _HERE, "_ref/liblily_metal_shim.so", "-B",
                            f"REFERENCE={reference_dir()}"], check=True, capture_output=True)
    return _LIB_PATH if os.path.exists(_LIB_PATH) else None


def available() -> bool:
    return build() is not None


def lib():
    global _lib
    if _lib is None:
        path = build()
        if path is None:
            raise RuntimeError("the Metal sampler's CPU build is absent and no reference checkout is at hand")
        L = C.CDLL(path)
        L.lily_metal_shim_draw.restype = C.c_int
        L.lily_metal_shim_draw.argtypes = [
            _f32p, C.c_uint32, _u32p, C.c_float, C.c_uint32, C.c_float, C.c_float, C.c_float, C.c_float,
            C.c_float, C.c_uint64, C.c_uint32, C.c_int, C.c_uint32, C.c_int, _u32p, _f32p, _u32p, _u32p,
            _u32p, _f32p, C.POINTER(C.c_int)]
        L.lily_metal_shim_uniform.restype = C.c_float
        L.lily_metal_shim_uniform.argtypes = [C.c_uint64, C.c_uint32]
        _lib = L
    return _lib


def _ptr(a, typ):
    return None if a is None else a.ctypes.data_as(typ)


class Dist:
    """A draft's exported kept distribution (src/kernels/sample.rs:184-199)."""

    def __init__(self):
        self.ids = np.zeros(K_CAP, dtype=np.uint32)
        self.probs = np.zeros(K_CAP, dtype=np.float32)
        self.n = np.zeros(1, dtype=np.uint32)

    def kept(self):
        n = int(self.n[0])
        return self.ids[:n].copy(), self.probs[:n].copy()


def uniform_for(seed: int, step: int) -> float:
    return float(lib().lily_metal_shim_uniform(seed, step))


def draw(logits, counts, *, temperature, top_k, top_p=1.0, min_p=0.0, presence_penalty=0.0,
         frequency_penalty=0.0, repetition_penalty=1.0, seed=0, step=0, mode=PLAIN, dist: Dist | None = None,
         draft: int | None = None, two_phase: bool = True, local_groups: int = 64, want_adjusted=False):
    """One draw as src/kernels/sample.rs:250-372 encodes it. `counts` (u32 [V])
    is read for the penalties and bumped at the drawn id when penalties are in
    use, as the shader does. Returns (token, used_two_phase[, adjusted])."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    assert counts.dtype == np.uint32 and counts.flags.c_contiguous and counts.size == logits.size
    out = np.full(1, 0xFFFFFFFF, dtype=np.uint32)
    adjusted = np.zeros(logits.size, dtype=np.float32) if want_adjusted else None
    d = np.array([0 if draft is None else draft], dtype=np.uint32)
    used = C.c_int(0)
    st = lib().lily_metal_shim_draw(
        _ptr(logits, _f32p), logits.size, _ptr(counts, _u32p), temperature, top_k, top_p, min_p,
        presence_penalty, frequency_penalty, repetition_penalty, seed, step, int(two_phase), local_groups,
        mode, _ptr(dist.ids if dist else None, _u32p), _ptr(dist.probs if dist else None, _f32p),
        _ptr(dist.n if dist else None, _u32p), _ptr(d, _u32p), _ptr(out, _u32p), _ptr(adjusted, _f32p),
        C.byref(used))
    if st != OK:
        raise RuntimeError(f"lily_metal_shim_draw: status {st}")
    res = (int(out[0]), bool(used.value))
    return res + (adjusted,) if want_adjusted else res
