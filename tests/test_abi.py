"""The C-ABI library loads here (no GPU) and exports every symbol the headers
declare; the host-only entry points are checked against the oracle."""
import ctypes as C
import glob
import os
import re

import numpy as np

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(lily_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported(lily):
    L = lily.lib()
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(L, name), f"{name} is declared in include/ but not exported"


def test_struct_layouts_match_the_header(lily):
    assert C.sizeof(lily.SamplingParams) == 40
    assert C.sizeof(oracle.Params) == 40
    assert lily.SamplingParams.seed.offset == 32
    assert lily.lib().lily_abi_version() == 1


def test_layouts_of_the_later_structs(lily):
    """lily_lmhead_t with its code width, lily_peer_exchange_t, and the size of an
    exchange buffer: a flag word per (rank, row) rounded up to 256 bytes, then two
    slots of n_shards x max_rows records of 520 bytes."""
    assert C.sizeof(lily.LmHead) == 48 and lily.LmHead.code_bits.offset == 40
    assert C.sizeof(lily.PeerExchangeStruct) == 16 + 16 * 8
    assert lily.PeerExchangeStruct.buffers.offset == 16
    L = lily.lib()
    for n, rows in ((1, 1), (2, 24), (8, 64), (16, 64)):
        flags = (n * rows * 4 + 255) // 256 * 256
        assert L.lily_peer_buffer_bytes(n, rows) == flags + 2 * n * rows * 520
    # Host-side refusals need no GPU.
    buf, handle = C.c_void_p(), (C.c_ubyte * 64)()
    assert L.lily_peer_buffer_create(0, 0, 8, C.byref(buf), handle) == lily.ERR_ARG
    assert L.lily_peer_buffer_create(0, 17, 8, C.byref(buf), handle) == lily.ERR_ARG
    assert L.lily_peer_buffer_open(0, None, C.byref(buf)) == lily.ERR_ARG


def test_uniform_for_matches_the_oracle(lily):
    for seed in (0, 7, 0xDEADBEEF, (1 << 64) - 1):
        for step in (0, 1, 77, 0x40000001, 0x80000002):
            assert lily.uniform_for(seed, step) == oracle.uniform_for(seed, step)
    assert lily.draft_step(5) == 5 | 0x40000000
    assert lily.residual_step(5) == 5 | 0x80000000


def test_params_helpers_match_the_reference_rules(lily):
    # src/kernels/sample.rs:34-95
    g = lily.SamplingParams.greedy()
    assert g.is_greedy() and not g.uses_penalties()
    assert g.effective() == (1.0, 1)
    p = lily.SamplingParams(temperature=0.8, top_k=0, top_p=0.9)
    assert not p.is_greedy() and p.effective()[1] == 1024
    assert lily.SamplingParams(temperature=0.8, top_k=5000).effective()[1] == 1024
    assert lily.SamplingParams(temperature=0.8, top_k=1).is_greedy()
    assert lily.SamplingParams(repetition_penalty=1.1).uses_penalties()
    d = lily.draft_params(lily.SamplingParams(temperature=0.7, top_k=20, presence_penalty=0.5,
                                              frequency_penalty=0.2, repetition_penalty=1.3, seed=9))
    assert not d.uses_penalties() and d.top_k == 20 and d.seed == 9
    assert abs(d.temperature - 0.7) < 1e-7
    for bad in (dict(temperature=-1.0), dict(top_p=0.0), dict(min_p=2.0),
                dict(repetition_penalty=0.0), dict(presence_penalty=float("nan"))):
        try:
            lily.SamplingParams(**bad).validate()
        except lily.LilyError as e:
            assert e.code == lily.ERR_PARAMS
        else:
            raise AssertionError(f"{bad} accepted")


def test_device_calls_fail_loudly_without_a_gpu(lily):
    import torch

    if torch.cuda.is_available():
        return
    h = C.c_void_p()
    st = lily.lib().lily_sampler_create(0, 1000, 1, 16, 16, 0, C.byref(h))
    assert st == lily.ERR_CUDA and not h
    try:
        lily.SamplerScratch(1000, device=0)
    except lily.LilyError as e:
        assert e.code == lily.ERR_CUDA
    else:
        raise AssertionError("a sampler was created without a GPU")


def test_no_product_file_touches_the_oracle():
    pkg = os.path.join(ROOT, "lily-qwen3.8-flash-next_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f
