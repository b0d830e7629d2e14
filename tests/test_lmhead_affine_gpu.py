"""The LM head in the reference's own storage (MLX affine, 8 and 4 bits: unsigned
codes, a bf16 scale and bias per 64 columns; src/weights.rs:21-36), on the GPU
through the C ABI, against the oracle's restatement of the reference's test
for gemv_quant (tests/unit/kernels/quant.rs:368-434: dequantise, then an fp32
product; tolerance 2e-2 + 2e-2 |x|). Bit for bit where every sum is exact."""
from __future__ import annotations

import numpy as np
import pytest

import oracle
from gpu_util import np_u32, t_f32
from test_lmhead_gpu import _bf16, _check_against_oracle, _records, _to_bf16_bits

pytestmark = pytest.mark.gpu


def _widen(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _affine_inputs(rng, tokens, hidden, rows, exact=False, bits=8):
    """codes as the reference stores them: U32 [rows, hidden * bits / 32], low code first."""
    codes = rng.integers(0, 2 ** 32, size=(rows, hidden * bits // 32), dtype=np.uint64).astype(np.uint32)
    groups = hidden // 64
    if exact:
        h = _to_bf16_bits(rng.integers(-4, 5, size=(tokens, hidden)).astype(np.float32))
        sc = 2.0 ** rng.integers(-6, -2, size=(rows, groups)).astype(np.float32)
        s = _to_bf16_bits(sc)
        b = _to_bf16_bits(sc * rng.integers(-(1 << (bits - 1)), 1, size=(rows, groups)).astype(np.float32))
    else:
        # tests/unit/kernels/quant.rs:370-385, 423: the reference's own distributions.
        h = _to_bf16_bits(rng.uniform(-1.0, 1.0, size=(tokens, hidden)).astype(np.float32))
        s = _to_bf16_bits(rng.uniform(0.005, 0.1, size=(rows, groups)).astype(np.float32))
        b = _to_bf16_bits(rng.uniform(-1.0, 0.0, size=(rows, groups)).astype(np.float32))
    return h, codes, s, b


def _gpu_affine(torch, scratch, h, codes, s, b, bits=8):
    rows, tokens = codes.shape[0], h.shape[0]
    q = torch.from_numpy(codes.view(np.uint8).reshape(rows, -1)).cuda()  # the same memory, as bytes
    out = torch.full((tokens, rows), float("nan"), dtype=torch.float32, device="cuda")
    scratch.lmhead_logits(q, _bf16(torch, s), _bf16(torch, h), out, biases=_bf16(torch, b), code_bits=bits)
    torch.cuda.synchronize()
    assert scratch.status() == 0
    return out.cpu().numpy()


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("tokens,hidden,rows", [(64, 512, 256), (5, 1024, 1000), (1, 2048, 4096),
                                                (33, 512, 40_000)])
def test_affine_head_is_exact_where_the_sums_are(cuda, lily, tokens, hidden, rows, bits):
    rng = np.random.default_rng([81, tokens, hidden, rows, bits])
    h, codes, s, b = _affine_inputs(rng, tokens, hidden, rows, exact=True, bits=bits)
    scratch = lily.SamplerScratch(rows, max_rows=64)
    got = _gpu_affine(cuda, scratch, h, codes, s, b, bits)
    want = oracle.lmhead_affine(h, codes, s, b, 64, bits)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    scratch.close()


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("tokens,hidden,rows", [(1, 2048, 256), (17, 4096, 777), (64, 1024, 2048)])
def test_affine_head_matches_the_dequantised_product(cuda, lily, tokens, hidden, rows, bits):
    """bits = 4: the storage gemv_q4_bf16 reads (src/kernels/metal/quant.metal:44-66)."""
    rng = np.random.default_rng([82, tokens, hidden, rows, bits])
    h, codes, s, b = _affine_inputs(rng, tokens, hidden, rows, bits=bits)
    scratch = lily.SamplerScratch(rows, max_rows=64)
    got = _gpu_affine(cuda, scratch, h, codes, s, b, bits)
    want = oracle.lmhead_affine(h, codes, s, b, 64, bits)
    # The reference's bound for its own kernel (cpu_ref::assert_close, 2e-2, 2e-2).
    assert np.all(np.abs(got - want) <= 2e-2 + 2e-2 * np.abs(want))
    # And far inside it: against the product in binary64 of the same dequantised weights.
    w = oracle.dequant_affine(codes, _widen(s), _widen(b), rows, hidden, 64, bits).astype(np.float64)
    exact = _widen(h).astype(np.float64) @ w.T
    scale = np.abs(exact).max()
    assert np.abs(got - exact).max() <= 2e-5 * scale, (np.abs(got - exact).max(), scale)
    assert np.abs(want - exact).max() <= 2e-4 * scale
    scratch.close()


def test_affine_head_refuses_what_it_cannot_do(cuda, lily):
    torch = cuda
    rng = np.random.default_rng(83)
    h, codes, s, b = _affine_inputs(rng, 4, 512, 256)
    scratch = lily.SamplerScratch(256, max_rows=64)
    q = torch.from_numpy(codes.view(np.uint8).reshape(256, -1)).cuda()
    out = torch.zeros((4, 256), dtype=torch.float32, device="cuda")
    bias = _bf16(torch, np.concatenate([b.reshape(-1), b.reshape(-1)[:1]]))
    with pytest.raises(lily.LilyError) as e:  # biases not 16-byte aligned
        scratch.lmhead_logits(q, _bf16(torch, s), _bf16(torch, h), out, biases=bias[1:])
    assert e.value.code == lily.ERR_ARG
    scratch.close()


@pytest.mark.parametrize("bits", [8, 4])
def test_affine_head_then_sharded_draw(cuda, lily, bits):
    """Two vocabulary shards of an affine head, each through the fused call,
    merged; the oracle draws from the logits the GPU head produced."""
    torch = cuda
    rng = np.random.default_rng([84, bits])
    tokens, hidden, vocab, n_shards = 16, 1024, 8192, 2
    per = vocab // n_shards
    h, codes, s, b = _affine_inputs(rng, tokens, hidden, vocab, bits=bits)
    q = torch.from_numpy(codes.view(np.uint8).reshape(vocab, -1)).cuda()
    sd, bd, hd = _bf16(torch, s), _bf16(torch, b), _bf16(torch, h)
    plist = [dict(temperature=0.7, top_k=40, top_p=0.95, seed=900 + t) for t in range(tokens)]
    params = [lily.SamplingParams(**p) for p in plist]
    uniforms = np.array([oracle.uniform_for(900 + t, 0) for t in range(tokens)], dtype=np.float32)
    rec = _records(torch, n_shards, tokens)
    shard = lily.SamplerScratch(per, max_rows=tokens, lmhead=True)
    for i in range(n_shards):
        lo, hi = i * per, (i + 1) * per
        shard.lmhead_shard_candidates(q[lo:hi], sd[lo:hi], hd, params, rec[i], first_id=lo,
                                      want_sums=True, biases=bd[lo:hi], code_bits=bits)
    out = torch.full((tokens,), -1, dtype=torch.int32, device="cuda")
    status = torch.full((tokens,), -1, dtype=torch.int32, device="cuda")
    kept_n = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    kept_ids = torch.zeros((tokens, 64), dtype=torch.int32, device="cuda")
    kept_probs = torch.zeros((tokens, 64), dtype=torch.float32, device="cuda")
    lse = torch.zeros(tokens, dtype=torch.float32, device="cuda")
    shard.merge_draw(rec, params, out, uniforms=t_f32(torch, uniforms), out_status=status,
                     kept_n=kept_n, kept_ids=kept_ids, kept_probs=kept_probs, out_lse=lse)
    torch.cuda.synchronize()
    assert shard.status() == 0
    whole = lily.SamplerScratch(vocab, max_rows=tokens)
    lf = _gpu_affine(cuda, whole, h, codes, s, b, bits)
    got = (np_u32(out), np_u32(status), np_u32(kept_n), np_u32(kept_ids), kept_probs.cpu().numpy(),
           lse.cpu().numpy())
    _check_against_oracle(lf, plist, uniforms, got)
    shard.close()
    whole.close()
