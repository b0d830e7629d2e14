"""Seeded synthetic inputs for the five benchmark configurations.

Shapes, sizes and value distributions follow the configurations the
benchmark names; no public dataset or checkpoint is involved. Everything is
numpy (PCG64), so the CPU checker and the GPU path read identical bytes.
bf16 tensors are carried as uint16 bit patterns (round-to-nearest-even of the
f32 draw).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

VOCAB = 151_936


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns, round to nearest even (no NaN inputs here)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def uniform_for(seed: int, step: int) -> np.float32:
    """The reference's draw for (seed, step): src/kernels/sample.rs:435-441."""
    m = (1 << 64) - 1
    z = (seed + step * 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z ^= z >> 31
    return np.float32(z >> 40) * np.float32(1.0 / 16777216.0)


def zipf_logits(rng: np.random.Generator, rows: int, vocab: int, sigma: float = 3.0,
                s: float = 1.1) -> np.ndarray:
    """N(0, sigma^2) plus a Zipf(s) bump s*ln(vocab/rank) over a seeded
    permutation of the vocabulary (one permutation per row)."""
    out = np.empty((rows, vocab), dtype=np.float32)
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    bump = (s * np.log(vocab / ranks)).astype(np.float32)
    for r in range(rows):
        perm = rng.permutation(vocab)
        row = (rng.standard_normal(vocab, dtype=np.float32) * np.float32(sigma))
        row[perm] += bump
        out[r] = row
    return out


@dataclass
class Batch:
    """One step's inputs for lily_sample_batch (host arrays)."""

    logits: np.ndarray                  # [B, V] float32, or uint16 bf16 bits
    bf16: bool
    params: list                        # B dicts of SamplingParams fields
    uniforms: np.ndarray                # [B] float32
    history: np.ndarray | None = None   # [B, H] uint32
    history_len: np.ndarray | None = None
    bias_ids: np.ndarray | None = None  # [B, L] uint32
    bias_vals: np.ndarray | None = None
    bias_len: np.ndarray | None = None
    ban_ids: np.ndarray | None = None
    ban_len: np.ndarray | None = None
    forced: np.ndarray | None = None    # [B] int32, -1 = none
    meta: dict = field(default_factory=dict)

    def logits_f32(self) -> np.ndarray:
        return bf16_bits_to_f32(self.logits) if self.bf16 else self.logits


def config1_step(step: int, vocab: int = VOCAB, seed: int = 1001, greedy: bool = False) -> Batch:
    """Single row: f32 logits N(0, 2.5^2) with 20 seeded ids spiked by +12,
    history of 4096 uniform ids, T 0.7 / top-k 20 / top-p 0.95 / repetition
    1.05, or the greedy pass."""
    rng = np.random.default_rng([seed, step])
    logits = (rng.standard_normal(vocab, dtype=np.float32) * np.float32(2.5))
    spikes = rng.choice(vocab, size=min(20, vocab), replace=False)
    logits[spikes] += np.float32(12.0)
    history = rng.integers(0, vocab, size=4096, dtype=np.uint32)
    p = dict(temperature=0.0 if greedy else 0.7, top_k=1 if greedy else 20,
             top_p=1.0 if greedy else 0.95, repetition_penalty=1.0 if greedy else 1.05,
             seed=seed)
    u = np.array([uniform_for(seed, step)], dtype=np.float32)
    return Batch(logits[None, :], False, [p], u, history[None, :],
                 np.array([4096], dtype=np.uint32), meta={"step": step})


def config2_step(step: int, vocab: int = VOCAB, seed: int = 2002, rows: int = 4,
                 history: int = 8192) -> Batch:
    """Server batch: bf16 rows, mixed params, presence 0.5 / frequency 0.2
    over 8192-id histories, one forced end-of-think id on row 2, 8 banned ids
    on every row, 64 bias entries of +-5 per row."""
    rng = np.random.default_rng([seed, step])
    logits = to_bf16_bits(zipf_logits(rng, rows, vocab))
    temps = [0.0, 0.6, 0.8, 1.0]
    ks = [0, 20, 40]
    ps = [1.0, 0.95, 0.8]
    params = []
    for r in range(rows):
        params.append(dict(temperature=temps[(r + step) % 4], top_k=ks[(r + step) % 3],
                           top_p=ps[(r + 2 * step) % 3], presence_penalty=0.5,
                           frequency_penalty=0.2, seed=seed + r))
    # Histories as a decode would see them: skewed towards frequent tokens.
    hist = (rng.zipf(1.3, size=(rows, history)) % vocab).astype(np.uint32)
    ban = rng.choice(vocab, size=8, replace=False).astype(np.uint32)
    ban_ids = np.tile(ban, (rows, 1))
    bias_ids = np.stack([rng.choice(vocab, size=64, replace=False) for _ in range(rows)]).astype(np.uint32)
    bias_vals = (rng.integers(0, 2, size=(rows, 64)).astype(np.float32) * 10.0 - 5.0)
    forced = np.full(rows, -1, dtype=np.int32)
    if rows > 2:
        forced[2] = int(rng.integers(0, vocab))
    u = np.array([uniform_for(seed + r, step) for r in range(rows)], dtype=np.float32)
    return Batch(logits, True, params, u, hist, np.full(rows, history, dtype=np.uint32),
                 bias_ids, bias_vals, np.full(rows, 64, dtype=np.uint32), ban_ids,
                 np.full(rows, 8, dtype=np.uint32), forced, meta={"step": step})


@dataclass
class SpecStep:
    target: np.ndarray      # [m, V] uint16 bf16 bits
    q: np.ndarray           # [m-1, V] float32 draft probabilities
    draft_ids: np.ndarray   # [m-1] uint32
    u_accept: np.ndarray    # [m] float32
    u_resid: np.ndarray     # [m-1] float32
    params: dict

    def target_f32(self) -> np.ndarray:
        return bf16_bits_to_f32(self.target)


def config3_step(step: int, vocab: int = VOCAB, seed: int = 3003, drafts: int = 2,
                 greedy: bool = False) -> SpecStep:
    """Speculative verification: target bf16 [drafts+1, V]; draft-head
    probabilities = softmax of N(0, 2^2) logits correlated 0.8 with the
    target; draft ids sampled from them; uniforms from (seed, step) with the
    residual draw on the step's high-bit domain."""
    rng = np.random.default_rng([seed, step])
    m = drafts + 1
    z = rng.standard_normal((m, vocab), dtype=np.float32)
    target = to_bf16_bits(z * np.float32(2.0))
    noise = rng.standard_normal((drafts, vocab), dtype=np.float32)
    dl = (np.float32(0.8) * z[:drafts] + np.float32(0.6) * noise) * np.float32(2.0)
    dl64 = dl.astype(np.float64)
    dl64 -= dl64.max(axis=1, keepdims=True)
    e = np.exp(dl64)
    q = (e / e.sum(axis=1, keepdims=True)).astype(np.float32)
    draft_ids = np.empty(drafts, dtype=np.uint32)
    for j in range(drafts):
        if greedy:
            draft_ids[j] = np.argmax(q[j])
        else:
            cdf = np.cumsum(q[j].astype(np.float64))
            draft_ids[j] = min(int(np.searchsorted(cdf, rng.random() * cdf[-1], side="right")),
                               vocab - 1)
    base = step * m
    u_accept = np.array([uniform_for(seed, base + j) for j in range(m)], dtype=np.float32)
    u_resid = np.array([uniform_for(seed, (base + j) | 0x80000000) for j in range(drafts)],
                       dtype=np.float32)
    p = dict(temperature=0.0 if greedy else 1.0, top_k=1 if greedy else 20,
             top_p=1.0 if greedy else 0.95, seed=seed)
    return SpecStep(target, q, draft_ids, u_accept, u_resid, p)


def config4_batch(rows: int = 256, vocab: int = VOCAB, seed: int = 4004,
                  history: int = 32768, step: int = 0) -> Batch:
    """Large-batch throughput: bf16 rows as in the server batch; top-k 50,
    top-p 0.9, min-p 0.05, T 0.8, repetition 1.1 over 32768-id histories."""
    rng = np.random.default_rng([seed, step])
    logits = to_bf16_bits(zipf_logits(rng, rows, vocab))
    params = [dict(temperature=0.8, top_k=50, top_p=0.9, min_p=0.05, repetition_penalty=1.1,
                   seed=seed + r) for r in range(rows)]
    hist = rng.integers(0, vocab, size=(rows, history), dtype=np.uint32)
    u = np.array([uniform_for(seed + r, step) for r in range(rows)], dtype=np.float32)
    return Batch(logits, True, params, u, hist, np.full(rows, history, dtype=np.uint32),
                 meta={"step": step})


@dataclass
class LmHead:
    hidden: np.ndarray   # [T, H] uint16 bf16 bits
    weight: np.ndarray   # [N, H] int8
    scales: np.ndarray   # [N, H / group] uint16 bf16 bits
    group: int
    params: dict
    uniforms: np.ndarray


def config5(tokens: int = 64, hidden: int = 4096, vocab: int = 262_144, group: int = 64,
            seed: int = 5005) -> LmHead:
    """Vocab-sharded fused LM head: hidden bf16 N(0,1), int8 symmetric weights,
    bf16 scales U(0.002, 0.02) per 64 columns; top-k 40 / top-p 0.95 / T 0.7."""
    rng = np.random.default_rng(seed)
    h = to_bf16_bits(rng.standard_normal((tokens, hidden), dtype=np.float32))
    w = rng.integers(-127, 128, size=(vocab, hidden), dtype=np.int8)
    s = to_bf16_bits(rng.uniform(0.002, 0.02, size=(vocab, hidden // group)).astype(np.float32))
    u = np.array([uniform_for(seed + t, 0) for t in range(tokens)], dtype=np.float32)
    return LmHead(h, w, s, group, dict(temperature=0.7, top_k=40, top_p=0.95, seed=seed), u)
