"""Per-block phase times of one sampler launch, from the time stamps the
kernel leaves with LILY_FLAG_PHASE_CLOCKS (the counterpart of the reference's
LILY_KERNEL_PROFILE, src/metal.rs:140-198).

    python phase_trace.py b4 [step ...]     # the 4-row server batch
    python phase_trace.py b256 [rows]       # the 256-row batch, or its first rows (summary)

Stamps are nanoseconds of the GPU's global timer, so stamps of different
blocks of a launch can be compared with each other.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NAMES = ["start", "bitmaps", "lists", "pass 2 / stream", "adjust + select", "merge", "sort", "end",
         "first threshold", "pass 1", "pass 1 met", "maxima", "search", "threshold set",
         "threshold taken", "collected", "entry"]
ENTRY = 16
# The small-batch kernel (a cluster of eight blocks per row) leaves its own stamps;
# block r of a row's cluster is listed as "slice" r.
CLUSTER_NAMES = {0: "slice loaded, cluster running", 1: "history counted", 2: "lists, penalties, block maximum",
                 3: "cluster maximum", 9: "histogram", 4: "cluster barrier", 5: "histograms summed, k-th bin",
                 10: "candidates placed in every block", 6: "cluster barrier", 11: "ranked within bins",
                 8: "cluster barrier", 7: "draw written"}
CLUSTER_ORDER = [16, 0, 1, 2, 3, 9, 4, 5, 10, 6, 11, 8, 7]
# The order in which a block of the two-pass route reaches its stamps.
ORDER = [16, 0, 1, 14, 15, 9, 10, 11, 12, 13, 8, 2, 3, 4, 5, 6, 7]


def _device_batch(torch, lily, x):
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).view(dt)).cuda()
    kw = dict(uniforms=t(x.uniforms, np.float32))
    if x.history is not None:
        kw.update(history_ids=t(x.history, np.int32), history_len=t(x.history_len, np.int32))
    if x.bias_ids is not None:
        kw.update(bias_ids=t(x.bias_ids, np.int32), bias_vals=t(x.bias_vals, np.float32),
                  bias_len=t(x.bias_len, np.int32))
    if x.ban_ids is not None:
        kw.update(ban_ids=t(x.ban_ids, np.int32), ban_len=t(x.ban_len, np.int32))
    if x.forced is not None:
        kw.update(forced_ids=t(x.forced, np.int32))
    logits = t(x.logits, np.int16).view(torch.bfloat16) if x.bf16 else t(x.logits, np.float32)
    return logits, [lily.SamplingParams(**p) for p in x.params], kw


def trace(torch, lily, scratch, x, launches: int = 3):
    """Runs `x` `launches` times; returns the stamps of the last launch,
    int64 [rows, slices, phases] (0 where a block did not pass)."""
    logits, params, kw = _device_batch(torch, lily, x)
    out = torch.zeros(len(params), dtype=torch.int32, device="cuda")
    clk = None
    for _ in range(launches):
        scratch.sample_batch(logits, params, out, **kw)
        clk = scratch.read_phase_clocks()
    return clk


def segments(stamps, cluster=False):
    """[(phase name, microseconds since the previous stamp)] of one block."""
    order, names = (CLUSTER_ORDER, CLUSTER_NAMES) if cluster else (ORDER, NAMES)
    out, prev = [], float(stamps[order[0]])
    for i in order[1:]:
        if stamps[i] != 0:
            out.append((names[i], (float(stamps[i]) - prev) / 1e3))
            prev = float(stamps[i])
    return out


def main(argv) -> None:
    import torch

    import lily_b200 as lily
    import workloads as w

    which = argv[1] if len(argv) > 1 else "b4"
    if which == "b4":
        steps = [int(a) for a in argv[2:]] or [0, 3]
        scratch = lily.SamplerScratch(w.VOCAB, max_rows=4, max_list=128, phase_clocks=True)
        for step in steps:
            x = w.config2_step(step)
            clk = trace(torch, lily, scratch, x)
            t0 = clk[:, :, ENTRY][clk[:, :, ENTRY] != 0].min()
            print(f"step {step}: (T, top_k, top_p) per row",
                  [(p.get("temperature"), p.get("top_k"), p.get("top_p")) for p in x.params])
            for r in range(clk.shape[0]):
                for sl in range(clk.shape[1]):
                    c = clk[r, sl]
                    if c[ENTRY] == 0:
                        continue
                    last = max(int(v) for v in c)
                    # (The 4-row batch goes to the small-batch kernel: eight blocks per row.)
                    cluster = clk.shape[0] <= 8 and c[13] == 0 and c[12] == 0
                    print(f"  row {r} block {sl}: enters {(c[ENTRY] - t0) / 1e3:5.1f}, leaves "
                          f"{(last - t0) / 1e3:5.1f} us after the launch's first block | " +
                          " | ".join(f"{n} {us:.1f}" for n, us in segments(c, cluster)))
    else:
        rows = int(argv[2]) if len(argv) > 2 else 256
        scratch = lily.SamplerScratch(w.VOCAB, max_rows=256, phase_clocks=True)
        clk = trace(torch, lily, scratch, w.config4_batch(rows=rows), launches=4)
        live = clk[clk[:, :, ENTRY] != 0].astype(np.float64)
        t0 = live[:, ENTRY].min()
        print("blocks", len(live))
        print(f"  block entry after the first block's: mean {(live[:, ENTRY] - t0).mean() / 1e3:6.2f} us"
              f"  max {(live[:, ENTRY] - t0).max() / 1e3:6.2f}")
        prev = ENTRY
        for i in ORDER[1:]:
            ok = (live[:, i] != 0) & (live[:, prev] != 0)
            if ok.any():
                d = (live[ok, i] - live[ok, prev]) / 1e3
                at = (live[ok, i] - t0) / 1e3
                q = np.percentile(at, [10, 50, 90])
                print(f"  {NAMES[i]:18s} mean {d.mean():6.2f} us  max {d.max():6.2f}   reached at "
                      f"{at.mean():6.2f} (mean), p10 / p50 / p90 {q[0]:.2f} / {q[1]:.2f} / {q[2]:.2f}, "
                      f"{at.max():6.2f} (last block)")
                prev = i
        tot = (live[:, 7] - live[:, ENTRY]) / 1e3
        print(f"  block lifetime mean {tot.mean():.1f} us, max {tot.max():.1f}; "
              f"last block ends {(live[:, 7].max() - t0) / 1e3:.1f} us after the first block enters")
    scratch.close()


if __name__ == "__main__":
    main(sys.argv)
