#!/usr/bin/env python
"""Benchmark of the sampling hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: the large-batch configuration, B=256 rows of bf16 logits at
V=151,936 with 32,768-id histories per row (top-k 50, top-p 0.9, min-p 0.05,
T 0.8, repetition 1.1). A step is one pass of the sampler over one batch.
With N GPUs the 256 rows are split evenly: rank r draws rows
[r * 256 / N, (r + 1) * 256 / N) of every batch (rows are independent: no
collective), so `value` is 256 rows per step time and the scaling is strong.
`weak_scaling` has the other figure: every rank drawing 256 rows of its own.

`value`   rows/s with inputs resident in HBM (CUDA events around K steps).
`e2e`     the same through the C ABI with HOST buffers: pinned host logits,
          histories and uniforms copied in, token ids copied out, per step.
`roofline` algorithmic bytes (logits + history read once) / kernel time
          against the measured HBM copy bandwidth.
`cpu_baseline` the CPU oracle (a port of the reference's CPU sampler) timed
          on this host's cores on a bounded sample.
`--impl reference` times only that CPU port, on all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np

ROWS = 256
HISTORY = 32_768
NB = 4  # distinct resident batches rotated through, 445 MB in all (> the 126 MB L2)
METRIC = "sampled rows/s at B=256,V=151,936"
UNIT = "rows/s"


def workload_config(world: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    alg_bytes = ROWS * (151_936 * 2 + HISTORY * 4)
    return {"workload": "large-batch B=256 V=151936 bf16 history=32768 "
                        "(top-k 50, top-p 0.9, min-p 0.05, T 0.8, repetition 1.1)",
            "rows_per_gpu": ROWS // world, "global_rows": ROWS, "vocab": 151_936, "history": HISTORY,
            "logits_dtype": "bf16", "parallelism": f"rows x{world}, no collective",
            "l2": f"{NB} resident batches rotated ({NB * alg_bytes / 1e6:.0f} MB > 126 MB L2)"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def ncu_traffic(key="stream_rows_kernel_b256_dram_bytes_per_launch"):
    """DRAM bytes per launch of a kernel from the committed ncu summary, if
    one has been recorded."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get(key)
    return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during a timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


class CpuSampler:
    """The CPU oracle over the rows of one batch on `threads` host threads
    (ctypes releases the GIL). The thread pool, the parameter structs and the
    widened logits are made once: a timed pass is only the sampler."""

    def __init__(self, batch, threads: int, mode: int = 1):
        from concurrent.futures import ThreadPoolExecutor

        import oracle

        self.oracle = oracle
        self.batch = batch
        self.mode = mode
        self.rows = batch.logits.shape[0]
        self.logits = [oracle.widen_bf16(batch.logits[r]) for r in range(self.rows)]
        self.params = [oracle.params(**p) for p in batch.params]
        self.pool = ThreadPoolExecutor(max_workers=threads)

    def _one(self, r):
        b = self.batch
        return self.oracle.sample(self.logits[r], self.params[r], float(b.uniforms[r]),
                                  history=b.history[r, :b.history_len[r]], mode=self.mode).token

    def one_pass(self):
        return list(self.pool.map(self._one, range(self.rows)))

    def rows_per_s(self, min_seconds: float):
        done = 0
        t0 = time.perf_counter()
        while True:
            self.one_pass()
            done += self.rows
            if time.perf_counter() - t0 >= min_seconds:
                break
        dt = time.perf_counter() - t0
        return done / dt, done, dt

    def close(self):
        self.pool.shutdown()


def run_reference(args):
    """The reference arm: the CPU port of the reference's sampler on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import workloads as w
    import oracle

    oracle.build()
    cores = os.cpu_count() or 1
    batch = w.config4_batch(rows=ROWS, history=HISTORY)
    cpu = CpuSampler(batch, cores)
    # One step = one 256-row batch through the CPU sampler.
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        cpu.one_pass()
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    cpu.close()
    total = sum(times)
    value = ROWS * len(times) / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded numpy; shapes and distributions of the large-batch configuration)",
        "config": workload_config(max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{len(times)} steps of one 256-row batch, partial-selection "
                                   "variant of the CPU sampler (identical outputs to the full sort)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--b4-steps", type=int, default=300)
    ap.add_argument("--lmhead-steps", type=int, default=30,
                    help="steps of the vocab-sharded LM head + sampling leg (0 = skip)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    import lily_b200 as lily
    import workloads as w

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler has no CPU fallback")
    lily.lib()  # fails loudly if the CUDA library has not been built
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    vocab = w.VOCAB
    import lily_b200.shard as sh

    rows_here = sh.row_range(ROWS, world, rank)       # this rank's rows of every 256-row batch
    lo, hi_row = rows_here.start, rows_here.stop
    n_here = hi_row - lo
    # Seeded host batches, the same on every rank (pinned: the end-to-end leg copies from them).
    host = []
    for b in range(NB):
        batch = w.config4_batch(rows=ROWS, history=HISTORY, seed=4004, step=b)
        lg = torch.from_numpy(batch.logits.view(np.int16)).pin_memory()
        hi = torch.from_numpy(batch.history.view(np.int32)).pin_memory()
        un = torch.from_numpy(batch.uniforms).pin_memory()
        host.append((batch, lg, hi, un))
    params = [lily.SamplingParams(**p) for p in host[0][0].params]
    hist_len = torch.full((ROWS,), HISTORY, dtype=torch.int32, device=dev)
    resident = [(lg.to(dev).view(torch.bfloat16), hi.to(dev), un.to(dev)) for _, lg, hi, un in host]
    raw = np.frombuffer(b"".join(bytes(p) for p in params), dtype=np.uint8).copy()
    d_params = torch.from_numpy(raw).to(dev)
    out = torch.zeros(ROWS, dtype=torch.int32, device=dev)
    scratch = lily.SamplerScratch(vocab, max_rows=ROWS, max_history=HISTORY, device=local)
    stream = torch.cuda.current_stream()

    # The argument block of each resident batch is built once: the timed loop
    # is then one C-ABI call per step, so that the host keeps ahead of the GPU.
    def prepare(first, last):
        return [scratch.prepare_sample_batch(lg[first:last], d_params[40 * first:40 * last], out[first:last],
                                             uniforms=un[first:last], history_ids=hi[first:last],
                                             history_len=hist_len[first:last], params_on_device=True)
                for lg, hi, un in resident]

    split = prepare(lo, hi_row)                        # the 256 rows split over the ranks
    whole = prepare(0, ROWS) if world > 1 else split   # every rank its own 256 rows

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def timed(prepared, steps):
        """Exactly `steps` steps between two events, nothing else in the stream (an
        event between two launches would keep a launch from being set up while
        the one before it drains). Max over ranks."""
        e_first, e_last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e_first.record(stream)
        for i in range(steps):
            scratch.sample_prepared(prepared[i % NB], stream=stream)
        e_last.record(stream)
        barrier()
        return max_over_ranks(e_first.elapsed_time(e_last))

    # ---- device-resident throughput -------------------------------------
    for i in range(args.warmup):
        scratch.sample_prepared(split[i % NB], stream=stream)
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    time.sleep(0.3)
    total_ms = timed(split, args.steps)
    # The same steps once more with an event after every launch: the spread of
    # single launches (each then pays its own start-up).
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record(stream)
    for i in range(args.steps):
        scratch.sample_prepared(split[i % NB], stream=stream)
        ev[i + 1].record(stream)
    barrier()
    per_launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    weak = None
    if world > 1:
        for i in range(3):
            scratch.sample_prepared(whole[i % NB], stream=stream)
        weak_ms = timed(whole, args.steps)
        weak = {"value": world * ROWS * args.steps / (weak_ms * 1e-3), "unit": UNIT,
                "us_per_step": weak_ms * 1e3 / args.steps, "rows_per_gpu": ROWS,
                "scaling": "weak: every rank draws 256 rows of its own per step"}
    # Keep the GPU busy a little longer so that nvidia-smi sees it under load.
    t_end = time.time() + 1.0
    i = 0
    while time.time() < t_end:
        scratch.sample_prepared(split[i % NB], stream=stream)
        i += 1
    torch.cuda.synchronize()
    clock_info = clocks.stop()
    ms_per_step = total_ms / args.steps
    value = ROWS * args.steps / (total_ms * 1e-3)
    assert scratch.status(stream) == lily.OK

    # ---- end to end through the C ABI with host buffers ------------------
    # Every rank copies in its own rows of the step's batch and copies its ids out.
    d_lg = torch.empty_like(resident[0][0][lo:hi_row])
    d_hi = torch.empty_like(resident[0][1][lo:hi_row])
    d_un = torch.empty_like(resident[0][2][lo:hi_row])
    h_out = torch.zeros(n_here, dtype=torch.int32).pin_memory()
    params_here = params[lo:hi_row]

    def step_e2e(i):
        _, lg, hi, un = host[i % NB]
        d_lg.view(torch.int16).copy_(lg[lo:hi_row], non_blocking=True)
        d_hi.copy_(hi[lo:hi_row], non_blocking=True)
        d_un.copy_(un[lo:hi_row], non_blocking=True)
        scratch.sample_batch(d_lg, params_here, out[lo:hi_row], uniforms=d_un, history_ids=d_hi,
                             history_len=hist_len[lo:hi_row], stream=stream)
        h_out.copy_(out[lo:hi_row], non_blocking=True)

    e2e_steps = max(10, min(args.steps, 50))
    for i in range(3):
        step_e2e(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(e2e_steps):
        step_e2e(i)
    e1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    e2e_value = ROWS * e2e_steps / (e2e_ms * 1e-3)
    h2d_rank = n_here * vocab * 2 + n_here * HISTORY * 4 + n_here * 4 + n_here * 40
    h2d = ROWS * vocab * 2 + ROWS * HISTORY * 4 + ROWS * 4 + ROWS * 40
    d2h = ROWS * 4
    check = host[(e2e_steps - 1) % NB][0]

    # ---- p50 latency of the 4-row server batch ----------------------------
    b4 = None
    if rank == 0 and args.b4_steps > 0:
        cs = ClockSampler(local)
        cs.start()
        b4 = b4_latency(torch, lily, w, dev, stream, args.b4_steps)
        b4["clocks"] = cs.stop()

    # ---- vocab-sharded 8-bit LM head + sampling (every rank takes part) -----
    lm = None
    if args.lmhead_steps > 0:
        cs = ClockSampler(local)
        cs.start()
        lm = lmhead_sharded(torch, dist, lily, dev, stream, world, rank, args.lmhead_steps)
        lm["clocks"] = cs.stop()

    # ---- roofline ----------------------------------------------------------
    # Algorithmic bytes of one launch on this GPU: its rows' logits and history, read once.
    alg_bytes = n_here * (vocab * 2 + HISTORY * 4)
    kernel_ms = total_ms / args.steps  # average launch duration over the timed region (one launch per step)
    peak, peak_kind = peaks()
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    kernel_name = ("stream_rows_kernel<bf16> (one block per row)" if n_here * 8 > 148
                   else "cluster_rows_kernel<bf16> (a cluster of eight blocks per row)")
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": ncu_traffic() if world == 1 else None,
                "peak_kind": peak_kind, "kernel": kernel_name, "kernel_ms": kernel_ms,
                "single_launch_ms_mean": statistics.mean(per_launch_ms),
                "single_launch_ms_p50": statistics.median(per_launch_ms),
                "algorithmic_bytes_per_launch": alg_bytes, "rows_per_launch": n_here}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle

        oracle.build()
        cores = os.cpu_count() or 1
        sampler = CpuSampler(host[0][0], cores)
        v, done, dt = sampler.rows_per_s(args.cpu_seconds)
        sampler.close()
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{done} rows (the 256-row batch repeated for {dt:.1f} s), "
                         "partial-selection variant of the CPU sampler"}
        # The last end-to-end step's tokens, checked against the CPU port.
        want = [oracle.sample(oracle.widen_bf16(check.logits[r]), oracle.params(**check.params[r]),
                              float(check.uniforms[r]), history=check.history[r]).token
                for r in range(0, ROWS, 16)]
        got = h_out.numpy().view(np.uint32)[::16].tolist()
        assert got == want, "bench: the end-to-end tokens differ from the CPU port"

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (seeded numpy; shapes and distributions of the large-batch configuration)",
            "config": workload_config(world),
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps,
                    "h2d_bytes_per_step_per_gpu": h2d_rank,
                    "h2d_gbs_per_gpu": h2d_rank / (e2e_ms / e2e_steps * 1e-3) / 1e9,
                    "note": "bound by the host-to-device copy of the step's logits and histories "
                            "(all GPUs of the box copy through the same host)"},
            "gpu_launches": args.steps, "clocks": clock_info, "weak_scaling": weak, "latency_b4": b4,
            "lmhead_sharded": lm,
            "us_per_step": ms_per_step * 1e3,
        }
        print(json.dumps(line), flush=True)
    scratch.close()
    if world > 1:
        dist.destroy_process_group()


def lmhead_sharded(torch, dist, lily, dev, stream, world, rank, steps):
    """The vocab-sharded configuration: hidden bf16 [64, 4096] against an int8
    head [262144, 4096] with bf16 scales per 64 columns, the vocabulary cut
    into `world` shards (strong scaling: the head is fixed, a rank holds
    1/world of it). A step is, on every rank: the head over the rank's rows and
    its 520-byte candidate records, one all-gather of the records, the merged
    draw (top-k 40, top-p 0.95, T 0.7). Weights are seeded random int8 made on
    the device; a rank whose shard is smaller than the L2 rotates two copies."""
    import lily_b200.shard as sh

    tokens, hidden, vocab = 64, 4096, 262_144
    per = vocab // world
    g = torch.Generator(device=dev)
    g.manual_seed(5005 + rank)
    copies = 1 if per * hidden > 600e6 else 2
    ws = [torch.randint(-127, 128, (per, hidden), dtype=torch.int8, device=dev, generator=g)
          for _ in range(copies)]
    sc = (torch.rand((per, hidden // 64), device=dev, generator=g) * 0.018 + 0.002).to(torch.bfloat16)
    gh = torch.Generator(device=dev)
    gh.manual_seed(5005)  # the same hidden states on every rank
    h = torch.randn((tokens, hidden), device=dev, generator=gh).to(torch.bfloat16)
    params = [lily.SamplingParams(temperature=0.7, top_k=40, top_p=0.95, seed=5005 + t)
              for t in range(tokens)]
    u = torch.tensor([lily.uniform_for(5005 + t, 0) for t in range(tokens)], dtype=torch.float32,
                     device=dev)
    scratch = lily.SamplerScratch(per, max_rows=tokens, lmhead=True, device=dev.index)
    rec = torch.empty((tokens, sh.RECORD_BYTES), dtype=torch.uint8, device=dev)
    out = torch.zeros(tokens, dtype=torch.int32, device=dev)
    logits = torch.empty((tokens, per), dtype=torch.float32, device=dev)

    # More than one rank: the records travel by the ranks' own stores into each
    # other's memory (lily_shard_publish / lily_merge_draw_peer); the all-gather
    # through NCCL is timed beside it.
    exchange, exchange_note = None, "one rank"
    if world > 1:
        exchange_note = "peer stores + flags (lily_merge_draw_peer)"
        try:
            exchange = sh.PeerExchange(dev.index, max_rows=tokens)
        except Exception as e:  # no peer access between the GPUs of this box: every rank alike
            exchange_note = f"NCCL all-gather (peer memory unavailable: {e})"
        ok = torch.tensor([1 if exchange is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0 and exchange is not None:
            exchange.close()
            exchange, exchange_note = None, "NCCL all-gather (peer memory unavailable on another rank)"

    def step(i):
        sh.sharded_lmhead_draw(scratch, ws[i % copies], sc, h, params, out, first_id=rank * per,
                               uniforms=u, records=rec, want_sums=True, stream=stream, exchange=exchange)

    def step_nccl(i):
        sh.sharded_lmhead_draw(scratch, ws[i % copies], sc, h, params, out, first_id=rank * per,
                               uniforms=u, records=rec, want_sums=True, stream=stream)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        for i in range(3):
            fn(i)
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(n):
            fn(i)
        e1.record(stream)
        sync()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / n

    step_ms = timed(step, steps)
    nccl_ms, same = None, True
    if world > 1:
        step(0)
        torch.cuda.synchronize()
        by_peer = out.clone()
        nccl_ms = timed(step_nccl, steps)
        step_nccl(0)
        torch.cuda.synchronize()
        same = bool(torch.equal(by_peer, out))
    head_ms = timed(lambda i: scratch.lmhead_logits(ws[i % copies], sc, h, logits, stream=stream), steps)
    # The same head read as the reference's MLX affine 8-bit storage (the
    # bytes as unsigned codes, plus a bias per 64 columns).
    bi = (-torch.rand((per, hidden // 64), device=dev, generator=g)).to(torch.bfloat16)
    affine_ms = timed(lambda i: scratch.lmhead_logits(ws[i % copies], sc, h, logits, stream=stream,
                                                      biases=bi), steps)
    # And in MLX affine 4-bit storage: the same bytes read as twice as many columns
    # (a head of 2 * hidden columns; its hidden states and groups are synthetic too).
    h4 = torch.cat([h, h], dim=1).contiguous()
    sc4 = torch.cat([sc, sc], dim=1).contiguous()
    bi4 = torch.cat([bi, bi], dim=1).contiguous()
    logits4 = torch.empty((tokens, per), dtype=torch.float32, device=dev)
    q4_ms = None
    if 2 * hidden <= 8192:
        q4_ms = timed(lambda i: scratch.lmhead_logits(ws[i % copies].view(torch.uint8), sc4, h4, logits4,
                                                      stream=stream, biases=bi4, code_bits=4), steps)
    assert scratch.status(stream) == lily.OK
    agree = True
    if world > 1:
        every = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(every, out)
        agree = all(bool(torch.equal(every[0], e)) for e in every)
    if exchange is not None:
        exchange.close()
    scratch.close()
    head_bytes = per * hidden + per * (hidden // 64) * 2 + tokens * hidden * 2
    peak, peak_kind = peaks()
    gbs = head_bytes / (head_ms * 1e-3) / 1e9
    return {"workload": "hidden bf16 [64,4096] x int8 head [262144,4096], bf16 scales per 64 columns, "
                        f"{world} vocabulary shard(s); top-k 40, top-p 0.95, T 0.7",
            "n_gpus": world, "scaling": "strong", "us_per_step": step_ms * 1e3,
            "exchange": exchange_note,
            "us_per_step_nccl_allgather": None if nccl_ms is None else nccl_ms * 1e3,
            "peer_equals_nccl": same,
            "rows_per_s": tokens / (step_ms * 1e-3), "steps": steps,
            "head_kernel_us": head_ms * 1e3, "head_bytes_per_gpu": head_bytes,
            "head_gbs_per_gpu": gbs, "head_frac_of_hbm": gbs / peak, "peak_kind": peak_kind,
            "head_traffic_1gpu": ncu_traffic("lmhead_int8_kernel_dram_bytes_per_launch"),
            "affine_head_us": affine_ms * 1e3,
            "affine_head_frac_of_hbm": (head_bytes + per * (hidden // 64) * 2) / (affine_ms * 1e-3) / 1e9 / peak,
            "affine4_head_us": None if q4_ms is None else q4_ms * 1e3,
            "affine4_head_workload": f"the same {per} x {hidden} bytes as 4-bit codes of a head of {2 * hidden} columns",
            "affine4_head_frac_of_hbm": None if q4_ms is None else
            (per * hidden + per * (2 * hidden // 64) * 4 + tokens * 2 * hidden * 2) / (q4_ms * 1e-3) / 1e9 / peak,
            "allgather_bytes_per_rank": tokens * sh.RECORD_BYTES, "ranks_agree": agree,
            "l2": "one 1.07 GB shard" if copies == 1 else "two weight copies rotated"}


def b4_latency(torch, lily, w, dev, stream, steps):
    """p50 / p90 microseconds per step of the 4-row server batch (mixed params,
    8192-id histories, bias, ban and one forced row), inputs resident."""
    vocab = w.VOCAB
    nb = 16
    batches = []
    for b in range(nb):
        x = w.config2_step(b)
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).view(dt)).to(dev)
        batches.append(dict(
            logits=t(x.logits, np.int16).view(torch.bfloat16), params=[lily.SamplingParams(**p) for p in x.params],
            uniforms=t(x.uniforms, np.float32), history_ids=t(x.history, np.int32),
            history_len=t(x.history_len, np.int32), bias_ids=t(x.bias_ids, np.int32),
            bias_vals=t(x.bias_vals, np.float32), bias_len=t(x.bias_len, np.int32),
            ban_ids=t(x.ban_ids, np.int32), ban_len=t(x.ban_len, np.int32),
            forced_ids=t(x.forced, np.int32)))
    s = lily.SamplerScratch(vocab, max_rows=4, max_list=64, device=dev.index)
    out = torch.zeros(4, dtype=torch.int32, device=dev)

    # The argument blocks are built once, as a decode loop that draws from the
    # same buffers every step would (host params are still staged every call).
    prepared = []
    for b in batches:
        kw = dict(b)
        lg, ps = kw.pop("logits"), kw.pop("params")
        prepared.append(s.prepare_sample_batch(lg, ps, out, **kw))

    def go(i):
        s.sample_prepared(prepared[i % nb], stream=stream)

    for i in range(20):
        go(i)
    torch.cuda.synchronize()
    us = []
    for i in range(steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        go(i)
        b.record(stream)
        b.synchronize()
        us.append(a.elapsed_time(b) * 1e3)
    # Back-to-back, no host sync between steps: what a pipelined decode loop sees.
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        go(i)
    e1.record(stream)
    torch.cuda.synchronize()
    s.close()
    us.sort()
    return {"p50_us": us[len(us) // 2], "p90_us": us[int(len(us) * 0.9)], "steps": steps,
            "back_to_back_us": e0.elapsed_time(e1) * 1e3 / steps,
            "workload": "server batch B=4 V=151936 bf16, host params, prepared argument blocks, events around each call"}


if __name__ == "__main__":
    main()
