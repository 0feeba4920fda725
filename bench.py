#!/usr/bin/env python
"""Benchmark of the `gemm_fp4` hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the 27B MLP gate/up prefill projection the headline metric is quoted on,
m = 512, n = 17408, k = 5120, f16 x ~ N(0,1), seeded synthetic NVFP4 weights.  One step is one
`gemm_fp4` launch; consecutive steps use different weight copies (8 copies, about 400 MB, more
than the L2) as crates/lex-rt/examples/gemm_bench.rs:99-115 does.  The decode matvec
(m = 1 and m = 4, same matrix) is timed the same way and reported under "matvec".

With N > 1 the weight rows are split column-parallel, n/N per GPU; each rank computes its
columns of y.  The step does not gather y (the next operator of the MLP consumes it sharded);
the variant that all-gathers y over NCCL is timed separately and reported under "allgather".

`--impl reference` times the CPU restatement of the reference interpreter (the reference is
Rust and cannot be built here) on the host cores, on a bounded sample of the same workload.

`--only gemm|matvec` times one kernel alone (short runs for profilers), `--no-sustained` leaves out
the seconds-long run of the headline steps, and `--only gemm --tokens M` runs the headline matrices
at another token count (other tile shapes of the same kernel); the full run is always m = 512.
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
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M, N_ROWS, K = 512, 17408, 5120
# DRAM bytes per launch of the block-scaled matmul_q_x kernel at (17408, 5120), from an ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum): 50.26 MB read, 9 KB written
MQ_TRAFFIC = 50.27e6
METRIC = "gemm_fp4 TFLOP/s at m=512 (27B MLP gate/up: n=17408 k=5120)"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        rows = []
        for ts, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                rows.append((ts, parts))
        inside = [p for ts, p in rows if t0 - 0.05 <= ts <= t1 + 0.15] or [p for _, p in rows]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = [float(p[0]) for p in inside if p[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(p[3 + i].lower().startswith("active") for p in inside)]
        bins = {}
        for v in mhz:
            key = str(int(v // 100 * 100))
            bins[key] = bins.get(key, 0) + 1
        return {"sm_mhz": statistics.median(mhz) if mhz else None,
                "sm_max_mhz": float(inside[0][1]) if inside[0][1].replace(".", "").isdigit() else None,
                "samples": len(inside), "reasons": reasons, "samples_by_100mhz": bins}


def host_cores() -> int:
    """Cores this process may run on.  The launcher of multi-rank runs exports OMP_NUM_THREADS=1, so the count is
    passed to the oracle explicitly rather than left to OpenMP's default."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _cpu_time_rows(x, rows: int):
    from lex_gpu_b200 import inputs
    from oracle import oracle as O
    wq, ws, wg = inputs.make_weights(rows, K)
    t = time.perf_counter()
    O.gemm_fp4(x, wq, ws, wg, threads=host_cores())
    return time.perf_counter() - t


def cpu_leg(target_seconds: float = 12.0):
    """The oracle on the host cores: whole rows of W, all m tokens, sized to about target_seconds."""
    from lex_gpu_b200 import inputs
    from oracle import oracle as O
    x = inputs.make_x(M, K)
    _cpu_time_rows(x, 128)                                         # load + warm
    probe = 512
    dt = _cpu_time_rows(x, probe)
    rows = int(min(N_ROWS, max(probe, probe * target_seconds / max(dt, 1e-6))) // 128 * 128)
    dt = _cpu_time_rows(x, rows)
    tflops = 2.0 * M * rows * K / dt / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": host_cores(), "kind": "port",
            "sample": f"{rows} of {N_ROWS} weight rows, all {M} tokens, k={K}: {dt:.2f} s"}


def run_reference(args):
    """The reference's CPU path (restated: the reference is Rust, no toolchain here) on the host
    cores.  One step = the m=512 product over a slice of weight rows, sized so that
    warmup + steps together take about 90 seconds."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from lex_gpu_b200 import inputs
    from oracle import oracle as O
    x = inputs.make_x(M, K)
    _cpu_time_rows(x, 128)
    probe = 512
    dt = _cpu_time_rows(x, probe)
    total = max(1, args.warmup + args.steps)
    rows = int(min(N_ROWS, max(128, probe * (90.0 / total) / max(dt, 1e-6))) // 128 * 128)
    for _ in range(args.warmup):
        _cpu_time_rows(x, rows)
    secs = 0.0
    for _ in range(args.steps):
        secs += _cpu_time_rows(x, rows)
    val = 2.0 * M * rows * K * args.steps / secs / 1e12
    info = {"value": val, "unit": "TFLOP/s", "cores": host_cores(), "kind": "port",
            "sample": f"{rows} of {N_ROWS} weight rows per step, all {M} tokens, k={K}"}
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * secs / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16*fp4->f32",
            "data": "synthetic", "config": {"workload": f"gemm_fp4 m={M} n={N_ROWS} k={K} (27B MLP gate/up prefill)",
                                            "note": "CPU restatement of the reference interpreter; each step a row-slice sample"},
            "cpu_baseline": info,
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def run_ours(args):
    import torch
    import lex_gpu_b200 as L
    from lex_gpu_b200 import build, inputs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.gpus != world:
        if rank == 0:
            sys.stderr.write(f"--gpus {args.gpus} but WORLD_SIZE={world}; using WORLD_SIZE\n")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    build.build()
    gpu = L.Gpu(local)
    stream = torch.cuda.Stream(device=dev)
    gpu.set_stream(stream.cuda_stream)
    peaks = measured_peaks()

    n0, n1 = L.shard_rows(N_ROWS, world, rank)
    n_local = n1 - n0

    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- resident inputs: x, and COPIES weight sets of this rank's rows
    x_np = inputs.make_x(M, K)
    x_t = torch.from_numpy(x_np.view(np.int16)).to(dev)
    xb = gpu.wrap_tensor(x_t)
    weights = []
    w0_host = None
    # enough copies of this rank's slab to exceed the L2 (126 MB) several times over
    wbytes_one = n_local * K // 2 + n_local * K // 16 + 4 * n_local
    COPIES = max(8, -(-400_000_000 // wbytes_one))
    for c in range(COPIES):
        if world == 1:
            wq, ws, wg = inputs.make_weights(N_ROWS, K, copy=c)
        else:
            # a rank generates only its own slab (same distributions, its own seed): generating and
            # slicing the whole matrix on every rank would cost minutes of host time
            wq, ws, wg = inputs.make_weights(n_local, K, seed_base=10_000 * (rank + 1), copy=c)
        if c == 0:
            w0_host = (wq, ws, wg)
        t = [torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (wq, ws, wg)]
        weights.append((t, [gpu.wrap_tensor(v) for v in t]))
    y_t = torch.empty((M, n_local), dtype=torch.float32, device=dev)
    yb = gpu.wrap_tensor(y_t)
    torch.cuda.synchronize(dev)

    def timed(pipe, steps_fn, steps, warmup, sample_clocks=False):
        """Device time of exactly `steps` steps (events on the launch stream), max over ranks."""
        with torch.cuda.stream(stream):
            for i in range(warmup):
                steps_fn(i)
        barrier()
        sampler = ClockSampler(local) if sample_clocks else None
        if sampler:
            sampler.start()
            time.sleep(0.25)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(steps):
                steps_fn(warmup + i)
            e1.record(stream)
        barrier()
        t1 = time.time()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop(t0, t1) if sampler else None
        if dist is not None:
            tt = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms * 1e-3, clocks

    # ---- headline: m = 512 GEMM
    pipe = gpu.plan_gemm_fp4(M, n_local, K)
    desc = pipe.describe()

    def gemm_step(i):
        _, bufs = weights[i % COPIES]
        gpu.run(pipe, [xb, bufs[0], bufs[1], bufs[2], yb])

    # ---- parity gate: before anything is timed, 128-row slices of this rank's y against the oracle (the checker);
    # a run that fails it prints no value
    from oracle import oracle as O

    def slice_errors(y_np, w_host, col0, slices, x_host=x_np):
        worst = (0.0, 0.0)
        for lo, hi in slices:
            want = O.gemm_fp4(x_host, *w_host, rows=(lo, hi), threads=host_cores())[:, lo:hi]
            err, scale, rel = O.err_of_scale(y_np[:, col0 + lo:col0 + hi], want)
            if not (scale > 1e-3 and np.isfinite(y_np[:, col0 + lo:col0 + hi]).all()):
                return (float("inf"), float("inf"))
            worst = (max(worst[0], err), max(worst[1], rel))
        return worst

    def all_ranks_max(v):
        if dist is None:
            return v
        tt = torch.tensor(list(v), device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return tuple(float(t) for t in tt)

    GATE = 2e-3
    y_t.fill_(float("nan"))
    with torch.cuda.stream(stream):
        gemm_step(0)
    barrier()
    row_slices = [(0, 128), (n_local // 2 // 128 * 128, n_local // 2 // 128 * 128 + 128), (n_local - 128, n_local)]
    p_err, p_rel = all_ranks_max(slice_errors(y_t.cpu().numpy(), w0_host, 0, row_slices))
    parity = {"gate_of_scale": GATE, "of_scale": p_err, "per_element_floor_1e-3_of_scale": p_rel,
              "checked": f"{len(row_slices)} slices of 128 weight rows x all {M} tokens of every rank's y against the CPU oracle",
              "ok": bool(p_err <= GATE)}
    if not parity["ok"]:
        raise SystemExit(f"parity gate failed before timing: {p_err:e} of scale (gate {GATE:e}); no value is reported")

    # long enough for the clock sampler to see the load: repeat the measured block
    full = args.only == "all"
    if args.only == "matvec":
        secs, clocks = timed(pipe, gemm_step, 1, 3)
    else:
        secs, clocks = timed(pipe, gemm_step, args.steps, args.warmup, sample_clocks=full)
    status = gpu.status_word()
    flops_step = 2.0 * M * N_ROWS * K
    tflops = flops_step * args.steps / secs / 1e12
    per_launch = secs / args.steps
    local_flops = 2.0 * M * n_local * K
    # DRAM bytes per launch (read + write) from an ncu capture of this kernel
    # (m=512 n=17408 k=5120 on one GPU: 55.5 MB read, 3.2 MB written, y still in L2); only for that shape
    gemm_traffic = 58.7e6 if world == 1 and M == 512 else None
    roofline = {"bound": "tensor", "achieved": local_flops / per_launch / 1e12, "peak": peaks["tflops"],
                "unit": "TFLOP/s", "frac": local_flops / per_launch / 1e12 / peaks["tflops"], "traffic": gemm_traffic,
                "peak_source": f"{peaks['source']} bf16 burst (cuBLAS 8192^3)", "kernel": desc.entry.decode(),
                "frac_of_nominal_2250": local_flops / per_launch / 1e12 / 2250.0}

    # ---- the same steps for seconds, not milliseconds: what the kernel holds under the power cap, with the clocks
    # sampled over this very region and the fraction taken against the sustained cuBLAS figure
    sustained = None
    if full and args.sustained:
        n_sus = int(min(200_000, max(args.steps, 2.5 / per_launch)))
        s_sus, c_sus = timed(pipe, gemm_step, n_sus, 3, sample_clocks=True)
        tf_sus = flops_step * n_sus / s_sus / 1e12
        peak_sus = peaks.get("tflops_sustained") or peaks["tflops"]
        sustained = {"value": tf_sus, "unit": "TFLOP/s", "steps": n_sus, "seconds": s_sus, "ms_per_step": 1e3 * s_sus / n_sus,
                     "frac_of_sustained_peak": (local_flops * n_sus / s_sus / 1e12) / peak_sus, "sustained_peak": peak_sus,
                     "frac_of_nominal_2250": (local_flops * n_sus / s_sus / 1e12) / 2250.0, "clocks": c_sus,
                     "us_x_median_mhz": (1e6 * s_sus / n_sus) * c_sus["sm_mhz"] if c_sus and c_sus.get("sm_mhz") else None}
        if (clocks or {}).get("samples", 0) < 3 and c_sus and c_sus.get("sm_mhz"):
            # the headline's timed region is shorter than the sampler's period: the record of the same steps held
            # for seconds stands in (its own figure is under "sustained")
            clocks = dict(c_sus)
            clocks["note"] = "the timed region is shorter than the sampler's period; sampled over the sustained run of the same steps"

    # ---- e2e: host x -> device, launch, y -> host, every step, through the C ABI call
    e2e, checksum = None, None
    if full:
        hx = L.HostBuffer(x_np.nbytes)
        hx.array(np.float16, (M, K))[:] = x_np
        hy = L.HostBuffer(M * n_local * 4)
        xd, yd = gpu.alloc(x_np.nbytes), gpu.alloc(M * n_local * 4)
        e2e_steps = max(5, min(args.steps, 50))
        for i in range(3):
            b = weights[i % COPIES][1]
            gpu.run_host(pipe, hx.ptr, xd, b[0], b[1], b[2], None, yd, hy.ptr)
        barrier()
        t = time.perf_counter()
        for i in range(e2e_steps):
            b = weights[i % COPIES][1]
            gpu.run_host(pipe, hx.ptr, xd, b[0], b[1], b[2], None, yd, hy.ptr)
        torch.cuda.synchronize(dev)
        e2e_secs = time.perf_counter() - t
        if dist is not None:
            tt = torch.tensor([e2e_secs], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e_secs = float(tt.item())
        checksum = float(hy.array(np.float32, (M, n_local))[0, :8].sum())
        serial_secs = e2e_secs
        # The same steps double-buffered: two streams, two sets of staging buffers, lexb_gemm_fp4_enqueue_host.
        # Every step still copies its x in and its y out inside the timed region; step i's copy back overlaps
        # step i+1's copy in and launch.
        # Each lane has its own pipeline: a pipeline planned with a K split owns one split-K workspace, and two
        # launches of it must not overlap on two streams.
        stream2 = torch.cuda.Stream(device=dev)
        lanes = [(stream, hx, hy, xd, yd, pipe)]
        hx2 = L.HostBuffer(x_np.nbytes)
        hx2.array(np.float16, (M, K))[:] = x_np
        hy2 = L.HostBuffer(M * n_local * 4)
        lanes.append((stream2, hx2, hy2, gpu.alloc(x_np.nbytes), gpu.alloc(M * n_local * 4), gpu.plan_gemm_fp4(M, n_local, K)))

        def piped(nsteps, first):
            for i in range(nsteps):
                st, h_x, h_y, d_x, d_y, lane_pipe = lanes[i % 2]
                gpu.set_stream(st.cuda_stream)
                b = weights[(first + i) % COPIES][1]
                gpu.enqueue_host(lane_pipe, h_x.ptr, d_x, b[0], b[1], b[2], None, d_y, h_y.ptr)
            torch.cuda.synchronize(dev)

        piped(4, 0)
        barrier()
        t = time.perf_counter()
        piped(e2e_steps, 4)
        e2e_secs = time.perf_counter() - t
        gpu.set_stream(stream.cuda_stream)
        if dist is not None:
            tt = torch.tensor([e2e_secs], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e_secs = float(tt.item())
        # what each lane brought back last, against the same weight sets run one step at a time on one stream
        lanes_ok = True
        for lane, i_last in ((0, e2e_steps - 2 + (e2e_steps % 2)), (1, e2e_steps - 1 - (e2e_steps % 2))):
            got_lane = lanes[lane][2].array(np.float32, (M, n_local)).copy()
            b = weights[(4 + i_last) % COPIES][1]
            gpu.run_host(pipe, hx.ptr, xd, b[0], b[1], b[2], None, yd, hy.ptr)
            lanes_ok = lanes_ok and np.array_equal(got_lane, hy.array(np.float32, (M, n_local)))
        if all_ranks_max((0.0 if lanes_ok else 1.0,))[0] != 0.0:
            raise SystemExit("the double-buffered end-to-end leg returned a y that differs from the single-stream result")
        e2e = {"value": flops_step * e2e_steps / e2e_secs / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(x_np.nbytes), "d2h_bytes_per_step": int(M * n_local * 4), "steps": e2e_steps,
               "ms_per_step": 1e3 * e2e_secs / e2e_steps,
               "note": "lexb_gemm_fp4_enqueue_host on two streams: every step copies pinned x in and y out, weights "
                       "resident; one step's copy back overlaps the next step's copy in and launch",
               "one_stream": {"value": flops_step * e2e_steps / serial_secs / 1e12, "ms_per_step": 1e3 * serial_secs / e2e_steps,
                              "note": "lexb_gemm_fp4_run_host, one step at a time"},
               "lanes_equal_single_stream": True}

    # ---- matvec (m = 1, 4): GB/s of weight bytes
    matvec = {}
    wbytes_local = n_local * K // 2 + n_local * K // 16 + 4 * n_local
    for mm in ((1, 4) if args.only != "gemm" else ()):
        p_mv = gpu.plan_gemm_fp4(mm, n_local, K)
        xs = gpu.wrap_tensor(x_t[:mm].contiguous())
        ys_t = torch.empty((mm, n_local), dtype=torch.float32, device=dev)
        ys = gpu.wrap_tensor(ys_t)

        def mv_step(i, p_mv=p_mv, xs=xs, ys=ys):
            b = weights[i % COPIES][1]
            gpu.run(p_mv, [xs, b[0], b[1], b[2], ys])

        mv_steps = max(args.steps, 200) if full else args.steps
        s_mv, _ = timed(p_mv, mv_step, mv_steps, max(args.warmup, 20) if full else args.warmup)
        per = s_mv / mv_steps
        gbs = wbytes_local / per / 1e9
        matvec[f"m{mm}"] = {"gbs_weight_bytes": gbs * world, "us_per_launch": per * 1e6,
                            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                         "frac": gbs / peaks["hbm_gbs"], "traffic": 50.24e6 if world == 1 else None,
                                         "frac_of_nominal_8000": gbs / 8000.0}}
        # the same bindings through matmul_q_x (the operator the model decodes with: weights not rounded
        # to f16), on the block-scaled FP4 tensor-core kernel
        p_mq = gpu.plan_matmul_fp4(mm, n_local, K)

        def mq_step(i, p_mq=p_mq, xs=xs, ys=ys):
            b = weights[i % COPIES][1]
            gpu.run(p_mq, [xs, b[0], b[1], b[2], ys])

        s_mq, _ = timed(p_mq, mq_step, mv_steps, max(args.warmup, 20) if full else args.warmup)
        per_q_single = s_mq / mv_steps
        # launched one at a time the kernel reads in order; with the caller's promise that nothing writes the
        # weights (LEXB_SCHED_WEIGHTS_CONSTANT) it loads them while the launch ahead still runs
        p_mq_c = gpu.plan_matmul_fp4(mm, n_local, K, weights_constant=True)
        s_mqc, _ = timed(p_mq_c, lambda i, p_mq_c=p_mq_c, xs=xs, ys=ys: gpu.run(p_mq_c, [xs] + list(weights[i % COPIES][1]) + [ys]),
                         mv_steps, max(args.warmup, 20) if full else args.warmup)
        per_q_single_const = s_mqc / mv_steps
        # The same launches as step lists through lexb_run_launches (Gpu::run_launches, how the runtime issues a
        # layer's dispatches).  The library runs consecutive steps that do not depend on one another as one
        # persistent kernel whose blocks stride over all their row tiles; a step that reads or overwrites what
        # an earlier step of the run touches starts a new launch.  Two patterns:
        #  "pairs": outputs alternate between two buffers, so every second step overwrites a buffer of the run
        #           before it - runs of two, the gate/up pair of one MLP (the same x, two weight matrices);
        #  "independent": every step has its own output - one run over the whole list (an upper bound: the
        #           q/k/v + gate/up + experts pattern with nothing in between).
        def list_seconds(n_outputs, pipe=p_mq):
            outs_t = [torch.empty((mm, n_local), dtype=torch.float32, device=dev) for _ in range(n_outputs)]
            outs = [gpu.wrap_tensor(t) for t in outs_t]
            lst = [(pipe, [xs] + list(weights[i % COPIES][1]) + [outs[i % n_outputs]]) for i in range(mv_steps)]
            gpu.run_launches(lst[:max(args.warmup, 8)])
            lst = L.StepList(lst)                 # marshalled outside the timed region
            gpu.run_launches(lst)                 # (job tables of the runs are kept by content from here on)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                e0.record(stream)
                gpu.run_launches(lst)
                e1.record(stream)
            barrier()
            sec = e0.elapsed_time(e1) * 1e-3
            if dist is not None:
                tt = torch.tensor([sec], device=dev, dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                sec = float(tt.item())
            return sec / mv_steps

        def hbm(per):
            g = wbytes_local / per / 1e9
            return {"bound": "hbm", "achieved": g, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": g / peaks["hbm_gbs"],
                    "traffic": MQ_TRAFFIC if world == 1 else None, "frac_of_nominal_8000": g / 8000.0}

        per_q = list_seconds(2)
        per_q_run = list_seconds(mv_steps)
        # A shard with few row tiles is planned with K split over blocks, which fills the GPU for a launch on its
        # own but keeps the step out of runs; planned with one K range per block the same lists run as runs.
        unsplit = None
        if p_mq.describe().k_splits > 1:
            p_one = gpu.plan_matmul_fp4(mm, n_local, K, k_splits=1)
            a2, ar = list_seconds(2, p_one), list_seconds(mv_steps, p_one)
            unsplit = {"plan": "k_splits = 1", "runs_of_two": {"us_per_launch": a2 * 1e6, "gbs_weight_bytes": wbytes_local / a2 / 1e9 * world},
                       "one_run": {"us_per_launch": ar * 1e6, "gbs_weight_bytes": wbytes_local / ar / 1e9 * world}}
        matvec[f"m{mm}"]["matmul_q_x"] = {
            "kernel": p_mq.describe().entry.decode(), "gbs_weight_bytes": wbytes_local / per_q / 1e9 * world,
            "us_per_launch": per_q * 1e6,
            "issued_as": "one step list (lexb_run_launches), outputs alternating between two buffers: runs of two steps",
            "us_per_launch_issued_one_by_one": per_q_single * 1e6,
            "us_per_launch_issued_one_by_one_weights_declared_constant": per_q_single_const * 1e6, "roofline": hbm(per_q),
            "independent_steps": {"issued_as": "one step list, every step with its own output: one run",
                                  "gbs_weight_bytes": wbytes_local / per_q_run / 1e9 * world,
                                  "us_per_launch": per_q_run * 1e6, "roofline": hbm(per_q_run)},
            "k_splits": p_mq.describe().k_splits, "lists_planned_unsplit": unsplit}

    # ---- all-gather variant (N > 1): y shards -> [N][m][n/N] on every rank
    allgather = None
    if dist is not None and full:
        from lex_gpu_b200.shard import RowShard, all_gather_y
        shard = RowShard.of(N_ROWS, world, rank)

        def ag_step(i):
            gemm_step(i)
            all_gather_y(y_t, shard)        # NCCL, ordered after the launch on the same stream

        s_ag, _ = timed(pipe, ag_step, args.steps, args.warmup)
        # the floor of any gather: the NCCL all-gather of the same bytes with nothing else in the step
        s_only, _ = timed(pipe, lambda i: all_gather_y(y_t, shard), args.steps, args.warmup)
        allgather = {"value": flops_step * args.steps / s_ag / 1e12, "unit": "TFLOP/s",
                     "ms_per_step": 1e3 * s_ag / args.steps, "bytes_per_rank": int(M * shard.max_rows() * 4),
                     "layout": "[N][m][max rows per rank]", "gather_only_us": 1e6 * s_only / args.steps,
                     "gemm_only_us": 1e6 * per_launch}
        # the same gather fused into the kernel: peer stores into every rank's y[m, n] (symmetric memory),
        # one cross-rank barrier per step
        try:
            from lex_gpu_b200.shard import SymmetricY
            with torch.cuda.stream(stream):
                sy = SymmetricY(M, N_ROWS, dist.group.WORLD)

                def fused_step(i):
                    b = weights[i % COPIES][1]
                    gpu.run_gather(pipe, xb, b[0], b[1], b[2], None, sy.ptrs, N_ROWS, n0)
                    sy.barrier()

                s_fu, _ = timed(pipe, fused_step, args.steps, args.warmup)
                # parity of the gathered y: the columns another rank stored here, against the oracle on that
                # rank's weights (regenerated on the host from its seed)
                sy.tensor.fill_(float("nan"))
                sy.barrier()
                fused_step(0)
                torch.cuda.synchronize(dev)
                other = (rank + 1) % world
                o0, o1 = L.shard_rows(N_ROWS, world, other)
                w_other = inputs.make_weights(o1 - o0, K, seed_base=10_000 * (other + 1), copy=0)
                g_err, g_rel = all_ranks_max(slice_errors(sy.tensor.cpu().numpy(), w_other, o0, [(0, 128), (o1 - o0 - 128, o1 - o0)]))
                sy.barrier()
            if not g_err <= GATE:
                raise SystemExit(f"parity gate failed on the gathered y: {g_err:e} of scale")
            allgather["fused_peer_stores"] = {"value": flops_step * args.steps / s_fu / 1e12, "unit": "TFLOP/s",
                                              "ms_per_step": 1e3 * s_fu / args.steps, "layout": "[m][n] on every rank",
                                              "note": "epilogue stores to all ranks over NVLink + one barrier per step",
                                              "parity_of_scale": g_err}
        except SystemExit:
            raise
        except Exception as e:      # symmetric memory unavailable on this machine
            allgather["fused_peer_stores"] = {"unavailable": repr(e)[:200]}

    # ---- the MLP around the headline GEMM (crates/lex-rt/src/qwen_run.rs:3165-3189) at m = 512: gate and up in ONE
    # launch over their interleaved rows with silu(gate) * up formed in the epilogue (f16 activation out), then down
    # with the residual.  N = 1: against the same layer as three GEMM launches and an elementwise launch.  N > 1: rows
    # sharded, the f16 activation gathered by the epilogue's peer stores (2 bytes per element cross NVLink).
    mlp = None
    if full:
        def rolled_sets(rows, cols_k, seed, copies):
            """`copies` weight sets of one seeded slab, each the slab rolled by whole 128-row tiles (same bytes
            and distributions, distinct memory), on the device."""
            wq, ws, wg = inputs.make_weights(rows, cols_k, seed_base=seed)
            base = [torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (wq, ws, wg)]
            out = []
            for c in range(copies):
                t = [torch.roll(b, shifts=128 * c, dims=0).contiguous() for b in base]
                out.append((t, [gpu.wrap_tensor(v) for v in t]))
            return out

        gu_rows = 2 * n_local                                   # this rank's gate and up rows, interleaved
        gu_bytes = gu_rows * K // 2 + gu_rows * K // 16 + 4 * gu_rows
        gu_sets = rolled_sets(gu_rows, K, 30_000 * (rank + 1), max(3, -(-300_000_000 // gu_bytes)))
        pipe_gu = gpu.plan_gemm_fp4(M, gu_rows, K)
        act_t = torch.empty((M, n_local), dtype=torch.float16, device=dev)
        act_b = gpu.wrap_tensor(act_t)
        flops_gu = 2.0 * M * (2 * N_ROWS) * K

        def gu_fused(i):
            b = gu_sets[i % len(gu_sets)][1]
            gpu.run_silu(pipe_gu, xb, b[0], b[1], b[2], act_b)

        s_gu, _ = timed(None, gu_fused, args.steps, args.warmup)
        d_gu = pipe_gu.describe()
        mlp = {"gate_up_fused": {"us_per_launch": 1e6 * s_gu / args.steps, "value": flops_gu * args.steps / s_gu / 1e12, "unit": "TFLOP/s",
                                 "kernel": d_gu.entry.decode(), "k_splits": d_gu.k_splits, "out": "f16 [m, ffn/N] activation",
                                 "bytes_written_per_launch": int(M * n_local * 2)}}
        if world == 1:
            ygu_t = torch.empty((M, gu_rows), dtype=torch.float32, device=dev)
            ygu_b = gpu.wrap_tensor(ygu_t)

            def gu_unfused(i):
                b = gu_sets[i % len(gu_sets)][1]
                gpu.run(pipe_gu, [xb, b[0], b[1], b[2], ygu_b])
                gpu.silu_mul(M, n_local, ygu_b, ygu_b, act_b, out_f16=True, gate_pitch=gu_rows, up_offset=n_local, up_pitch=gu_rows)

            s_un, _ = timed(None, gu_unfused, args.steps, args.warmup)
            mlp["gate_up_then_silu_mul_launch"] = {"us_per_step": 1e6 * s_un / args.steps,
                                                   "note": "one GEMM launch over [m, 2 ffn] f32, then the elementwise launch"}
            # the whole layer: fused gate/up, then down (n = 5120, k = 17408) with the residual
            dn_sets = rolled_sets(K, N_ROWS, 31_000, 4)
            pipe_dn = gpu.plan_gemm_fp4(M, K, N_ROWS, residual=True)
            res_t = torch.zeros((M, K), dtype=torch.float32, device=dev)
            out_t = torch.empty((M, K), dtype=torch.float32, device=dev)
            res_b, out_b = gpu.wrap_tensor(res_t), gpu.wrap_tensor(out_t)

            def layer(i):
                gu_fused(i)
                b = dn_sets[i % len(dn_sets)][1]
                gpu.run(pipe_dn, [act_b, b[0], b[1], b[2], res_b, out_b])

            s_ly, _ = timed(None, layer, args.steps, args.warmup)
            flops_layer = flops_gu + 2.0 * M * K * N_ROWS
            mlp["layer"] = {"us_per_layer": 1e6 * s_ly / args.steps, "value": flops_layer * args.steps / s_ly / 1e12, "unit": "TFLOP/s",
                            "config": "m=512: gate+up fused with silu_mul (ffn 17408, k 5120), down (n 5120, k 17408) + residual"}
            # end to end through host buffers: x in (f16), the layer, y [m, 5120] f32 out - what a prefill chunk's
            # MLP moves across PCIe when the activation stays on the device
            hx_l, hy_l = L.HostBuffer(x_np.nbytes), L.HostBuffer(M * K * 4)
            hx_l.array(np.float16, (M, K))[:] = x_np
            x_dev_l = torch.empty((M, K), dtype=torch.float16, device=dev)

            def layer_host(i):
                with torch.cuda.stream(stream):
                    x_dev_l.copy_(torch.from_numpy(hx_l.array(np.float16, (M, K))), non_blocking=True)
                    b = gu_sets[i % len(gu_sets)][1]
                    gpu.run_silu(pipe_gu, gpu.wrap_tensor(x_dev_l), b[0], b[1], b[2], act_b)
                    b = dn_sets[i % len(dn_sets)][1]
                    gpu.run(pipe_dn, [act_b, b[0], b[1], b[2], res_b, out_b])
                    torch.from_numpy(hy_l.array(np.float32, (M, K))).copy_(out_t, non_blocking=True)

            for i in range(3):
                layer_host(i)
            torch.cuda.synchronize(dev)
            t_h = time.perf_counter()
            n_h = max(5, min(args.steps, 50))
            for i in range(n_h):
                layer_host(i)
            torch.cuda.synchronize(dev)
            t_h = time.perf_counter() - t_h
            mlp["layer_e2e_host_buffers"] = {"us_per_layer": 1e6 * t_h / n_h, "value": flops_layer * n_h / t_h / 1e12, "unit": "TFLOP/s",
                                             "h2d_bytes_per_step": int(x_np.nbytes), "d2h_bytes_per_step": int(M * K * 4)}
        else:
            try:
                from lex_gpu_b200.shard import SymmetricY
                with torch.cuda.stream(stream):
                    sa = SymmetricY(M, N_ROWS, dist.group.WORLD, dtype=torch.float16)

                    def gu_gather(i):
                        b = gu_sets[i % len(gu_sets)][1]
                        gpu.run_silu_gather(pipe_gu, xb, b[0], b[1], b[2], sa.ptrs, 2 * N_ROWS, 2 * n0)
                        sa.barrier()

                    s_gg, _ = timed(None, gu_gather, args.steps, args.warmup)
                    # parity of the gathered activation: this rank's own columns against its unfused result
                    sa.tensor.fill_(0)
                    sa.barrier()
                    gu_gather(0)
                    gu_fused(0)
                    torch.cuda.synchronize(dev)
                    same = bool(torch.equal(sa.tensor[:, n0:n1], act_t))
                    sa.barrier()
                if all_ranks_max((0.0 if same else 1.0,))[0] != 0.0:
                    raise SystemExit("the gathered f16 activation differs from the rank's own fused result")
                mlp["gate_up_fused_gathered"] = {"us_per_step": 1e6 * s_gg / args.steps, "value": flops_gu * args.steps / s_gg / 1e12,
                                                 "unit": "TFLOP/s", "bytes_into_every_gpu": int(M * (N_ROWS - n_local) * 2),
                                                 "note": "f16 activation [m, ffn] on every rank by peer stores + one barrier per step"}
            except SystemExit:
                raise
            except Exception as e:
                mlp["gate_up_fused_gathered"] = {"unavailable": repr(e)[:200]}
        del gu_sets

    # ---- one layer of the 27B MLP stack at m = 4096 (the 64-layer stack configuration), n-sharded: gate, up (n=17408,
    # k=5120) and down (n=5120, k=17408), independent calls, y not chained.  Reported, not the headline.
    stack = None
    if full and args.stack:
        m4 = 4096
        shapes = [("gate", N_ROWS, K), ("up", N_ROWS, K), ("down", K, N_ROWS)]
        steps4, flops4 = [], 0.0
        keep = []
        for name, nn, kk in shapes:
            a0, a1 = L.shard_rows(nn, world, rank)
            nl = a1 - a0
            xx = torch.from_numpy(inputs.make_x(m4, kk, seed_base=5).view(np.int16)).to(dev)
            yy = torch.empty((m4, nl), dtype=torch.float32, device=dev)
            sets = []
            slab = nl * kk // 2 + nl * kk // 16 + 4 * nl
            for c in range(max(3, -(-400_000_000 // (3 * slab)))):      # rotate through more than the L2 holds
                w = inputs.make_weights(nl, kk, seed_base=20_000 * (rank + 1) + (0 if name != "up" else 7), copy=c)
                tt = [torch.from_numpy(np.ascontiguousarray(v)).to(dev) for v in w]
                sets.append(tt)
            pp = gpu.plan_gemm_fp4(m4, nl, kk)
            keep.append((xx, yy, sets, pp))
            steps4.append((pp, gpu.wrap_tensor(xx), [[gpu.wrap_tensor(v) for v in tt] for tt in sets], gpu.wrap_tensor(yy)))
            flops4 += 2.0 * m4 * nn * kk

        def layer_step(i):
            for pp, xbuf, wsets, ybuf in steps4:
                b = wsets[i % len(wsets)]
                gpu.run(pp, [xbuf, b[0], b[1], b[2], ybuf])

        n_layers = 16
        s4, _ = timed(None, layer_step, n_layers, 3)
        stack = {"value": flops4 * n_layers / s4 / 1e12, "unit": "TFLOP/s", "ms_per_layer": 1e3 * s4 / n_layers,
                 "config": f"m=4096, gate+up (n=17408,k=5120) + down (n=5120,k=17408) per layer, n-sharded x{world}, no gather",
                 "layers_timed": n_layers}
        del keep

    # ---- the reference's own CUDA kernels, compiled for sm_100a from its tree (oracle/_ref): the bar on this box.
    # Same shapes, same rotation of weight copies, same event timing; f32 x for its matvec, as it is emitted.
    ref_box = None
    if world == 1 and full:
        from oracle import refkernels as R
        ref_box = {}
        try:
            entry = R.gemm_entry(M, N_ROWS, K)
            yr = torch.empty((M, N_ROWS), dtype=torch.float32, device=dev)

            def ref_gemm_step(i):
                t = weights[i % COPIES][0]
                R.run_torch(entry, [x_t, t[0], t[1], t[2], yr], stream.cuda_stream)

            n_ref = max(8, min(args.steps, 24))
            s_ref, _ = timed(None, ref_gemm_step, n_ref, 3)
            err, scale, _ = O.err_of_scale(yr[:, :128].cpu().numpy(),
                                           O.gemm_fp4(x_np, *inputs.make_weights(N_ROWS, K, copy=(3 + n_ref - 1) % COPIES), rows=(0, 128),
                                                      threads=host_cores())[:, :128])
            ref_box["gemm"] = {"kernel": R.info(entry), "tflops": flops_step * n_ref / s_ref / 1e12, "us_per_launch": 1e6 * s_ref / n_ref,
                               "source": "crates/lex-msl/src/gemm.rs:89-320 instantiated for this shape, nvcc sm_100a",
                               "of_scale_vs_oracle": err, "ours_over_reference": (s_ref / n_ref) / per_launch}
        except Exception as e:
            ref_box["gemm"] = {"unavailable": repr(e)[:200]}
        try:
            x32 = x_t[:1].view(torch.float16).float().contiguous()
            yv = torch.empty((1, N_ROWS), dtype=torch.float32, device=dev)

            def ref_mv_step(i):
                t = weights[i % COPIES][0]
                R.run_torch(R.MATVEC_ENTRY, [x32, t[0], t[1], t[2], yv], stream.cuda_stream)

            s_rv, _ = timed(None, ref_mv_step, 200, 20)
            per_rv = s_rv / 200
            ref_box["matvec"] = {"kernel": R.info(R.MATVEC_ENTRY), "us_per_launch": 1e6 * per_rv,
                                 "gbs_weight_bytes": wbytes_local / per_rv / 1e9, "frac_of_hbm_peak": wbytes_local / per_rv / 1e9 / peaks["hbm_gbs"],
                                 "source": "crates/lex-msl/tests/golden/matvec_nvfp4_17408x5120_cuda.cu unchanged, nvcc sm_100a"}
        except Exception as e:
            ref_box["matvec"] = {"unavailable": repr(e)[:200]}

    if rank == 0:
        info = cpu_leg() if (world == 1 and full) else None
        line = {"metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": 1e3 * per_launch, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16*fp4->f32", "data": "synthetic",
                "config": {"workload": f"gemm_fp4 m={M} n={N_ROWS} k={K} (27B MLP gate/up prefill)",
                           "parallelism": f"n-sharded x{world}, {n_local} rows on rank 0, no gather in the step",
                           "k_splits": desc.k_splits,
                           "l2": f"{COPIES} weight copies rotated per step ({COPIES * wbytes_local / 1e6:.0f} MB per GPU > L2)",
                           "schedule": {"bm": desc.bm, "bn": desc.bn, "bk": desc.bk, "stages": desc.stages,
                                        "grid": desc.grid, "threads": desc.threads, "smem": desc.threadgroup_bytes}},
                "roofline": roofline, "cpu_baseline": info, "e2e": e2e, "gpu_launches": args.steps,
                "clocks": clocks, "matvec": matvec, "allgather": allgather, "device_status": status,
                "checksum": checksum, "only": args.only, "stack_m4096": stack, "parity": parity, "sustained": sustained,
                "reference_kernels_on_this_box": ref_box, "mlp_m512": mlp}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-stack", dest="stack", action="store_false",
                    help="skip the m=4096 stack-layer leg (reported under stack_m4096)")
    ap.add_argument("--no-sustained", dest="sustained", action="store_false",
                    help="skip the seconds-long run of the headline steps (short runs for profilers)")
    ap.add_argument("--only", default="all", choices=["all", "gemm", "matvec"],
                    help="time one kernel only (short runs for profilers); the JSON line then omits the other legs")
    ap.add_argument("--tokens", type=int, default=M,
                    help="with --only gemm: another token count m for the same matrices (profiler runs of other tile shapes); "
                         "the metric's own m is the default")
    args = ap.parse_args()
    if args.tokens != M:
        if args.only != "gemm" or args.impl != "ours":
            ap.error("--tokens is for --only gemm runs of this implementation")
        globals()["M"] = args.tokens
        globals()["METRIC"] = METRIC.replace("m=512", f"m={args.tokens}")
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
