#!/usr/bin/env python3
"""Benchmark of the tiled execution path: ResNet-50 batch 32 per GPU through the ASPEN C API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload resnet50|bert_base]

One step = one pass of the tile graph (nasm) of a batch-32 inference over synthetic N(0,1) input
with seeded He-normal weights (no pretrained weights or dataset exist in this tree).  With N > 1
(launched by torch.distributed.run, one rank per GPU) every rank runs its own batch-32 graph on
its own GPU -- independent shards, no collective on the data path, weak scaling -- and rank 0
prints one JSON line with the whole-job inferences/s, timed on the device (CUDA events on the
engine's stream) as the maximum over ranks.

`--impl reference` times the unmodified reference's pthread/AVX2 path (oracle/_ref, built from the
reference sources) on the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    # name: (cfg builder, batch per GPU, seq, weight scheme, weight seed, input seed, per-sample input shape)
    "resnet50": ("resnet50", 32, 0, "he", 1, 0),
    "bert_base": ("bert_base", 32, 128, "n002", 3, 3),
}
# DRAM bytes per scheduler launch, from the ncu capture summarised in profiles/ (batch-4 case scaled by 8).
TRAFFIC_BYTES = {"resnet50": 2.3e9}
# Tiling of the nasm per workload: (row quantum, column quantum, min_ninst_per_ldata).  Tensor-core shaped
# quanta; the values a graph computes do not depend on them.  Each is the best of a measured sweep
# (quanta 64-256, min_ninst 100-592).
TILING = {"resnet50": (128, 128, 180), "bert_base": (256, 128, 296)}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def prepare_files(workload: str, workdir: str):
    from aspen_b200 import cfgs, weights
    builder, batch, seq, scheme, wseed, _ = WORKLOADS[workload]
    cfg = os.path.join(workdir, f"{workload}.cfg")
    wfile = os.path.join(workdir, f"{workload}.bin")
    wl = cfgs.write_cfg(builder, cfg)
    weights.write_aspen_data(wfile, weights.make_weights(wl, wseed, scheme))
    return cfg, wfile


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.rows, self.proc = index, [], None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])
        except Exception:
            pass

    def stop(self):
        if self.proc:
            self.proc.terminate()
        self.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({names[i] for r in self.rows if len(r) >= 7 for i in range(4) if r[3 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def reduce_max(value: float, world: int, use_cuda: bool) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device="cuda" if use_cuda else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int, use_cuda: bool):
    if world == 1:
        return
    import torch
    import torch.distributed as dist
    dist.barrier()
    if use_cuda:
        torch.cuda.synchronize()


def init_dist(world: int, local_rank: int, use_cuda: bool):
    if world == 1:
        return
    import torch
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if use_cuda:
        torch.cuda.set_device(local_rank)
    dist.init_process_group(backend="nccl" if use_cuda else "gloo")


def job_value(units_per_rank: int, steps: int, world: int, max_ms: float) -> float:
    """Whole-job throughput: units all ranks processed / slowest rank's device time."""
    return units_per_rank * steps * world / (max_ms * 1e-3)


class _StdoutToStderr:
    """The reference library prints progress with printf; the bench line must be the only thing on stdout."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def __exit__(self, *exc):
        try:
            import ctypes
            ctypes.CDLL(None).fflush(None)
        except Exception:  # noqa: BLE001
            pass
        os.dup2(self.saved, 1)
        os.close(self.saved)


def cpu_reference_rate(workload: str, cfg: str, wfile: str, batch: int, steps: int, warmup: int, workdir: str):
    """Times the reference's own DSE path (main.c:116-123 loop) on the host cores.  The graph file is
    written by this library and loaded by the reference (identical graphs; the reference's own
    generator needs minutes at this size)."""
    from aspen_b200 import api
    from oracle import ref
    _, _, seq, *_ = WORKLOADS[workload]
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    api.lib().aspen_b200_set_tile_profile(0)
    dnn = api.Dnn(cfg, None)
    nasm = api.Nasm(dnn, batch, seq, 100)
    nfile = os.path.join(workdir, f"{workload}_B{batch}_ref.nasm")
    nasm.save(nfile)
    nasm.close()
    dnn.close()
    with _StdoutToStderr():
        rn = ref.RefNet(cfg, wfile, batch, seq, nasm_file=nfile)
        i0 = rn.ldata_info(0)
        x = np.random.default_rng(0).standard_normal((i0["W"], i0["H"]), dtype=np.float32)
        sec = rn.bench_dse(x, cores, warmup, steps)
        rn.close()
    return batch / sec, cores


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    from oracle import ref
    workload = args.workload
    _, batch, seq, *_ = WORKLOADS[workload]
    if not ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libaspen_ref.so is not built (run make -C oracle ref where the reference sources are mounted)"}))
        return
    wd = tempfile.mkdtemp(prefix="aspen_bench_")
    cfg, wfile = prepare_files(workload, wd)
    rate, cores = cpu_reference_rate(workload, cfg, wfile, batch, args.steps, args.warmup, wd)
    ms = batch / rate * 1e3
    line = {
        "impl": "reference", "metric": "inferences_per_sec", "value": rate, "unit": "inf/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": f"{workload}_bs{batch}_per_gpu", "seq_len": seq or None, "tile_profile": "reference 64x12",
                                       "min_ninst_per_ldata": 100},
        "cpu_baseline": {"value": rate, "unit": "inf/s", "cores": cores, "kind": "reference",
                         "sample": f"reference DSE path, {cores} pthread workers, {args.steps} timed passes of one batch-{batch} graph"},
        "e2e": {"value": rate, "unit": "inf/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="resnet50", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--dry-run", action="store_true", help="no GPU: exercise launch, barrier and aggregation with fake timings")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.dry_run else args.warmup
    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    use_cuda = not args.dry_run
    init_dist(world, local_rank, use_cuda)
    workload = args.workload
    builder, batch, seq, scheme, wseed, iseed = WORKLOADS[workload]

    if args.dry_run:
        barrier(world, False)
        my_ms = 10.0 * args.steps * (1.0 + 0.1 * rank)
        max_ms = reduce_max(my_ms, world, False)
        barrier(world, False)
        if rank == 0:
            print(json.dumps({"metric": "inferences_per_sec", "value": job_value(batch, args.steps, world, max_ms), "unit": "inf/s",
                              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": max_ms / args.steps,
                              "scaling": "weak", "data": "dry-run", "higher_is_better": True}), flush=True)
        return

    import torch
    from aspen_b200 import api
    L = api.lib()
    if L.aspen_b200_set_device(local_rank) != 0:
        raise SystemExit("no CUDA device for this rank: " + api.last_error())
    wd = tempfile.mkdtemp(prefix=f"aspen_bench_r{rank}_")
    cfg, wfile = prepare_files(workload, wd)

    q_h, q_w, min_ninst = TILING[workload]
    L.aspen_b200_set_tile_quanta(q_h, q_w, 100000000)
    dnn = api.Dnn(cfg, wfile)
    nasm = api.Nasm(dnn, batch, seq, min_ninst)
    L.aspen_b200_set_tile_profile(0)
    rpool = api.Rpool()
    group = api.DseGroup(0, 0)
    group.set_rpool(rpool)
    i0 = nasm.ldata_info(0)
    in_shape = (i0["W"], i0["H"])
    x_pinned = torch.empty(in_shape, dtype=torch.float32).pin_memory()
    x_pinned.copy_(torch.from_numpy(np.random.default_rng(iseed).standard_normal(in_shape, dtype=np.float32)))
    x = x_pinned.numpy()
    rpool.add(nasm, x)
    arena_bytes = sum(nasm.ldata_info(i)["mem_size"] for i in range(nasm.num_ldata))
    flops = nasm.total_flops

    # ---- device-timed runs (inputs resident in HBM) ----
    group.time_runs(1, 1)                                   # first touch outside the timed region
    barrier(world, True)
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    ms, launches = group.time_runs(args.warmup, args.steps)
    clocks = sampler.stop()
    max_ms = reduce_max(ms, world, True)
    barrier(world, True)

    # ---- end to end through the public API: host input -> H2D -> run -> D2H result ----
    order = [api.BATCH, api.OUT_C, api.OUT_H, api.OUT_W] if seq == 0 else [api.BATCH, api.MAT_N, api.MAT_M]
    for _ in range(2):
        rpool.add(nasm, x); group.run(); group.wait(nasm); group.stop(); out = nasm.result(order)
    barrier(world, True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        rpool.add(nasm, x)            # rpool_add_nasm_raw_input: host -> device copy of this step's input
        group.run()
        group.wait(nasm)
        group.stop()
        out = nasm.result(order)      # dse_get_nasm_result: device -> host read of the step's result
    serial_ms = (time.perf_counter() - t0) * 1e3
    serial_max = reduce_max(serial_ms, world, True)
    barrier(world, True)
    assert np.isfinite(out).all()

    # Same calls, two graphs of the same network in flight (the serving loop of a user who double-buffers):
    # while the scheduler kernel works on one graph, the next step's input uploads and the previous step's
    # result downloads on the library's transfer stream.  Every timed iteration still contains one
    # host -> device input copy, one completed graph and one device -> host result read.
    L.aspen_b200_set_tile_quanta(q_h, q_w, 100000000)
    nasm2 = api.Nasm(dnn, batch, seq, min_ninst)
    L.aspen_b200_set_tile_profile(0)
    pair = [nasm, nasm2]
    for n_ in pair:                                           # both images built and warm
        rpool.add(n_, x); group.run(); group.wait(n_); group.stop(); out = n_.result(order)
    cur = 0
    barrier(world, True)
    t0 = time.perf_counter()
    rpool.add(pair[cur], x); group.run()      # step 1 starts inside the timed region
    for _ in range(args.steps - 1):
        nxt = cur ^ 1
        rpool.add(pair[nxt], x)       # upload of the next step's input, under the current graph's kernel
        group.wait(pair[cur])
        group.stop()
        group.run()                   # next graph starts
        out = pair[cur].result(order) # result of the finished graph, under the next graph's kernel
        cur = nxt
    group.wait(pair[cur]); group.stop(); out2 = pair[cur].result(order)
    e2e_ms = (time.perf_counter() - t0) * 1e3     # exactly `steps` uploads, runs and downloads
    if args.steps < 2:
        out = out2
    e2e_max = reduce_max(e2e_ms, world, True)
    barrier(world, True)
    assert np.isfinite(out).all() and np.array_equal(out, out2)

    # Extra, not the headline: both graphs armed in ONE scheduler launch (the reference's co-inference: several
    # nasms in one rpool).  Twice the ready tiles per layer for the same 148 SMs.
    co_iters = max(args.steps // 2, 1)
    co_ms, _ = group.time_runs(2, co_iters)
    co_max = reduce_max(co_ms, world, True)
    co_value = 2 * batch * co_iters * world / (co_max * 1e-3)
    barrier(world, True)

    if rank == 0:
        report(args, world, workload, batch, seq, nasm, flops, arena_bytes, ms, max_ms, e2e_max, serial_max, launches, clocks, x, out, cfg, wfile, wd, co_value)
    group.close(); nasm2.close(); nasm.close(); rpool.close(); dnn.close()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def report(args, world, workload, batch, seq, nasm, flops, arena_bytes, ms, max_ms, e2e_max, serial_max, launches, clocks, x, out, cfg, wfile, wd, co_value):
    from aspen_b200 import api
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak_tf = float(peaks.get("bf16_tflops_sustained", 0) or 0) or 1400.0
    peak_src = "of measured (MEASURED_PEAKS.json bf16_tflops_sustained)" if peaks else "of fallback (1.4 PFLOP/s sustained bf16)"
    achieved_tf = flops * args.steps / (ms * 1e-3) / 1e12
    value = job_value(batch, args.steps, world, max_ms)
    line = {
        "metric": "inferences_per_sec", "value": value, "unit": "inf/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": max_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32",
        "data": "synthetic",
        "config": {"workload": f"{workload}_bs{batch}_per_gpu", "seq_len": seq or None, "tile_profile": "b200 tensor-core quanta",
                   "tile_quanta": list(TILING[workload][:2]), "min_ninst_per_ldata": TILING[workload][2], "tiles": nasm.num_ninst, "flops_per_step": flops,
                   "l2": f"no flush: each step streams a {arena_bytes / 1e9:.2f} GB activation arena (> 126 MB L2)"},
        "clocks": clocks,
        "e2e": {"value": job_value(batch, args.steps, world, e2e_max), "unit": "inf/s", "h2d_bytes_per_step": int(x.nbytes),
                "d2h_bytes_per_step": int(out.nbytes), "ms_per_step": e2e_max / args.steps,
                "mode": "two graphs in flight: input upload and result download overlap the other graph's kernel",
                "serial_value": job_value(batch, args.steps, world, serial_max), "serial_ms_per_step": serial_max / args.steps},
        "gpu_launches": launches,
        "co_inference": {"graphs_per_launch": 2, "value": co_value, "unit": "inf/s",
                         "note": "two batch-sized graphs of the network in one rpool and one scheduler launch, inputs resident"},
        "roofline": {"bound": "tensor", "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved_tf / peak_tf,
                     "traffic": TRAFFIC_BYTES.get(workload), "peak_source": peak_src,
                     "note": "kernel = persistent scheduler_kernel<true> (whole tile graph, all layer types); operands are TF32, whose dense "
                             "peak is half the bf16 figure used as denominator"},
    }
    if not args.no_cpu_baseline and world == 1:
        from oracle import ref
        if ref.available():
            try:
                rate, cores = cpu_reference_rate(workload, cfg, wfile, 4, 10, 2, wd)
                line["cpu_baseline"] = {"value": rate, "unit": "inf/s", "cores": cores, "kind": "reference",
                                        "sample": f"reference DSE path ({cores} pthread workers), 10 timed passes of a batch-4 graph of the same network"}
            except Exception as exc:  # noqa: BLE001
                line["cpu_baseline"] = {"value": None, "unit": "inf/s", "cores": 0, "kind": "reference", "sample": f"failed: {exc}"}
        else:
            line["cpu_baseline"] = cpu_port_rate(workload)
    print(json.dumps(line), flush=True)


def cpu_port_rate(workload: str):
    """Fallback when the reference build is absent: the plain-C oracle on one sample."""
    from aspen_b200 import cfgs, weights
    from oracle import port
    builder, _, seq, scheme, wseed, _ = WORKLOADS[workload]
    text, wl = cfgs.BUILDERS[builder]()
    w = weights.make_weights(wl, wseed, scheme)
    first = port.parse_cfg(text)[0]["opts"]
    shape = (seq, int(first["M"])) if "M" in first else (int(first["height"]) * int(first["width"]), int(first["channels"]))
    x = np.random.default_rng(0).standard_normal(shape, dtype=np.float32)
    t0 = time.perf_counter()
    port.run(text, w, x, 1, seq)
    dt = time.perf_counter() - t0
    return {"value": 1.0 / dt, "unit": "inf/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": "plain-C oracle (OpenMP), one pass over one sample of the same network"}


if __name__ == "__main__":
    main()
