#!/usr/bin/env python3
"""Benchmark of the tiled execution path: ResNet-50 batch 32 per GPU through the ASPEN C API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload resnet50|bert_base]

One step = one pass of the tile graph (nasm) of a batch-32 inference over synthetic N(0,1) input
with seeded He-normal weights (no pretrained weights or dataset exist in this tree).  With N > 1
(launched by torch.distributed.run, one rank per GPU) every rank runs its own batch-32 graph on
its own GPU -- independent shards, no collective on the data path, weak scaling -- and rank 0
prints one JSON line with the whole-job inferences/s, timed on the device (CUDA events on the
engine's stream) as the maximum over ranks.

The device-timed region is repeated `--blocks` times (each exactly `--steps` passes) and the median
block is reported.  Beside the headline the line carries: `e2e` (host input -> H2D -> run -> D2H through
the public calls), `bert_base` (BERT-base S128 batch 32, the other half of the metric), and for N > 1
`strong` (the global batch of 32 split 32/N per GPU, results gathered on rank 0 in batch order) and
`by_model` (ResNet-50 batch 16 on one half of the GPUs, VGG-16 batch 16 on the other half).

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
    "vgg16": ("vgg16", 16, 0, "he", 2, 2),
}
# DRAM bytes per pass, from the ncu capture of the service-mode kernel summarised in profiles/ (265 MB per batch-4 pass, scaled by 8:
# activation traffic grows with the batch).  A timed launch serves `steps` passes.
TRAFFIC_BYTES_PER_STEP = {"resnet50": 2.12e9}
# Tiling of the nasm per workload: (row quantum, column quantum, min_ninst_per_ldata).  Tensor-core shaped
# quanta; the values a graph computes do not depend on them.  Each is the best of a measured sweep
# (quanta 64-256, min_ninst 100-592).
TILING = {"resnet50": (128, 128, 100), "bert_base": (256, 128, 148), "vgg16": (128, 128, 180)}
# The tile counts above are the best of a sweep in service mode (consecutive passes overlap, so fewer, larger tiles win); a graph
# that is launched by itself is latency bound in its narrow layers and wants more tiles per layer (180 / 296).


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

    def wait_first(self, timeout: float):
        """Blocks until the first sample has arrived (nvidia-smi needs a second or more to start, longer when eight
        ranks start one each), so that the timed region that follows is covered."""
        t0 = time.time()
        while not self.rows and time.time() - t0 < timeout:
            time.sleep(0.05)
        if not self.rows:
            log(f"clock sampler: no nvidia-smi sample for GPU {self.index} after {timeout:.0f} s")
        self.rows.clear()       # samples taken before the timed region do not count

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


class Net:
    """One network on this rank's GPU, driven through the public API: dnn + `graphs` tile graphs (nasms) of the same
    batch in one rpool, one dse group, a pinned host input."""

    def __init__(self, workload: str, batch: int, workdir: str, graphs: int = 1, min_ninst: int | None = None, group=None, rpool=None,
                 tokens: int = 0):
        import torch
        from aspen_b200 import api
        self.api, self.L = api, api.lib()
        self.workload, self.batch = workload, batch
        builder, _, self.seq, scheme, wseed, iseed = WORKLOADS[workload]
        self.cfg, self.wfile = prepare_files(workload, workdir)
        q_h, q_w, mn = TILING[workload]
        self.tiling = (q_h, q_w, min_ninst or mn)
        self.L.aspen_b200_set_tile_quanta(q_h, q_w, 100000000)
        self.dnn = api.Dnn(self.cfg, self.wfile)
        self.ids = None
        if tokens:
            # token-id input: seeded N(0, 0.02) token and position tables, ids uniform over the vocabulary (no tokenised text
            # exists in this tree); the hidden states are gathered on the device from 4 bytes per token
            rng = np.random.default_rng(iseed)
            i0m = int(open(self.cfg).read().split("M=")[1].split()[0])
            self.dnn.set_embedding((0.02 * rng.standard_normal((tokens, i0m))).astype(np.float32),
                                   (0.02 * rng.standard_normal((max(self.seq, 1), i0m))).astype(np.float32))
            self.ids = rng.integers(0, tokens, size=(batch, self.seq), dtype=np.int32)
        self.nasms = [api.Nasm(self.dnn, batch, self.seq, self.tiling[2]) for _ in range(graphs)]
        self.L.aspen_b200_set_tile_profile(0)
        self.own_group = group is None
        self.rpool = rpool or api.Rpool()
        self.group = group or api.DseGroup(0, 0)
        if self.own_group:
            self.group.set_rpool(self.rpool)
        i0 = self.nasms[0].ldata_info(0)
        shape = (i0["W"], i0["H"])
        self.x_pinned = torch.empty(shape, dtype=torch.float32).pin_memory()
        self.x_pinned.copy_(torch.from_numpy(np.random.default_rng(iseed).standard_normal(shape, dtype=np.float32)))
        self.x = self.x_pinned.numpy()
        self.order = [api.BATCH, api.OUT_C, api.OUT_H, api.OUT_W] if self.seq == 0 else [api.BATCH, api.MAT_N, api.MAT_M]
        self.flops = self.nasms[0].total_flops
        self.arena_bytes = sum(self.nasms[0].ldata_info(i)["mem_size"] for i in range(self.nasms[0].num_ldata))
        self.out = None

    def feed(self, n_):
        """This step's input: host hidden states / image (rpool_add_nasm_raw_input) or host token ids (aspen_b200_rpool_add_nasm_tokens)."""
        if self.ids is not None:
            self.rpool.add_tokens(n_, self.ids)
        else:
            self.rpool.add(n_, self.x)

    @property
    def h2d_bytes(self) -> int:
        return int(self.ids.nbytes if self.ids is not None else self.x.nbytes)

    def add_graph(self):
        """One more tile graph of the same network in the same rpool (the graphs in rotation of the service-mode legs).  Not
        before the per-launch timed blocks: a timed launch drains every graph of the pool."""
        q_h, q_w, mn = self.tiling
        self.L.aspen_b200_set_tile_quanta(q_h, q_w, 100000000)
        n_ = self.api.Nasm(self.dnn, self.batch, self.seq, mn)
        self.L.aspen_b200_set_tile_profile(0)
        self.nasms.append(n_)
        self.feed(n_); self.group.run(); self.group.wait(n_); self.group.stop(); self.out = n_.result(self.order)

    def warm(self):
        """Device images built, first touch done, one graph armed for the device-timed runs."""
        for n_ in self.nasms:
            self.feed(n_); self.group.run(); self.group.wait(n_); self.group.stop(); self.out = n_.result(self.order)
        self.feed(self.nasms[0])

    def time_blocks(self, warmup: int, steps: int, blocks: int):
        """`blocks` device-timed regions (CUDA events on the engine's stream) of exactly `steps` back-to-back passes of one graph."""
        ms, launches = [], 0
        for b in range(blocks):
            t, launches = self.group.time_runs(warmup if b == 0 else 1, steps)
            ms.append(t)
        return ms, launches

    def serve(self, graphs: int = 4):
        """Service mode (aspen_b200_dse_group_set_service) with `graphs` tile graphs of the network in rotation, each run once."""
        while len(self.nasms) < graphs:
            self.add_graph()
        self.group.set_service(True)
        for n_ in self.nasms:
            self.feed(n_)
        self.group.run()
        for n_ in self.nasms:
            self.group.wait(n_)
        self.group.stop()

    def time_served(self, warmup: int, steps: int, blocks: int):
        """`blocks` device-timed regions (CUDA events on the engine's stream) of exactly `steps` passes, dealt round robin to
        the graphs in rotation, inside one resident scheduler launch per region; every pass starts with the input layer's
        tiles (scatter / rounding of the resident input)."""
        ms, launches = [], 0
        for b in range(blocks):
            t, launches = self.group.time_passes(warmup if b == 0 else 2, steps)
            ms.append(t)
        return ms, launches

    def e2e_served(self, steps: int) -> float:
        """The serving loop in service mode: dse_group_run once, then per step rpool_add_nasm_raw_input (host -> device copy of
        the step's input, next to the graphs being computed), dse_wait_for_nasm_completion and dse_get_nasm_result (device ->
        host) of the oldest request; all graphs but one are in the kernel while that one uploads."""
        g, n = self.nasms, len(self.nasms)
        depth = n - 1                                # requests in the kernel while one more uploads
        t0 = time.perf_counter()
        self.feed(g[0]); self.group.run()
        for k in range(1, min(depth, steps)):
            self.feed(g[k % n])
        out = None
        for k in range(steps):
            if k + depth < steps:
                self.feed(g[(k + depth) % n])
            self.group.wait(g[k % n])
            out = g[k % n].result(self.order)
        self.group.stop()
        ms = (time.perf_counter() - t0) * 1e3     # exactly `steps` uploads, completed passes and downloads
        assert self.group.status() == 0 and np.isfinite(out).all()
        self.out = out
        return ms

    def e2e_serial(self, steps: int) -> float:
        nasm = self.nasms[0]
        t0 = time.perf_counter()
        for _ in range(steps):
            self.feed(nasm)                   # rpool_add_nasm_raw_input: host -> device copy of this step's input
            self.group.run()
            self.group.wait(nasm)
            self.group.stop()
            self.out = nasm.result(self.order)  # dse_get_nasm_result: device -> host read of the step's result
        return (time.perf_counter() - t0) * 1e3

    def close(self):
        if self.own_group:
            self.group.close()
        for n_ in reversed(self.nasms):
            n_.close()
        if self.own_group:
            self.rpool.close()
        self.dnn.close()


def measure_matmul_peaks():
    """Dense TF32 tensor peak of this GPU, measured the way MEASURED_PEAKS.json measures bf16: torch.matmul 8192^3
    with TF32 enabled, best of 10 (burst) and back to back for about 2 s (sustained)."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    n = 8192
    a = torch.randn(n, n, device="cuda"); b = torch.randn(n, n, device="cuda")
    for _ in range(3):
        a @ b
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); a @ b; e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0, k = time.time(), 0
    e0.record()
    while time.time() - t0 < 2.0:
        for _ in range(20):
            a @ b
        k += 20
        torch.cuda.synchronize()
    e1.record(); torch.cuda.synchronize()
    flop = 2.0 * n ** 3
    del a, b
    torch.cuda.empty_cache()
    return {"tf32_tflops": flop / best / 1e9, "tf32_tflops_sustained": flop * k / e0.elapsed_time(e1) / 1e9}


def gather_rows(local: np.ndarray, world: int):
    """Results of all ranks on rank 0, in rank (= batch) order.  NCCL moves a few KB of logits after the timed region;
    the data path itself has no collective."""
    import torch
    import torch.distributed as dist
    t = torch.from_numpy(np.ascontiguousarray(local)).cuda()
    parts = [torch.empty_like(t) for _ in range(world)] if dist.get_rank() == 0 else None
    dist.gather(t, parts, dst=0)
    return np.concatenate([p.cpu().numpy() for p in parts]) if parts else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--blocks", type=int, default=5, help="repetitions of the device-timed region; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="resnet50", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--keep-hidden-states", action="store_true",
                    help="also materialise the pre-add output of every layer whose residual add is fused into it (the library's default)")
    ap.add_argument("--no-extras", action="store_true", help="headline only: no BERT-base, strong-scaling or by-model legs")
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
    batch = WORKLOADS[workload][1]

    if args.dry_run:
        barrier(world, False)
        my_ms = 10.0 * args.steps * (1.0 + 0.1 * rank)
        max_ms = reduce_max(my_ms, world, False)
        # strong split of the global batch (32 samples -> 32 / world per rank) and the by-model split, as the GPU path shards them
        shard = strong_shard(batch, rank, world)
        model = by_model_assignment(rank, world)
        parts = gather_objects((rank, shard, model), world)
        barrier(world, False)
        if rank == 0:
            print(json.dumps({"metric": "inferences_per_sec", "value": job_value(batch, args.steps, world, max_ms), "unit": "inf/s",
                              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": max_ms / args.steps,
                              "scaling": "weak", "data": "dry-run", "higher_is_better": True,
                              "strong": {"shards": [p[1] for p in parts], "graphs_in_rotation": graphs_in_rotation(batch // world)},
                              "by_model": {"assignment": [p[2] for p in parts]}}), flush=True)
        return

    from aspen_b200 import api
    L = api.lib()
    if L.aspen_b200_set_device(local_rank) != 0:
        raise SystemExit("no CUDA device for this rank: " + api.last_error())
    wd = tempfile.mkdtemp(prefix=f"aspen_bench_r{rank}_")
    # A convolution / matmul with the residual add fused into its epilogue writes the sum; its own pre-add matrix has no reader
    # but a debugging read, and is not written unless asked for.  Every other layer's output stays readable.
    L.aspen_b200_set_hidden_states(1 if args.keep_hidden_states else 0)

    sampler = ClockSampler(local_rank)
    sampler.start()
    net = Net(workload, batch, wd)
    net.warm()
    sampler.wait_first(5.0)

    # ---- one scheduler launch per step, one graph (inputs scattered beforehand): the explanatory figure ----
    barrier(world, True)
    pl_ms, _ = net.time_blocks(args.warmup, args.steps, 3)
    pl_max = float(np.median([reduce_max(t, world, True) for t in pl_ms]))
    barrier(world, True)
    net.e2e_serial(2)
    barrier(world, True)
    serial_max = reduce_max(net.e2e_serial(args.steps), world, True)
    single_out = net.out.copy()

    # ---- the headline: service mode, device-timed (inputs resident in HBM): `blocks` regions of exactly `steps` passes ----
    net.serve(4)
    barrier(world, True)
    block_ms, launches = net.time_served(args.warmup, args.steps, args.blocks)
    clocks = sampler.stop()
    block_max = [reduce_max(t, world, True) for t in block_ms]
    barrier(world, True)
    ms, max_ms = float(np.median(block_ms)), float(np.median(block_max))

    # ---- end to end through the public API: host input -> H2D -> pass -> D2H result, every step ----
    net.e2e_served(4)
    barrier(world, True)
    e2e_max = reduce_max(net.e2e_served(args.steps), world, True)
    barrier(world, True)
    out = net.out
    served_ok = bool(np.array_equal(out, single_out))      # a served pass gives the values of a launched run, bit for bit
    if not served_ok:
        log("served result differs from the launched run's")
    net.group.set_service(False)
    per_launch = {"value": job_value(batch, args.steps, world, pl_max), "unit": "inf/s", "ms_per_step": pl_max / args.steps,
                  "served_result_identical": served_ok,
                  "note": "one graph, dse_group_run launches the scheduler once per step, input scattered before the timed region"}

    extras = {}
    if not args.no_extras:
        extras = extra_legs(args, rank, world, wd, net, workload)

    if rank == 0:
        report(args, world, workload, batch, net, ms, max_ms, block_max, e2e_max, serial_max, launches, clocks, out, wd, per_launch, extras)
    net.close()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def graphs_in_rotation(samples: int) -> int:
    """Graphs a GPU keeps in rotation in service mode for shards of `samples` samples.  A small shard leaves most SMs idle in its
    narrow layers, so more of them are kept in flight (measured on one GPU: 12 graphs of 4 samples run at 0.39 ms per pass,
    8 at 0.43, 4 at 0.65; batch-32 graphs gain nothing beyond 4)."""
    return max(4, min(12, 96 // max(samples, 1)))


def strong_shard(global_batch: int, rank: int, world: int):
    """Samples [lo, hi) of the global batch that rank `rank` of `world` computes (configs[1]: 32 -> 32 / N per GPU)."""
    per = global_batch // world
    return [rank * per, (rank + 1) * per]


def by_model_assignment(rank: int, world: int):
    """configs[2]: ResNet-50 batch 16 on the first half of the GPUs, VGG-16 batch 16 on the second half; each model's
    batch is split evenly over its GPUs.  Returns (network, samples on this rank)."""
    if world < 2:
        return None
    half = world // 2
    return ["resnet50", 16 // half] if rank < half else ["vgg16", 16 // (world - half)]


def gather_objects(obj, world: int):
    if world == 1:
        return [obj]
    import torch.distributed as dist
    parts = [None] * world
    dist.all_gather_object(parts, obj)
    return parts


def extra_legs(args, rank, world, wd, net, workload):
    """The other half of the metric (BERT-base batch 32) and the two multi-GPU splits the configurations name."""
    extras = {}
    steps = args.steps
    # ---- BERT-base S128 batch 32 per GPU (configs[3]) ----
    if workload == "resnet50":
        b = Net("bert_base", WORKLOADS["bert_base"][1], wd, tokens=30522)
        b.warm()
        barrier(world, True)
        pms, _ = b.time_blocks(3, steps, 3)
        pmax = float(np.median([reduce_max(t, world, True) for t in pms]))
        b.serve(4)
        barrier(world, True)
        bms, _ = b.time_served(3, steps, 3)
        bmax = float(np.median([reduce_max(t, world, True) for t in bms]))
        b.e2e_served(4)
        barrier(world, True)
        be2e = reduce_max(b.e2e_served(steps), world, True)
        barrier(world, True)
        b.group.set_service(False)
        tf = b.flops * steps / (float(np.median(bms)) * 1e-3) / 1e12
        extras["bert_base"] = {"metric": "sequences_per_sec", "config": {"workload": "bert_base_s128_bs32_per_gpu", "tile_quanta": list(b.tiling[:2]),
                                                                          "min_ninst_per_ldata": b.tiling[2], "tiles": b.nasms[0].num_ninst},
                               "value": job_value(b.batch, steps, world, bmax), "unit": "seq/s", "ms_per_step": bmax / steps,
                               "e2e": {"value": job_value(b.batch, steps, world, be2e), "unit": "seq/s", "h2d_bytes_per_step": b.h2d_bytes,
                                       "input": "token ids (int32), embedded on the device",
                                       "d2h_bytes_per_step": int(b.out.nbytes)},
                               "per_launch": {"value": job_value(b.batch, steps, world, pmax), "unit": "seq/s", "ms_per_step": pmax / steps},
                               "achieved_tflops": tf, "flops_per_step": b.flops}
        b.close()
    # ---- strong scaling (configs[1]): the global batch of 32 split 32 / N per GPU, results gathered on rank 0 ----
    gb = WORKLOADS[workload][1]
    if world > 1 and gb % world == 0:
        lo, hi = strong_shard(gb, rank, world)
        # every GPU serves its samples of one global batch after the other
        rotation = graphs_in_rotation(hi - lo)
        s = Net(workload, hi - lo, wd, graphs=1)
        rows = net.x.shape[0] // gb
        s.x_pinned.copy_(net.x_pinned[lo * rows:hi * rows])       # this rank's samples of the global batch
        s.warm()
        s.serve(rotation)
        barrier(world, True)
        sms, _ = s.time_served(3, steps, 3)
        smax = float(np.median([reduce_max(t, world, True) for t in sms]))
        s.e2e_served(rotation)
        barrier(world, True)
        se2e = reduce_max(s.e2e_served(steps), world, True)
        s.group.set_service(False)
        local = s.out.reshape(hi - lo, -1)
        whole = gather_rows(local, world)
        ok = None
        if rank == 0:
            want = net.out.reshape(gb, -1)
            ok = bool(whole.shape == want.shape and np.abs(whole - want).max() <= 2e-3 * np.abs(want).max()
                      and (whole.argmax(1) == want.argmax(1)).all())
        extras["strong"] = {"config": {"workload": f"{workload}_global_bs{gb}", "per_gpu_batch": hi - lo, "tiles_per_gpu": s.nasms[0].num_ninst,
                                       "execution": f"service mode, {rotation} shards in rotation per GPU"},
                            "value": gb * steps / (smax * 1e-3), "unit": "inf/s", "ms_per_step": smax / steps, "scaling": "strong",
                            "e2e_value": gb * steps / (se2e * 1e-3), "gathered_equals_single_gpu_batch": ok}
        s.close()
    # ---- by model (configs[2]): ResNet-50 batch 16 on one half of the GPUs, VGG-16 batch 16 on the other ----
    assign = by_model_assignment(rank, world)
    if assign and assign[1] >= 1:
        name, nb = assign
        m = Net(name, nb, wd, graphs=1)
        m.warm()
        m_rotation = graphs_in_rotation(nb)
        m.serve(m_rotation)
        barrier(world, True)
        mms, _ = m.time_served(3, steps, 3)
        mmax = float(np.median([reduce_max(t, world, True) for t in mms]))
        barrier(world, True)
        m.group.set_service(False)
        mine = gather_objects((name, nb, float(np.median(mms)) / steps), world)
        extras["by_model"] = {"config": {"workload": "resnet50_bs16_plus_vgg16_bs16", "assignment": [[p[0], p[1]] for p in mine],
                                         "execution": f"service mode, {m_rotation} graphs in rotation per GPU"},
                              "value": 32 * steps / (mmax * 1e-3), "unit": "inf/s", "ms_per_step": mmax / steps,
                              "ms_per_step_per_rank": [p[2] for p in mine]}
        m.close()
    return extras


def report(args, world, workload, batch, net, ms, max_ms, block_max, e2e_max, serial_max, launches, clocks, out, wd, per_launch, extras):
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    seq, flops, nasm = net.seq, net.flops, net.nasms[0]
    peak_tf = float(peaks.get("bf16_tflops_sustained", 0) or 0) or 1400.0
    peak_src = "of measured (MEASURED_PEAKS.json bf16_tflops_sustained)" if peaks else "of fallback (1.4 PFLOP/s sustained bf16)"
    achieved_tf = flops * args.steps / (ms * 1e-3) / 1e12
    value = job_value(batch, args.steps, world, max_ms)
    spread = (max(block_max) - min(block_max)) / max_ms if block_max else 0.0
    line = {
        "metric": "inferences_per_sec", "value": value, "unit": "inf/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": max_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32",
        "data": "synthetic",
        "config": {"workload": f"{workload}_bs{batch}_per_gpu", "seq_len": seq or None, "tile_profile": "b200 tensor-core quanta",
                   "tile_quanta": list(net.tiling[:2]), "min_ninst_per_ldata": net.tiling[2], "tiles": nasm.num_ninst, "flops_per_step": flops,
                   "execution": f"service mode: {len(net.nasms)} tile graphs of batch {batch} in rotation inside one resident scheduler launch per "
                                "timed block; every step is one complete pass of one graph, input layer's scatter included",
                   "hidden_states": "all materialised" if args.keep_hidden_states else
                                    "pre-add outputs of layers with a fused residual add are not materialised; every other layer's output is",
                   "l2": f"no flush: each step streams a {net.arena_bytes / 1e9:.2f} GB activation arena (> 126 MB L2)"},
        "timing": {"blocks": len(block_max), "block_ms": [round(t, 4) for t in block_max], "reported": "median block", "spread_frac": spread},
        "clocks": clocks,
        "e2e": {"value": job_value(batch, args.steps, world, e2e_max), "unit": "inf/s", "h2d_bytes_per_step": net.h2d_bytes,
                "d2h_bytes_per_step": int(out.nbytes), "ms_per_step": e2e_max / args.steps,
                "mode": "service mode: per step one rpool_add_nasm_raw_input (upload), one completed pass, one dse_get_nasm_result (download); "
                        f"{len(net.nasms) - 1} requests in the resident kernel while one more uploads",
                "serial_value": job_value(batch, args.steps, world, serial_max), "serial_ms_per_step": serial_max / args.steps},
        "gpu_launches": launches,
        "per_launch": per_launch,
        "roofline": {"bound": "tensor", "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved_tf / peak_tf,
                     "traffic": TRAFFIC_BYTES_PER_STEP[workload] * args.steps if workload in TRAFFIC_BYTES_PER_STEP else None,
                     "traffic_per_step": TRAFFIC_BYTES_PER_STEP.get(workload), "peak_source": peak_src,
                     "note": "kernel = persistent scheduler_kernel<true, false, true> (whole tile graphs, all layer types; one launch per timed block); "
                             "operands are TF32: see peak_tf32"},
    }
    if world == 1 and not args.no_extras:
        try:
            tf32 = measure_matmul_peaks()
            line["roofline"]["peak_tf32"] = tf32
            line["roofline"]["frac_tf32"] = achieved_tf / tf32["tf32_tflops_sustained"]
            if "bert_base" in extras:
                extras["bert_base"]["roofline"] = {"bound": "tensor", "achieved": extras["bert_base"]["achieved_tflops"], "peak": peak_tf, "unit": "TFLOP/s",
                                                   "frac": extras["bert_base"]["achieved_tflops"] / peak_tf,
                                                   "frac_tf32": extras["bert_base"]["achieved_tflops"] / tf32["tf32_tflops_sustained"]}
        except Exception as exc:  # noqa: BLE001
            line["roofline"]["peak_tf32"] = f"not measured: {exc}"
    line.update(extras)
    if not args.no_cpu_baseline and world == 1:
        from oracle import ref
        if ref.available():
            try:
                passes = 8
                rate, cores = cpu_reference_rate(workload, net.cfg, net.wfile, batch, passes, 2, wd)
                line["cpu_baseline"] = {"value": rate, "unit": "inf/s", "cores": cores, "kind": "reference",
                                        "sample": f"reference DSE path ({cores} pthread workers), {passes} timed passes of one batch-{batch} graph of the same network"}
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
