"""Command-line driver in the spirit of the reference's main.c (<dnn> <batch> <iterations> ... [seq]):

    python -m aspen_b200.run_case resnet50 --batch 4 --iters 3 [--seq 128] [--precision tf32|fp32]
                                  [--profile reference|b200] [--quanta H W] [--min-ninst 100] [--layer-table]

Builds the network from a generated cfg with seeded synthetic weights, runs it `iters` times
through rpool / dse and prints the device time per run.  Used for profiler captures of the
persistent scheduler kernel on small cases.

`--layer-table` (sets ASPEN_B200_PROFILE=1 before the library loads) prints, per layer shape class,
the tiles per run, the executors' microseconds per tile and what that is per SM: TFLOP/s for the
contraction tiles (2 M N K per tile), GB/s of algorithmic bytes for the memory-bound tiles
(residual 12 B per element, layernorm 8 B, pooling 4 B x (inputs read once + outputs), softmax 8 B),
each with its fraction of one SM's share of the roof given by --tensor-peak / --hbm-peak.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile

import numpy as np

GEMM_TYPES = {"CONV", "FC", "MATMUL", "K_ATTENTION", "V_ATTENTION"}


def layer_table(api, nasm, dnn, prof, runs, n_sms, tensor_peak_tf, hbm_peak_gbs):
    """Markdown rows from the scheduler's per-layer accounting, identical layers merged into one shape class."""
    classes = {}
    for l, v in sorted(prof["layers"].items()):
        li = nasm.ldata_info(l)
        p = dnn.layer_params(l)
        tname = api.LAYER_TYPES[li["type"]]
        k = li["flop_per_output"] // 2
        key = (tname, li["H"], li["W"], k, li["tile_h"], li["tile_w"])
        c = classes.setdefault(key, {"layers": 0, "ns": 0, "tiles": 0, "flop": 0.0, "bytes": 0.0})
        c["layers"] += 1
        c["ns"] += v["ns"]
        c["tiles"] += v["tiles"]
        elems = float(li["H"]) * li["W"] * runs
        if tname in GEMM_TYPES:
            c["flop"] += float(li["flop_per_output"]) * elems
        elif tname == "RESIDUAL":
            c["bytes"] += 12.0 * elems
        elif tname in ("LAYERNORM", "SOFTMAX"):
            c["bytes"] += 8.0 * elems
        elif tname in ("MAXPOOL", "AVGPOOL"):
            ratio = (p[api.IN_H] * p[api.IN_W]) / max(p[api.OUT_H] * p[api.OUT_W], 1)
            c["bytes"] += 4.0 * elems * (1.0 + ratio)
        else:
            c["bytes"] += 8.0 * elems
    tf_sm, gb_sm = tensor_peak_tf / n_sms, hbm_peak_gbs / n_sms
    out = ["| layer type | out rows x cols | K | tile | layers | tiles/run | us/tile | per SM | of one SM's roof |", "|---|---|---|---|---|---|---|---|---|"]
    for (tname, H, W, k, th, tw), c in classes.items():
        us = c["ns"] / max(c["tiles"], 1) / 1e3
        if tname in GEMM_TYPES:
            rate = c["flop"] / max(c["ns"], 1) / 1e3            # FLOP per ns = GFLOP/s -> /1e3 = TFLOP/s
            per, frac = f"{rate:.2f} TFLOP/s", rate / tf_sm
        else:
            rate = c["bytes"] / max(c["ns"], 1)                  # bytes per ns = GB/s
            per, frac = f"{rate:.1f} GB/s", rate / gb_sm
        out.append(f"| {tname} | {H} x {W} | {k if tname in GEMM_TYPES else '-'} | {th} x {tw} | {c['layers']} | {c['tiles'] // runs} | {us:.1f} | {per} | {frac:.3f} |")
    return "\n".join(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("net")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--min-ninst", type=int, default=100)
    ap.add_argument("--precision", default="tf32", choices=["tf32", "fp32"])
    ap.add_argument("--profile", default="b200", choices=["reference", "b200"])
    ap.add_argument("--quanta", type=int, nargs=2, metavar=("H", "W"), help="tile row / column quanta (overrides --profile)")
    ap.add_argument("--service", type=int, default=0, metavar="GRAPHS",
                    help="service mode: this many graphs of the network in rotation inside one resident scheduler launch")
    ap.add_argument("--drop-pre-add", action="store_true", help="aspen_b200_set_hidden_states(0): outputs that only a fused residual add reads are not written")
    ap.add_argument("--layer-table", action="store_true", help="per-layer-class time accounting (see the module docstring)")
    ap.add_argument("--tensor-peak", type=float, default=1353.0, help="TFLOP/s the per-SM tensor fractions are quoted against")
    ap.add_argument("--hbm-peak", type=float, default=6454.9, help="GB/s the per-SM bandwidth fractions are quoted against")
    args = ap.parse_args()
    if args.layer_table:
        os.environ["ASPEN_B200_PROFILE"] = "1"
    from . import api, cfgs, weights
    if args.net not in cfgs.BUILDERS:
        raise SystemExit(f"unknown net {args.net}; one of {sorted(cfgs.BUILDERS)}")
    wd = tempfile.mkdtemp(prefix="aspen_case_")
    cfg, wfile = os.path.join(wd, "net.cfg"), os.path.join(wd, "net.bin")
    wl = cfgs.write_cfg(args.net, cfg)
    weights.write_aspen_data(wfile, weights.make_weights(wl, 1, "n002" if args.seq else "he"))
    L = api.lib()
    if args.quanta:
        L.aspen_b200_set_tile_quanta(args.quanta[0], args.quanta[1], 100000000)
    else:
        L.aspen_b200_set_tile_profile(1 if args.profile == "b200" else 0)
    if args.drop_pre_add:
        L.aspen_b200_set_hidden_states(0)
    dnn = api.Dnn(cfg, wfile)
    nasm = api.Nasm(dnn, args.batch, args.seq, args.min_ninst)
    others = [api.Nasm(dnn, args.batch, args.seq, args.min_ninst) for _ in range(max(args.service - 1, 0))]
    L.aspen_b200_set_tile_profile(0)
    rpool = api.Rpool()
    group = api.DseGroup(0, 0 if args.precision == "tf32" else 1)
    group.set_rpool(rpool)
    i0 = nasm.ldata_info(0)
    x = np.random.default_rng(0).standard_normal((i0["W"], i0["H"]), dtype=np.float32)
    rpool.add(nasm, x)
    if args.service:
        # every graph once (images built, first touch), then the timed passes dealt round robin inside resident launches
        group.set_service(True)
        for n_ in others:
            rpool.add(n_, x)
        group.run()
        for n_ in [nasm] + others:
            group.wait(n_)
        group.stop()
        if args.layer_table:
            group.profile()
        timed = group.time_passes
    else:
        if args.layer_table:
            group.time_runs(1, 1)
            group.profile()                               # clears the counters of the first-touch run
        timed = group.time_runs
    ms, launches = timed(args.warmup, args.iters)
    flops = nasm.total_flops
    print(f"{args.net} batch {args.batch} seq {args.seq}: {nasm.num_ninst} tiles, {ms / args.iters:.3f} ms/run, "
          f"{flops * args.iters / ms / 1e9:.1f} TFLOP/s, {launches} launches, status {group.status()}")
    if args.layer_table:
        p = group.profile()
        if p is None:
            print("no profile: the library was loaded before ASPEN_B200_PROFILE was set", file=sys.stderr)
        else:
            runs = args.warmup + args.iters
            n = p["ctas"] * runs
            busy = sum(v["ns"] for v in p["layers"].values())
            print(f"per CTA and run (us): tiles {busy / n / 1e3:.1f}, waiting for a ready tile {p['wait_ns'] / n / 1e3:.1f}, "
                  f"completion + child updates (scheduler warp) {p['complete_ns'] / n / 1e3:.1f}; {p['ctas']} CTAs")
            print(layer_table(api, nasm, dnn, p, runs, p["ctas"], args.tensor_peak, args.hbm_peak))
    group.close()
    for n_ in others:
        n_.close()
    nasm.close(); rpool.close(); dnn.close()


if __name__ == "__main__":
    main()
