"""Command-line driver in the spirit of the reference's main.c (<dnn> <batch> <iterations> ... [seq]):

    python -m aspen_b200.run_case resnet50 --batch 4 --iters 3 [--seq 128] [--precision tf32|fp32]
                                  [--profile reference|b200] [--min-ninst 100]

Builds the network from a generated cfg with seeded synthetic weights, runs it `iters` times
through rpool / dse and prints the device time per run.  Used for profiler captures of the
persistent scheduler kernel on small cases.
"""
from __future__ import annotations

import argparse
import os
import tempfile

import numpy as np

from . import api, cfgs, weights


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("net", choices=sorted(cfgs.BUILDERS))
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--min-ninst", type=int, default=100)
    ap.add_argument("--precision", default="tf32", choices=["tf32", "fp32"])
    ap.add_argument("--profile", default="b200", choices=["reference", "b200"])
    args = ap.parse_args()
    wd = tempfile.mkdtemp(prefix="aspen_case_")
    cfg, wfile = os.path.join(wd, "net.cfg"), os.path.join(wd, "net.bin")
    wl = cfgs.write_cfg(args.net, cfg)
    weights.write_aspen_data(wfile, weights.make_weights(wl, 1, "n002" if args.seq else "he"))
    L = api.lib()
    L.aspen_b200_set_tile_profile(1 if args.profile == "b200" else 0)
    dnn = api.Dnn(cfg, wfile)
    nasm = api.Nasm(dnn, args.batch, args.seq, args.min_ninst)
    rpool = api.Rpool()
    group = api.DseGroup(0, 0 if args.precision == "tf32" else 1)
    group.set_rpool(rpool)
    i0 = nasm.ldata_info(0)
    x = np.random.default_rng(0).standard_normal((i0["W"], i0["H"]), dtype=np.float32)
    rpool.add(nasm, x)
    ms, launches = group.time_runs(args.warmup, args.iters)
    flops = nasm.total_flops
    print(f"{args.net} batch {args.batch} seq {args.seq}: {nasm.num_ninst} tiles, {ms / args.iters:.3f} ms/run, "
          f"{flops * args.iters / ms / 1e9:.1f} TFLOP/s, {launches} launches, status {group.status()}")
    group.close(); nasm.close(); rpool.close(); dnn.close()


if __name__ == "__main__":
    main()
