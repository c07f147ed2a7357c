"""Shared plumbing of the parity tests: build a seeded network for both libraries, run the
reference's layer walk (CPU) and this library's device engine, and compare every layer."""
from __future__ import annotations

import os

import numpy as np

from aspen_b200 import api, cfgs, weights

# name -> (builder kwargs, weight scheme, seeds (weights, input))
NETS = {
    "tiny_cnn": ({}, "he", (11, 10)),
    "tiny_transformer": ({}, "n002", (13, 12)),
    "tiny_gpt": ({"masked": True, "pre_ln": True}, "n002", (15, 14)),
    # head size 32: the smallest the fused attention tile takes (the 4-head variants above have head size 16)
    "tiny_attn": ({"heads": 2}, "n002", (21, 20)),
    "tiny_attn_causal": ({"heads": 2, "masked": True, "pre_ln": True}, "n002", (23, 22)),
    "custom": ({}, "he", (5, 6)),
    "tiny_yolo": ({}, "he", (17, 16)),
    "tiny_acts": ({}, "he", (19, 18)),
    "resnet50": ({}, "he", (1, 0)),
    "vgg16": ({}, "he", (2, 2)),
    "bert_base": ({}, "n002", (3, 3)),
    "gpt2_124M": ({}, "n002", (4, 4)),
    # GPT-2 with the tail the reference's cfg leaves out: final layernorm and the 50257-row output head
    "gpt2_lm": ({"with_lm_head": True}, "n002", (4, 4)),
}
_BUILDER = {"tiny_gpt": "tiny_transformer", "gpt2_lm": "gpt2_124M", "tiny_attn": "tiny_transformer", "tiny_attn_causal": "tiny_transformer"}


def prepare(name: str, workdir: str):
    """Writes <name>.cfg and <name>.bin (seeded weights) into workdir; returns their paths."""
    kw, scheme, (wseed, _) = NETS[name]
    cfg = os.path.join(workdir, name + ".cfg")
    wfile = os.path.join(workdir, name + ".bin")
    if not (os.path.exists(cfg) and os.path.exists(wfile)):
        wl = cfgs.write_cfg(_BUILDER.get(name, name), cfg, **kw)
        weights.write_aspen_data(wfile, weights.make_weights(wl, wseed, scheme))
    return cfg, wfile


def make_input(name: str, shape) -> np.ndarray:
    """Packed input as rpool_add_nasm_raw_input takes it: [columns W][rows H] == NHWC / [B][S][M]."""
    return weights.make_input(shape, NETS[name][2][1])


def compare(a: np.ndarray, b: np.ndarray, rel: float, abs_floor: float):
    """Mismatch rule of the reference's compare_float_array (src/util.c:368-391): an element
    differs when BOTH its relative and its absolute error exceed their thresholds.  Returns
    (number of mismatches, max abs error, max rel error among elements above the floor)."""
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    err = np.abs(a - b)
    denom = np.maximum(np.abs(b), 1e-30)
    relerr = err / denom
    bad = (relerr >= rel) & (err >= abs_floor)
    big = err >= abs_floor
    return int(bad.sum()), float(err.max(initial=0.0)), float(relerr[big].max(initial=0.0))


class Device:
    """One network on the device engine, driven like the reference's example programs."""

    def __init__(self, cfg: str, wfile: str | None, batch: int, seq: int = 0, min_ninst: int = 100, precision: int = 0,
                 profile: int = 0):
        L = api.lib()
        if profile in (0, 1):
            L.aspen_b200_set_tile_profile(profile)   # any other value: keep the quanta the caller has set
        self.dnn = api.Dnn(cfg, wfile)
        self.nasm = api.Nasm(self.dnn, batch, seq, min_ninst)
        L.aspen_b200_set_tile_profile(0)
        self.rpool = api.Rpool()
        self.group = api.DseGroup(0, precision)
        self.group.set_rpool(self.rpool)

    def input_shape(self):
        i0 = self.nasm.ldata_info(0)
        return (i0["W"], i0["H"])

    def run(self, x: np.ndarray) -> int:
        self.rpool.add(self.nasm, x)
        self.group.run()
        self.group.wait(self.nasm)
        self.group.stop()
        return self.group.status()

    def rerun(self) -> int:
        self.rpool.reset(self.nasm)
        self.group.run()
        self.group.wait(self.nasm)
        self.group.stop()
        return self.group.status()

    def close(self):
        self.group.close()
        self.nasm.close()
        self.rpool.close()
        self.dnn.close()


def layer_report(dev: Device, refnet, rel: float, abs_scale: float = 1e-5):
    """Per-layer comparison rows: (idx, type, mismatches, max abs err, max rel err, ref max |x|)."""
    rows = []
    for i in range(1, dev.nasm.num_ldata):
        got = dev.nasm.ldata(i)
        want = refnet.ldata(i)
        scale = float(np.abs(want).max(initial=0.0))
        bad, ea, er = compare(got, want, rel, abs_scale * max(scale, 1e-30) + 1e-30)
        rows.append((i, api.LAYER_TYPES[dev.nasm.ldata_info(i)["type"]], bad, ea, er, scale))
    return rows
