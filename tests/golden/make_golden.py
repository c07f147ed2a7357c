"""Generates the committed fixtures under tests/golden/ by running the UNMODIFIED reference
(oracle/_ref/libaspen_ref.so, built from the reference sources by oracle/Makefile).

    python tests/golden/make_golden.py [net ...]      (no names: every fixture)

Inputs and weights are seeded (tests/harness.py), so only outputs are stored:
  values_<net>.npz   reference layer-walk activations (final layer + a few hidden layers)
  graph_<net>.json   reference tiler geometry per layer + sha256 of the reference's .nasm text
"""
import hashlib
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import harness  # noqa: E402
from oracle import ref  # noqa: E402

VALUE_CASES = [("tiny_cnn", 2, 0, 20), ("tiny_transformer", 2, 16, 20), ("tiny_gpt", 2, 16, 20), ("custom", 2, 0, 50),
               ("tiny_yolo", 2, 0, 8), ("tiny_acts", 3, 0, 8)]
GRAPH_CASES = [("tiny_yolo", 2, 0, 8), ("tiny_acts", 3, 0, 8), ("tiny_cnn", 2, 0, 20), ("tiny_transformer", 2, 16, 20), ("custom", 2, 0, 50), ("resnet50", 1, 0, 50),
               ("resnet50", 4, 0, 100), ("vgg16", 1, 0, 100), ("bert_base", 1, 32, 20), ("bert_base", 4, 128, 100),
               ("gpt2_124M", 2, 64, 50)]


def nasm_digest(path):
    h = hashlib.sha256()
    for line in open(path, "rb"):
        if not line.startswith(b"DNN_NAME"):
            h.update(line)
    return h.hexdigest()


def main():
    wd = tempfile.mkdtemp()
    only = set(sys.argv[1:])
    for name, batch, seq, mn in VALUE_CASES:
        if only and name not in only:
            continue
        cfg, wf = harness.prepare(name, wd)
        rn = ref.RefNet(cfg, wf, batch, seq, min_ninst=mn)
        i0 = rn.ldata_info(0)
        x = harness.make_input(name, (i0["W"], i0["H"]))
        rn.walk(x, threads=1)
        keep = sorted(set([1, 2, rn.num_ldata // 2, rn.num_ldata - 2, rn.num_ldata - 1]) | set(range(1, min(rn.num_ldata, 14))))
        arrays = {f"layer_{i}": rn.ldata(i) for i in keep if 0 < i < rn.num_ldata}
        np.savez_compressed(os.path.join(HERE, f"values_{name}.npz"), **arrays)
        rn.close()
        print("values", name, {k: v.shape for k, v in arrays.items()})
    for name, batch, seq, mn in GRAPH_CASES:
        if only and name not in only:
            continue
        cfg, _ = harness.prepare(name, wd)
        rn = ref.RefNet(cfg, None, batch, seq, min_ninst=mn, with_parents=True)
        out = os.path.join(wd, "g.nasm")
        rn.save_nasm(out)
        info = {
            "net": name, "batch": batch, "seq": seq, "min_ninst": mn, "num_ninst": rn.num_ninst,
            "ldata": [[rn.ldata_info(i)[k] for k in ref.LDATA_FIELDS] for i in range(rn.num_ldata)],
            "nasm_sha256": nasm_digest(out),
        }
        with open(os.path.join(HERE, f"graph_{name}_B{batch}_S{seq}.json"), "w") as f:
            json.dump(info, f)
        rn.close()
        print("graph", name, batch, seq, rn.num_ninst)


if __name__ == "__main__":
    main()
