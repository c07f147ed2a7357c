"""TEST INFRASTRUCTURE ONLY: whole-network driver of the CPU oracle (oracle/oracle_tiles.c).

Parses a cfg with the reference's rules (section/key mapping: reference src/darknet_parser.c:455-552,
size inference: src/input_parser.c:35-129), then evaluates the layers one after the other with the
plain-C layer functions.  Returns every layer's activations packed as [columns][rows] -- the same
view `refwalk_get_ldata` and `aspen_b200_nasm_get_ldata_packed` give.  Nothing in the product
imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_lib = None

ACT = {None: 0, "logistic": 1, "linear": 0, "none": 0, "tanh": 3, "relu": 4, "leaky": 5, "elu": 6, "selu": 7, "gelu": 8,
       "gelu_acc": 9}
TYPE = {"[net]": "input", "[network]": "input", "[conv]": "conv", "[convolutional]": "conv", "[shortcut]": "residual",
        "[max]": "maxpool", "[maxpool]": "maxpool", "[avg]": "avgpool", "[avgpool]": "avgpool", "[conn]": "fc",
        "[connected]": "fc", "[soft]": "softmax", "[softmax]": "softmax", "[matmul]": "matmul",
        "[attention_k]": "attn_k", "[attention_v]": "attn_v", "[layernorm]": "layernorm", "[yolo]": "yolo", "[append]": "append"}


def build() -> str:
    src = os.path.join(_HERE, "oracle_tiles.c")
    if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.run(["gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-Wall", "-o", _LIB, src, "-lm"], check=True)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def parse_cfg(text: str):
    """-> list of dicts {type, opts}; blanks anywhere in a line are dropped, '#'/';' start comments."""
    layers = []
    for raw in text.splitlines():
        line = "".join(ch for ch in raw if ch not in " \t\r\n")
        if not line or line[0] in "#;":
            continue
        if line[0] == "[":
            if line in TYPE:
                layers.append({"type": TYPE[line], "opts": {}})
            else:
                layers.append(None)          # unsupported section: dropped, its options too
            continue
        if layers and layers[-1] is not None and "=" in line:
            k, v = line.split("=", 1)
            layers[-1]["opts"].setdefault(k, v)
    return [l for l in layers if l is not None]


def run(cfg_text: str, weight_list, x: np.ndarray, batch: int, seq: int = 0):
    """weight_list: [(weight, bias)] in weight-file order (see aspen_b200/weights.py).
    x: packed input [columns][rows].  Returns list of packed per-layer outputs."""
    L = lib()
    layers = parse_cfg(cfg_text)
    outs, shapes = [], []      # shapes: dict with C/H/W or M per layer
    wi = 0
    for i, lay in enumerate(layers):
        o, t = lay["opts"], lay["type"]
        geti = lambda k, d=0: int(o.get(k, d))
        act = ACT[o.get("activation")]
        par = None if t == "input" else i + (geti("parent") or -1)
        frm = i + geti("from") if geti("from") else None
        if t == "input":
            if geti("M"):
                sh = {"M": geti("M")}
            else:
                sh = {"C": geti("channels"), "H": geti("height"), "W": geti("width")}
            out = np.ascontiguousarray(x, dtype=np.float32).copy()
        elif t == "conv":
            ps = shapes[par]
            k, s, p, oc = geti("size"), geti("stride") or 1, geti("pad"), geti("filters") or geti("output")
            oh = (ps["H"] + 2 * p - (k - 1) - 1) // s + 1
            ow = (ps["W"] + 2 * p - (k - 1) - 1) // s + 1
            w, b = weight_list[wi]; wi += 1
            out = np.empty((batch * oh * ow, oc), np.float32)
            L.oracle_conv2d(_p(outs[par]), _p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(b)), _p(out), batch, ps["H"], ps["W"],
                            ps["C"], oc, k, k, s, p, act)
            sh = {"C": oc, "H": oh, "W": ow}
        elif t in ("maxpool", "avgpool"):
            ps = shapes[par]
            k, s, p = geti("size"), geti("stride") or 1, geti("pad")
            oh = (ps["H"] + 2 * p - (k - 1) - 1) // s + 1
            ow = (ps["W"] + 2 * p - (k - 1) - 1) // s + 1
            out = np.empty((batch * oh * ow, ps["C"]), np.float32)
            fn = L.oracle_maxpool2d if t == "maxpool" else L.oracle_avgpool2d
            fn(_p(outs[par]), _p(out), batch, ps["H"], ps["W"], ps["C"], k, k, s, p, act)
            sh = {"C": ps["C"], "H": oh, "W": ow}
        elif t == "fc":
            ps = shapes[par]
            oc = geti("filters") or geti("output")
            w, b = weight_list[wi]; wi += 1
            out = np.empty((batch, oc), np.float32)
            L.oracle_fully_connected(_p(outs[par]), _p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(b)), _p(out), batch, ps["H"],
                                     ps["W"], ps["C"], oc, act)
            sh = {"C": oc, "H": 1, "W": 1}
        elif t == "residual":
            a, b2 = outs[par], outs[frm]
            out = np.empty_like(a)
            L.oracle_residual(_p(a), _p(b2), _p(out), C.c_size_t(a.size), act)
            sh = dict(shapes[par])
        elif t == "softmax":
            a = outs[par]
            out = np.empty_like(a)
            L.oracle_softmax(_p(a), _p(out), a.shape[0], a.shape[1])
            sh = dict(shapes[par])
        elif t == "matmul":
            a = outs[par]
            m = geti("M")
            w, b = weight_list[wi]; wi += 1
            out = np.empty((a.shape[0], m), np.float32)
            L.oracle_matmul(_p(a), _p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(b)), _p(out), a.shape[0], a.shape[1], m, act)
            sh = {"M": m}
        elif t == "layernorm":
            a = outs[par]
            w, b = weight_list[wi]; wi += 1
            out = np.empty_like(a)
            L.oracle_layernorm(_p(a), _p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(b)), _p(out), a.shape[0], a.shape[1])
            sh = dict(shapes[par])
        elif t == "attn_k":
            q, k = outs[par], outs[frm]          # PARENT_0 = queries, PARENT_1 = keys
            heads, hidden = geti("n_head"), geti("n_embd")
            out = np.empty((batch * heads * seq, seq), np.float32)
            L.oracle_k_attention(_p(q), _p(k), _p(out), batch, seq, heads, hidden, geti("masked"))
            sh = {"M": seq}
        elif t == "attn_v":
            p, v = outs[par], outs[frm]          # PARENT_0 = probabilities, PARENT_1 = values
            heads, hidden = geti("n_head"), geti("n_embd")
            out = np.empty((batch * seq, hidden), np.float32)
            L.oracle_v_attention(_p(p), _p(v), _p(out), batch, seq, heads, hidden)
            sh = {"M": hidden}
        elif t == "yolo":
            ps = shapes[par]
            c = geti("classes") + 5
            # anchors of the three masked boxes (reference src/darknet_parser.c:487-549)
            masks = [int(v) for v in o["mask"].split(",")]
            allanch = [float(v) for v in o["anchors"].split(",")]
            anch = np.array([allanch[2 * m + j] for m in masks[:3] for j in (0, 1)], np.float32)
            a_num = ps["C"] // c
            out = np.empty((batch * a_num * ps["H"] * ps["W"], c), np.float32)
            L.oracle_yolo(_p(outs[par]), _p(anch), _p(out), batch, ps["H"], ps["W"], ps["C"], c, geti("stride"))
            sh = {"C": c, "H": 1, "W": ps["H"] * ps["W"] * a_num}
        elif t == "append":
            ps, ps2 = shapes[par], shapes[frm]
            s = geti("stride") or 1
            out = np.empty((batch * ps["H"] * s * ps["W"] * s, ps["C"] + ps2["C"]), np.float32)
            L.oracle_append(_p(outs[par]), _p(outs[frm]), _p(out), batch, ps["H"], ps["W"], ps["C"], ps2["C"], s)
            sh = {"C": ps["C"] + ps2["C"], "H": ps["H"] * s, "W": ps["W"] * s}
        else:
            raise ValueError(t)
        outs.append(out)
        shapes.append(sh)
    return outs
