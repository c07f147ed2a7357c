"""TEST INFRASTRUCTURE ONLY: ctypes view of oracle/_ref/libaspen_ref.so.

That library is the unmodified ASPEN reference (its own C sources, compiled by oracle/Makefile)
plus oracle/ref_walk.c.  Nothing in the product imports this module; tests, the smoke check
and the benchmark's CPU-baseline leg do.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libaspen_ref.so")

_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(LIB_PATH, mode=os.RTLD_LOCAL | os.RTLD_NOW) if hasattr(os, "RTLD_LOCAL") else C.CDLL(LIB_PATH)
        vp, u, cp = C.c_void_p, C.c_uint, C.c_char_p
        L.apu_create_dnn.restype = vp
        L.apu_create_dnn.argtypes = [cp, cp]
        L.apu_destroy_dnn.argtypes = [vp]
        L.apu_create_nasm.restype = vp
        L.apu_create_nasm.argtypes = [vp, u, u]
        L.apu_create_transformer_nasm.restype = vp
        L.apu_create_transformer_nasm.argtypes = [vp, u, u, u]
        L.apu_load_nasm_from_file.restype = vp
        L.apu_load_nasm_from_file.argtypes = [cp, vp]
        L.apu_save_nasm_to_file.argtypes = [vp, cp]
        L.apu_destroy_nasm.argtypes = [vp]
        L.refwalk_create_nasm.restype = vp
        L.refwalk_create_nasm.argtypes = [vp, u, u, u]
        L.refwalk_run.restype = C.c_int
        L.refwalk_run.argtypes = [vp, vp, C.c_int]
        L.refwalk_get_ldata.restype = C.c_long
        L.refwalk_get_ldata.argtypes = [vp, u, vp]
        L.refwalk_num_ldata.restype = u
        L.refwalk_num_ldata.argtypes = [vp]
        L.refwalk_num_ninst.restype = u
        L.refwalk_num_ninst.argtypes = [vp]
        L.refwalk_total_flops.restype = C.c_ulong
        L.refwalk_total_flops.argtypes = [vp]
        L.refwalk_ldata_info.argtypes = [vp, u, vp]
        L.refwalk_ninst_info.argtypes = [vp, u, vp]
        L.refwalk_layer_params.argtypes = [vp, u, vp]
        L.refwalk_num_layers.restype = u
        L.refwalk_num_layers.argtypes = [vp]
        L.refbench_dse.restype = C.c_double
        L.refbench_dse.argtypes = [vp, vp, u, u, u]
        L.dse_get_nasm_result.restype = C.c_ssize_t
        L.dse_get_nasm_result.argtypes = [vp, vp, C.POINTER(vp)]
        L.dse_get_ldata_result.restype = C.c_ssize_t
        L.dse_get_ldata_result.argtypes = [vp, u, vp, C.POINTER(vp)]
        _lib = L
    return _lib


LDATA_FIELDS = ("type", "act", "H", "W", "stride", "tile_h", "tile_w", "num_ninst", "flop_per_output",
                "parent0", "parent1", "mem_size")
NINST_FIELDS = ("pos_h", "pos_w", "tile_h", "tile_w", "num_parents", "num_children", "num_input_pos")


class RefNet:
    """One reference dnn + nasm pair."""

    def __init__(self, cfg_path: str, weight_path: str | None, batch: int, seq: int = 0, min_ninst: int = 100,
                 with_parents: bool = False, nasm_file: str | None = None):
        L = lib()
        self.L = L
        self.dnn = L.apu_create_dnn(cfg_path.encode(), weight_path.encode() if weight_path else None)
        assert self.dnn, "reference apu_create_dnn failed"
        if nasm_file is not None:
            self.nasm = L.apu_load_nasm_from_file(nasm_file.encode(), self.dnn)
        elif with_parents:
            self.nasm = (L.apu_create_transformer_nasm(self.dnn, min_ninst, batch, seq) if seq
                         else L.apu_create_nasm(self.dnn, min_ninst, batch))
        else:
            self.nasm = L.refwalk_create_nasm(self.dnn, min_ninst, batch, seq)
        assert self.nasm, "reference nasm creation failed"
        self.num_ldata = L.refwalk_num_ldata(self.nasm)
        self.num_ninst = L.refwalk_num_ninst(self.nasm)

    def ldata_info(self, idx: int) -> dict:
        buf = (C.c_uint * 12)()
        self.L.refwalk_ldata_info(self.nasm, idx, buf)
        return dict(zip(LDATA_FIELDS, list(buf)))

    def ninst_info(self, idx: int) -> dict:
        buf = (C.c_uint * 7)()
        self.L.refwalk_ninst_info(self.nasm, idx, buf)
        return dict(zip(NINST_FIELDS, list(buf)))

    def layer_params(self, idx: int) -> list[int]:
        buf = (C.c_uint * 23)()
        self.L.refwalk_layer_params(self.dnn, idx, buf)
        return list(buf)

    def walk(self, x: np.ndarray, threads: int = 0) -> None:
        x = np.ascontiguousarray(x, dtype=np.float32)
        rc = self.L.refwalk_run(self.nasm, x.ctypes.data, threads or (os.cpu_count() or 1))
        assert rc == 0

    def ldata(self, idx: int) -> np.ndarray:
        info = self.ldata_info(idx)
        out = np.empty((info["W"], info["H"]), dtype=np.float32)
        n = self.L.refwalk_get_ldata(self.nasm, idx, out.ctypes.data)
        assert n == out.size, (n, out.size)
        return out

    def bench_dse(self, x: np.ndarray, num_dse: int, warmup: int, iters: int) -> float:
        x = np.ascontiguousarray(x, dtype=np.float32)
        return float(self.L.refbench_dse(self.nasm, x.ctypes.data, num_dse, warmup, iters))

    def save_nasm(self, path: str) -> None:
        self.L.apu_save_nasm_to_file(self.nasm, path.encode())

    def close(self) -> None:
        if self.nasm:
            self.L.apu_destroy_nasm(self.nasm)
            self.nasm = None
        if self.dnn:
            self.L.apu_destroy_dnn(self.dnn)
            self.dnn = None
