"""ctypes binding of libaspen_b200.so -- the same calls, in the same order, a C program makes
through the ASPEN public header (reference include/aspen.h:90-133).  Used by the tests, the
benchmark and the smoke check; it adds no logic of its own.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None

# LAYER_PARAMS ids (reference include/aspen.h:56-60)
(OUT_W, OUT_H, OUT_C, BATCH, IN_W, IN_H, IN_C, WEIGHT_W, WEIGHT_H, SUB_C, STRIDE, PADDING, DILATION, GROUPS,
 NUM_HIDDEN, NUM_HEAD, NUM_SEQ, MAT_M, MAT_N, MAT_K, SUB_M, MASKED, FORM_BYTES, NUM_PARAM_ELEMENTS) = range(24)

LAYER_TYPES = ["NO_LAYER_TYPE", "INPUT", "CONV", "FC", "RESIDUAL", "BATCHNORM", "YOLO", "APPEND", "ACTIVATION", "MAXPOOL",
               "AVGPOOL", "ROUTE", "SOFTMAX", "MATMUL", "LAYERNORM", "K_ATTENTION", "V_ATTENTION"]

LDATA_FIELDS = ("type", "act", "H", "W", "stride", "tile_h", "tile_w", "num_ninst", "flop_per_output",
                "parent0", "parent1", "mem_size")
NINST_FIELDS = ("pos_h", "pos_w", "tile_h", "tile_w", "num_parents", "num_children", "num_input_pos")

EXPORTS = """apu_create_dnn apu_destroy_dnn apu_save_dnn_to_file apu_load_dnn_from_file apu_generate_nasm
apu_generate_transformer_nasm apu_create_nasm apu_create_transformer_nasm apu_destroy_nasm apu_load_nasm_from_file
apu_save_nasm_to_file apu_reset_nasm rpool_init rpool_destroy rpool_add_nasm_raw_input rpool_add_nasm rpool_reset_queue
rpool_reset_nasm dse_group_init dse_group_set_rpool dse_group_destroy dse_group_run dse_group_stop
dse_group_run_until_nasm_completion dse_wait_for_nasm_completion dse_check_nasm_completion dse_get_ldata_result
dse_get_nasm_result aspen_flush_dynamic_memory print_aspen_build_info print_dnn_info print_layer_info print_tensor_info
print_nasm_info print_ldata_info print_ninst_info print_rpool_queue_info print_rpool_queue_group_info print_rpool_info
aspen_b200_last_error aspen_b200_group_status aspen_b200_set_tile_profile aspen_b200_set_tile_quanta
aspen_b200_set_precision aspen_b200_set_device aspen_b200_dnn_num_layers aspen_b200_dnn_layer_params
aspen_b200_dnn_layer_type aspen_b200_nasm_num_ldata aspen_b200_nasm_num_ninst aspen_b200_nasm_total_flops
aspen_b200_nasm_ldata_info aspen_b200_nasm_ninst_info aspen_b200_nasm_ninst_parents aspen_b200_nasm_ninst_children
aspen_b200_nasm_get_ldata_packed aspen_b200_group_time_runs aspen_b200_group_time_passes aspen_b200_dse_group_set_service aspen_b200_group_profile aspen_b200_generate_nasm aspen_b200_set_hidden_states aspen_b200_dnn_set_embedding
aspen_b200_rpool_add_nasm_tokens aspen_b200_matmul_noalloc""".split()


def lib():
    """Loads (building first if the sources are newer) the shared library and types its entry points."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.build()
    L = C.CDLL(path)
    vp, u, cp, i = C.c_void_p, C.c_uint, C.c_char_p, C.c_int
    sig = {
        "apu_create_dnn": (vp, [cp, cp]), "apu_destroy_dnn": (None, [vp]),
        "apu_save_dnn_to_file": (None, [vp, cp]), "apu_load_dnn_from_file": (vp, [cp]),
        "apu_generate_nasm": (vp, [vp, u, u]), "apu_generate_transformer_nasm": (vp, [vp, u, u, u]),
        "apu_create_nasm": (vp, [vp, u, u]), "apu_create_transformer_nasm": (vp, [vp, u, u, u]),
        "apu_destroy_nasm": (None, [vp]), "apu_load_nasm_from_file": (vp, [cp, vp]),
        "apu_save_nasm_to_file": (None, [vp, cp]), "apu_reset_nasm": (None, [vp]),
        "rpool_init": (vp, []), "rpool_destroy": (None, [vp]),
        "rpool_add_nasm_raw_input": (None, [vp, vp, vp]), "rpool_add_nasm": (None, [vp, vp, cp]),
        "rpool_reset_queue": (None, [vp]), "rpool_reset_nasm": (None, [vp, vp]),
        "dse_group_init": (vp, [u]), "dse_group_set_rpool": (None, [vp, vp]), "dse_group_destroy": (None, [vp]),
        "dse_group_run": (None, [vp]), "dse_group_stop": (None, [vp]),
        "dse_group_run_until_nasm_completion": (None, [vp, vp]),
        "dse_wait_for_nasm_completion": (None, [vp]), "dse_check_nasm_completion": (u, [vp]),
        "dse_get_ldata_result": (C.c_ssize_t, [vp, u, vp, C.POINTER(vp)]),
        "dse_get_nasm_result": (C.c_ssize_t, [vp, vp, C.POINTER(vp)]),
        "aspen_flush_dynamic_memory": (None, []), "print_aspen_build_info": (None, []),
        "print_dnn_info": (None, [vp, i]), "print_nasm_info": (None, [vp, i, i]), "print_rpool_info": (None, [vp]),
        "aspen_b200_last_error": (cp, []), "aspen_b200_group_status": (i, [vp]),
        "aspen_b200_set_tile_profile": (None, [i]), "aspen_b200_set_tile_quanta": (None, [u, u, u]),
        "aspen_b200_set_precision": (None, [i]), "aspen_b200_set_hidden_states": (None, [i]), "aspen_b200_set_device": (i, [i]),
        "aspen_b200_dnn_num_layers": (u, [vp]), "aspen_b200_dnn_layer_params": (None, [vp, u, vp]),
        "aspen_b200_dnn_layer_type": (i, [vp, u]),
        "aspen_b200_nasm_num_ldata": (u, [vp]), "aspen_b200_nasm_num_ninst": (u, [vp]),
        "aspen_b200_nasm_total_flops": (C.c_uint64, [vp]),
        "aspen_b200_nasm_ldata_info": (None, [vp, u, vp]), "aspen_b200_nasm_ninst_info": (None, [vp, u, vp]),
        "aspen_b200_nasm_ninst_parents": (u, [vp, u, vp, u]), "aspen_b200_nasm_ninst_children": (u, [vp, u, vp, u]),
        "aspen_b200_nasm_get_ldata_packed": (C.c_long, [vp, u, vp]),
        "aspen_b200_group_time_runs": (C.c_double, [vp, u, u, C.POINTER(C.c_ulonglong)]),
        "aspen_b200_group_time_passes": (C.c_double, [vp, u, u, C.POINTER(C.c_ulonglong)]),
        "aspen_b200_dse_group_set_service": (C.c_int, [vp, C.c_int]),
        "aspen_b200_group_profile": (i, [vp, vp, C.POINTER(u)]),
        "aspen_b200_generate_nasm": (vp, [vp, u, u, C.POINTER(u)]),
        "aspen_b200_matmul_noalloc": (i, [vp, vp, vp, vp, u, u, u, i, vp]),
        "aspen_b200_dnn_set_embedding": (i, [vp, vp, u, vp, u]), "aspen_b200_rpool_add_nasm_tokens": (None, [vp, vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _libc = C.CDLL(None)
    _libc.free.argtypes = [vp]
    L._free = _libc.free
    _lib = L
    return L


def last_error() -> str:
    return lib().aspen_b200_last_error().decode(errors="replace")


class Dnn:
    def __init__(self, cfg_path: str, weight_path: str | None = None):
        self.h = lib().apu_create_dnn(cfg_path.encode(), weight_path.encode() if weight_path else None)
        if not self.h:
            raise RuntimeError("apu_create_dnn failed: " + last_error())

    @property
    def num_layers(self) -> int:
        return lib().aspen_b200_dnn_num_layers(self.h)

    def layer_params(self, idx: int) -> list[int]:
        buf = (C.c_uint * NUM_PARAM_ELEMENTS)()
        lib().aspen_b200_dnn_layer_params(self.h, idx, buf)
        return list(buf)

    def layer_type(self, idx: int) -> int:
        return lib().aspen_b200_dnn_layer_type(self.h, idx)

    def set_embedding(self, token_table: np.ndarray, position_table: np.ndarray | None = None) -> None:
        tok = np.ascontiguousarray(token_table, dtype=np.float32)
        pos = None if position_table is None else np.ascontiguousarray(position_table, dtype=np.float32)
        rc = lib().aspen_b200_dnn_set_embedding(self.h, tok.ctypes.data, tok.shape[0], pos.ctypes.data if pos is not None else None,
                                                pos.shape[0] if pos is not None else 0)
        if rc != 0:
            raise RuntimeError("aspen_b200_dnn_set_embedding failed: " + last_error())

    def close(self):
        if self.h:
            lib().apu_destroy_dnn(self.h)
            self.h = None


class Nasm:
    def __init__(self, dnn: Dnn, batch: int, seq: int = 0, min_ninst: int = 100, handle=None):
        L = lib()
        self.dnn = dnn
        if handle is not None:
            self.h = handle
        elif seq:
            self.h = L.apu_create_transformer_nasm(dnn.h, min_ninst, batch, seq)
        else:
            self.h = L.apu_create_nasm(dnn.h, min_ninst, batch)
        if not self.h:
            raise RuntimeError("nasm creation failed: " + last_error())

    @classmethod
    def tuned(cls, dnn: Dnn, batch: int, seq: int = 0):
        """aspen_b200_generate_nasm: tile-shape search on the device.  Returns (nasm, (row quantum, column quantum, min_ninst))."""
        chosen = (C.c_uint * 3)()
        h = lib().aspen_b200_generate_nasm(dnn.h, batch, seq, chosen)
        if not h:
            raise RuntimeError("aspen_b200_generate_nasm failed: " + last_error())
        return cls(dnn, 0, handle=h), tuple(chosen)

    @classmethod
    def load(cls, dnn: Dnn, path: str) -> "Nasm":
        h = lib().apu_load_nasm_from_file(path.encode(), dnn.h)
        if not h:
            raise RuntimeError("apu_load_nasm_from_file failed: " + last_error())
        return cls(dnn, 0, handle=h)

    def save(self, path: str) -> None:
        lib().apu_save_nasm_to_file(self.h, path.encode())

    @property
    def num_ldata(self) -> int:
        return lib().aspen_b200_nasm_num_ldata(self.h)

    @property
    def num_ninst(self) -> int:
        return lib().aspen_b200_nasm_num_ninst(self.h)

    @property
    def total_flops(self) -> int:
        return int(lib().aspen_b200_nasm_total_flops(self.h))

    def ldata_info(self, idx: int) -> dict:
        buf = (C.c_uint * 12)()
        lib().aspen_b200_nasm_ldata_info(self.h, idx, buf)
        return dict(zip(LDATA_FIELDS, list(buf)))

    def ninst_info(self, idx: int) -> dict:
        buf = (C.c_uint * 7)()
        lib().aspen_b200_nasm_ninst_info(self.h, idx, buf)
        return dict(zip(NINST_FIELDS, list(buf)))

    def parents(self, idx: int) -> list[int]:
        n = lib().aspen_b200_nasm_ninst_parents(self.h, idx, None, 0)
        buf = (C.c_uint * max(n, 1))()
        lib().aspen_b200_nasm_ninst_parents(self.h, idx, buf, n)
        return list(buf)[:n]

    def children(self, idx: int) -> list[int]:
        n = lib().aspen_b200_nasm_ninst_children(self.h, idx, None, 0)
        buf = (C.c_uint * max(n, 1))()
        lib().aspen_b200_nasm_ninst_children(self.h, idx, buf, n)
        return list(buf)[:n]

    def ldata(self, idx: int) -> np.ndarray:
        """Packed activations of one layer after a run: array [W columns][H rows]."""
        info = self.ldata_info(idx)
        out = np.empty((info["W"], info["H"]), dtype=np.float32)
        n = lib().aspen_b200_nasm_get_ldata_packed(self.h, idx, out.ctypes.data)
        if n != out.size:
            raise RuntimeError("reading layer output failed: " + last_error())
        return out

    def result(self, order) -> np.ndarray:
        arr = (C.c_int * len(order))(*order)
        ptr = C.c_void_p()
        nbytes = lib().dse_get_nasm_result(self.h, arr, C.byref(ptr))
        if nbytes < 0:
            raise RuntimeError("dse_get_nasm_result failed: " + last_error())
        return np.asarray(_OwnedBuffer(ptr, nbytes))      # the library's buffer itself, no copy

    def close(self):
        if self.h:
            lib().apu_destroy_nasm(self.h)
            self.h = None


class _OwnedBuffer:
    """A malloc'ed float buffer handed over by the library: numpy arrays made from it (and their views) keep this object
    as their base, and the buffer is freed with it."""

    def __init__(self, ptr: C.c_void_p, nbytes: int):
        self._ptr = ptr
        self.__array_interface__ = {"data": (ptr.value, False), "shape": (nbytes // 4,), "typestr": "<f4", "version": 3}

    def __del__(self):
        try:
            lib()._free(self._ptr)
        except Exception:  # noqa: BLE001 -- interpreter shutdown: the process's memory goes away with it
            pass


class Rpool:
    def __init__(self):
        self.h = lib().rpool_init()

    def add(self, nasm: Nasm, x: np.ndarray | None) -> None:
        if x is None:
            lib().rpool_add_nasm_raw_input(self.h, nasm.h, None)
        else:
            x = np.ascontiguousarray(x, dtype=np.float32)
            lib().rpool_add_nasm_raw_input(self.h, nasm.h, x.ctypes.data)

    def add_tokens(self, nasm: Nasm, ids: np.ndarray) -> None:
        """aspen_b200_rpool_add_nasm_tokens: ids [batch][seq] int32, embedded on the device."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        lib().aspen_b200_rpool_add_nasm_tokens(self.h, nasm.h, ids.ctypes.data)

    def reset(self, nasm: Nasm) -> None:
        lib().rpool_reset_queue(self.h)
        lib().rpool_reset_nasm(self.h, nasm.h)

    def close(self):
        if self.h:
            lib().rpool_destroy(self.h)
            self.h = None


class DseGroup:
    def __init__(self, num_dse: int = 0, precision: int | None = None):
        if precision is not None:
            lib().aspen_b200_set_precision(precision)
        self.h = lib().dse_group_init(num_dse)
        if not self.h:
            raise RuntimeError("dse_group_init failed: " + last_error())

    def set_rpool(self, rpool: Rpool) -> None:
        lib().dse_group_set_rpool(self.h, rpool.h)

    def run(self) -> None:
        lib().dse_group_run(self.h)

    def stop(self) -> None:
        lib().dse_group_stop(self.h)

    def wait(self, nasm: Nasm) -> None:
        lib().dse_wait_for_nasm_completion(nasm.h)

    def status(self) -> int:
        return lib().aspen_b200_group_status(self.h)

    def time_runs(self, warmup: int, iters: int) -> tuple[float, int]:
        n = C.c_ulonglong(0)
        ms = lib().aspen_b200_group_time_runs(self.h, warmup, iters, C.byref(n))
        if ms < 0:
            raise RuntimeError("timed runs failed: " + last_error())
        return ms, int(n.value)

    def set_service(self, on: bool) -> None:
        """Service mode: dse_group_run launches one resident kernel that serves every later rpool add until stop()."""
        if lib().aspen_b200_dse_group_set_service(self.h, 1 if on else 0) != 0:
            raise RuntimeError("service mode: " + last_error())

    def time_passes(self, warmup: int, passes: int) -> tuple[float, int]:
        n = C.c_ulonglong(0)
        ms = lib().aspen_b200_group_time_passes(self.h, warmup, passes, C.byref(n))
        if ms < 0:
            raise RuntimeError("timed passes failed: " + last_error())
        return ms, int(n.value)

    def profile(self):
        """Scheduler time accounting (needs ASPEN_B200_PROFILE=1): summed nanoseconds and tile counts per layer."""
        buf = (C.c_ulonglong * 516)()
        n = C.c_uint(0)
        if lib().aspen_b200_group_profile(self.h, buf, C.byref(n)) != 0:
            return None
        return {"ctas": n.value, "idle_polls": buf[0], "complete_ns": buf[1], "wait_ns": buf[515],
                "layers": {l: {"ns": buf[2 + l], "tiles": buf[258 + l]} for l in range(256) if buf[258 + l]}}

    def close(self):
        if self.h:
            lib().dse_group_destroy(self.h)
            self.h = None
