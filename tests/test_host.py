"""Host side of the library on CPU: cfg parsing, the tiler and dependency graph against the
reference's geometry (fixtures and, when present, the reference itself), file codecs, the error
conventions of the C API, and that the shared library exports every declared entry point."""
import ctypes as C
import hashlib
import json
import glob
import os
import re

import numpy as np
import pytest

import harness
from aspen_b200 import api, cfgs
from oracle import ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
REFDIR = os.environ.get("ASPEN_REFERENCE", "/root/reference")


def _digest(path):
    h = hashlib.sha256()
    for line in open(path, "rb"):
        if not line.startswith(b"DNN_NAME"):
            h.update(line)
    return h.hexdigest()


def test_library_exports_every_declared_symbol():
    L = api.lib()
    header = open(os.path.join(ROOT, "include", "aspen_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = set(re.findall(r"\b([a-z_0-9]+)\s*\(", header)) - {"defined", "sizeof"}
    declared = {n for n in names if re.match(r"^(apu_|rpool_|dse_|print_|aspen_)", n)}
    assert len(declared) >= 55
    assert declared == set(api.EXPORTS), declared ^ set(api.EXPORTS)
    for n in declared:
        assert hasattr(L, n), n


GRAPHS = sorted(glob.glob(os.path.join(GOLDEN, "graph_*.json")))


@pytest.mark.parametrize("path", GRAPHS, ids=[os.path.basename(p)[6:-5] for p in GRAPHS])
def test_tiler_and_graph_match_reference_fixture(path, workdir):
    g = json.load(open(path))
    if g["net"] in ("vgg16",) and os.environ.get("ASPEN_FAST_TESTS"):
        pytest.skip("large")
    cfg = os.path.join(workdir, g["net"] + "_g.cfg")
    cfgs.write_cfg(harness._BUILDER.get(g["net"], g["net"]), cfg, **harness.NETS[g["net"]][0])
    dnn = api.Dnn(cfg)
    nasm = api.Nasm(dnn, g["batch"], g["seq"], g["min_ninst"])
    assert nasm.num_ninst == g["num_ninst"]
    for i, row in enumerate(g["ldata"]):
        info = nasm.ldata_info(i)
        assert [info[k] for k in api.LDATA_FIELDS] == row, (i, info, row)
    out = os.path.join(workdir, "mine.nasm")
    nasm.save(out)
    assert _digest(out) == g["nasm_sha256"]          # parent order, child order, num_input_pos: all identical
    # a file written here loads back to the same graph
    again = api.Nasm.load(dnn, out)
    for t in (0, nasm.num_ninst // 2, nasm.num_ninst - 1):
        assert again.parents(t) == nasm.parents(t) and again.children(t) == nasm.children(t)
    again.close()
    nasm.close()
    dnn.close()


@pytest.mark.skipif(not os.path.isdir(REFDIR), reason="reference tree not mounted")
@pytest.mark.parametrize("net,fname", [("resnet50", "resnet50_B2.nasm"), ("resnet50", "resnet50_B4.nasm")])
def test_shipped_nasm_files_load(net, fname, workdir):
    cfg = os.path.join(workdir, net + "_s.cfg")
    cfgs.write_cfg(net, cfg)
    dnn = api.Dnn(cfg)
    path = os.path.join(REFDIR, "files", net, fname)
    nasm = api.Nasm.load(dnn, path)
    out = os.path.join(workdir, "reload.nasm")
    nasm.save(out)
    assert _digest(out) == _digest(path)
    nasm.close()
    dnn.close()


@pytest.mark.skipif(not os.path.isdir(REFDIR), reason="reference tree not mounted")
@pytest.mark.parametrize("net", ["resnet50", "vgg16", "bert_base", "gpt2_124M", "custom"])
def test_generated_cfg_equals_reference_cfg(net, workdir):
    """The cfg builders stand in for the reference's files/*.cfg on machines without the reference."""
    mine = os.path.join(workdir, net + "_c.cfg")
    cfgs.write_cfg(net, mine)
    theirs = os.path.join(REFDIR, "files", "custom.cfg" if net == "custom" else f"{net}/{net}_aspen.cfg")
    a, b = api.Dnn(mine), api.Dnn(theirs)
    assert a.num_layers == b.num_layers
    for i in range(a.num_layers):
        assert a.layer_type(i) == b.layer_type(i) and a.layer_params(i) == b.layer_params(i), i
    a.close()
    b.close()


@pytest.mark.skipif(not ref.available(), reason="reference build (oracle/_ref) not present")
def test_layer_params_match_reference_parser(workdir):
    for net in ("tiny_cnn", "tiny_gpt", "resnet50"):
        cfg, _ = harness.prepare(net, workdir)
        mine = api.Dnn(cfg)
        rn = ref.RefNet(cfg, None, 1, 8 if "gpt" in net else 0, min_ninst=1)
        for i in range(mine.num_layers):
            assert mine.layer_params(i) == rn.layer_params(i)[:api.NUM_PARAM_ELEMENTS], (net, i)
        rn.close()
        mine.close()


def test_b200_tile_profile_only_changes_geometry(workdir):
    cfg, _ = harness.prepare("resnet50", workdir)
    dnn = api.Dnn(cfg)
    a = api.Nasm(dnn, 4, 0, 100)
    api.lib().aspen_b200_set_tile_profile(1)
    b = api.Nasm(dnn, 4, 0, 100)
    api.lib().aspen_b200_set_tile_profile(0)
    assert a.total_flops == b.total_flops == 4 * 8185945088
    for i in range(a.num_ldata):
        ia, ib = a.ldata_info(i), b.ldata_info(i)
        assert (ia["H"], ia["W"]) == (ib["H"], ib["W"])
        if ib["type"] == 2 and ib["W"] >= 128:
            # conv tiles are whole blocks: 128 columns, or whole output rows / samples for the strided layers
            # (OW = 28 -> 4 rows = 112, OW = 14 -> 7 rows = 98, 7 x 7 -> two samples = 98)
            p = dnn.layer_params(i)
            strided = p[api.STRIDE] > 1 and p[api.IN_C] % 32 == 0
            block = {28: 112, 14: 98, 7: 98}[p[api.OUT_W]] if strided else 128
            assert ib["tile_w"] % block == 0, (i, ib["tile_w"], block)
    # every tile has parents, parents precede children
    for t in range(b.ldata_info(0)["num_ninst"], b.num_ninst, 97):
        ps = b.parents(t)
        assert ps and max(ps) < t
    a.close(); b.close(); dnn.close()


def test_weight_file_and_aspen_codec_roundtrip(workdir):
    cfg, wf = harness.prepare("tiny_cnn", workdir)
    L = api.lib()
    dnn = api.Dnn(cfg, wf)
    path = os.path.join(workdir, "tiny.aspen").encode()
    L.apu_save_dnn_to_file(dnn.h, path)
    h2 = L.apu_load_dnn_from_file(path)
    assert h2
    assert L.aspen_b200_dnn_num_layers(h2) == dnn.num_layers
    for i in range(dnn.num_layers):
        buf = (C.c_uint * api.NUM_PARAM_ELEMENTS)()
        L.aspen_b200_dnn_layer_params(h2, i, buf)
        assert list(buf) == dnn.layer_params(i)
    path2 = os.path.join(workdir, "tiny2.aspen").encode()
    L.apu_save_dnn_to_file(h2, path2)
    assert open(path, "rb").read() == open(path2, "rb").read()
    L.apu_destroy_dnn(h2)
    dnn.close()


@pytest.mark.skipif(not ref.available(), reason="reference build (oracle/_ref) not present")
def test_aspen_file_is_readable_by_reference(workdir):
    cfg, wf = harness.prepare("tiny_cnn", workdir)
    L, R = api.lib(), ref.lib()
    dnn = api.Dnn(cfg, wf)
    mine = os.path.join(workdir, "m.aspen").encode()
    L.apu_save_dnn_to_file(dnn.h, mine)
    R.apu_load_dnn_from_file.restype = C.c_void_p
    R.apu_load_dnn_from_file.argtypes = [C.c_char_p]
    R.apu_save_dnn_to_file.argtypes = [C.c_void_p, C.c_char_p]
    rd = R.apu_load_dnn_from_file(mine)
    assert rd
    theirs = os.path.join(workdir, "t.aspen").encode()
    R.apu_save_dnn_to_file(rd, theirs)
    a, b = open(mine, "rb").read(), open(theirs, "rb").read()
    strip = lambda s: re.sub(rb"ASPEN_BUILD:[^\n]*\n", b"", s)
    assert strip(a) == strip(b)                      # same tensors, same packed weight layout, byte for byte
    dnn.close()


def test_error_conventions(workdir, capfd):
    L = api.lib()
    assert L.apu_create_dnn(b"/nonexistent/x.cfg", None) is None
    assert "Couldn't open" in api.last_error() or "no sections" in api.last_error()
    assert L.apu_create_dnn(b"model.txt", None) is None
    cfg, _ = harness.prepare("tiny_cnn", workdir)
    dnn = api.Dnn(cfg)
    assert L.apu_create_nasm(dnn.h, 0, 1) is None          # min_ninst_per_ldata must be >= 1
    nasm = api.Nasm(dnn, 1, 0, 4)
    L.apu_destroy_dnn(dnn.h)                                # refused: a nasm still references the dnn
    assert "still referencing" in api.last_error()
    assert dnn.num_layers == 11
    assert L.apu_load_nasm_from_file(b"/nonexistent.nasm", dnn.h) is None
    ptr = C.c_void_p()
    assert L.dse_get_nasm_result(None, None, C.byref(ptr)) == -1
    assert L.dse_get_nasm_result(nasm.h, None, None) == -1
    rp = L.rpool_init()
    L.rpool_add_nasm_raw_input(rp, None, None)
    assert "nasm is NULL" in api.last_error()
    L.rpool_destroy(rp)
    # service mode and its timer need a dse group
    assert L.aspen_b200_dse_group_set_service(None, 1) == -1
    assert "dse_group is NULL" in api.last_error()
    assert L.aspen_b200_group_time_passes(None, 1, 1, None) < 0
    nasm.close()
    dnn.close()
    capfd.readouterr()


def test_corrupt_nasm_file_is_rejected(workdir):
    cfg, _ = harness.prepare("tiny_cnn", workdir)
    dnn = api.Dnn(cfg)
    nasm = api.Nasm(dnn, 1, 0, 4)
    good = os.path.join(workdir, "good.nasm")
    nasm.save(good)
    text = open(good).read()
    bad = os.path.join(workdir, "bad.nasm")
    open(bad, "w").write(text.replace("NINST_IDX:5\n", "NINST_IDX:6\n", 1))
    assert api.lib().apu_load_nasm_from_file(bad.encode(), dnn.h) is None
    open(bad, "w").write(text[: len(text) // 2])
    assert api.lib().apu_load_nasm_from_file(bad.encode(), dnn.h) is None
    nasm.close()
    dnn.close()


def test_engine_refuses_to_run_without_gpu():
    """No CPU fallback: without a usable sm_100 device a dse group cannot be created."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    assert api.lib().dse_group_init(4) is None
    assert "CUDA" in api.last_error() or "device" in api.last_error()


def _aspen_tensors(path):
    """The raw tensors of a .aspen file, in file order (layout: reference src/apu_file_io.c:434-501)."""
    blob = open(path, "rb").read()
    out, pos = [], 0
    while True:
        start = blob.find(b"\t\tNUM_DIMS:", pos)
        if start < 0:
            return out
        data = blob.find(b"\t\tTENSOR_DATA:\n", start)
        head = blob[start:data].decode()
        nd = int(re.search(r"NUM_DIMS:(\d+)", head).group(1))
        order = [int(v) for v in re.findall(r"\t\t\t\d+ (\d+)\n", head.split("DATA_DIM_ORDER:")[1].split("DATA_DIM_ORDER_END")[0])]
        dims = [int(v) for v in re.findall(r"\t\t\t\d+ (\d+)\n", head.split("TENSOR_DIMS:")[1].split("TENSOR_DIMS_END")[0])]
        n = int(np.prod([dims[order[k]] for k in range(nd)]))
        data += len(b"\t\tTENSOR_DATA:\n")
        out.append(np.frombuffer(blob[data:data + 4 * n], np.float32))
        assert blob[data + 4 * n:data + 4 * n + 18] == b"\t\tTENSOR_DATA_END\n"
        pos = data + 4 * n


def _bn_weight_file(path, tensors, bn):
    """ASPEN_DATA file whose conv layers carry BN_VAR / BN_MEAN / BN_WEIGHT blocks next to WEIGHT and BIAS
    (the writer side of reference examples/3. custom_example/custom_net.py; reader src/apu_file_io.c:135-140,346-413)."""
    with open(path, "wb") as f:
        f.write(b"ASPEN_DATA\n")
        for i, (w, b) in enumerate(tensors, start=1):
            blocks = [("WEIGHT", w), ("BIAS", b)]
            if i in bn:
                blocks += [("BN_VAR", bn[i][0]), ("BN_MEAN", bn[i][1]), ("BN_WEIGHT", bn[i][2])]
            for name, arr in blocks:
                raw = np.ascontiguousarray(arr, dtype="<f4").tobytes()
                f.write(f"LAYER:{i}\nTENSOR_TYPE:{name}\nDATA_SIZE:{len(raw)}\nDATA_START:\n".encode() + raw + b"DATA_END\nLAYER_END\n")


def test_batchnorm_is_folded_on_load_like_the_reference(workdir):
    """Weight files may carry batch-norm statistics per convolution; both libraries fold them into weight and bias
    while loading (reference src/apu_file_io.c:400-413, src/util.c:259-276: w *= g / sqrt(var + 1e-5),
    b -= g * mean / sqrt(var + 1e-5))."""
    from aspen_b200 import weights
    kw, scheme, (wseed, _) = harness.NETS["tiny_cnn"]
    text, wl = cfgs.BUILDERS["tiny_cnn"](**kw)
    cfg = os.path.join(workdir, "bn.cfg")
    open(cfg, "w").write(text)
    tensors = weights.make_weights(wl, wseed, scheme)
    rng = np.random.default_rng(23)
    bn = {}
    for i, (kind, shape, _) in enumerate(wl, start=1):
        if kind == "conv" and i != 2:          # one convolution stays without statistics
            n = shape[0]
            bn[i] = (rng.uniform(0.5, 2.0, n).astype(np.float32), rng.standard_normal(n).astype(np.float32),
                     rng.uniform(0.5, 1.5, n).astype(np.float32))
    wf = os.path.join(workdir, "bn.bin")
    _bn_weight_file(wf, tensors, bn)
    L = api.lib()
    dnn = api.Dnn(cfg, wf)
    mine = os.path.join(workdir, "bn_mine.aspen")
    L.apu_save_dnn_to_file(dnn.h, mine.encode())
    dnn.close()
    got = _aspen_tensors(mine)
    # the same file without statistics gives the unfolded tensors in the same (packed) layout
    plain = os.path.join(workdir, "bn_plain.bin")
    weights.write_aspen_data(plain, tensors)
    dnn = api.Dnn(cfg, plain)
    base = os.path.join(workdir, "bn_base.aspen")
    L.apu_save_dnn_to_file(dnn.h, base.encode())
    dnn.close()
    raw = _aspen_tensors(base)
    assert len(got) == len(raw) == 2 * len(wl)
    changed = 0
    for i in range(1, len(wl) + 1):
        w0, b0, w1, b1 = raw[2 * i - 2], raw[2 * i - 1], got[2 * i - 2], got[2 * i - 1]
        if i not in bn:
            assert np.array_equal(w0, w1) and np.array_equal(b0, b1)
            continue
        var, mean, g = bn[i]
        inv = np.sqrt((var.astype(np.float64) + 1e-5).astype(np.float32))
        np.testing.assert_allclose(b1, b0 - g * mean / inv, rtol=2e-6, atol=1e-7)
        # packed weight layout [rows/8][K][8] (reference src/apu.c:14-40): element (r, k) at ((r // 8) * K + k) * 8 + r % 8
        rows = len(b0)
        k = w0.size // (8 * ((rows + 7) // 8))
        scale = np.zeros(8 * ((rows + 7) // 8), np.float32)
        scale[:rows] = g / inv
        want = (w0.reshape(-1, k, 8) * scale.reshape(-1, 1, 8)).ravel()
        np.testing.assert_allclose(w1, want, rtol=2e-6, atol=1e-9)
        changed += 1
    assert changed == len(bn) >= 4
    if ref.available():
        R = ref.lib()
        R.apu_save_dnn_to_file.argtypes = [C.c_void_p, C.c_char_p]
        rd = R.apu_create_dnn(cfg.encode(), wf.encode())
        assert rd
        theirs = os.path.join(workdir, "bn_ref.aspen")
        R.apu_save_dnn_to_file(rd, theirs.encode())
        R.apu_destroy_dnn(rd)
        want = _aspen_tensors(theirs)
        assert len(want) == len(got)
        for a, b in zip(got, want):
            np.testing.assert_allclose(a, b, rtol=2e-6, atol=1e-9)   # the reference is built with -Ofast: not bit-exact


def test_result_arrays_own_the_library_buffer():
    """Nasm.result hands back the malloc'ed buffer of dse_get_nasm_result without copying it: the array and every view
    of it keep the buffer alive, and it is freed exactly once when the last of them goes."""
    import ctypes as C
    import gc
    libc = C.CDLL(None)
    libc.malloc.restype = C.c_void_p
    libc.malloc.argtypes = [C.c_size_t]
    freed = []
    real_free = api.lib()._free
    api.lib()._free = lambda p: (freed.append(p.value), real_free(p))
    try:
        ptr = C.c_void_p(libc.malloc(64))
        C.memset(ptr, 0, 64)
        arr = np.asarray(api._OwnedBuffer(ptr, 64))
        arr[:] = np.arange(16, dtype=np.float32)
        view = arr.reshape(4, 4)[1:]
        del arr
        gc.collect()
        assert not freed and view.sum() == sum(range(4, 16))
        del view
        gc.collect()
        assert freed == [ptr.value]
    finally:
        api.lib()._free = real_free
