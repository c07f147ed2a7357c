"""Parity of the device engine (through the C ABI) with the CPU oracle, layer by layer.

Oracle: the unmodified reference's own tile kernels walked layer by layer (oracle/_ref, built from
the reference sources) when that build is present, else the plain-C restatement (oracle/port.py).

Tolerances (written here once):
  fp32 FFMA mode  : an element differs when rel >= 1e-4 AND abs >= 1e-5 * max|layer|  -> none may differ
                    (the mismatch rule of the reference's compare_float_array, src/util.c:368-391)
  TF32 tensor-core mode : max|got - want| <= 1e-2 * max|want| for every layer (logits and every hidden
                    state), and the top-1 class of every sample is identical for classifier networks.
"""
import ctypes as C
import os

import numpy as np
import pytest

import harness
from aspen_b200 import api, cfgs, weights
from oracle import port, ref

pytestmark = pytest.mark.gpu

FP32_REL, FP32_ABS = 1e-4, 1e-5
TF32_NORM = 1e-2
# TF32 mode, second bound in the form of the reference's compare_float_array: no element may be off by
# rel >= 1e-2 AND abs >= 5e-3 * max|layer| at once: an error in the upper half of the normalised bound is only
# accepted on an element large enough for it to stay below 1 % of that element.
TF32_REL, TF32_ABS = 1e-2, 5e-3
CLASSIFIERS = {"tiny_cnn", "custom", "resnet50", "vgg16"}


def oracle_layers(name, cfg, wf, batch, seq, min_ninst, x):
    if ref.available():
        rn = ref.RefNet(cfg, wf, batch, seq, min_ninst=min_ninst)
        rn.walk(x)
        outs = [None] + [rn.ldata(i) for i in range(1, rn.num_ldata)]
        rn.close()
        return outs
    kw, scheme, (wseed, _) = harness.NETS[name]
    text, wl = cfgs.BUILDERS[harness._BUILDER.get(name, name)](**kw)
    return port.run(text, weights.make_weights(wl, wseed, scheme), x, batch, seq)


def check_layers(dev, outs, precision, name):
    worst = 0.0
    for i in range(1, dev.nasm.num_ldata):
        got, want = dev.nasm.ldata(i), outs[i]
        assert got.shape == want.shape
        scale = float(np.abs(want).max())
        if precision == 1:
            bad, ea, er = harness.compare(got, want, FP32_REL, FP32_ABS * scale)
            assert bad == 0, f"{name} layer {i}: {bad} mismatches (max abs {ea:.3e}, max rel {er:.3e})"
        else:
            err = float(np.abs(got.astype(np.float64) - want).max()) / max(scale, 1e-30)
            worst = max(worst, err)
            assert err <= TF32_NORM, f"{name} layer {i}: normalised error {err:.3e}"
            bad, ea, er = harness.compare(got, want, TF32_REL, TF32_ABS * scale)
            assert bad == 0, f"{name} layer {i}: {bad} elements off by rel >= {TF32_REL} and abs >= {TF32_ABS} * max (max abs {ea:.3e}, max rel {er:.3e})"
    if name in CLASSIFIERS:
        last = dev.nasm.num_ldata - 1
        assert (dev.nasm.ldata(last).argmax(1) == outs[last].argmax(1)).all()
    return worst


CASES = [
    # net, batch, seq, min_ninst, precision (0 tf32 / 1 fp32), tile profile (0 reference / 1 b200)
    ("tiny_cnn", 2, 0, 20, 1, 0), ("tiny_cnn", 2, 0, 20, 0, 0), ("tiny_cnn", 5, 0, 3, 0, 1),
    ("tiny_transformer", 2, 16, 20, 1, 0), ("tiny_transformer", 2, 16, 20, 0, 0), ("tiny_transformer", 3, 40, 5, 0, 1),
    ("tiny_gpt", 2, 16, 20, 1, 0), ("tiny_gpt", 2, 16, 20, 0, 0), ("tiny_gpt", 1, 100, 7, 0, 1), ("tiny_gpt", 1, 100, 7, 1, 1),
    # head size 32 (the smallest the fused attention tile takes; see test_fused_attention_* for the fused runs)
    ("tiny_attn", 3, 40, 5, 0, 1), ("tiny_attn", 2, 40, 5, 1, 1), ("tiny_attn_causal", 2, 100, 5, 0, 1),
    ("custom", 2, 0, 50, 1, 0), ("custom", 7, 0, 50, 0, 1),
    ("resnet50", 1, 0, 50, 1, 0), ("resnet50", 4, 0, 100, 0, 0), ("resnet50", 4, 0, 100, 0, 1),
    ("bert_base", 1, 128, 20, 1, 0), ("bert_base", 4, 128, 100, 0, 0), ("bert_base", 4, 128, 100, 0, 1),
    ("gpt2_124M", 2, 64, 50, 0, 0), ("gpt2_124M", 1, 512, 100, 0, 1),
    ("vgg16", 1, 0, 100, 0, 1), ("vgg16", 16, 0, 180, 0, 1),
    ("gpt2_124M", 16, 512, 100, 0, 1),
    # detection heads: yolo box decode and upsample-and-concatenate (reference src/tiled_kernels.c:675-741)
    ("tiny_yolo", 2, 0, 8, 1, 0), ("tiny_yolo", 2, 0, 8, 0, 0), ("tiny_yolo", 5, 0, 4, 0, 1),
    # logistic / tanh / elu / selu epilogues (reference src/naive_kernels.c:11-57)
    ("tiny_acts", 3, 0, 8, 1, 0), ("tiny_acts", 3, 0, 8, 0, 0), ("tiny_acts", 6, 0, 4, 0, 1),
]


@pytest.mark.parametrize("name,batch,seq,mn,precision,profile", CASES)
def test_every_layer_matches_oracle(name, batch, seq, mn, precision, profile, workdir):
    if not ref.available() and name in ("resnet50", "bert_base", "gpt2_124M", "vgg16"):
        pytest.skip("plain-C oracle is too slow for this size; needs the reference build")
    cfg, wf = harness.prepare(name, workdir)
    dev = harness.Device(cfg, wf, batch, seq, mn, precision, profile)
    x = harness.make_input(name, dev.input_shape())
    assert dev.run(x) == 0, api.last_error()
    outs = oracle_layers(name, cfg, wf, batch, seq, mn, x)
    check_layers(dev, outs, precision, name)
    dev.close()


@pytest.mark.skipif(not ref.available(), reason="needs the reference build")
@pytest.mark.parametrize("env", [{"ASPEN_B200_NO_ROW_BOXES": "1"}, {"ASPEN_B200_IM2COL": "0"}, {"ASPEN_B200_IM2COL": "2"},
                                 {"ASPEN_B200_NO_FUSE": "1", "ASPEN_B200_IM2COL": "2"}])
def test_every_operand_staging_matches_oracle(env, workdir, monkeypatch):
    """ResNet-50 with each way of staging the convolution operands forced: stem by gather instead of row boxes,
    strided layers by gather instead of strided boxes, every 3x3 layer by strided boxes instead of shifted
    box + fix-up.  All must meet the same per-layer bound against the reference."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    cfg, wf = harness.prepare("resnet50", workdir)
    dev = harness.Device(cfg, wf, 3, 0, 100, 0, 1)
    x = harness.make_input("resnet50", dev.input_shape())
    assert dev.run(x) == 0, api.last_error()
    outs = oracle_layers("resnet50", cfg, wf, 3, 0, 100, x)
    worst = check_layers(dev, outs, 0, "resnet50")
    assert worst < TF32_NORM
    dev.close()


@pytest.mark.skipif(not ref.available(), reason="needs the reference build")
@pytest.mark.parametrize("name,batch,seq", [("resnet50", 32, 0), ("bert_base", 32, 128)])
def test_benchmark_configuration_matches_oracle(name, batch, seq, workdir):
    """The benchmark's own workload (batch 32, bench.py's tile quanta and min_ninst, TF32) against the reference."""
    import bench
    q_h, q_w, mn = bench.TILING[name]
    cfg, wf = harness.prepare(name, workdir)
    api.lib().aspen_b200_set_tile_quanta(q_h, q_w, 100000000)
    dev = harness.Device(cfg, wf, batch, seq, mn, 0, 2)      # profile 2: keep the quanta just set
    x = harness.make_input(name, dev.input_shape())
    assert dev.run(x) == 0, api.last_error()
    outs = oracle_layers(name, cfg, wf, batch, seq, mn, x)
    worst = check_layers(dev, outs, 0, name)
    assert worst < TF32_NORM
    dev.close()


def test_rerun_is_bitwise_identical_and_batch_samples_are_independent(workdir):
    cfg, wf = harness.prepare("resnet50", workdir)
    dev = harness.Device(cfg, wf, 4, 0, 100, 0, 1)
    x = harness.make_input("resnet50", dev.input_shape())
    assert dev.run(x) == 0
    last = dev.nasm.num_ldata - 1
    first = dev.nasm.ldata(last).copy()
    mid = dev.nasm.ldata(40).copy()
    assert dev.rerun() == 0                    # rpool_reset_nasm keeps the input resident in layer 0
    assert np.array_equal(first, dev.nasm.ldata(last)) and np.array_equal(mid, dev.nasm.ldata(40))
    dev.close()
    # sample 2 alone gives the same logits as sample 2 inside the batch (tiles never mix samples) ...
    one = harness.Device(cfg, wf, 1, 0, 50, 0, 1)
    per = x.shape[0] // 4
    assert one.run(x[2 * per:3 * per]) == 0
    np.testing.assert_array_equal(one.nasm.ldata(last)[0], first[2])
    one.close()
    # ... and with the reference's tile geometry too, up to the TF32 summation order of the input
    # convolution (its k axis is staged in a different order when the tiles are whole MMA blocks)
    ref_geom = harness.Device(cfg, wf, 1, 0, 50, 0, 0)
    assert ref_geom.run(x[2 * per:3 * per]) == 0
    got = ref_geom.nasm.ldata(last)[0]
    assert np.abs(got - first[2]).max() <= 2e-3 * np.abs(first[2]).max()
    assert int(got.argmax()) == int(first[2].argmax())
    ref_geom.close()


def test_result_api_orders(workdir):
    cfg, wf = harness.prepare("tiny_cnn", workdir)
    dev = harness.Device(cfg, wf, 3, 0, 4, 1, 0)
    x = harness.make_input("tiny_cnn", dev.input_shape())
    assert dev.run(x) == 0
    # layer 7 is a conv output: native [B][H][W][C]; ask for NCHW like the reference's main.c:131
    native = dev.nasm.ldata(7)
    info = dev.nasm.ldata_info(7)
    arr = (C.c_int * 4)(api.BATCH, api.OUT_C, api.OUT_H, api.OUT_W)
    ptr = C.c_void_p()
    n = api.lib().dse_get_ldata_result(dev.nasm.h, 7, arr, C.byref(ptr))
    assert n == native.size * 4
    got = np.frombuffer(C.string_at(ptr, n), np.float32).reshape(3, info["H"], 5, 5)
    api.lib()._free(ptr)
    np.testing.assert_array_equal(got, native.reshape(3, 5, 5, info["H"]).transpose(0, 3, 1, 2))
    # final softmax layer: [B][C]
    res = dev.nasm.result([api.BATCH, api.OUT_C, api.OUT_H, api.OUT_W])
    np.testing.assert_array_equal(res.reshape(3, 10), dev.nasm.ldata(dev.nasm.num_ldata - 1))
    np.testing.assert_allclose(res.reshape(3, 10).sum(1), 1.0, rtol=1e-5)
    dev.close()


def test_input_from_nchw_file_and_null_input(workdir):
    cfg, wf = harness.prepare("tiny_cnn", workdir)
    dev = harness.Device(cfg, wf, 2, 0, 4, 1, 0)
    nchw = harness.make_input("tiny_cnn", (2, 3, 20, 20))
    path = os.path.join(workdir, "in.tensor")
    nchw.tofile(path)
    L = api.lib()
    L.rpool_add_nasm(dev.rpool.h, dev.nasm.h, path.encode())
    dev.group.run(); dev.group.wait(dev.nasm); dev.group.stop()
    a = dev.nasm.ldata(dev.nasm.num_ldata - 1).copy()
    assert dev.run(np.ascontiguousarray(nchw.transpose(0, 2, 3, 1)).reshape(-1, 3)) == 0
    np.testing.assert_array_equal(a, dev.nasm.ldata(dev.nasm.num_ldata - 1))
    L.rpool_add_nasm(dev.rpool.h, dev.nasm.h, None)          # NULL file: zeros (ref src/apu.c:646-649)
    dev.group.run(); dev.group.wait(dev.nasm); dev.group.stop()
    assert np.all(dev.nasm.ldata(0) == 0)
    dev.close()


def test_co_inference_two_networks_in_one_rpool(workdir):
    """Several nasms in one rpool interleave in one scheduler run (reference examples/2.
    batched_execution_example/aspen_execute.c:48-67)."""
    cfg_a, wf_a = harness.prepare("tiny_cnn", workdir)
    cfg_b, wf_b = harness.prepare("custom", workdir)
    L = api.lib()
    da, db = api.Dnn(cfg_a, wf_a), api.Dnn(cfg_b, wf_b)
    na, nb, nc = api.Nasm(da, 2, 0, 8), api.Nasm(db, 3, 0, 8), api.Nasm(da, 1, 0, 8)
    rp, grp = api.Rpool(), api.DseGroup(0, 1)
    grp.set_rpool(rp)
    xs = []
    for name, nasm in (("tiny_cnn", na), ("custom", nb), ("tiny_cnn", nc)):
        i0 = nasm.ldata_info(0)
        xs.append(harness.make_input(name, (i0["W"], i0["H"])))
        rp.add(nasm, xs[-1])
    grp.run()
    for nasm in (na, nb, nc):
        grp.wait(nasm)
        assert L.dse_check_nasm_completion(nasm.h) == 1
    grp.stop()
    assert grp.status() == 0
    together = [n.ldata(n.num_ldata - 1).copy() for n in (na, nb, nc)]
    # each alone gives the same bits
    for idx, (nasm, x) in enumerate(zip((na, nb, nc), xs)):
        rp2, g2 = api.Rpool(), api.DseGroup(0, 1)
        g2.set_rpool(rp2)
        solo = api.Nasm(nasm.dnn, nasm.ldata_info(0)["W"] // (400 if idx != 1 else 1024), 0, 8)
        rp2.add(solo, x)
        g2.run(); g2.wait(solo); g2.stop()
        np.testing.assert_array_equal(solo.ldata(solo.num_ldata - 1), together[idx])
        g2.close(); solo.close(); rp2.close()
    grp.close()
    for n in (na, nb, nc):
        n.close()
    rp.close(); da.close(); db.close()


@pytest.mark.skipif(not ref.available(), reason="needs the reference build")
def test_resnet50_and_vgg16_co_inference_on_the_tensor_cores(workdir):
    """ResNet-50 batch 16 and VGG-16 batch 16 armed in one rpool and drained by one scheduler launch in TF32 mode
    (the two-model co-inference of the reference's second example at the batch sizes of the benchmark
    configuration); every layer of both against the reference."""
    L = api.lib()
    nets = []
    L.aspen_b200_set_tile_profile(1)
    for name in ("resnet50", "vgg16"):
        cfg, wf = harness.prepare(name, workdir)
        dnn = api.Dnn(cfg, wf)
        nets.append((name, cfg, wf, dnn, api.Nasm(dnn, 16, 0, 180)))
    L.aspen_b200_set_tile_profile(0)
    rp, grp = api.Rpool(), api.DseGroup(0, 0)
    grp.set_rpool(rp)
    xs = []
    for name, _, _, _, nasm in nets:
        i0 = nasm.ldata_info(0)
        xs.append(harness.make_input(name, (i0["W"], i0["H"])))
        rp.add(nasm, xs[-1])
    grp.run()
    for *_, nasm in nets:
        grp.wait(nasm)
    grp.stop()
    assert grp.status() == 0, api.last_error()
    for (name, cfg, wf, dnn, nasm), x in zip(nets, xs):
        outs = oracle_layers(name, cfg, wf, 16, 0, 180, x)

        class _View:           # check_layers wants an object with a .nasm
            pass
        v = _View()
        v.nasm = nasm
        assert check_layers(v, outs, 0, name) < TF32_NORM
    grp.close()
    for *_, dnn, nasm in nets:
        nasm.close()
    rp.close()
    for *_, dnn, _n in nets:
        dnn.close()


def test_detection_heads_are_packed_per_sample_like_the_reference(workdir):
    """dse_get_nasm_result of a network that ends in a yolo layer returns every yolo layer's rows, sample by sample
    (reference src/dse.c:476-511).  At batch 1 the reference's own call gives the bytes to compare with; at larger
    batches its copy runs past its buffers, so there the expectation is stated from the per-layer outputs."""
    cfg, wf = harness.prepare("tiny_yolo", workdir)
    order = [api.BATCH, api.OUT_C, api.OUT_H, api.OUT_W]
    for batch in (1, 3):
        dev = harness.Device(cfg, wf, batch, 0, 8, 1, 0)
        x = harness.make_input("tiny_yolo", dev.input_shape())
        assert dev.run(x) == 0, api.last_error()
        got = dev.nasm.result(order)
        heads = [i for i in range(dev.nasm.num_ldata) if api.LAYER_TYPES[dev.nasm.ldata_info(i)["type"]] == "YOLO"]
        assert len(heads) == 2
        parts = []
        for b in range(batch):
            for i in heads:
                a = dev.nasm.ldata(i)                     # [B * boxes][C] -> per sample [C][boxes]
                per = a.shape[0] // batch
                parts.append(a[b * per:(b + 1) * per].T.ravel())
        np.testing.assert_array_equal(got, np.concatenate(parts))
        if batch == 1 and ref.available():
            rn = ref.RefNet(cfg, wf, 1, 0, min_ninst=8)
            rn.walk(x, threads=2)
            arr = (C.c_int * 4)(*order)
            ptr = C.c_void_p()
            n = rn.L.dse_get_nasm_result(rn.nasm, arr, C.byref(ptr))
            want = np.frombuffer(C.string_at(ptr, n), np.float32).copy()
            api.lib()._free(ptr)
            rn.close()
            assert want.shape == got.shape
            bad, ea, er = harness.compare(got, want, FP32_REL, FP32_ABS * float(np.abs(want).max()))
            assert bad == 0, f"{bad} mismatches, max abs {ea:.3e}, max rel {er:.3e}"
        dev.close()


def test_token_ids_are_embedded_on_the_device(workdir):
    """aspen_b200_rpool_add_nasm_tokens: layer 0 = token_table[id] + position_table[s], gathered by a kernel; the
    network then runs as if the caller had passed those hidden states (which is what the oracle is given)."""
    name, batch, seq, vocab = "tiny_gpt", 3, 24, 97
    cfg, wf = harness.prepare(name, workdir)
    rng = np.random.default_rng(31)
    tok = (0.02 * rng.standard_normal((vocab, 64))).astype(np.float32)
    pos = (0.02 * rng.standard_normal((seq + 5, 64))).astype(np.float32)
    ids = rng.integers(0, vocab, size=(batch, seq), dtype=np.int32)
    hidden = (tok[ids] + pos[None, :seq]).reshape(batch * seq, 64).astype(np.float32)
    for precision in (1, 0):
        dnn = api.Dnn(cfg, wf)
        dnn.set_embedding(tok, pos)
        nasm = api.Nasm(dnn, batch, seq, 20)
        rp, grp = api.Rpool(), api.DseGroup(0, precision)
        grp.set_rpool(rp)
        rp.add_tokens(nasm, ids)
        grp.run(); grp.wait(nasm); grp.stop()
        assert grp.status() == 0, api.last_error()
        got0 = nasm.ldata(0)
        if precision == 1:
            np.testing.assert_array_equal(got0, hidden)
        else:
            assert np.abs(got0 - hidden).max() <= 1e-3 * np.abs(hidden).max()      # layer 0 is kept rounded to TF32
        outs = oracle_layers(name, cfg, wf, batch, seq, 20, hidden)

        class _View:
            pass
        v = _View()
        v.nasm = nasm
        check_layers(v, outs, precision, name)
        # the same graph again with other ids: a second upload reuses the staging buffers
        ids2 = ids[::-1].copy()
        rp.add_tokens(nasm, ids2)
        grp.run(); grp.wait(nasm); grp.stop()
        want0 = (tok[ids2] + pos[None, :seq]).reshape(batch * seq, 64)
        assert np.abs(nasm.ldata(0) - want0).max() <= 1e-3 * np.abs(want0).max()
        grp.close(); nasm.close(); rp.close(); dnn.close()


@pytest.mark.skipif(not ref.available(), reason="needs the reference build")
def test_gpt2_with_final_layernorm_and_tied_output_head(workdir):
    """GPT-2 124M plus the tail the reference's cfg leaves out -- final layernorm and the 50257-row output head,
    expressed with the layer types both libraries already have (a derived cfg, the same file for both) -- fed
    with token ids; the head's weights are the token table (tied).  Every layer, logits included, against the
    reference."""
    name, batch, seq = "gpt2_lm", 2, 64
    cfg, wf = harness.prepare(name, workdir)
    kw, scheme, (wseed, _) = harness.NETS[name]
    _, wl = cfgs.BUILDERS["gpt2_124M"](**kw)
    tok = weights.make_weights(wl, wseed, scheme)[-1][0]          # [50257][768]: the head's weight matrix
    assert tok.shape == (50257, 768)
    rng = np.random.default_rng(4)
    pos = (0.02 * rng.standard_normal((1024, 768))).astype(np.float32)
    ids = rng.integers(0, 50257, size=(batch, seq), dtype=np.int32)
    hidden = (tok[ids] + pos[None, :seq]).reshape(batch * seq, 768).astype(np.float32)
    L = api.lib()
    L.aspen_b200_set_tile_profile(1)
    dnn = api.Dnn(cfg, wf)
    dnn.set_embedding(tok, pos)
    nasm = api.Nasm(dnn, batch, seq, 100)
    L.aspen_b200_set_tile_profile(0)
    rp, grp = api.Rpool(), api.DseGroup(0, 0)
    grp.set_rpool(rp)
    rp.add_tokens(nasm, ids)
    grp.run(); grp.wait(nasm); grp.stop()
    assert grp.status() == 0, api.last_error()
    outs = oracle_layers(name, cfg, wf, batch, seq, 100, hidden)

    class _View:
        pass
    v = _View()
    v.nasm = nasm
    assert check_layers(v, outs, 0, name) < TF32_NORM
    last = nasm.num_ldata - 1
    assert nasm.ldata(last).shape == (batch * seq, 50257)
    assert (nasm.ldata(last).argmax(1) == outs[last].argmax(1)).mean() >= 0.95      # next-token choice; near-ties may flip in TF32
    grp.close(); nasm.close(); rp.close(); dnn.close()


def test_unsatisfiable_graph_reports_stall_instead_of_hanging(workdir, monkeypatch):
    """A tile that lists the same parent twice can never reach its count: the bounded ready-queue
    wait gives up, the run ends with ASPEN_B200_ERR_STALL and the context stays usable."""
    monkeypatch.setenv("ASPEN_B200_STALL_MS", "300")
    cfg, wf = harness.prepare("tiny_cnn", workdir)
    dnn = api.Dnn(cfg, wf)
    good = api.Nasm(dnn, 1, 0, 4)
    path = os.path.join(workdir, "stall.nasm")
    good.save(path)
    lines = open(path).read().split("\n")
    t = sum(good.ldata_info(i)["num_ninst"] for i in range(9))      # first tile of the connected layer
    k = lines.index(f"\tNINST_IDX:{t}")
    n_par = int(lines[k + 2].split(":")[1])
    first_parent = lines[k + 4]
    lines[k + 2] = f"\tNUM_PARENT_NINSTS:{n_par + 1}"
    lines.insert(k + 4 + n_par, f"\t\t{n_par} {first_parent.split()[1]}")
    open(path, "w").write("\n".join(lines))
    bad = api.Nasm.load(dnn, path)
    rp, grp = api.Rpool(), api.DseGroup(0, 1)
    grp.set_rpool(rp)
    rp.add(bad, None)
    grp.run()
    grp.wait(bad)
    grp.stop()
    assert grp.status() == 1                                   # ASPEN_B200_ERR_STALL
    assert api.lib().dse_check_nasm_completion(bad.h) == 0
    # the same group still runs a healthy graph afterwards
    rp2 = api.Rpool()
    grp.close(); bad.close(); rp.close()
    g2 = api.DseGroup(0, 1)
    g2.set_rpool(rp2)
    rp2.add(good, None)
    g2.run(); g2.wait(good); g2.stop()
    assert g2.status() == 0 and api.lib().dse_check_nasm_completion(good.h) == 1
    g2.close(); good.close(); rp2.close(); dnn.close()


def test_stop_then_run_again_completes(workdir):
    cfg, wf = harness.prepare("resnet50", workdir)
    dev = harness.Device(cfg, wf, 4, 0, 100, 0, 1)
    x = harness.make_input("resnet50", dev.input_shape())
    dev.rpool.add(dev.nasm, x)
    dev.group.run()
    dev.group.stop()                       # cooperative stop, possibly mid-graph
    dev.group.run()                        # unfinished graph restarts
    dev.group.wait(dev.nasm)
    dev.group.stop()
    assert dev.group.status() == 0 and api.lib().dse_check_nasm_completion(dev.nasm.h) == 1
    a = dev.nasm.ldata(dev.nasm.num_ldata - 1).copy()
    assert dev.rerun() == 0
    np.testing.assert_array_equal(a, dev.nasm.ldata(dev.nasm.num_ldata - 1))
    dev.close()


@pytest.mark.parametrize("name,batch,seq,mn,profile", [("resnet50", 2, 0, 100, 1), ("resnet50", 1, 0, 50, 0), ("tiny_transformer", 3, 24, 20, 0),
                                                       ("bert_base", 2, 128, 100, 1)])
def test_residual_fused_into_producer_equals_separate_layer(name, batch, seq, mn, profile, workdir, monkeypatch):
    """The residual layers computed in the producing convolution / matmul epilogue (the default) give,
    bit for bit, what the separate residual tiles (ref src/tiled_kernels.c:503-541) give, in every layer."""
    cfg, wf = harness.prepare(name, workdir)
    outs = []
    for no_fuse in ("0", "1"):
        monkeypatch.setenv("ASPEN_B200_NO_FUSE", no_fuse)
        dev = harness.Device(cfg, wf, batch, seq, mn, 0, profile)
        x = harness.make_input(name, dev.input_shape())
        assert dev.run(x) == 0
        outs.append([dev.nasm.ldata(i).copy() for i in range(1, dev.nasm.num_ldata)])
        types = [api.LAYER_TYPES[dev.nasm.ldata_info(i)["type"]] for i in range(1, dev.nasm.num_ldata)]
        dev.close()
    assert "RESIDUAL" in types
    for i, (a, b) in enumerate(zip(*outs)):
        assert np.array_equal(a, b), f"layer {i + 1} ({types[i]}) differs"


@pytest.mark.parametrize("name,batch,seq,mn", [("resnet50", 2, 0, 100), ("tiny_transformer", 3, 24, 20), ("tiny_attn", 2, 64, 5)])
def test_dropping_pre_add_outputs_changes_no_other_layer(name, batch, seq, mn, workdir, monkeypatch):
    """aspen_b200_set_hidden_states(0): a convolution / matmul whose output only feeds the residual add fused into
    its own epilogue does not write that output.  Every other layer and the result stay bit-identical; the dropped
    layers read as zeros."""
    if name == "tiny_attn":
        monkeypatch.setenv("ASPEN_B200_ATTN_FUSE", "1")      # then the attention_k matrices are dropped as well
    cfg, wf = harness.prepare(name, workdir)
    L = api.lib()
    runs = []
    for keep in (1, 0):
        L.aspen_b200_set_hidden_states(keep)
        try:
            dev = harness.Device(cfg, wf, batch, seq, mn, 0, 1)
            x = harness.make_input(name, dev.input_shape())
            assert dev.run(x) == 0, api.last_error()
        finally:
            L.aspen_b200_set_hidden_states(1)
        runs.append([dev.nasm.ldata(i).copy() for i in range(1, dev.nasm.num_ldata)])
        types = [api.LAYER_TYPES[dev.nasm.ldata_info(i)["type"]] for i in range(1, dev.nasm.num_ldata)]
        dev.close()
    dropped = [i for i, (a, b) in enumerate(zip(*runs)) if not np.array_equal(a, b)]
    assert dropped, "no layer was dropped"
    for i in dropped:
        assert types[i] in ("CONV", "MATMUL", "K_ATTENTION")
        assert not runs[1][i].any(), f"layer {i + 1} differs but is not all zero"
        assert runs[0][i].any()
    assert np.array_equal(runs[0][-1], runs[1][-1])
    n_res = sum(1 for t in types if t == "RESIDUAL")
    n_conv_like = sum(1 for i in dropped if types[i] != "K_ATTENTION")
    assert n_res - 1 <= n_conv_like <= n_res          # a residual add whose other operand is the network input stays a layer of its own


@pytest.mark.parametrize("name,batch,seq,mn,profile", [("tiny_attn", 3, 40, 5, 1), ("tiny_attn", 2, 128, 5, 1), ("tiny_attn_causal", 2, 100, 5, 1),
                                                       ("tiny_attn_causal", 3, 24, 5, 0), ("bert_base", 2, 128, 100, 1), ("gpt2_124M", 2, 64, 50, 1)])
def test_fused_attention_one_key_group_still_writes_the_probabilities(name, batch, seq, mn, profile, workdir, monkeypatch):
    """ASPEN_B200_ATTN_FUSE=1: attention_k + attention_v run as one tile.  With at most 128 keys the tile also writes the
    attention_k layer's matrix, so every layer is compared with the oracle as usual."""
    if not ref.available() and name in ("bert_base", "gpt2_124M"):
        pytest.skip("needs the reference build")
    monkeypatch.setenv("ASPEN_B200_ATTN_FUSE", "1")
    cfg, wf = harness.prepare(name, workdir)
    dev = harness.Device(cfg, wf, batch, seq, mn, 0, profile)
    x = harness.make_input(name, dev.input_shape())
    assert dev.run(x) == 0, api.last_error()
    outs = oracle_layers(name, cfg, wf, batch, seq, mn, x)
    check_layers(dev, outs, 0, name)
    dev.close()


@pytest.mark.parametrize("name,batch,seq,mn", [("tiny_attn", 2, 256, 20), ("tiny_attn", 2, 192, 20), ("tiny_attn_causal", 2, 384, 20),
                                               ("tiny_attn_causal", 1, 512, 20)])
def test_fused_attention_over_several_key_groups(name, batch, seq, mn, workdir, monkeypatch):
    """Sequences longer than one group of 128 keys: the fused attention tile accumulates P x V over the groups (and, with a
    causal mask, skips the groups above its queries).  The probabilities then never reach memory, so this needs
    aspen_b200_set_hidden_states(0); every layer that is still written is compared with the oracle."""
    monkeypatch.setenv("ASPEN_B200_ATTN_FUSE", "1")
    cfg, wf = harness.prepare(name, workdir)
    L = api.lib()
    L.aspen_b200_set_hidden_states(0)
    try:
        dev = harness.Device(cfg, wf, batch, seq, mn, 0, 1)
        x = harness.make_input(name, dev.input_shape())
        assert dev.run(x) == 0, api.last_error()
    finally:
        L.aspen_b200_set_hidden_states(1)
    outs = oracle_layers(name, cfg, wf, batch, seq, mn, x)
    types = [api.LAYER_TYPES[dev.nasm.ldata_info(i)["type"]] for i in range(dev.nasm.num_ldata)]
    fused = 0
    for i in range(1, dev.nasm.num_ldata):
        got, want = dev.nasm.ldata(i), outs[i]
        if not got.any():
            assert types[i] in ("K_ATTENTION", "MATMUL")          # never written: fused away
            fused += types[i] == "K_ATTENTION"
            continue
        err = float(np.abs(got.astype(np.float64) - want).max()) / float(np.abs(want).max())
        assert err <= TF32_NORM, f"{name} layer {i} ({types[i]}): normalised error {err:.3e}"
    assert fused == 2                                            # both attention_k layers
    dev.close()


def test_two_graphs_in_flight_upload_and_download_overlap_a_run(workdir):
    """The serving loop of bench.py's end-to-end leg: while one graph is being computed, the next graph's
    input is uploaded and the previous graph's result is read.  Every result must equal the one the same
    input gives when nothing overlaps."""
    cfg, wf = harness.prepare("resnet50", workdir)
    L = api.lib()
    L.aspen_b200_set_tile_profile(1)
    dnn = api.Dnn(cfg, wf)
    pair = [api.Nasm(dnn, 4, 0, 100), api.Nasm(dnn, 4, 0, 100)]
    L.aspen_b200_set_tile_profile(0)
    rpool = api.Rpool()
    group = api.DseGroup(0, 0)
    group.set_rpool(rpool)
    i0 = pair[0].ldata_info(0)
    rng = np.random.default_rng(11)
    xs = [rng.standard_normal((i0["W"], i0["H"]), dtype=np.float32) for _ in range(5)]
    order = [api.BATCH, api.OUT_C, api.OUT_H, api.OUT_W]
    want = []
    for x in xs:                                   # nothing overlaps
        rpool.add(pair[0], x); group.run(); group.wait(pair[0]); group.stop()
        want.append(pair[0].result(order).copy())
    got = []
    cur = 0
    rpool.add(pair[cur], xs[0]); group.run()
    for step in range(len(xs)):
        nxt = cur ^ 1
        if step + 1 < len(xs):
            rpool.add(pair[nxt], xs[step + 1])     # upload under the running graph
        group.wait(pair[cur]); group.stop()
        assert group.status() == 0
        if step + 1 < len(xs):
            group.run()
        got.append(pair[cur].result(order).copy()) # download under the next graph's run
        cur = nxt
    for a, b in zip(want, got):
        assert np.array_equal(a, b)
    assert not np.array_equal(want[0], want[1])
    group.close(); pair[1].close(); pair[0].close(); rpool.close(); dnn.close()


def test_tile_shape_search_returns_a_working_graph(workdir):
    """aspen_b200_generate_nasm times tensor-core shaped tilings on the device and returns the fastest; whatever it
    picks, the values are the ones of a default graph (up to TF32 summation order of the input convolution)."""
    cfg, wf = harness.prepare("tiny_cnn", workdir)
    dnn = api.Dnn(cfg, wf)
    tuned, chosen = api.Nasm.tuned(dnn, 6)
    assert chosen[0] in (128, 256) and chosen[1] in (128, 256) and chosen[2] in (100, 148, 180, 222, 296)
    plain = api.Nasm(dnn, 6, 0, 20)
    rpool = api.Rpool()
    group = api.DseGroup(0, 0)
    group.set_rpool(rpool)
    i0 = plain.ldata_info(0)
    x = np.random.default_rng(5).standard_normal((i0["W"], i0["H"]), dtype=np.float32)
    outs = []
    for n_ in (tuned, plain):
        rpool.add(n_, x); group.run(); group.wait(n_); group.stop()
        assert group.status() == 0
        outs.append(n_.ldata(n_.num_ldata - 1).copy())
    assert outs[0].shape == outs[1].shape
    assert np.abs(outs[0] - outs[1]).max() <= 2e-3 * np.abs(outs[1]).max()
    group.close(); plain.close(); tuned.close(); rpool.close(); dnn.close()
