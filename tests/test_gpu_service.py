"""Service mode of a dse group (aspen_b200_dse_group_set_service): one resident scheduler kernel serves every
rpool add between dse_group_run and dse_group_stop, the way the reference's DSE threads do (src/dse.c:20-108).

Every result is compared bit for bit with the result the same graph and input give when the scheduler is launched
per run (that path is what the parity tests compare with the oracle), and one case is compared with the oracle
directly."""
import time

import numpy as np
import pytest

import harness
from aspen_b200 import api
from test_gpu_parity import check_layers, oracle_layers

pytestmark = pytest.mark.gpu

IMG = [api.BATCH, api.OUT_C, api.OUT_H, api.OUT_W]
SEQ = [api.BATCH, api.MAT_N, api.MAT_M]


def _net(name, workdir, batch, seq, mn, precision, graphs=1, profile=0):
    cfg, wf = harness.prepare(name, workdir)
    L = api.lib()
    L.aspen_b200_set_tile_profile(profile)
    dnn = api.Dnn(cfg, wf)
    nasms = [api.Nasm(dnn, batch, seq, mn) for _ in range(graphs)]
    L.aspen_b200_set_tile_profile(0)
    rpool, group = api.Rpool(), api.DseGroup(0, precision)
    group.set_rpool(rpool)
    i0 = nasms[0].ldata_info(0)
    return cfg, wf, dnn, nasms, rpool, group, (i0["W"], i0["H"])


def _close(dnn, nasms, rpool, group):
    group.close()
    for n_ in reversed(nasms):
        n_.close()
    rpool.close()
    dnn.close()


def _per_launch_layers(nasm, rpool, group, x):
    rpool.add(nasm, x); group.run(); group.wait(nasm); group.stop()
    assert group.status() == 0, api.last_error()
    return [nasm.ldata(i).copy() for i in range(nasm.num_ldata)]


@pytest.mark.parametrize("name,batch,seq,mn,precision,profile", [
    ("tiny_cnn", 3, 0, 20, 1, 0), ("tiny_cnn", 3, 0, 20, 0, 0), ("resnet50", 2, 0, 100, 0, 1), ("tiny_transformer", 3, 24, 20, 0, 0),
    ("tiny_yolo", 2, 0, 20, 0, 0),
])
def test_a_served_pass_equals_a_launched_run_in_every_layer(name, batch, seq, mn, precision, profile, workdir):
    cfg, wf, dnn, nasms, rpool, group, shape = _net(name, workdir, batch, seq, mn, precision, profile=profile)
    nasm = nasms[0]
    rng = np.random.default_rng(5)
    xs = [rng.standard_normal(shape, dtype=np.float32) for _ in range(3)]
    want = [_per_launch_layers(nasm, rpool, group, x) for x in xs]
    group.set_service(True)
    for k, x in enumerate(xs):
        rpool.add(nasm, x)
        if k == 0:
            group.run()                       # from here on the kernel is resident: the later adds go to it
        group.wait(nasm)
        assert group.status() == 0, api.last_error()
        for i in range(1, nasm.num_ldata):
            assert np.array_equal(nasm.ldata(i), want[k][i]), f"{name}: pass {k}, layer {i}"
    group.stop()
    assert group.status() == 0
    # and against the oracle itself for the last input
    outs = oracle_layers(name, cfg, wf, batch, seq, mn, xs[-1])

    class _View:
        pass
    v = _View()
    v.nasm = nasm
    check_layers(v, outs, precision, name)
    group.set_service(False)                  # back to one launch per run: same values
    again = _per_launch_layers(nasm, rpool, group, xs[0])
    for i in range(1, nasm.num_ldata):
        assert np.array_equal(again[i], want[0][i])
    _close(dnn, nasms, rpool, group)


def test_requests_for_three_graphs_overlap_and_keep_their_own_results(workdir):
    """The serving loop of bench.py's end-to-end leg: three graphs of one network rotate; while two are being computed the
    third one's input uploads and a finished one's result downloads."""
    cfg, wf, dnn, nasms, rpool, group, shape = _net("resnet50", workdir, 4, 0, 100, 0, graphs=3, profile=1)
    rng = np.random.default_rng(11)
    xs = [rng.standard_normal(shape, dtype=np.float32) for _ in range(8)]
    want = []
    for x in xs:
        rpool.add(nasms[0], x); group.run(); group.wait(nasms[0]); group.stop()
        want.append(nasms[0].result(IMG).copy())
    group.set_service(True)
    got = [None] * len(xs)
    rpool.add(nasms[0], xs[0]); rpool.add(nasms[1], xs[1])
    group.run()
    for k in range(len(xs)):
        if k + 2 < len(xs):
            rpool.add(nasms[(k + 2) % 3], xs[k + 2])          # upload next to two running graphs
        group.wait(nasms[k % 3])
        got[k] = nasms[k % 3].result(IMG).copy()
    group.stop()
    assert group.status() == 0, api.last_error()
    for k in range(len(xs)):
        assert np.array_equal(got[k], want[k]), f"request {k}"
    assert not np.array_equal(want[0], want[1])
    _close(dnn, nasms, rpool, group)


def test_two_networks_are_served_by_one_kernel(workdir):
    cfg_a, wf_a = harness.prepare("tiny_cnn", workdir)
    cfg_b, wf_b = harness.prepare("tiny_transformer", workdir)
    dnn_a, dnn_b = api.Dnn(cfg_a, wf_a), api.Dnn(cfg_b, wf_b)
    na, nb = api.Nasm(dnn_a, 2, 0, 20), api.Nasm(dnn_b, 2, 24, 20)
    rpool, group = api.Rpool(), api.DseGroup(0, 0)
    group.set_rpool(rpool)
    rng = np.random.default_rng(3)
    ia, ib = na.ldata_info(0), nb.ldata_info(0)
    xa = [rng.standard_normal((ia["W"], ia["H"]), dtype=np.float32) for _ in range(3)]
    xb = [rng.standard_normal((ib["W"], ib["H"]), dtype=np.float32) for _ in range(3)]
    want_a, want_b = [], []
    for k in range(3):
        rpool.add(na, xa[k]); rpool.add(nb, xb[k]); group.run(); group.wait(na); group.wait(nb); group.stop()
        want_a.append(na.result(IMG).copy()); want_b.append(nb.result(SEQ).copy())
    group.set_service(True)
    for k in range(3):
        rpool.add(na, xa[k]); rpool.add(nb, xb[k])
        group.run()                           # a second dse_group_run while the kernel is resident changes nothing
        group.wait(nb); group.wait(na)
        assert np.array_equal(na.result(IMG), want_a[k]) and np.array_equal(nb.result(SEQ), want_b[k])
    group.stop()
    assert group.status() == 0
    group.close(); nb.close(); na.close(); rpool.close(); dnn_b.close(); dnn_a.close()


def test_token_ids_are_embedded_by_the_input_tiles(workdir):
    name, batch, seq, vocab = "tiny_gpt", 3, 24, 97
    cfg, wf = harness.prepare(name, workdir)
    rng = np.random.default_rng(31)
    tok = (0.02 * rng.standard_normal((vocab, 64))).astype(np.float32)
    pos = (0.02 * rng.standard_normal((seq + 5, 64))).astype(np.float32)
    dnn = api.Dnn(cfg, wf)
    dnn.set_embedding(tok, pos)
    nasm = api.Nasm(dnn, batch, seq, 20)
    rpool, group = api.Rpool(), api.DseGroup(0, 0)
    group.set_rpool(rpool)
    ids = [rng.integers(0, vocab, size=(batch, seq), dtype=np.int32) for _ in range(3)]
    want = []
    for i_ in ids:
        rpool.add_tokens(nasm, i_); group.run(); group.wait(nasm); group.stop()
        want.append([nasm.ldata(i).copy() for i in range(nasm.num_ldata)])
    group.set_service(True)
    for k, i_ in enumerate(ids):
        rpool.add_tokens(nasm, i_)
        group.run()
        group.wait(nasm)
        for i in range(nasm.num_ldata):
            assert np.array_equal(nasm.ldata(i), want[k][i]), f"ids {k}, layer {i}"
    group.stop()
    assert group.status() == 0, api.last_error()
    group.close(); nasm.close(); rpool.close(); dnn.close()


def test_the_kernel_leaves_when_idle_and_is_launched_again_on_demand(workdir, monkeypatch):
    monkeypatch.setenv("ASPEN_B200_IDLE_MS", "2")
    cfg, wf, dnn, nasms, rpool, group, shape = _net("tiny_cnn", workdir, 2, 0, 20, 0)
    nasm = nasms[0]
    rng = np.random.default_rng(9)
    xs = [rng.standard_normal(shape, dtype=np.float32) for _ in range(4)]
    want = []
    for x in xs:
        rpool.add(nasm, x); group.run(); group.wait(nasm); group.stop()
        want.append(nasm.result(IMG).copy())
    group.set_service(True)
    rpool.add(nasm, xs[0]); group.run(); group.wait(nasm)
    assert np.array_equal(nasm.result(IMG), want[0])
    time.sleep(0.05)                          # far beyond the idle limit: the kernel has left
    rpool.add(nasm, xs[1])                    # nobody is there to take it ...
    group.wait(nasm)                          # ... so the wait launches the kernel again
    assert np.array_equal(nasm.result(IMG), want[1])
    time.sleep(0.05)
    rpool.add(nasm, xs[2]); group.run(); group.wait(nasm)
    assert np.array_equal(nasm.result(IMG), want[2])
    group.stop(); group.stop()                # a second stop finds nothing to do
    rpool.reset(nasm)                         # same input once more (rpool_reset_nasm keeps layer 0's source)
    group.run(); group.wait(nasm); group.stop()
    assert np.array_equal(nasm.result(IMG), want[2])
    assert group.status() == 0, api.last_error()
    _close(dnn, nasms, rpool, group)


def test_timed_passes_complete_and_leave_valid_results(workdir):
    cfg, wf, dnn, nasms, rpool, group, shape = _net("resnet50", workdir, 2, 0, 100, 0, graphs=2, profile=1)
    x = np.random.default_rng(2).standard_normal(shape, dtype=np.float32)
    rpool.add(nasms[0], x); group.run(); group.wait(nasms[0]); group.stop()
    want = nasms[0].result(IMG).copy()
    group.set_service(True)
    for n_ in nasms:
        rpool.add(n_, x)
    group.run()
    for n_ in nasms:
        group.wait(n_)
    group.stop()
    ms, launches = group.time_passes(3, 11)
    assert ms > 0 and launches >= 2
    assert group.status() == 0, api.last_error()
    for n_ in nasms:
        assert np.array_equal(n_.result(IMG), want)
    _close(dnn, nasms, rpool, group)
