"""The CPU oracle (oracle/oracle_tiles.c driven by oracle/port.py) against fixtures produced by
the unmodified reference (tests/golden/make_golden.py) and, where the reference build is present,
against the reference run live."""
import os

import numpy as np
import pytest

import harness
from aspen_b200 import cfgs, weights
from oracle import port, ref

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = [("tiny_cnn", 2, 0), ("tiny_transformer", 2, 16), ("tiny_gpt", 2, 16), ("custom", 2, 0), ("tiny_yolo", 2, 0), ("tiny_acts", 3, 0)]
# The oracle sums in plain k order in fp32, the reference in 8-wide vectors over K-blocks of 368:
# agreement is to rounding, not bit-exact.
REL, ABS = 1e-4, 1e-5


def _net(name):
    kw, scheme, (wseed, _) = harness.NETS[name]
    text, wl = cfgs.BUILDERS[harness._BUILDER.get(name, name)](**kw)
    return text, weights.make_weights(wl, wseed, scheme)


def _input_shape(name, batch, seq):
    text, _ = _net(name)
    first = port.parse_cfg(text)[0]["opts"]
    if "M" in first:
        return (batch * seq, int(first["M"]))
    return (batch * int(first["height"]) * int(first["width"]), int(first["channels"]))


@pytest.mark.parametrize("name,batch,seq", CASES)
def test_port_matches_reference_fixtures(name, batch, seq):
    text, w = _net(name)
    x = harness.make_input(name, _input_shape(name, batch, seq))
    outs = port.run(text, w, x, batch, seq)
    gold = np.load(os.path.join(GOLDEN, f"values_{name}.npz"))
    assert len(gold.files) >= 5
    for key in gold.files:
        idx = int(key.split("_")[1])
        want = gold[key]
        got = outs[idx]
        assert got.shape == want.shape, (key, got.shape, want.shape)
        scale = float(np.abs(want).max())
        bad, ea, er = harness.compare(got, want, REL, ABS * scale)
        assert bad == 0, f"{name} {key}: {bad} mismatches, max abs {ea:.3e}, max rel {er:.3e}"


@pytest.mark.skipif(not ref.available(), reason="reference build (oracle/_ref) not present")
@pytest.mark.parametrize("name,batch,seq", [("tiny_cnn", 3, 0), ("tiny_gpt", 1, 24), ("tiny_yolo", 3, 0), ("tiny_acts", 2, 0)])
def test_port_matches_reference_live(name, batch, seq, workdir):
    cfg, wf = harness.prepare(name, workdir)
    text, w = _net(name)
    rn = ref.RefNet(cfg, wf, batch, seq, min_ninst=7)
    i0 = rn.ldata_info(0)
    x = harness.make_input(name, (i0["W"], i0["H"]))
    rn.walk(x, threads=2)
    outs = port.run(text, w, x, batch, seq)
    for i in range(1, rn.num_ldata):
        want = rn.ldata(i)
        scale = float(np.abs(want).max())
        bad, ea, er = harness.compare(outs[i], want, REL, ABS * scale)
        assert bad == 0, f"{name} layer {i}: {bad} mismatches, max abs {ea:.3e}"
    rn.close()


def test_activation_edge_values():
    L = port.lib()
    x = np.array([-3.0, -0.0, 0.0, 1e-8, 2.5, -1e4, 1e4], np.float32)
    for act, fn in ((4, lambda v: np.maximum(v, 0)), (5, lambda v: np.where(v > 0, v, 0.1 * v))):
        y = x.copy()
        L.oracle_activate(y.ctypes.data_as(port.C.c_void_p), port.C.c_size_t(y.size), act)
        np.testing.assert_allclose(y, fn(x).astype(np.float32), rtol=1e-6)


def test_maxpool_all_padding_is_minus_inf():
    # a window that lies entirely in the padding yields -inf (reference src/tiled_kernels.c:428-436)
    L = port.lib()
    x = np.ones((1 * 2 * 2, 1), np.float32)
    out = np.zeros((1 * 3 * 3, 1), np.float32)      # k=1, stride=2, pad=2 -> 3x3 outputs, corners outside
    L.oracle_maxpool2d(x.ctypes.data_as(port.C.c_void_p), out.ctypes.data_as(port.C.c_void_p), 1, 2, 2, 1, 1, 1, 2, 2, 0)
    assert np.isneginf(out[0, 0]) and out[4, 0] == 1.0


def test_masked_attention_rows_sum_to_one_and_are_causal():
    L = port.lib()
    B, S, heads, hidden = 2, 12, 2, 16
    rng = np.random.default_rng(0)
    q = rng.standard_normal((B * S, hidden), dtype=np.float32)
    k = rng.standard_normal((B * S, hidden), dtype=np.float32)
    out = np.empty((B * heads * S, S), np.float32)
    L.oracle_k_attention(q.ctypes.data_as(port.C.c_void_p), k.ctypes.data_as(port.C.c_void_p), out.ctypes.data_as(port.C.c_void_p),
                         B, S, heads, hidden, 1)
    np.testing.assert_allclose(out.sum(1), 1.0, rtol=1e-5)
    p = out.reshape(B, heads, S, S)
    assert np.all(np.triu(p, 1) == 0.0)
