"""aspen_b200_matmul_noalloc: the entry point for callers that may not allocate device memory (plug-ins
that run inside a fixed memory budget, loops that cannot take the device-wide synchronisation of an
allocation).  It must give what the regular, allocating API gives for the same matmul layer -- and what
the CPU oracle gives -- on repeated calls that share its fixed scratch array.  Collected last on purpose:
the scratch array is process-wide state."""
import os

import numpy as np
import pytest

import harness
from aspen_b200 import api, weights
from oracle import port

pytestmark = pytest.mark.gpu

RELU, GELU, TANH = 4, 8, 3


def oracle_matmul(x, w, b, act):
    """out[n][m] = act(bias[m] + sum_k w[m][k] x[n][k]) by the plain-C oracle (oracle/oracle_tiles.c)."""
    out = np.empty((x.shape[0], w.shape[0]), np.float32)
    p = lambda a: a.ctypes.data_as(port.C.c_void_p) if a is not None else None
    port.lib().oracle_matmul(p(np.ascontiguousarray(x)), p(np.ascontiguousarray(w)), p(b), p(out), x.shape[0], x.shape[1], w.shape[0], act)
    return out


def regular_api_matmul(workdir, tag, x, w, b, act_name):
    """The same layer through cfg -> dnn -> nasm -> rpool -> dse (fp32 FFMA mode)."""
    n, k = x.shape
    m = w.shape[0]
    cfg = os.path.join(workdir, f"mm_{tag}.cfg")
    with open(cfg, "w") as f:
        f.write(f"[net]\nM={k}\nheight=1\nfilters={k}\n\n[matmul]\nM={m}\nactivation={act_name}\n")
    wf = os.path.join(workdir, f"mm_{tag}.bin")
    weights.write_aspen_data(wf, [(w, b)])
    dev = harness.Device(cfg, wf, 1, n, 4, precision=1, profile=1)
    assert dev.run(x) == 0, api.last_error()
    out = dev.nasm.ldata(1).copy()
    dev.close()
    return out


def test_noalloc_matmul_matches_regular_api_on_two_calls_in_a_row(workdir):
    import torch
    L = api.lib()
    rng = np.random.default_rng(7)
    # second call is smaller and differently shaped: stale descriptors of the first call must not matter
    for call, (n, k, m, act, act_name) in enumerate([(300, 192, 260, RELU, "relu"), (130, 64, 72, GELU, "gelu")]):
        x = rng.standard_normal((n, k), dtype=np.float32)
        w = (rng.standard_normal((m, k), dtype=np.float32) / np.sqrt(k)).astype(np.float32)
        b = rng.standard_normal((m,), dtype=np.float32)
        want = regular_api_matmul(workdir, str(call), x, w, b, act_name)
        xd, wd, bd = (torch.from_numpy(a).cuda() for a in (x, w, b))
        od = torch.full((n, m), float("nan"), device="cuda")
        torch.cuda.synchronize()
        rc = L.aspen_b200_matmul_noalloc(xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), od.data_ptr(), n, k, m, act, None)
        assert rc == 0, api.last_error()
        got = od.cpu().numpy()
        scale = float(np.abs(want).max())
        bad, ea, er = harness.compare(got, want, 1e-4, 1e-5 * scale)      # the fp32 rule of the parity tests
        assert bad == 0, f"call {call}: {bad} mismatches, max abs {ea:.3e}, max rel {er:.3e}"
        bad, ea, er = harness.compare(got, oracle_matmul(x, w, b, act), 1e-4, 1e-5 * scale)
        assert bad == 0, f"call {call} vs CPU oracle: {bad} mismatches, max abs {ea:.3e}, max rel {er:.3e}"


def test_noalloc_matmul_odd_shapes_no_bias_and_unaligned_input_match_the_oracle():
    """Shapes whose tiles are clipped in both directions, k not a multiple of 4 (scalar loads), no bias,
    and an input that starts 4 bytes off a 16-byte boundary."""
    import torch
    L = api.lib()
    rng = np.random.default_rng(9)
    for n, k, m, act, with_bias, offset in [(37, 50, 130, TANH, False, 0), (129, 64, 257, RELU, True, 1), (5, 3, 2, 0, True, 0)]:
        x = rng.standard_normal((n, k), dtype=np.float32)
        w = (rng.standard_normal((m, k), dtype=np.float32) / np.sqrt(k)).astype(np.float32)
        b = rng.standard_normal((m,), dtype=np.float32) if with_bias else None
        flat = torch.zeros(n * k + 4, device="cuda")
        flat[offset:offset + n * k] = torch.from_numpy(x).cuda().reshape(-1)
        xd = flat[offset:offset + n * k]
        wd = torch.from_numpy(w).cuda()
        bd = torch.from_numpy(b).cuda() if with_bias else None
        od = torch.full((n, m), float("nan"), device="cuda")
        torch.cuda.synchronize()
        rc = L.aspen_b200_matmul_noalloc(xd.data_ptr(), wd.data_ptr(), bd.data_ptr() if with_bias else None, od.data_ptr(), n, k, m, act, None)
        assert rc == 0, api.last_error()
        want = oracle_matmul(x, w, b, act)
        bad, ea, er = harness.compare(od.cpu().numpy(), want, 1e-4, 1e-5 * float(np.abs(want).max()))
        assert bad == 0, f"({n},{k},{m}): {bad} mismatches, max abs {ea:.3e}, max rel {er:.3e}"


def test_noalloc_matmul_rejects_oversized_and_bad_arguments():
    import torch
    L = api.lib()
    t = torch.zeros(16, device="cuda")
    # 65 x 64 tiles of 128 x 128 = 4160 > 4096
    assert L.aspen_b200_matmul_noalloc(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 64 * 128, 4, 65 * 128, 0, None) == -2
    assert "4096" in api.last_error()
    # sizes near 2^32 must not wrap into a small tile count
    assert L.aspen_b200_matmul_noalloc(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 4, 4, 2**32 - 5, 0, None) == -2
    assert L.aspen_b200_matmul_noalloc(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 2**32 - 100, 4, 4, 0, None) == -2
    assert L.aspen_b200_matmul_noalloc(None, t.data_ptr(), None, t.data_ptr(), 4, 4, 4, 0, None) == -1
    assert L.aspen_b200_matmul_noalloc(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 4, 4, 4, 99, None) == -1
