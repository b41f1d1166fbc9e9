"""The oracle reproduces the committed golden vectors (tests/golden/*.npz, made by
tests/golden/make_golden.py).  CPU only."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SIGN, SCALE = 0x12345678, 0x9ABCDEF0


def load(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


def test_four_six_golden(oracle):
    g = load("four_six.npz")
    x = g["x"]
    b, s, gs = oracle.four_six(x, oracle.tensor_amax(x)[1], rowwise=False)
    assert np.array_equal(b, g["fs_tensor_bytes"]) and np.array_equal(s, g["fs_tensor_scales"])
    assert np.array_equal(gs, g["fs_tensor_gs"])
    b, s, gs = oracle.four_six(x, oracle.row_amax(x), rowwise=True)
    assert np.array_equal(b, g["fs_row_bytes"]) and np.array_equal(s, g["fs_row_scales"])
    assert np.array_equal(gs, g["fs_row_gs"]) and np.array_equal(oracle.scale_pack(s, 24, 128), g["fs_row_packed"])
    assert gs[7] == 1.0 and not b.reshape(24, -1)[7].any()  # the all-zero row


def test_ms_eden_golden(oracle):
    g = load("ms_eden.npz")
    e, gs = g["e"], float(g["gs"])
    r = oracle.ms_eden(0, e, 40, 128, gs, SIGN, SCALE)
    t = oracle.ms_eden(1, e, 96, 64, gs, SIGN, SCALE ^ 0x85EBCA6B)
    for got, key in zip(r, ("rows_bytes", "rows_scales", "rows_gs", "rows_chunk_amax")):
        assert np.array_equal(got, g[key]), key
    for got, key in zip(t, ("t_bytes", "t_scales", "t_gs", "t_chunk_amax")):
        assert np.array_equal(got, g[key]), key


def test_gemm_golden(oracle):
    g = load("gemm.npz")
    a = (g["a_bytes"], g["a_scales"], g["a_gs"])
    w = (g["w_bytes"], g["w_scales"], g["w_gs"])
    raw = oracle.gemm(a, w, 48, 128, 40, 2)
    assert np.array_equal(raw, g["raw"])
    relu2, pre = oracle.gemm(a, w, 48, 128, 40, 2, bias=g["bias"], epi=2, want_pre=True)
    assert np.array_equal(relu2, g["relu2"]) and np.array_equal(pre, g["pre"])
