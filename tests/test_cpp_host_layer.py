"""The C++ host layer (include/nvfp4_b200.hpp): a C++ program walks one MLP block forward and backward
through the module structs (tests/cpp/mlp_layer_driver.cpp); its results must equal, byte for byte, those
of the same call sequence made through the ctypes mirror, and match the CPU oracle's dequantized
reference within the GEMM tolerance."""
from __future__ import annotations

import importlib.util
import os
import struct
import subprocess

import numpy as np
import pytest
import torch

from helpers import normal, rel_fro

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MAGIC = 0x4D4C5031
GEMM_TOL = 1e-3  # relative Frobenius error against the FP32 product of the dequantized operands


def _driver() -> str:
    spec = importlib.util.spec_from_file_location("nvfp4_build_script",
                                                  os.path.join(ROOT, "nanogpt-120a_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build_cpp_driver()


def test_cpp_driver_builds_and_reports_errors(tmp_path):
    """The header compiles as C++17 against the built library, and a failing step surfaces as a message
    and exit code 1 (no abort, no exception escaping)."""
    exe = _driver()
    assert os.access(exe, os.X_OK)
    r = subprocess.run([exe, str(tmp_path / "missing.bin"), str(tmp_path / "out.bin")], capture_output=True, text=True)
    assert r.returncode == 1 and "cannot open" in r.stderr
    bad = tmp_path / "bad.bin"
    bad.write_bytes(struct.pack("<8I", 1, 2, 3, 4, 5, 6, 7, 8))
    r = subprocess.run([exe, str(bad), str(tmp_path / "out.bin")], capture_output=True, text=True)
    assert r.returncode == 1 and "bad header" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,d_model,d_mlp", [(256, 128, 512), (384, 192, 768)])
def test_cpp_mlp_block_equals_ctypes_path(pkg, oracle, dev, tmp_path, tokens, d_model, d_mlp):
    exe = _driver()
    seeds = (0x12345678, 0x9ABCDEF0, 0x0BADF00D, 0x600DCAFE)
    f32 = lambda seed, shape, std: np.ascontiguousarray(normal(seed, shape, std), dtype=np.float32)
    x, dy = f32(701, (tokens, d_model), 1.0), f32(706, (tokens, d_model), 1e-3)
    w_fc, b_fc = f32(702, (d_mlp, d_model), 0.02), f32(703, (d_mlp,), 0.02)
    w_proj, b_proj = f32(704, (d_model, d_mlp), 0.02), f32(705, (d_model,), 0.02)
    src, dst = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(src, "wb") as f:
        f.write(struct.pack("<8I", MAGIC, tokens, d_model, d_mlp, *seeds))
        for a in (x, w_fc, b_fc, w_proj, b_proj, dy):
            f.write(a.tobytes())
    r = subprocess.run([exe, str(src), str(dst)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    raw = dst.read_bytes()
    sizes = [tokens * d_model, tokens * d_model, d_mlp * d_model, d_mlp, d_model * d_mlp, d_model]
    got, off = [], 0
    for n in sizes:
        got.append(np.frombuffer(raw, dtype=np.float32, count=n, offset=off))
        off += 4 * n
    chunk_count, status = struct.unpack_from("<2I", raw, off)
    assert off + 8 == len(raw) and status == 0 and chunk_count > 0

    # the same sequence through the ctypes mirror
    q, gemm, mlp, bwd = pkg.Nvfp4QuantModule(), pkg.Nvfp4GemmModule(), pkg.MlpModule(), pkg.LinearBackwardModule()
    t = lambda a: torch.from_numpy(a).to(dev)
    wq_fc = q.quantize_four_six(t(w_fc), rowwise=False, packed=True)
    wq_proj = q.quantize_four_six(t(w_proj), rowwise=False, packed=True)
    xq = q.quantize_four_six(t(x), rowwise=True, packed=True, decoded_amax=True)
    pre = torch.empty((tokens, d_mlp), dtype=torch.float32, device=dev)
    hidden = gemm.gemm(xq, wq_fc, bias=t(b_fc), epilogue=pkg.EPI_RELU2, out_dtype=torch.float32, aux=pre)
    hq = q.quantize_four_six(hidden, rowwise=True, packed=True, decoded_amax=True)
    y = gemm.gemm(hq, wq_proj, bias=t(b_proj), epilogue=pkg.EPI_BIAS, out_dtype=torch.float32)
    sc_proj = pkg.LinearBackwardScratch(tokens, d_mlp, d_model, dev)
    sc_fc = pkg.LinearBackwardScratch(tokens, d_model, d_mlp, dev)
    d_hidden, dw_proj, db_proj = bwd.backward_ms_eden(e=t(dy), weight=wq_proj, input=hq, scratch=sc_proj,
                                                      sign_seed=seeds[0], scale_seed=seeds[1])
    d_pre, chunks = mlp.relu2_backward_amax(pre, d_hidden, sc_fc.e_h["chunk_amax"])
    assert chunks == chunk_count
    dx, dw_fc, db_fc = bwd.backward_ms_eden(e=d_pre, weight=wq_fc, input=xq, scratch=sc_fc, sign_seed=seeds[2],
                                            scale_seed=seeds[3], precomputed_e_amax_chunks=chunks)
    want = [y, dx, dw_fc, db_fc, dw_proj, db_proj]
    for name, g, w in zip(("y", "dx", "dw_fc", "db_fc", "dw_proj", "db_proj"), got, want):
        assert g.tobytes() == w.cpu().numpy().tobytes(), name

    # the fc pre-activation the C++ program's results rest on, against the oracle: bit-exact quantizer
    # bytes, GEMM within the tolerance of the FP32 product of the dequantized operands
    ox = oracle.four_six(x, oracle.row_amax(x), True)
    ow = oracle.four_six(w_fc, oracle.tensor_amax(w_fc)[1], False)
    assert np.array_equal(xq.bytes.cpu().numpy(), ox[0]) and np.array_equal(wq_fc.bytes.cpu().numpy(), ow[0])
    want_pre = oracle.gemm(ox, ow, tokens, d_model, d_mlp, 2, bias=b_fc, epi=1)
    assert rel_fro(pre.cpu().numpy(), want_pre) <= GEMM_TOL
