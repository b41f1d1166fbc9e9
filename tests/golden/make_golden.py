"""Generates the committed golden vectors of tests/golden/*.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference ships no byte-level golden vectors for this path and cannot be run here, so
these fixtures freeze the oracle's outputs (which the known-answer tests pin to the
reference's own cases) on small seeded inputs: they catch regressions of the oracle on the
CPU and give the GPU tests inputs/outputs that do not depend on the oracle being rebuilt.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from helpers import normal  # noqa: E402
from oracle import oracle  # noqa: E402

SIGN, SCALE = 0x12345678, 0x9ABCDEF0


def bf16_round(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def main():
    x = normal(1, (24, 128))
    x[3, 5] *= 50.0
    x[7] = 0.0
    x = bf16_round(x)  # every fixture input is exactly representable in bf16
    out = {"x": x}
    b, s, g = oracle.four_six(x, oracle.tensor_amax(x)[1], rowwise=False)
    out.update(fs_tensor_bytes=b, fs_tensor_scales=s, fs_tensor_gs=g)
    b, s, g = oracle.four_six(x, oracle.row_amax(x), rowwise=True)
    out.update(fs_row_bytes=b, fs_row_scales=s, fs_row_gs=g, fs_row_packed=oracle.scale_pack(s, 24, 128))
    np.savez_compressed(os.path.join(HERE, "four_six.npz"), **out)

    e = bf16_round(normal(2, (40, 96), 1e-3))
    gs = oracle.ms_eden_global_scale(float(np.abs(e).max()))
    out = {"e": e, "gs": np.float32(gs)}
    r = oracle.ms_eden(0, e, 40, 128, gs, SIGN, SCALE)
    t = oracle.ms_eden(1, e, 96, 64, gs, SIGN, SCALE ^ 0x85EBCA6B)
    out.update(rows_bytes=r[0], rows_scales=r[1], rows_gs=r[2], rows_chunk_amax=r[3], t_bytes=t[0], t_scales=t[1],
               t_gs=t[2], t_chunk_amax=t[3])
    src = oracle.four_six(x, oracle.row_amax(x), rowwise=True)
    gsx = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(*src, 24, 128, True)[1][0]))
    xt = oracle.ms_eden(3, (*src, 24, 128), 128, 64, gsx, SIGN, SCALE ^ 0xC2B2AE35)
    out.update(xt_gs_scalar=np.float32(gsx), xt_bytes=xt[0], xt_scales=xt[1])
    np.savez_compressed(os.path.join(HERE, "ms_eden.npz"), **out)

    rng = np.random.default_rng(3)
    m, n, k = 48, 40, 128
    a = (rng.integers(0, 256, m * k // 2, dtype=np.uint8), rng.integers(0x30, 0x48, m * k // 16, dtype=np.uint8),
         (0.5 + rng.random(m)).astype(np.float32))
    w = (rng.integers(0, 256, n * k // 2, dtype=np.uint8), rng.integers(0x30, 0x48, n * k // 16, dtype=np.uint8),
         np.array([0.75], np.float32))
    bias = rng.normal(0, 10, n).astype(np.float32)
    raw = oracle.gemm(a, w, m, k, n, 2)
    relu2, pre = oracle.gemm(a, w, m, k, n, 2, bias=bias, epi=2, want_pre=True)
    np.savez_compressed(os.path.join(HERE, "gemm.npz"), a_bytes=a[0], a_scales=a[1], a_gs=a[2], w_bytes=w[0],
                        w_scales=w[1], w_gs=w[2], bias=bias, raw=raw, relu2=relu2, pre=pre)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
