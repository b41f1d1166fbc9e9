"""GPU parity tests: the sm_100a kernels, called through the C ABI, against the CPU oracle on
the same seeded inputs.  Bit-exact for every byte / index / scale output; GEMM outputs within
a relative Frobenius error of 1e-3 of the FP32 dequantized oracle (the tolerance the path's
specification states).  bf16 GEMM outputs are compared with the oracle result rounded to bf16
(bf16 rounding alone is ~1.1e-3 RMS)."""
import numpy as np
import pytest
import torch

from helpers import bf16_normal, normal, rel_fro, set_e2m1_one, with_outliers

pytestmark = pytest.mark.gpu

GEMM_TOL = 1e-3
SIGN, SCALE = 0x12345678, 0x9ABCDEF0  # crates/cuda-kernels/tests/nvfp4_quant.rs:70-71


def cpu(t):
    return t.detach().cpu().numpy()


def assert_no_timeouts(pkg):
    torch.cuda.synchronize()
    assert pkg.read_device_status() == 0


# ------------------------------------------------------------------------------------------ amax

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 16), (7, 48), (128, 768), (33, 1000), (5, 1024 + 8)])
def test_amax(pkg, oracle, dev, dtype, shape):
    q = pkg.Nvfp4QuantModule()
    x = bf16_normal(11, shape).to(dtype)
    x[0, 0] = float("nan")  # max.f32 drops NaN operands
    xf = x.float().numpy()
    got_row = cpu(q.row_amax(x.to(dev)))
    assert np.array_equal(got_row, oracle.row_amax(xf))
    chunks, amax = q.tensor_amax(x.to(dev))
    o_chunks, o_amax = oracle.tensor_amax(xf)
    assert np.array_equal(cpu(chunks), o_chunks) and np.array_equal(cpu(amax), o_amax)
    again = q.tensor_amax_from_chunks_f32(chunks, chunks.numel())
    assert np.array_equal(cpu(again), o_amax)


# ------------------------------------------------------------------------------------------ four-six

def _check_four_six(pkg, oracle, dev, x, rowwise, packed):
    q = pkg.Nvfp4QuantModule()
    xf = x.float().numpy()
    rows, cols = xf.shape
    amax = oracle.row_amax(xf) if rowwise else oracle.tensor_amax(xf)[1]
    ob, os_, og = oracle.four_six(xf, amax, rowwise)
    t = q.quantize_four_six(x.to(dev), rowwise=rowwise, packed=packed)
    assert np.array_equal(cpu(t.bytes), ob)
    want_scales = oracle.scale_pack(os_, rows, cols) if packed else os_
    assert np.array_equal(cpu(t.scales), want_scales)
    assert np.array_equal(cpu(t.global_scales), og)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rowwise", [False, True])
@pytest.mark.parametrize("shape,packed", [((1, 16), False), ((3, 48), False), ((128, 768), True), ((200, 192), True),
                                          ((129, 64), True), ((64, 1024), False)])
def test_four_six_bit_exact(pkg, oracle, dev, dtype, rowwise, shape, packed):
    x = with_outliers(bf16_normal(21, shape), seed=5, every=97).to(dtype)
    _check_four_six(pkg, oracle, dev, x, rowwise, packed)


@pytest.mark.parametrize("shape,packed", [((1, 16), False), ((3, 48), False), ((37, 1040), False), ((200, 192), True),
                                          ((768, 768), True)])
@pytest.mark.parametrize("beta", [0.0, 0.9, 1.0])
def test_materialize_schedule_free(pkg, oracle, dev, shape, packed, beta):
    """gpt/optimizer/launcher/update.rs:11-58: amax and four-six of y = z + beta (x - z), bit-exact."""
    opt = pkg.OptimizerModule()
    z = torch.from_numpy(normal(61, shape, 0.02).astype(np.float32))
    x = z + torch.from_numpy(normal(62, shape, 0.003).astype(np.float32))
    x[0, 3] = 1.5  # an outlier decides the tensor scale
    t, amax = opt.materialize_schedule_free(z.to(dev), x.to(dev), beta, packed=packed)
    y = oracle.schedule_free_value(z.numpy(), x.numpy(), beta).reshape(shape)
    if beta == 0.0:
        assert np.array_equal(y, z.numpy())
    want_amax = oracle.tensor_amax(y)[1]
    assert cpu(amax).tobytes() == want_amax.tobytes()
    ob, os_, og = oracle.four_six(y, want_amax, False)
    assert np.array_equal(cpu(t.bytes), ob)
    assert np.array_equal(cpu(t.scales), oracle.scale_pack(os_, *shape) if packed else os_)
    assert np.array_equal(cpu(t.global_scales), og)


@pytest.mark.parametrize("n", [1, 8, 1000, 8 * 4096 + 5])
@pytest.mark.parametrize("kind", ["f32", "f16", "bf16"])
def test_relu2_backward(pkg, oracle, dev, n, kind):
    """gpt/mlp/kernels.rs:72-104, including -0, NaN and unaligned views."""
    mlp = pkg.MlpModule()
    pre = torch.from_numpy(normal(71, (n + 1,), 1.0).astype(np.float32))
    d = torch.from_numpy(normal(72, (n + 1,), 1e-3).astype(np.float32))
    pre[0] = -0.0
    if n > 4:
        pre[3] = float("nan")
    for off in (0, 1):  # offset 1: not 16-byte aligned
        p, g = pre[off:off + n], d[off:off + n]
        if kind == "bf16":
            p, g = p.bfloat16(), g.bfloat16()
            got = mlp.relu2_backward(p.to(dev)[:], g.to(dev)[:]).float()
            want = torch.from_numpy(oracle.relu2_backward(p.float().numpy(), g.float().numpy())).bfloat16().float()
        else:
            p = p.half() if kind == "f16" else p
            got = mlp.relu2_backward(p.to(dev), g.to(dev))
            want = torch.from_numpy(oracle.relu2_backward(p.float().numpy(), g.numpy()))
        assert cpu(got).tobytes() == want.numpy().tobytes()


def test_four_six_rowwise_long_rows(pkg, oracle, dev):
    """Rows longer than one thread block covers take the two-kernel path; a row that exactly fills
    a block (4096) and ragged row counts take the fused one."""
    for shape in [(3, 8192), (5, 4096), (7, 2048), (11, 48)]:
        x = with_outliers(bf16_normal(23, shape), seed=9, every=53)
        _check_four_six(pkg, oracle, dev, x, rowwise=True, packed=False)


@pytest.mark.parametrize("shape,packed,dtype", [((3001, 768), True, torch.bfloat16), ((9411, 192), True, torch.float32),
                                                ((23011, 80), False, torch.bfloat16), ((1300, 3072), True, torch.bfloat16)])
def test_four_six_rowwise_persistent_kernel(pkg, oracle, dev, shape, packed, dtype):
    """More row blocks than resident CTAs: the fused rowwise quantizer runs persistent CTAs that prefetch
    their next row block.  Ragged row counts, a group count that is not a multiple of four (byte stores
    instead of gathered words), decoded amax, and relu^2 on load."""
    q = pkg.Nvfp4QuantModule()
    x = with_outliers(bf16_normal(29, shape), seed=4, every=211).to(dtype)
    xf = x.float().numpy()
    t = q.quantize_four_six(x.to(dev), rowwise=True, packed=packed, decoded_amax=True)
    ob, os_, og = oracle.four_six(xf, oracle.row_amax(xf), True)
    assert np.array_equal(cpu(t.bytes), ob)
    assert np.array_equal(cpu(t.scales), oracle.scale_pack(os_, *shape) if packed else os_)
    assert np.array_equal(cpu(t.global_scales), og)
    assert cpu(t.decoded_amax).tobytes() == np.asarray(oracle.nvfp4_amax(ob, os_, og, *shape, True)[1], np.float32).tobytes()
    relu = np.maximum(xf, np.float32(0))
    act = relu * relu
    t = q.quantize_relu2_four_six_rowwise(x.to(dev), packed=packed)
    ob, os_, og = oracle.four_six(act, oracle.row_amax(act), True)
    assert np.array_equal(cpu(t.bytes), ob)
    assert np.array_equal(cpu(t.scales), oracle.scale_pack(os_, *shape) if packed else os_)
    assert np.array_equal(cpu(t.global_scales), og)


def test_four_six_edge_values(pkg, oracle, dev):
    """Zero rows, ties on the E2M1 grid, huge and tiny magnitudes, negative zero."""
    x = torch.zeros(8, 64)
    x[1] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 8)
    x[2] = -x[1]
    x[3] = 1e30
    x[4] = 1e-30
    x[5, ::2] = -0.0
    x[6] = torch.linspace(-3, 3, 64)
    x[7, 5] = 448.0 * 6 * 3
    for rowwise in (False, True):
        _check_four_six(pkg, oracle, dev, x, rowwise, packed=False)


def test_quantize_round_trip_8192x768(pkg, oracle, dev):
    """The round-trip case of the specification: [8192 x 768] bf16 ~N(0,1) with 0.1 % of the elements scaled
    by 50, per-tensor and rowwise scale, then the dequantize round trip."""
    x = with_outliers(bf16_normal(1, (8192, 768)), seed=2, every=1000, factor=50.0)
    _check_four_six(pkg, oracle, dev, x, rowwise=False, packed=True)
    _check_four_six(pkg, oracle, dev, x, rowwise=True, packed=False)
    q, d = pkg.Nvfp4QuantModule(), pkg.Nvfp4DecodeModule()
    t = q.quantize_four_six(x.to(dev), rowwise=True, packed=False)
    back = cpu(d.decode(t))
    want = oracle.decode(cpu(t.bytes), cpu(t.scales), cpu(t.global_scales), 8192, 768, rowwise=True, transpose=False)
    assert np.array_equal(back, want)
    assert rel_fro(back, x.float().numpy()) < 0.12  # 4-bit round trip error, sanity only


def test_four_six_reference_named_entries(pkg, oracle, dev):
    q = pkg.Nvfp4QuantModule()
    x = bf16_normal(31, (24, 80)).float()
    xf = x.numpy()
    amax = oracle.tensor_amax(xf)[1]
    t = q.fp32_to_nvfp4_four_six(x.to(dev), torch.from_numpy(amax).to(dev))
    ob, os_, og = oracle.four_six(xf, amax, rowwise=False)
    assert np.array_equal(cpu(t.bytes), ob) and np.array_equal(cpu(t.scales), os_) and np.array_equal(cpu(t.global_scales), og)
    ramax = oracle.row_amax(xf)
    t = q.fp32_to_nvfp4_four_six_rowwise(x.to(dev), torch.from_numpy(ramax).to(dev))
    ob, os_, og = oracle.four_six(xf, ramax, rowwise=True)
    assert np.array_equal(cpu(t.bytes), ob) and np.array_equal(cpu(t.scales), os_) and np.array_equal(cpu(t.global_scales), og)
    for transposed, (pr, pc) in ((False, (32, 96)), (True, (96, 32))):
        t = q.fp32_to_nvfp4_four_six_padded(x.to(dev), torch.from_numpy(amax).to(dev), pr, pc, transposed=transposed)
        ob, os_, og = oracle.four_six_padded(xf, amax, pr, pc, transposed)
        assert np.array_equal(cpu(t.bytes), ob) and np.array_equal(cpu(t.scales), os_)
        assert np.array_equal(cpu(t.global_scales), og)


# ------------------------------------------------------------------------------------------ MS-EDEN

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols,dst,packed", [(2, 32, 32, False), (5, 40, 64, False), (128, 768, 768, True),
                                                  (130, 100, 128, True), (64, 2304, 2304, False)])
def test_ms_eden_rows_bit_exact(pkg, oracle, dev, dtype, rows, cols, dst, packed):
    q = pkg.Nvfp4QuantModule()
    x = bf16_normal(41, (rows, cols), std=1e-3).to(dtype)
    xf = x.float().numpy()
    gs = oracle.ms_eden_global_scale(float(np.abs(xf).max()))
    ob, os_, og, oc = oracle.ms_eden(0, xf, rows, dst, gs, SIGN, SCALE)
    t, ca = q.ms_eden_quantize(src_kind=pkg.SRC_F32_ROWS, x=x.to(dev), rows=rows, cols=cols, dst_row_len=dst,
                               global_scale=gs, sign_seed=SIGN, scale_seed=SCALE, packed=packed, want_chunk_amax=True)
    assert np.array_equal(cpu(t.bytes), ob)
    assert np.array_equal(cpu(t.scales), oracle.scale_pack(os_, rows, dst) if packed else os_)
    assert np.array_equal(cpu(t.global_scales), og)
    assert np.array_equal(cpu(ca), oc)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols,packed", [(33, 16, False), (128, 64, True), (200, 48, False), (256, 96, True)])
def test_ms_eden_transposed_bit_exact(pkg, oracle, dev, dtype, rows, cols, packed):
    q = pkg.Nvfp4QuantModule()
    x = bf16_normal(43, (rows, cols), std=1e-3).to(dtype)
    xf = x.float().numpy()
    dst = pkg.padded_k(rows)
    gs = torch.tensor([oracle.ms_eden_global_scale(float(np.abs(xf).max()))], dtype=torch.float32)
    ob, os_, og, oc = oracle.ms_eden(1, xf, cols, dst, float(gs[0]), SIGN, SCALE, col_offset=7, group_offset=6)
    t, ca = q.ms_eden_quantize(src_kind=pkg.SRC_F32_TRANSPOSED, x=x.to(dev), rows=rows, cols=cols, dst_row_len=dst,
                               global_scale=gs.to(dev), sign_seed=SIGN, scale_seed=SCALE, packed=packed,
                               want_chunk_amax=True, col_offset=7, group_offset=6)
    assert np.array_equal(cpu(t.bytes), ob)
    assert np.array_equal(cpu(t.scales), oracle.scale_pack(os_, cols, dst) if packed else os_)
    assert np.array_equal(cpu(t.global_scales), og) and np.array_equal(cpu(ca), oc)


def test_ms_eden_transposed_long_destination(pkg, oracle, dev):
    """A destination longer than the tiled kernel covers takes the generic gather kernel."""
    q = pkg.Nvfp4QuantModule()
    rows, cols, dst = 33, 16, 192
    x = bf16_normal(44, (rows, cols), std=1e-3).float()
    ob, os_, og, oc = oracle.ms_eden(1, x.numpy(), cols, dst, 0.75, SIGN, SCALE, so=0.25)
    t, ca = q.ms_eden_quantize(src_kind=pkg.SRC_F32_TRANSPOSED, x=x.to(dev), rows=rows, cols=cols, dst_row_len=dst,
                               global_scale=0.75, sign_seed=SIGN, scale_seed=SCALE, scale_override=0.25,
                               want_chunk_amax=True)
    assert np.array_equal(cpu(t.bytes), ob) and np.array_equal(cpu(t.scales), os_)
    assert np.array_equal(cpu(t.global_scales), og) and np.array_equal(cpu(ca), oc)


@pytest.mark.parametrize("rowwise", [False, True])
@pytest.mark.parametrize("src_packed", [False, True])
def test_ms_eden_nvfp4_sources_bit_exact(pkg, oracle, dev, rowwise, src_packed):
    """NVFP4 -> NVFP4 transposed re-quantizers (weight W and saved activation X)."""
    q = pkg.Nvfp4QuantModule()
    rows, cols = 96, 128
    x = bf16_normal(45, (rows, cols))
    src = q.quantize_four_six(x.to(dev), rowwise=rowwise, packed=src_packed)
    xf = x.float().numpy()
    sb, ss, sg = oracle.four_six(xf, oracle.row_amax(xf) if rowwise else oracle.tensor_amax(xf)[1], rowwise)
    kind = 3 if rowwise else 2
    dst = pkg.padded_k(rows)
    _, o_amax = oracle.nvfp4_amax(sb, ss, sg, rows, cols, rowwise)
    gs = oracle.ms_eden_global_scale(float(o_amax[0]))
    ob, os_, og, oc = oracle.ms_eden(kind, (sb, ss, sg, rows, cols), cols, dst, gs, SIGN, SCALE)
    if not src_packed:
        fn = (q.rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale if rowwise
              else q.nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale)
        t, g_dev, ca = fn(src, dst, SIGN, SCALE)
        assert cpu(g_dev)[0] == np.float32(gs)
        assert np.array_equal(cpu(ca), oc)
    else:
        t, _ = q.ms_eden_quantize(src_kind=kind, src=src, rows=rows, cols=cols, dst_row_len=dst, global_scale=gs,
                                  sign_seed=SIGN, scale_seed=SCALE)
    assert np.array_equal(cpu(t.bytes), ob) and np.array_equal(cpu(t.scales), os_)
    assert np.array_equal(cpu(t.global_scales), og)


@pytest.mark.parametrize("rowwise", [False, True])
@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 384)])
def test_ms_eden_nvfp4_whole_tile_sources(pkg, oracle, dev, rowwise, rows, cols):
    """Whole 128 x 128 tiles with packed source scales take the two-rows-per-thread transposer;
    chunk amax, sign / group offsets and a packed destination included."""
    q = pkg.Nvfp4QuantModule()
    x = with_outliers(bf16_normal(46, (rows, cols)), seed=8, every=211)
    src = q.quantize_four_six(x.to(dev), rowwise=rowwise, packed=True)
    xf = x.float().numpy()
    sb, ss, sg = oracle.four_six(xf, oracle.row_amax(xf) if rowwise else oracle.tensor_amax(xf)[1], rowwise)
    kind = 3 if rowwise else 2
    gs = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(sb, ss, sg, rows, cols, rowwise)[1][0]))
    for packed_dst in (False, True):
        ob, os_, og, oc = oracle.ms_eden(kind, (sb, ss, sg, rows, cols), cols, rows, gs, SIGN, SCALE, col_offset=5,
                                         group_offset=10)
        t, ca = q.ms_eden_quantize(src_kind=kind, src=src, rows=rows, cols=cols, dst_row_len=rows, global_scale=gs,
                                   sign_seed=SIGN, scale_seed=SCALE, packed=packed_dst, want_chunk_amax=True,
                                   col_offset=5, group_offset=10)
        assert np.array_equal(cpu(t.bytes), ob)
        assert np.array_equal(cpu(t.scales), oracle.scale_pack(os_, cols, rows) if packed_dst else os_)
        assert np.array_equal(cpu(t.global_scales), og) and np.array_equal(cpu(ca), oc)


def test_ms_eden_reference_named_entries(pkg, oracle, dev):
    """derived-device-scale rows, the pair entry and the reference's 64-value ramp case."""
    q = pkg.Nvfp4QuantModule()
    ramp = ((torch.arange(64, dtype=torch.float32) - 31.5) * 0.03125).reshape(2, 32)
    t, ca = q.fp32_to_nvfp4_ms_eden(ramp.to(dev), 32, 1.0, pkg.QUARTET_MS_EDEN_SCALE_OVERRIDE, SIGN, SCALE)
    ob, os_, og, oc = oracle.ms_eden(0, ramp.numpy(), 2, 32, 1.0, SIGN, SCALE)
    assert np.array_equal(cpu(t.bytes), ob) and np.array_equal(cpu(t.scales), os_)
    assert np.array_equal(cpu(t.global_scales), og) and np.array_equal(cpu(ca), oc)

    x = bf16_normal(47, (96, 80), std=1e-3).float()
    xf = x.numpy()
    gs = oracle.ms_eden_global_scale(float(np.abs(xf).max()))
    t, g_dev, ca = q.fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale(x.to(dev), 128, SIGN, SCALE)
    ob, os_, og, oc = oracle.ms_eden(0, xf, 96, 128, gs, SIGN, SCALE)
    assert cpu(g_dev)[0] == np.float32(gs)
    assert np.array_equal(cpu(t.bytes), ob) and np.array_equal(cpu(t.scales), os_) and np.array_equal(cpu(ca), oc)

    r, tr, g_dev = q.fp32_pair_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
        x.to(dev), 128, 128, SIGN, SCALE, SCALE ^ 0x85EBCA6B)
    ot = oracle.ms_eden(1, xf, 80, 128, gs, SIGN, SCALE ^ 0x85EBCA6B)
    assert np.array_equal(cpu(r.bytes), ob) and np.array_equal(cpu(r.scales), os_)
    assert np.array_equal(cpu(tr.bytes), ot[0]) and np.array_equal(cpu(tr.scales), ot[1])
    assert np.array_equal(cpu(tr.global_scales), ot[2])


def test_kernels_match_committed_golden_vectors(pkg, dev):
    """The CUDA path against tests/golden/*.npz (no oracle involved at run time)."""
    import os

    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    q, gemm = pkg.Nvfp4QuantModule(), pkg.Nvfp4GemmModule()
    g = dict(np.load(os.path.join(golden, "four_six.npz")))
    x = torch.from_numpy(g["x"]).to(dev)
    t = q.quantize_four_six(x.to(torch.bfloat16), rowwise=False, packed=False)
    assert np.array_equal(cpu(t.bytes), g["fs_tensor_bytes"]) and np.array_equal(cpu(t.scales), g["fs_tensor_scales"])
    t = q.quantize_four_six(x, rowwise=True, packed=True)
    assert np.array_equal(cpu(t.bytes), g["fs_row_bytes"]) and np.array_equal(cpu(t.scales), g["fs_row_packed"])
    assert np.array_equal(cpu(t.global_scales), g["fs_row_gs"])
    src = q.quantize_four_six(x, rowwise=True, packed=False)
    m = dict(np.load(os.path.join(golden, "ms_eden.npz")))
    e = torch.from_numpy(m["e"]).to(dev)
    r, tr, gs = q.fp32_pair_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
        e, 128, 64, SIGN, SCALE, SCALE ^ 0x85EBCA6B)
    assert cpu(gs)[0] == m["gs"]
    assert np.array_equal(cpu(r.bytes), m["rows_bytes"]) and np.array_equal(cpu(r.scales), m["rows_scales"])
    assert np.array_equal(cpu(tr.bytes), m["t_bytes"]) and np.array_equal(cpu(tr.scales), m["t_scales"])
    xt, xgs, _ = q.rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale(src, 64, SIGN,
                                                                                             SCALE ^ 0xC2B2AE35)
    assert cpu(xgs)[0] == m["xt_gs_scalar"]
    assert np.array_equal(cpu(xt.bytes), m["xt_bytes"]) and np.array_equal(cpu(xt.scales), m["xt_scales"])
    k = dict(np.load(os.path.join(golden, "gemm.npz")))
    A = _to_dev(pkg, dev, (k["a_bytes"], k["a_scales"], k["a_gs"]), 48, 128, True)
    W = _to_dev(pkg, dev, (k["w_bytes"], k["w_scales"], k["w_gs"]), 40, 128, False)
    assert rel_fro(cpu(gemm.gemm(A, W)), k["raw"]) <= GEMM_TOL
    aux = torch.empty((48, 40), dtype=torch.float32, device=dev)
    out = gemm.gemm(A, W, bias=torch.from_numpy(k["bias"]).to(dev), epilogue=pkg.EPI_RELU2, aux=aux)
    assert rel_fro(cpu(out), k["relu2"]) <= GEMM_TOL and rel_fro(cpu(aux), k["pre"]) <= GEMM_TOL


# ------------------------------------------------------------------------------------------ layout / decode / post-ops

def test_scale_pack_decode_pad(pkg, oracle, dev):
    rng = np.random.default_rng(3)
    logical = rng.integers(0, 255, size=(200 * 12,), dtype=np.uint8)
    packed = pkg.Sm120ScalePackModule().pack(torch.from_numpy(logical).to(dev), 200, 192)
    assert np.array_equal(cpu(packed), oracle.scale_pack(logical, 200, 192))

    # reference decode test: all-ones payload (crates/cuda-kernels/tests/nvfp4_decode.rs:18-51)
    t = pkg.Nvfp4Tensor(torch.full((16,), 0x22, dtype=torch.uint8, device=dev),
                        torch.full((2,), 0x38, dtype=torch.uint8, device=dev),
                        torch.tensor([1.0, 2.0], device=dev), 2, 16, rowwise=True)
    out = cpu(pkg.Nvfp4DecodeModule().decode_transpose_f32(t))
    assert np.array_equal(out.reshape(-1), np.tile([1.0, 2.0], 16).astype(np.float32))
    t.rowwise, t.global_scales = False, torch.tensor([3.0], device=dev)
    assert (cpu(pkg.Nvfp4DecodeModule().decode_transpose_f32(t)) == 3.0).all()

    pad = pkg.TmaMatrixPadModule()
    a = torch.from_numpy(normal(9, (5, 7)).astype(np.float32))
    p = cpu(pad.pad_f32(a.to(dev), 8, 16))
    assert np.array_equal(p[:5, :7], a.numpy()) and p[5:].sum() == 0 and p[:, 7:].sum() == 0
    pt = cpu(pad.transpose_pad_f32(a.to(dev), 8, 16))
    assert np.array_equal(pt[:7, :5], a.numpy().T) and pt[7:].sum() == 0
    assert np.array_equal(cpu(pad.crop_f32(torch.from_numpy(p).to(dev), 7)), p[:, :7])
    u4 = torch.arange(32, dtype=torch.uint8)
    padded = cpu(pad.pad_u4_rows(u4.to(dev), 4, 6, 16))
    assert np.array_equal(padded[:32], u4.numpy()) and not padded[32:].any()


def test_bias_grad_bit_exact(pkg, oracle, dev):
    bwd = pkg.LinearBackwardModule()
    for shape in [(64, 64), (1000, 100), (8192, 96), (3, 5)]:
        e = torch.from_numpy(normal(13, shape, 1e-3).astype(np.float32))
        assert np.array_equal(cpu(bwd.linear_bias_grad(e.to(dev))), oracle.bias_grad(e.numpy()))


def test_postops_bit_exact(pkg, oracle, dev):
    q, post = pkg.Nvfp4QuantModule(), pkg.ProjectionPostOpModule()
    rows, cols = 64, 48
    raw = torch.from_numpy(normal(15, (rows, cols)).astype(np.float32))
    res = torch.from_numpy(normal(16, (rows, cols)).astype(np.float32))
    bias_f = bf16_normal(17, (1, cols), 0.02)
    bias = q.quantize_four_six(bias_f.to(dev), rowwise=False, packed=False)
    bias_dec = oracle.decode(cpu(bias.bytes), cpu(bias.scales), cpu(bias.global_scales), 1, cols, False, False)[0]
    assert np.array_equal(cpu(post.bias_inplace(raw.clone().to(dev), bias)), raw.numpy() + bias_dec)
    want_res = np.float32(1.0) * (raw.numpy() + bias_dec) + res.numpy()
    assert np.array_equal(cpu(post.residual_add(raw.to(dev), bias, res.clone().to(dev))), want_res)
    pre = raw.clone().to(dev)
    out = cpu(post.relu2_inplace(pre, bias))
    assert np.array_equal(cpu(pre), raw.numpy() + bias_dec)
    assert np.array_equal(out, np.maximum(raw.numpy() + bias_dec, 0) ** 2)


# ------------------------------------------------------------------------------------------ GEMM

def _rand_nvfp4(rng, rows, k, rowwise):
    """Random NVFP4 tensor with scale bytes in a sane range (no NaN / inf encodings)."""
    b = rng.integers(0, 256, size=rows * k // 2, dtype=np.uint8)
    s = rng.integers(0x20, 0x50, size=rows * k // 16, dtype=np.uint8)
    g = (0.5 + rng.random(rows if rowwise else 1)).astype(np.float32)
    return b, s, g


def _to_dev(pkg, dev, t, rows, k, rowwise, packed_by=None):
    b, s, g = t
    return pkg.Nvfp4Tensor(torch.from_numpy(b).to(dev), torch.from_numpy(s).to(dev), torch.from_numpy(g).to(dev), rows, k,
                           packed=False, rowwise=rowwise)


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 128, 256), (256, 256, 512), (128, 256, 1024), (200, 136, 192),
                                   (1, 8, 64), (384, 768, 768), (130, 520, 320), (512, 1280, 2304)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_f32_vs_oracle(pkg, oracle, dev, m, n, k, mode):
    rng = np.random.default_rng(m * 7 + n * 3 + k + mode)
    a, b = _rand_nvfp4(rng, m, k, mode == 2), _rand_nvfp4(rng, n, k, False)
    want = oracle.gemm(a, b, m, k, n, mode)
    got = cpu(pkg.Nvfp4GemmModule().gemm(_to_dev(pkg, dev, a, m, k, mode == 2), _to_dev(pkg, dev, b, n, k, False), mode=mode))
    assert_no_timeouts(pkg)
    assert np.isfinite(got).all()
    assert rel_fro(got, want) <= GEMM_TOL, rel_fro(got, want)


def test_gemm_known_answers(pkg, oracle, dev):
    """crates/cuda-kernels/tests/lm_head.rs:25-72 and tests/linear_backward/quartet.rs:13-76 (exact)."""
    gemm = pkg.Nvfp4GemmModule()
    tokens, k, vocab = 2, 64, 16
    a = np.zeros(tokens * k // 2, np.uint8)
    for e in (0, 1, k + 2):
        set_e2m1_one(a, e)
    w = np.zeros(vocab * k // 2, np.uint8)
    for e in (0, k + 1, 2 * k + 2):
        set_e2m1_one(w, e)
    ones = lambda n: np.full(n // 16, 0x38, np.uint8)
    out = cpu(gemm.gemm(_to_dev(pkg, dev, (a, ones(tokens * k), np.ones(tokens, np.float32)), tokens, k, True),
                        _to_dev(pkg, dev, (w, ones(vocab * k), np.ones(1, np.float32)), vocab, k, False)))
    want = np.zeros((tokens, vocab), np.float32)
    want[0, 0] = want[0, 1] = want[1, 2] = 1.0
    assert np.array_equal(out, want)

    t = i = o = 64
    first_col = np.zeros(t * o // 2, np.uint8)
    for r in range(t):
        set_e2m1_one(first_col, r * o)
    first_row = np.zeros(o * t // 2, np.uint8)
    for c in range(t):
        set_e2m1_one(first_row, c)
    dinput = cpu(gemm.gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer(
        _to_dev(pkg, dev, (first_col, ones(t * o), np.ones(t, np.float32)), t, o, True),
        _to_dev(pkg, dev, (first_col.copy(), ones(i * o), np.ones(1, np.float32)), i, o, False)))
    assert (dinput == 1.0).all()
    dweight = cpu(gemm.gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer(
        _to_dev(pkg, dev, (first_row, ones(o * t), np.ones(o, np.float32)), o, t, True),
        _to_dev(pkg, dev, (np.full(i * t // 2, 0x22, np.uint8), ones(i * t), np.ones(1, np.float32)), i, t, False)))
    assert (dweight[0] == t).all() and (dweight[1:] == 0).all()


@pytest.mark.parametrize("epi", [1, 2, 3])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_epilogues(pkg, oracle, dev, epi, out_dtype):
    if epi == 3 and out_dtype == torch.bfloat16:
        pytest.skip("the residual stream is f32 in the reference")
    m, n, k = 256, 384, 256
    rng = np.random.default_rng(epi)
    a, b = _rand_nvfp4(rng, m, k, True), _rand_nvfp4(rng, n, k, False)
    bias = rng.normal(0, 50.0, n).astype(np.float32)
    res = rng.normal(0, 100.0, (m, n)).astype(np.float32)
    gemm = pkg.Nvfp4GemmModule()
    A, B = _to_dev(pkg, dev, a, m, k, True), _to_dev(pkg, dev, b, n, k, False)
    bias_d = torch.from_numpy(bias).to(dev)
    if epi == 2:
        want, want_pre = oracle.gemm(a, b, m, k, n, 2, bias=bias, epi=2, want_pre=True)
        aux = torch.empty((m, n), dtype=out_dtype, device=dev)
        got = gemm.gemm(A, B, bias=bias_d, epilogue=pkg.EPI_RELU2, out_dtype=out_dtype, aux=aux)
        if out_dtype == torch.bfloat16:
            want_pre = torch.from_numpy(want_pre).to(torch.bfloat16).float().numpy()
        assert rel_fro(cpu(aux.float()), want_pre) <= GEMM_TOL
    elif epi == 3:
        want = oracle.gemm(a, b, m, k, n, 2, bias=bias, epi=3, residual=res)
        got = gemm.gemm(A, B, bias=bias_d, epilogue=pkg.EPI_RESIDUAL, out=torch.from_numpy(res).to(dev).clone())
    else:
        want = oracle.gemm(a, b, m, k, n, 2, bias=bias, epi=1)
        got = gemm.gemm(A, B, bias=bias_d, epilogue=pkg.EPI_BIAS, out_dtype=out_dtype)
    if out_dtype == torch.bfloat16:
        assert rel_fro(cpu(got.float()), want) <= 2.5e-3  # bf16 rounding alone is ~1.1e-3 RMS
        want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    assert rel_fro(cpu(got.float()), want) <= GEMM_TOL
    assert_no_timeouts(pkg)


def test_gemm_split_k_and_padded_output(pkg, oracle, dev):
    """Long-K narrow GEMM (the dW shape, split-K path) and the padded-output entry."""
    gemm = pkg.Nvfp4GemmModule()
    m, n, k = 256, 128, 8192
    rng = np.random.default_rng(77)
    a, b = _rand_nvfp4(rng, m, k, True), _rand_nvfp4(rng, n, k, False)
    want = oracle.gemm(a, b, m, k, n, 2)
    got = cpu(gemm.gemm(_to_dev(pkg, dev, a, m, k, True), _to_dev(pkg, dev, b, n, k, False)))
    assert rel_fro(got, want) <= GEMM_TOL
    m, n, npad, k = 128, 200, 256, 128
    a, b = _rand_nvfp4(rng, m, k, True), _rand_nvfp4(rng, npad, k, False)
    want = oracle.gemm(a, (b[0][: n * k // 2], b[1][: n * k // 16], b[2]), m, k, n, 2)
    got = cpu(gemm.gemm_tma_nvfp4_rowwise_a_scale_padded_output(_to_dev(pkg, dev, a, m, k, True),
                                                                _to_dev(pkg, dev, b, npad, k, False), n))
    assert got.shape == (m, n) and rel_fro(got, want) <= GEMM_TOL
    assert_no_timeouts(pkg)


def test_gemm_resident_panel_with_tails(pkg, oracle, dev):
    """Short K with many row blocks runs with the B panel resident in shared memory; M, N and K
    all have ragged tails here (K = 448 is seven 64-element atoms: a full k-tile and a 3-atom one)."""
    gemm = pkg.Nvfp4GemmModule()
    m, n, k = 10000, 1000, 448
    rng = np.random.default_rng(5)
    a, b = _rand_nvfp4(rng, m, k, True), _rand_nvfp4(rng, n, k, False)
    bias = rng.normal(0, 30.0, n).astype(np.float32)
    want = oracle.gemm(a, b, m, k, n, 2, bias=bias, epi=1)
    A, B = _to_dev(pkg, dev, a, m, k, True), _to_dev(pkg, dev, b, n, k, False)
    got = cpu(gemm.gemm(A, B, bias=torch.from_numpy(bias).to(dev), epilogue=pkg.EPI_BIAS))
    assert rel_fro(got, want) <= GEMM_TOL
    got16 = cpu(gemm.gemm(A, B, bias=torch.from_numpy(bias).to(dev), epilogue=pkg.EPI_BIAS,
                          out_dtype=torch.bfloat16).float())
    assert rel_fro(got16, torch.from_numpy(want).to(torch.bfloat16).float().numpy()) <= GEMM_TOL
    assert_no_timeouts(pkg)


def test_gemm_rejects_bad_shapes(pkg, dev):
    gemm = pkg.Nvfp4GemmModule()
    rng = np.random.default_rng(0)
    a, b = _rand_nvfp4(rng, 16, 32, True), _rand_nvfp4(rng, 16, 32, False)
    A, B = _to_dev(pkg, dev, a, 16, 32, True), _to_dev(pkg, dev, b, 16, 32, False)
    A.scales = torch.zeros(512, dtype=torch.uint8, device=dev)
    B.scales = torch.zeros(512, dtype=torch.uint8, device=dev)
    A.packed = B.packed = True
    with pytest.raises(pkg.Nvfp4Error) as err:  # K = 32 is not a multiple of 64
        gemm.gemm(A, B)
    assert err.value.code == 1  # CUDA_ERROR_INVALID_VALUE, like utils/nvfp4_tma_matmul/launcher.rs:183-190


def test_c_attn_forward_8192_tokens(pkg, oracle, dev):
    """One forward projection of the c_attn shape: X [8192 x 768] ~N(0,1), W [2304 x 768] ~N(0,0.02),
    b ~N(0,0.02), per-tensor scales, bf16 out."""
    q, gemm = pkg.Nvfp4QuantModule(), pkg.Nvfp4GemmModule()
    m, k, n = 8192, 768, 2304
    x, w = bf16_normal(101, (m, k)), bf16_normal(102, (n, k), 0.02)
    bias = bf16_normal(103, (n,), 0.02).float()
    xq = q.quantize_four_six(x.to(dev), rowwise=False, packed=True)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=True)
    y = gemm.gemm(xq, wq, bias=bias.to(dev), epilogue=pkg.EPI_BIAS, out_dtype=torch.bfloat16)
    xf, wf = x.float().numpy(), w.float().numpy()
    ox = oracle.four_six(xf, oracle.tensor_amax(xf)[1], False)
    ow = oracle.four_six(wf, oracle.tensor_amax(wf)[1], False)
    assert np.array_equal(cpu(xq.bytes), ox[0]) and np.array_equal(cpu(wq.bytes), ow[0])
    want = oracle.gemm(ox, ow, m, k, n, 1, bias=bias.numpy(), epi=1)
    want_bf16 = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    got = cpu(y.float())
    assert rel_fro(got, want_bf16) <= GEMM_TOL
    y32 = gemm.gemm(xq, wq, bias=bias.to(dev), epilogue=pkg.EPI_BIAS, out_dtype=torch.float32)
    assert rel_fro(cpu(y32), want) <= GEMM_TOL
    assert_no_timeouts(pkg)


# ------------------------------------------------------------------------------------------ linear backward

@pytest.mark.parametrize("native", [False, True])
@pytest.mark.parametrize("tokens,in_dim,out_dim", [(64, 64, 64), (256, 128, 192), (200, 64, 100), (1024, 768, 2304),
                                                   (384, 256, 128)])
def test_linear_backward_vs_oracle(pkg, oracle, dev, tokens, in_dim, out_dim, native):
    """gpt/linear_backward/ms_eden.rs:15-55 composition: every quantized operand bit-exact, the two
    GEMMs within tolerance of the oracle GEMM over the same operands.  native=False is the
    reference's data flow (f32 dY, logical scale planes); native=True the B200 one (bf16 dY, packed
    scale planes, decoded amax handed over), which takes the whole-tile kernels where shapes allow."""
    q, bwd = pkg.Nvfp4QuantModule(), pkg.LinearBackwardModule()
    x, w = bf16_normal(201, (tokens, in_dim)), bf16_normal(202, (out_dim, in_dim), 0.02)
    if native:
        dy = bf16_normal(203, (tokens, out_dim), 1e-3)
        e_dev, dy = dy.to(dev), dy.float()
    else:
        dy = torch.from_numpy(normal(203, (tokens, out_dim), 1e-3).astype(np.float32))
        e_dev = dy.to(dev)
    xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=native, decoded_amax=native)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=native)
    scratch = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
    dx, dw, db = bwd.backward_ms_eden(e=e_dev, weight=wq, input=xq, scratch=scratch, sign_seed=SIGN, scale_seed=SCALE)
    dx, dw = dx.float(), dw.float()
    assert_no_timeouts(pkg)

    xf, wf, ef = x.float().numpy(), w.float().numpy(), dy.numpy()
    oxq = oracle.four_six(xf, oracle.row_amax(xf), True)
    owq = oracle.four_six(wf, oracle.tensor_amax(wf)[1], False)
    ok, tk = oracle.padded_k(out_dim), oracle.padded_k(tokens)
    gs_e = oracle.ms_eden_global_scale(float(np.abs(ef).max()))
    e_h = oracle.ms_eden(0, ef, tokens, ok, gs_e, SIGN, SCALE, want_chunk_amax=False)
    e_t = oracle.ms_eden(1, ef, out_dim, tk, gs_e, SIGN, SCALE ^ 0x85EBCA6B, want_chunk_amax=False)
    gs_w = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(*owq, out_dim, in_dim, False)[1][0]))
    w_t = oracle.ms_eden(2, (*owq, out_dim, in_dim), in_dim, ok, gs_w, SIGN, SCALE ^ 0x9E3779B9, want_chunk_amax=False)
    gs_x = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(*oxq, tokens, in_dim, True)[1][0]))
    x_t = oracle.ms_eden(3, (*oxq, tokens, in_dim), in_dim, tk, gs_x, SIGN, SCALE ^ 0xC2B2AE35, want_chunk_amax=False)
    for name, ref, rows, kk in (("e_h", e_h, tokens, ok), ("e_t_h", e_t, out_dim, tk), ("weight_t_h", w_t, in_dim, ok),
                                ("input_t_h", x_t, in_dim, tk)):
        op = getattr(scratch, name)
        assert np.array_equal(cpu(op["bytes"]), ref[0]), name
        assert np.array_equal(cpu(op["scales_packed"]), oracle.scale_pack(ref[1], rows, kk)), name
        assert np.array_equal(cpu(op["global_scales"]), ref[2]), name
    # dbias rides along with the tiled dY quantization: bit-exact against that summation order,
    # and equal to the reference-order sum up to f32 rounding (relative 1e-5 of the column scale)
    assert np.array_equal(cpu(db), oracle.bias_grad_tiled(ef))
    ref_db = oracle.bias_grad(ef)
    assert np.abs(cpu(db) - ref_db).max() <= 1e-5 * np.abs(ef).sum(0).max()
    want_dx = oracle.gemm(e_h[:3], (w_t[0], w_t[1], np.array([gs_w], np.float32)), tokens, ok, in_dim, 2)
    want_dw = oracle.gemm(e_t[:3], (x_t[0], x_t[1], np.array([gs_x], np.float32)), out_dim, tk, in_dim, 2)
    assert rel_fro(cpu(dx), want_dx) <= GEMM_TOL
    assert rel_fro(cpu(dw), want_dw) <= GEMM_TOL
    # and the quantized gradients approximate the real ones
    assert rel_fro(cpu(dx), ef @ wf) < 0.3
    assert rel_fro(cpu(dw), ef.T @ xf) < 0.3


@pytest.mark.parametrize("shape,packed", [((130, 192), True), ((64, 48), False), ((5, 4096), False), ((3, 8192), False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_four_six_fused_decoded_amax(pkg, oracle, dev, shape, packed, dtype):
    """The fused rowwise quantizer's by-product equals the amax of the decoded tensor
    (utils/nvfp4/quant/kernels/ms_eden/amax.rs:23-64), on the one- and the two-kernel path."""
    q = pkg.Nvfp4QuantModule()
    x = with_outliers(bf16_normal(77, shape), seed=3, every=61).to(dtype)
    t = q.quantize_four_six(x.to(dev), rowwise=True, packed=packed, decoded_amax=True)
    xf = x.float().numpy()
    ob, os_, og = oracle.four_six(xf, oracle.row_amax(xf), True)
    assert np.array_equal(cpu(t.bytes), ob)
    want = oracle.nvfp4_amax(ob, os_, og, shape[0], shape[1], True)[1]
    assert cpu(t.decoded_amax).tobytes() == np.asarray(want, np.float32).tobytes()
    assert float(want[0]) == np.abs(oracle.decode(ob, os_, og, shape[0], shape[1], True, False)).max()


def test_linear_backward_precomputed_x_amax(pkg, oracle, dev):
    """Handing the forward quantizer's decoded amax to the backward changes no output byte."""
    q, bwd = pkg.Nvfp4QuantModule(), pkg.LinearBackwardModule()
    tokens, in_dim, out_dim = 256, 192, 128
    x, w = bf16_normal(401, (tokens, in_dim)), bf16_normal(402, (out_dim, in_dim), 0.02)
    dy = bf16_normal(403, (tokens, out_dim), 1e-3).to(dev)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=True)
    outs = []
    for hand_over in (False, True):
        xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=True, decoded_amax=hand_over)
        assert (xq.decoded_amax is not None) == hand_over
        sc = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
        dx, dw, db = bwd.backward_ms_eden(e=dy, weight=wq, input=xq, scratch=sc, sign_seed=SIGN, scale_seed=SCALE)
        outs.append((cpu(sc.input_t_h["bytes"]), cpu(sc.input_t_h["scales_packed"]), cpu(sc.input_t_h["global_scale"]),
                     cpu(dx), cpu(dw), cpu(db)))
    for a, b in zip(*outs):
        assert a.tobytes() == b.tobytes()
    assert_no_timeouts(pkg)


@pytest.mark.parametrize("kind", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", [(256, 128), (384, 192), (200, 100)])
def test_relu2_backward_amax_hand_over(pkg, oracle, dev, kind, shape):
    """The ReLU^2 backward that emits the amax of its own output: same gradient bytes as the plain entry
    (and as the oracle, gpt/mlp/kernels.rs:72-104), chunk maxima whose max is the tensor amax, and a linear
    backward fed with them (precomputed_e_amax_chunks) that differs in no output byte from one that reads dY."""
    q, bwd, mlp = pkg.Nvfp4QuantModule(), pkg.LinearBackwardModule(), pkg.MlpModule()
    tokens, out_dim = shape
    in_dim = 128
    pre = torch.from_numpy(normal(601, (tokens, out_dim), 1.0).astype(np.float32))
    d = torch.from_numpy(normal(602, (tokens, out_dim), 1e-3).astype(np.float32))
    pre[0, 0], pre[1, 2] = -0.0, float("nan")
    if kind == "bf16":
        pre, d = pre.bfloat16(), d.bfloat16()
    elif kind == "f16":
        pre = pre.half()
    want = torch.from_numpy(oracle.relu2_backward(pre.float().numpy(), d.float().numpy()))
    want = want.bfloat16() if kind == "bf16" else want
    sc = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
    sc.e_h["chunk_amax"].fill_(float("inf"))  # stale content must not leak into the scale
    got, chunks = mlp.relu2_backward_amax(pre.to(dev), d.to(dev), sc.e_h["chunk_amax"])
    assert cpu(got.float()).tobytes() == want.float().numpy().tobytes()
    assert 0 < chunks <= sc.e_h["chunk_amax"].numel()
    finite = torch.nan_to_num(want.float(), nan=0.0).abs().max()
    assert float(sc.e_h["chunk_amax"][:chunks].max()) == float(finite)
    plain = mlp.relu2_backward(pre.to(dev), d.to(dev))
    assert cpu(plain.float()).tobytes() == cpu(got.float()).tobytes()

    x, w = bf16_normal(603, (tokens, in_dim)), bf16_normal(604, (out_dim, in_dim), 0.02)
    # the NaN the element-wise check carried would poison every GEMM output: drop it for the hand-over check
    pre_clean = torch.nan_to_num(pre.float(), nan=0.5).to(pre.dtype)
    xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=True, decoded_amax=True)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=True)
    outs = []
    for hand_over in (False, True):
        sc = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
        if hand_over:
            e, chunks = mlp.relu2_backward_amax(pre_clean.to(dev), d.to(dev), sc.e_h["chunk_amax"])
        else:
            e, chunks = mlp.relu2_backward(pre_clean.to(dev), d.to(dev)), 0
        dx, dw, db = bwd.backward_ms_eden(e=e, weight=wq, input=xq, scratch=sc, sign_seed=SIGN, scale_seed=SCALE,
                                          precomputed_e_amax_chunks=chunks)
        outs.append((cpu(sc.e_h["global_scale"]), cpu(sc.e_h["bytes"]), cpu(sc.e_t_h["bytes"]),
                     cpu(sc.e_t_h["scales_packed"]), cpu(dx), cpu(dw), cpu(db)))
    for a, b in zip(*outs):
        assert a.tobytes() == b.tobytes()
    assert_no_timeouts(pkg)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_backward_edge_values_whole_tiles(pkg, oracle, dev, dtype):
    """The whole-tile quantizers (two chunks per thread, integer scale rounding with its range
    checks) on the values that leave their fast paths: zero rows and columns, groups 2^20 below the
    tensor amax (sub-normal block scales), one huge outlier (saturating scales), negative zeros."""
    q, bwd = pkg.Nvfp4QuantModule(), pkg.LinearBackwardModule()
    tokens, in_dim, out_dim = 256, 128, 128
    dy = bf16_normal(501, (tokens, out_dim), 1e-3)
    dy[3] = 0.0
    dy[:, 7] = 0.0
    dy[16:48] *= 2.0 ** -20
    dy[100, 100] = 3.0e4
    dy[5, ::2] = -0.0
    x = bf16_normal(502, (tokens, in_dim))
    x[9] = 0.0
    x[64:96] *= 2.0 ** -18
    x[200, 5] = 1.0e4
    w = bf16_normal(503, (out_dim, in_dim), 0.02)
    w[:, 3] = 0.0
    xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=True, decoded_amax=True)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=True)
    scratch = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
    e_dev = dy.to(dev) if dtype == torch.bfloat16 else dy.float().to(dev)
    bwd.backward_ms_eden(e=e_dev, weight=wq, input=xq, scratch=scratch, sign_seed=SIGN, scale_seed=SCALE)
    assert_no_timeouts(pkg)
    xf, wf, ef = x.float().numpy(), w.float().numpy(), dy.float().numpy()
    oxq = oracle.four_six(xf, oracle.row_amax(xf), True)
    owq = oracle.four_six(wf, oracle.tensor_amax(wf)[1], False)
    assert np.array_equal(cpu(xq.bytes), oxq[0])
    gs_e = oracle.ms_eden_global_scale(float(np.abs(ef).max()))
    e_h = oracle.ms_eden(0, ef, tokens, out_dim, gs_e, SIGN, SCALE, want_chunk_amax=False)
    e_t = oracle.ms_eden(1, ef, out_dim, tokens, gs_e, SIGN, SCALE ^ 0x85EBCA6B, want_chunk_amax=False)
    gs_w = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(*owq, out_dim, in_dim, False)[1][0]))
    w_t = oracle.ms_eden(2, (*owq, out_dim, in_dim), in_dim, out_dim, gs_w, SIGN, SCALE ^ 0x9E3779B9, want_chunk_amax=False)
    gs_x = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(*oxq, tokens, in_dim, True)[1][0]))
    x_t = oracle.ms_eden(3, (*oxq, tokens, in_dim), in_dim, tokens, gs_x, SIGN, SCALE ^ 0xC2B2AE35, want_chunk_amax=False)
    for name, ref, rows, kk in (("e_h", e_h, tokens, out_dim), ("e_t_h", e_t, out_dim, tokens),
                                ("weight_t_h", w_t, in_dim, out_dim), ("input_t_h", x_t, in_dim, tokens)):
        op = getattr(scratch, name)
        assert np.array_equal(cpu(op["bytes"]), ref[0]), name
        assert np.array_equal(cpu(op["scales_packed"]), oracle.scale_pack(ref[1], rows, kk)), name
        assert np.array_equal(cpu(op["global_scales"]), ref[2]), name


def test_linear_backward_sharded_equals_whole(pkg, oracle, dev):
    """Token sharding (two shards run back to back on one GPU): with the shared dY scale and the
    token offsets, shard dX rows equal the unsharded rows and the shard dW sum matches."""
    q, bwd = pkg.Nvfp4QuantModule(), pkg.LinearBackwardModule()
    tokens, in_dim, out_dim = 512, 128, 256
    x, w = bf16_normal(301, (tokens, in_dim)), bf16_normal(302, (out_dim, in_dim), 0.02)
    dy = torch.from_numpy(normal(303, (tokens, out_dim), 1e-3).astype(np.float32)).to(dev)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=False)
    xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=False)
    whole = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
    dx, dw, _ = bwd.backward_ms_eden(e=dy, weight=wq, input=xq, scratch=whole, sign_seed=SIGN, scale_seed=SCALE)
    gs = whole.e_h["global_scale"].clone()
    half = tokens // 2
    dws = []
    for s in range(2):
        xs = q.quantize_four_six(x[s * half:(s + 1) * half].contiguous().to(dev), rowwise=True, packed=False)
        sc = pkg.LinearBackwardScratch(half, in_dim, out_dim, dev)
        dxs, dwsh, _ = bwd.backward_ms_eden(e=dy[s * half:(s + 1) * half].contiguous(), weight=wq, input=xs, scratch=sc,
                                            sign_seed=SIGN, scale_seed=SCALE, token_offset=s * half, e_global_scale=gs)
        assert torch.equal(sc.e_h["bytes"], whole.e_h["bytes"].view(tokens, -1)[s * half:(s + 1) * half].reshape(-1))
        assert rel_fro(cpu(dxs), cpu(dx[s * half:(s + 1) * half])) <= 1e-5
        dws.append(dwsh)
    # X^T is re-quantized per shard (own amax-derived scale, own rounding), so the dW sum agrees with
    # the unsharded dW to quantization noise only; both approximate dY^T.X
    assert rel_fro(cpu(dws[0] + dws[1]), cpu(dw)) < 0.25
    true_dw = cpu(dy).T @ x.float().numpy()
    assert rel_fro(cpu(dws[0] + dws[1]), true_dw) < 0.3 and rel_fro(cpu(dw), true_dw) < 0.3
    assert_no_timeouts(pkg)


@pytest.mark.parametrize("m,n,k", [(1, 1, 65), (48, 40, 200), (256, 192, 1024)])
def test_tc_matmul_ms_eden(pkg, oracle, dev, m, n, k):
    """utils/nvfp4_tc_matmul/launcher.rs:23-87 (the (1, 1, 65) all-ones case is the reference's own test,
    tests/nvfp4_tc_matmul.rs:20-49): both quantized operands bit-exact, the product within the GEMM tolerance
    of the dequantized dot products."""
    mod = pkg.Nvfp4TcMatmulModule()
    if (m, n, k) == (1, 1, 65):
        a, b = torch.ones(m, k), torch.full((n, k), 0.5)
        ga = gb = 1.0
    else:
        a = torch.from_numpy(normal(81, (m, k)).astype(np.float32))
        b = torch.from_numpy(normal(82, (n, k), 0.02).astype(np.float32))
        ga = oracle.ms_eden_global_scale(float(a.abs().max()))
        gb = oracle.ms_eden_global_scale(float(b.abs().max()))
    out, ta, tb = mod.matmul_ms_eden(a.to(dev), b.to(dev), SIGN, SCALE, ga, gb)
    pk = oracle.padded_k(k)
    oa = oracle.ms_eden(0, a.numpy(), m, pk, ga, SIGN, SCALE, want_chunk_amax=False)
    ob = oracle.ms_eden(0, b.numpy(), n, pk, gb, SIGN, SCALE ^ 0x9E3779B9, want_chunk_amax=False)
    for t, o, rows in ((ta, oa, m), (tb, ob, n)):
        assert np.array_equal(cpu(t.bytes), o[0])
        assert np.array_equal(cpu(t.scales), oracle.scale_pack(o[1], rows, pk))
        assert np.array_equal(cpu(t.global_scales), o[2])
    want = oracle.gemm(oa[:3], (ob[0], ob[1], np.array([gb], np.float32)), m, pk, n, 2)
    assert rel_fro(cpu(out), want) <= GEMM_TOL
    if k == 65:
        assert abs(float(cpu(out)[0, 0]) - float(want[0, 0])) <= 1.0e-5 * max(1.0, abs(float(want[0, 0])))
    assert_no_timeouts(pkg)


# ------------------------------------------------------------------------------------------ projection set

def test_projection_set_step_streams_and_graph(pkg, dev):
    """The training-step projection set: the side-stream weight quantization changes no output, and a
    step replayed from a CUDA graph equals the eager step drawn with the same seeds."""
    from nanogpt_120a_b200.projection_set import ModelShape, ProjectionSet

    shape = ModelShape("tiny-proj-set", 2, 128, 256, 512)

    def buckets(ps):
        torch.cuda.synchronize()
        return [b.clone() for b in ps.buckets] + [ps.dx[w].clone() for w in sorted(ps.dx)]

    a = ProjectionSet(shape, 256, dev, seed=5)
    b = ProjectionSet(shape, 256, dev, seed=5, overlap_weight_quantization=False)
    a.step(), b.step()
    first_a, first_b = buckets(a), buckets(b)
    for x, y in zip(first_a, first_b):
        assert torch.equal(x, y)
    a.step()  # second eager step: the second pair of seeds per linear
    second_a = buckets(a)
    assert any(not torch.equal(x, y) for x, y in zip(first_a, second_a))  # the seeds did change the gradients
    graph = b.capture_step()  # capture draws the same second seeds
    graph.replay()
    for x, y in zip(second_a, buckets(b)):
        assert torch.equal(x, y)
    assert_no_timeouts(pkg)


def test_projection_set_reuses_packed_weights(pkg, dev):
    """A micro-step that keeps the packed NVFP4 weights of the previous step (no optimizer update in
    between) launches fewer kernels and yields the same gradients as one that re-quantizes them."""
    from nanogpt_120a_b200.projection_set import ModelShape, ProjectionSet

    shape = ModelShape("tiny-proj-set", 2, 128, 256, 512)
    a = ProjectionSet(shape, 256, dev, seed=9)
    b = ProjectionSet(shape, 256, dev, seed=9)
    a.step(), b.step()
    lib = pkg.library()
    n0 = lib.nvfp4_launch_count()
    a.step(weights_changed=True)
    n1 = lib.nvfp4_launch_count()
    b.step(weights_changed=False)
    n2 = lib.nvfp4_launch_count()
    torch.cuda.synchronize()
    assert (n1 - n0) - (n2 - n1) >= len(a.all_linears())  # at least the four-six launch of every weight
    for x, y in zip(a.buckets, b.buckets):
        assert torch.equal(x, y)
    for la, lb in zip(a.all_linears(), b.all_linears()):
        assert torch.equal(la.wq.bytes, lb.wq.bytes) and torch.equal(la.wq.scales, lb.wq.scales)
    assert_no_timeouts(pkg)


def test_split_k_deterministic_switch(pkg, oracle, dev):
    """Split-K dW GEMMs: with the switch on (at most two splits) repeated launches agree bit for bit; with it
    off (as many splits as fill the SMs) they stay within the GEMM tolerance of the same result."""
    gemm = pkg.Nvfp4GemmModule()
    rng = np.random.default_rng(77)
    m, n, k = 256, 256, 16384  # 2 x 1 wide tiles, 64 k-tiles: up to 8 splits
    a, b = _rand_nvfp4(rng, m, k, True), _rand_nvfp4(rng, n, k, False)
    A, B = _to_dev(pkg, dev, a, m, k, True), _to_dev(pkg, dev, b, n, k, False)
    A.scales, B.scales = pkg.Sm120ScalePackModule().pack(A.scales, m, k), pkg.Sm120ScalePackModule().pack(B.scales, n, k)
    A.packed = B.packed = True
    assert not pkg.deterministic_reductions()
    try:
        pkg.set_deterministic_reductions(True)
        assert pkg.deterministic_reductions()
        first = cpu(gemm.gemm(A, B, out_dtype=torch.float32))
        for _ in range(10):
            assert cpu(gemm.gemm(A, B, out_dtype=torch.float32)).tobytes() == first.tobytes()
    finally:
        pkg.set_deterministic_reductions(False)
    fast = cpu(gemm.gemm(A, B, out_dtype=torch.float32))
    assert rel_fro(fast, first) <= 1e-6
    want = oracle.gemm(a, b, m, k, n, 2)
    assert rel_fro(first, want) <= GEMM_TOL and rel_fro(fast, want) <= GEMM_TOL
    assert_no_timeouts(pkg)


@pytest.mark.gpu
def test_checkpoint_device_round_trip(pkg, oracle, dev, tmp_path):
    """A quantized weight and its bias leave the device through the checkpoint writer and come back through the
    reader byte for byte; the file equals the CPU restatement of the reference's container, and a tensor whose
    member lengths break bytes = len / 2, scales = len / 16 is refused on upload."""
    from oracle import checkpoint as oracle_ckpt
    q = pkg.Nvfp4QuantModule()
    w = torch.randn(384, 256, device=dev)
    t = q.quantize_four_six(w, packed=False)
    b = q.quantize_four_six(torch.randn(1, 384, device=dev), packed=False)
    path = str(tmp_path / "w.ckpt")
    wr = pkg.CheckpointWriter(path, 2)
    wr.write_tensor("blocks.0.attn_qkv.weight", 384 * 256, t.global_scales, t.bytes, t.scales)
    wr.write_tensor("blocks.0.attn_qkv.bias", 384, b.global_scales, b.bytes, b.scales)
    wr.finish()
    want = oracle_ckpt.write_checkpoint([
        ("blocks.0.attn_qkv.weight", 384 * 256, float(t.global_scales.item()), cpu(t.bytes).tobytes(), cpu(t.scales).tobytes()),
        ("blocks.0.attn_qkv.bias", 384, float(b.global_scales.item()), cpu(b.bytes).tobytes(), cpu(b.scales).tobytes())])
    assert open(path, "rb").read() == want
    r = pkg.CheckpointReader(path)
    assert r.read_header() == 2
    for src, name in ((t, "blocks.0.attn_qkv.weight"), (b, "blocks.0.attn_qkv.bias")):
        got = r.read_tensor_device(dev)
        assert got.name == name
        assert torch.equal(got.bytes, src.bytes.view(-1)) and torch.equal(got.scales, src.scales.view(-1))
        assert torch.equal(got.global_scale, src.global_scales.view(-1)[:1])
    r.close()
    bad = str(tmp_path / "bad.ckpt")
    open(bad, "wb").write(oracle_ckpt.write_checkpoint([("w", 64, 1.0, bytes(31), bytes(4))]))
    r = pkg.CheckpointReader(bad)
    with pytest.raises(pkg.Nvfp4Error, match="len / 2"):
        r.read_tensor_device(dev)
    r.close()
