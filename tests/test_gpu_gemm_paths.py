"""GPU parity of every GEMM instantiation and schedule the training-step workload runs, at the sizes it
runs them: tile widths 128 / 192 / 256, f32 and bf16 output, streaming and resident-B (banded and contiguous)
schedules, split-K, fused bias / ReLU^2 (+ saved pre-activation) epilogues, NVFP4-encoded bias, outputs larger
than 4 GB, and the one-layer / GPT-2-medium shapes.  Rows of a GEMM are independent, so a launch of any M is
checked on sampled 128-row blocks against the CPU oracle (relative Frobenius error <= 1e-3 of the FP32
dequantized product, the tolerance the path's specification states).  Every case asserts, through
nvfp4_gemm_plan_query, that the shape really selects the path it is meant to cover (on a 148-SM part), so a
change of the heuristics cannot silently un-test a path.  The reference tests its TMA GEMM the same way,
against a second implementation on model-sized patterned data
(crates/cuda-kernels/tests/projection_tma.rs:31-162)."""
import numpy as np
import pytest
import torch

from helpers import bf16_normal, normal, rel_fro

pytestmark = pytest.mark.gpu

GEMM_TOL = 1e-3
SIGN, SCALE = 0x12345678, 0x9ABCDEF0


def cpu(t):
    return t.detach().cpu().numpy()


def rand_nvfp4(rng, rows, k, rowwise):
    b = rng.integers(0, 256, size=rows * k // 2, dtype=np.uint8)
    s = rng.integers(0x28, 0x48, size=rows * k // 16, dtype=np.uint8)
    g = (0.5 + rng.random(rows if rowwise else 1)).astype(np.float32)
    return b, s, g


def to_dev(pkg, dev, t, rows, k, rowwise):
    """Device tensor with the scale plane packed on the GPU (bit-exactness of the pack is tested elsewhere)."""
    b, s, g = t
    logical = torch.from_numpy(s).to(dev)
    packed = pkg.Sm120ScalePackModule().pack(logical, rows, k)
    return pkg.Nvfp4Tensor(torch.from_numpy(b).to(dev), packed, torch.from_numpy(g).to(dev), rows, k, packed=True,
                           rowwise=rowwise)


def row_blocks(m, extra=()):
    """First block, one in the middle (another band of a banded schedule), the last (possibly ragged) one."""
    nb = (m + 127) // 128
    picks = sorted({0, nb // 2, nb - 1, *[b for b in extra if b < nb]})
    return [(b * 128, min(m, b * 128 + 128)) for b in picks]


def slice_rows(t, r0, r1, k, rowwise):
    b, s, g = t
    return b[r0 * k // 2:r1 * k // 2], s[r0 * k // 16:r1 * k // 16], (g[r0:r1] if rowwise else g)


def check_rows(oracle, a, b, m, k, n, got, *, mode=2, bias=None, epi=0, pre=None, blocks=None, bf16=False):
    worst = 0.0
    for r0, r1 in (blocks or row_blocks(m)):
        a_s = slice_rows(a, r0, r1, k, mode == 2)
        if epi == 2:
            want, want_pre = oracle.gemm(a_s, b, r1 - r0, k, n, mode, bias=bias, epi=2, want_pre=True)
        else:
            want, want_pre = oracle.gemm(a_s, b, r1 - r0, k, n, mode, bias=bias, epi=epi), None
        if bf16:
            want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
            want_pre = None if want_pre is None else torch.from_numpy(want_pre).to(torch.bfloat16).float().numpy()
        g = cpu(got[r0:r1].float())
        assert np.isfinite(g).all()
        err = rel_fro(g, want)
        assert err <= GEMM_TOL, (r0, err)
        worst = max(worst, err)
        if pre is not None:
            err = rel_fro(cpu(pre[r0:r1].float()), want_pre)
            assert err <= GEMM_TOL, ("pre", r0, err)
    return worst


def assert_plan(plan, **want):
    got = {k: getattr(plan, k) for k in want}
    for key, value in want.items():
        if callable(value):
            assert value(got[key]), (key, got)
        else:
            assert got[key] == value, (key, got)


def no_timeouts(pkg):
    torch.cuda.synchronize()
    assert pkg.read_device_status() == 0


@pytest.fixture
def tile(pkg):
    """Force a tile width for one test and restore the automatic choice afterwards."""
    def force(n, m=128):
        pkg.set_gemm_tile_override(n, m)
    yield force
    pkg.set_gemm_tile_override(0)


def run_case(pkg, oracle, dev, m, n, k, *, out_dtype, epi=0, want_plan=None, seed=0, blocks=None, with_pre=True):
    rng = np.random.default_rng(seed + m + 3 * n + 7 * k)
    a, b = rand_nvfp4(rng, m, k, True), rand_nvfp4(rng, n, k, False)
    A, B = to_dev(pkg, dev, a, m, k, True), to_dev(pkg, dev, b, n, k, False)
    bias = rng.normal(0, 40.0, n).astype(np.float32) if epi else None
    bias_d = None if bias is None else torch.from_numpy(bias).to(dev)
    gemm = pkg.Nvfp4GemmModule()
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    aux = torch.empty((m, n), dtype=out_dtype, device=dev) if (epi == 2 and with_pre) else None
    kw = dict(bias=bias_d, epilogue=epi, out=out, aux=aux)
    plan = gemm.plan(A, B, **kw)
    if want_plan:
        assert_plan(plan, **want_plan)
    gemm.gemm(A, B, **kw)
    no_timeouts(pkg)
    err = check_rows(oracle, a, b, m, k, n, out, bias=bias, epi=epi, pre=aux, blocks=blocks,
                     bf16=out_dtype == torch.bfloat16)
    return plan, err


# ------------------------------------------------------------------------------------------ wide tiles, forward

@pytest.mark.parametrize("width", [192, 256])
@pytest.mark.parametrize("epi", [1, 2])
def test_resident_banded_bf16(pkg, oracle, dev, tile, width, epi):
    """The forward GEMMs of the training step (K = 768, bf16 out, bias / ReLU^2 + pre-activation) with both wide
    tiles: B panel resident in shared memory, banded schedule; 192 columns with a double-buffered accumulator,
    256 columns with one buffer handed back early."""
    tile(width)
    run_case(pkg, oracle, dev, 19072, 2304, 768, out_dtype=torch.bfloat16, epi=epi,
             want_plan=dict(block_n=width, acc_stages=1 if width == 256 else 2, b_resident=1,
                            resident_cpn=lambda c: c >= 1, k_splits=1, tma_store=1))


@pytest.mark.parametrize("epi", [1, 2])
def test_resident_banded_256_auto(pkg, oracle, dev, epi):
    """N = 1024 does not divide into 192-column blocks: the automatic choice is the 256-column tile, resident B
    panel, banded schedule, bias staged through shared memory."""
    run_case(pkg, oracle, dev, 19072, 1024, 768, out_dtype=torch.bfloat16, epi=epi,
             want_plan=dict(block_n=256, acc_stages=1, b_resident=1, resident_cpn=lambda c: c >= 1, tma_store=1))


@pytest.mark.parametrize("width,epi", [(192, 0), (256, 1)])
def test_resident_contiguous_vocab(pkg, oracle, dev, tile, width, epi):
    """LM-head shape: 32000 columns (166 full 192-column blocks and one of 128, or 125 blocks of 256): more
    column blocks than CTAs, so the resident schedule walks contiguous tile ranges and reloads the panel when
    the column block changes."""
    tile(width)
    run_case(pkg, oracle, dev, 640, 32000, 768, out_dtype=torch.bfloat16, epi=epi,
             want_plan=dict(block_n=width, b_resident=1, resident_cpn=0))


def test_training_step_shapes_take_tested_paths(pkg, dev):
    """What the automatic choice picks for every GEMM of the GPT-2-small training step at 65536 tokens on a
    148-SM part: (tile height, tile width, K splits > 1, resident).  Each combination is covered by a parity test of this
    file with the same width, output type and schedule; a change of the heuristics shows up here first."""
    if torch.cuda.get_device_properties(dev).multi_processor_count != 148:
        pytest.skip("the expectations are for a 148-SM part")
    gemm = pkg.Nvfp4GemmModule()
    T, d, h, v = 65536, 768, 3072, 32000
    bf, f32 = torch.bfloat16, torch.float32
    want = {  # name: (m, n, k, out dtype, epilogue) -> (block_m, block_n, split, resident)
        "fwd c_attn": ((T, 3 * d, d, bf, 1), (128, 256, False, 1)), "fwd c_proj": ((T, d, d, bf, 1), (128, 256, False, 1)),
        "fwd fc": ((T, h, d, bf, 1), (128, 256, False, 1)), "fwd proj": ((T, d, h, bf, 1), (256, 192, False, 0)),
        "fwd lm_head": ((T, v, d, bf, 0), (128, 256, False, 1)), "dX c_attn": ((T, d, 3 * d, bf, 0), (256, 192, False, 0)),
        "dX c_proj": ((T, d, d, bf, 0), (128, 256, False, 1)), "dX fc": ((T, d, h, bf, 0), (256, 192, False, 0)),
        "dX proj": ((T, h, d, bf, 0), (128, 256, False, 1)), "dX lm_head": ((T, d, v, bf, 0), (256, 192, False, 0)),
        "dW c_attn": ((3 * d, d, T, f32, 0), (256, 192, True, 0)), "dW c_proj": ((d, d, T, f32, 0), (256, 192, True, 0)),
        "dW fc": ((h, d, T, f32, 0), (256, 192, True, 0)), "dW proj": ((d, h, T, f32, 0), (256, 192, True, 0)),
        "dW lm_head": ((v, d, T, f32, 0), (256, 192, False, 0)),
    }
    one = torch.ones(1, device=dev)
    for name, ((m, n, k, dt, epi), (block_m, block_n, split, resident)) in want.items():
        # the plan depends on shapes, types and alignment only: tiny placeholder buffers stand in for the operands
        stub = torch.zeros(16, dtype=torch.uint8, device=dev)
        A = pkg.Nvfp4Tensor(stub, stub, one, m, k, packed=True, rowwise=True)
        B = pkg.Nvfp4Tensor(stub, stub, one, n, k, packed=True, rowwise=False)
        out = torch.empty(16, dtype=dt, device=dev)
        plan = gemm.plan(A, B, out=out, epilogue=epi, bias=one if epi else None)
        got = (plan.block_m, plan.block_n, plan.k_splits > 1, plan.b_resident)
        assert got == (block_m, block_n, split, resident), (name, got)


# ------------------------------------------------------------------------------------------ streaming (long K)

@pytest.mark.parametrize("n,k,block_n,resident", [(1024, 1024, 256, 0), (1024, 2304, 256, 0), (1024, 4096, 256, 0),
                                                  (768, 2304, 192, 0), (768, 3072, 192, 0), (4096, 1024, 192, 1)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_streaming_wide(pkg, oracle, dev, n, k, block_n, resident, out_dtype):
    """dX-shaped GEMMs (M = tokens, long K): wide tiles streaming both operands, f32 and bf16 output; the
    d_model = 1024 up projection (four k-tiles) still fits its B panel in shared memory beside four A stages."""
    run_case(pkg, oracle, dev, 4864, n, k, out_dtype=out_dtype, epi=0,
             want_plan=dict(block_n=block_n, b_resident=resident))


SHAPES = [(128, 128), (128, 192), (128, 256), (256, 192)]  # (tile height, tile width)


@pytest.mark.parametrize("height,width", SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("epi", [0, 1, 2])
def test_every_tile_shape_with_tails(pkg, oracle, dev, tile, height, width, out_dtype, epi):
    """Each tile shape forced on one GEMM whose M, N and K are all ragged: 1000 columns (a last block of 104 /
    40 / 232 columns, odd and even 192-column blocks), 10000 rows (the last 256-row block holds 16 rows: its
    second half lies below the matrix), K = 448 = a full k-tile and a 3-atom one."""
    tile(width, height)
    run_case(pkg, oracle, dev, 10000, 1000, 448, out_dtype=out_dtype, epi=epi,
             want_plan=dict(block_m=height, block_n=width))


@pytest.mark.parametrize("height,width", SHAPES)
def test_every_tile_shape_streaming_odd_k(pkg, oracle, dev, tile, height, width):
    """Streaming schedule with a k-tile tail (K = 1216 = 19 atoms) for every shape, f32 output; 2200 rows end in
    the second half of a 256-row block."""
    tile(width, height)
    run_case(pkg, oracle, dev, 2200, 600, 1216, out_dtype=torch.float32, epi=1,
             want_plan=dict(block_m=height, block_n=width, b_resident=0))


@pytest.mark.parametrize("n,k", [(768, 2304), (768, 3072), (3072, 768 * 2)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_tall_tile_streaming_auto(pkg, oracle, dev, n, k, out_dtype):
    """dX-shaped GEMMs with enough rows: the automatic choice is the 256 x 192 tile (two MMAs per k-atom over one
    B stage, single-buffered accumulators, two scale-factor column sets)."""
    run_case(pkg, oracle, dev, 19072 + 128, n, k, out_dtype=out_dtype, epi=0,
             want_plan=dict(block_m=256, block_n=192, b_resident=0, acc_stages=1))


# ------------------------------------------------------------------------------------------ split-K (dW)

@pytest.mark.parametrize("m,n,k", [(3072, 768, 65536), (768, 768, 65536), (2304, 768, 65536), (768, 3072, 65536),
                                   (4096, 1024, 32768)])
def test_split_k_dw_shapes(pkg, oracle, dev, m, n, k):
    """dW = dY^T . X at the training step's shapes (K = tokens): f32 output, K split over CTAs, partial tiles
    summed by TMA reduce-add.  Checked on sampled output rows."""
    plan, _ = run_case(pkg, oracle, dev, m, n, k, out_dtype=torch.float32, epi=0,
                       want_plan=dict(b_resident=0), blocks=row_blocks(m)[:2])
    assert plan.k_splits >= 2 or plan.grid >= 96, (plan.k_splits, plan.grid)


@pytest.mark.parametrize("height,width", SHAPES)
def test_split_k_with_bias_every_tile_shape(pkg, oracle, dev, tile, height, width):
    """Split-K with a linear bias epilogue: the bias joins the sum exactly once (with the first split's partial
    tile), whatever the tile shape; ragged N so the last column block is clipped by the reduce-add."""
    tile(width, height)
    plan, _ = run_case(pkg, oracle, dev, 700, 840, 16384, out_dtype=torch.float32, epi=1,
                       want_plan=dict(block_m=height, block_n=width, b_resident=0))
    assert plan.k_splits >= 2, plan.k_splits


@pytest.mark.parametrize("height,width", [(128, 192), (128, 256), (256, 192)])
def test_lm_head_dw_unsplit_wide_f32(pkg, oracle, dev, tile, height, width):
    """LM-head dW: enough tiles to fill the SMs without a split -- the unsplit wide f32 instantiations."""
    tile(width, height)
    run_case(pkg, oracle, dev, 32000, 768, 4096, out_dtype=torch.float32, epi=0,
             want_plan=dict(block_m=height, block_n=width, k_splits=1, b_resident=0))


# ------------------------------------------------------------------------------------------ huge output

def test_output_larger_than_4gb(pkg, oracle, dev):
    """Logits of the full step: 65536 x 32000 bf16 = 4.19 GB in one launch (byte offsets beyond 2^32); first,
    middle and last row block checked."""
    run_case(pkg, oracle, dev, 65536, 32000, 768, out_dtype=torch.bfloat16, epi=0, want_plan=dict(b_resident=1))


# ------------------------------------------------------------------------------------------ NVFP4 bias, row amax

@pytest.mark.parametrize("height,width", SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_nvfp4_bias_and_relu2_row_amax(pkg, oracle, dev, tile, height, width, out_dtype):
    """An NVFP4-encoded bias decoded in the epilogue equals the f32 bias of its decoded values, and the
    epilogue's by-product row amax of relu(stored)^2 equals the one computed from the stored tensor, bit for
    bit; the ReLU^2-on-load quantizer fed with it produces the bytes of quantizing relu(stored)^2."""
    tile(width, height)
    q, gemm = pkg.Nvfp4QuantModule(), pkg.Nvfp4GemmModule()
    m, n, k = 1500, 832, 256
    rng = np.random.default_rng(width)
    a, b = rand_nvfp4(rng, m, k, True), rand_nvfp4(rng, n, k, False)
    A, B = to_dev(pkg, dev, a, m, k, True), to_dev(pkg, dev, b, n, k, False)
    bias_src = torch.from_numpy(rng.normal(0, 30.0, (1, n)).astype(np.float32)).to(dev)
    bias_q = q.quantize_four_six(bias_src, rowwise=False, packed=False)
    bias_dec = oracle.decode(cpu(bias_q.bytes), cpu(bias_q.scales), cpu(bias_q.global_scales), 1, n, False, False)[0]
    ramax = torch.full((m,), -1.0, dtype=torch.float32, device=dev)  # stale content must not survive
    pre = gemm.gemm(A, B, bias=bias_q, epilogue=pkg.EPI_BIAS, out_dtype=out_dtype, relu2_row_amax=ramax)
    ref = gemm.gemm(A, B, bias=torch.from_numpy(bias_dec).to(dev), epilogue=pkg.EPI_BIAS, out_dtype=out_dtype)
    assert torch.equal(pre, ref)
    check_rows(oracle, a, b, m, k, n, pre, bias=bias_dec, epi=1, bf16=out_dtype == torch.bfloat16)
    relu = torch.clamp(pre.float(), min=0.0)
    act = relu * relu  # f32: max(pre, 0) then one rounded multiply
    assert torch.equal(ramax, act.amax(dim=1))
    # relu^2 on load, with and without the producer's amax, against the oracle on the materialised activation
    actf = cpu(act)
    ob, os_, og = oracle.four_six(actf, oracle.row_amax(actf), True)
    for hand_over in (ramax, None):
        t = q.quantize_relu2_four_six_rowwise(pre, row_amax=hand_over, packed=True, decoded_amax=True)
        assert np.array_equal(cpu(t.bytes), ob)
        assert np.array_equal(cpu(t.scales), oracle.scale_pack(os_, m, n))
        assert np.array_equal(cpu(t.global_scales), og)
        want_dec = oracle.nvfp4_amax(ob, os_, og, m, n, True)[1]
        assert cpu(t.decoded_amax).tobytes() == np.asarray(want_dec, np.float32).tobytes()
    no_timeouts(pkg)


# ------------------------------------------------------------------------------------------ reference-style entries

def test_forward_projection_entries(pkg, oracle, dev):
    """qkv_projection, c_proj, up_relu2, down_residual, logits, logits_tma, NextLat projection with the reference's
    argument lists (rowwise NVFP4 X with logical scales, NVFP4 W, NVFP4 bias, f32 out; launchers cited in
    include/nvfp4_b200.h) against the oracle GEMM + post-op semantics (gpt/projection_postop.rs:97-162)."""
    q = pkg.Nvfp4QuantModule()
    tokens, d, h = 384, 128, 256
    x = bf16_normal(901, (tokens, d)).float()
    hid = bf16_normal(902, (tokens, h)).float()
    mods = pkg.AttentionModule(), pkg.MlpModule(), pkg.LmHeadModule(), pkg.NextLatModule()
    att, mlp, head, nextlat = mods

    def qw(seed, rows, cols):
        w = bf16_normal(seed, (rows, cols), 0.02).float()
        t = q.quantize_four_six(w.to(dev), rowwise=False, packed=False)
        return t, (cpu(t.bytes), cpu(t.scales), cpu(t.global_scales))

    def qb(seed, n):
        bsrc = bf16_normal(seed, (1, n), 0.02).float()
        t = q.quantize_four_six(bsrc.to(dev), rowwise=False, packed=False)
        return t, oracle.decode(cpu(t.bytes), cpu(t.scales), cpu(t.global_scales), 1, n, False, False)[0]

    def qx(t):
        tq = q.quantize_four_six(t.to(dev), rowwise=True, packed=False)
        return tq, (cpu(tq.bytes), cpu(tq.scales), cpu(tq.global_scales))

    xq, xo = qx(x)
    hq, ho = qx(hid)
    for packed_inputs in (False, True):
        if packed_inputs:  # this library's own layout: no scratch, same results
            xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=True)
            hq = q.quantize_four_six(hid.to(dev), rowwise=True, packed=True)
        w_attn, wo_attn = qw(903, 3 * d, d)
        b_attn, bd_attn = qb(904, 3 * d)
        want = oracle.gemm(xo, wo_attn, tokens, d, 3 * d, 2, bias=bd_attn, epi=1)
        assert rel_fro(cpu(att.qkv_projection(xq, w_attn, b_attn)), want) <= GEMM_TOL
        assert rel_fro(cpu(nextlat.projection(xq, w_attn, b_attn)), want) <= GEMM_TOL
        got16 = att.qkv_projection(xq, w_attn, b_attn, out_dtype=torch.bfloat16)
        assert rel_fro(cpu(got16.float()), torch.from_numpy(want).bfloat16().float().numpy()) <= GEMM_TOL

        w_proj, wo_proj = qw(905, d, d)
        b_proj, bd_proj = qb(906, d)
        res = torch.from_numpy(normal(907, (tokens, d)).astype(np.float32))
        want = oracle.gemm(xo, wo_proj, tokens, d, d, 2, bias=bd_proj, epi=3, residual=res.numpy())
        assert rel_fro(cpu(att.c_proj(xq, w_proj, b_proj, res.clone().to(dev))), want) <= GEMM_TOL

        w_fc, wo_fc = qw(908, h, d)
        b_fc, bd_fc = qb(909, h)
        want, want_pre = oracle.gemm(xo, wo_fc, tokens, d, h, 2, bias=bd_fc, epi=2, want_pre=True)
        pre, act = mlp.up_relu2(xq, w_fc, b_fc)
        assert rel_fro(cpu(pre), want_pre) <= GEMM_TOL and rel_fro(cpu(act), want) <= GEMM_TOL
        ramax = torch.empty(tokens, dtype=torch.float32, device=dev)
        pre_only, none = mlp.up_relu2(xq, w_fc, b_fc, store_activation=False, relu2_row_amax=ramax)
        assert none is None and torch.equal(pre_only, pre)
        relu = torch.clamp(pre, min=0.0)
        assert torch.equal(ramax, (relu * relu).amax(dim=1))

        w_down, wo_down = qw(910, d, h)
        b_down, bd_down = qb(911, d)
        want = oracle.gemm(ho, wo_down, tokens, h, d, 2, bias=bd_down, epi=3, residual=res.numpy())
        assert rel_fro(cpu(mlp.down_residual(hq, w_down, b_down, res.clone().to(dev))), want) <= GEMM_TOL

        w_head, wo_head = qw(912, 512, d)
        want = oracle.gemm(xo, wo_head, tokens, d, 512, 2)
        assert rel_fro(cpu(head.logits(xq, w_head)), want) <= GEMM_TOL
        assert torch.equal(head.logits_tma(xq, w_head), head.logits(xq, w_head))
    no_timeouts(pkg)


def test_lm_head_logits_known_answer(pkg, dev):
    """The reference's own LM-head case through `logits` (crates/cuda-kernels/tests/lm_head.rs:25-72): unit
    nibbles at chosen positions, unit scales -> exact small integers."""
    from helpers import set_e2m1_one

    tokens, k, vocab = 2, 64, 16
    a = np.zeros(tokens * k // 2, np.uint8)
    for e in (0, 1, k + 2):
        set_e2m1_one(a, e)
    w = np.zeros(vocab * k // 2, np.uint8)
    for e in (0, k + 1, 2 * k + 2):
        set_e2m1_one(w, e)
    ones = lambda n: torch.full((n // 16,), 0x38, dtype=torch.uint8, device=dev)
    X = pkg.Nvfp4Tensor(torch.from_numpy(a).to(dev), ones(tokens * k), torch.ones(tokens, device=dev), tokens, k,
                        rowwise=True)
    W = pkg.Nvfp4Tensor(torch.from_numpy(w).to(dev), ones(vocab * k), torch.ones(1, device=dev), vocab, k)
    want = np.zeros((tokens, vocab), np.float32)
    want[0, 0] = want[0, 1] = want[1, 2] = 1.0
    for tma in (False, True):
        assert np.array_equal(cpu(pkg.LmHeadModule().logits(X, W, tma=tma)), want)


def test_backward_device_scale_entries_and_map_cache(pkg, oracle, dev):
    """backward_device_scale{,_tma,_cta} / backward run the two gradient GEMMs over the operands
    backward_ms_eden left in the scratch and reproduce its dX / dW bit for bit (unsplit shapes); prepare_tma
    warms the tensor-map cache so the launches that follow encode nothing."""
    q, bwd = pkg.Nvfp4QuantModule(), pkg.LinearBackwardModule()
    tokens, in_dim, out_dim = 512, 256, 384
    x, w = bf16_normal(921, (tokens, in_dim)), bf16_normal(922, (out_dim, in_dim), 0.02)
    dy = bf16_normal(923, (tokens, out_dim), 1e-3).float().to(dev)
    xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=True, decoded_amax=True)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=True)
    sc = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
    dx, dw, _ = bwd.backward_ms_eden(e=dy, weight=wq, input=xq, scratch=sc, sign_seed=SIGN, scale_seed=SCALE)
    for variant in ("tma", "plain", "cta", "backward"):
        dx2, dw2 = torch.zeros_like(dx), torch.zeros_like(dw)
        bwd.backward_device_scale(sc, dx2, dw2, variant=variant)
        assert torch.equal(dx, dx2) and torch.equal(dw, dw2)
    gemm = pkg.Nvfp4GemmModule()
    e_h, w_t = sc.as_tensor("e_h"), sc.as_tensor("weight_t_h")
    w_t.rowwise, w_t.global_scales = False, sc.weight_t_h["global_scale"]
    out = torch.empty((tokens, in_dim), dtype=torch.float32, device=dev)
    gemm.prepare_tma_nvfp4_device_scales(e_h, w_t)
    gemm.gemm(e_h, w_t, out=out)  # encodes the output map once
    _, misses0 = pkg.tensor_map_cache_stats()
    hits0 = pkg.tensor_map_cache_stats()[0]
    for _ in range(3):
        gemm.gemm(e_h, w_t, out=out)
    hits1, misses1 = pkg.tensor_map_cache_stats()
    assert misses1 == misses0 and hits1 >= hits0 + 9
    assert torch.equal(out, dx)
    no_timeouts(pkg)


# ------------------------------------------------------------------------------------------ whole layers at size

LAYER_SMALL = [("c_attn", 768, 2304, 1), ("attn_c_proj", 768, 768, 1), ("mlp_fc", 768, 3072, 2), ("mlp_proj", 3072, 768, 1)]
LAYER_MEDIUM = [("c_attn", 1024, 3072, 1), ("mlp_fc", 1024, 4096, 2), ("mlp_proj", 4096, 1024, 1)]


def _layer_case(pkg, oracle, dev, tokens, name, in_dim, out_dim, epi, seed):
    """One linear, forward + backward_ms_eden, on the specification's distributions: every quantized operand
    bit-exact on the whole tensor, the three GEMMs on sampled row blocks."""
    q, gemm, bwd = pkg.Nvfp4QuantModule(), pkg.Nvfp4GemmModule(), pkg.LinearBackwardModule()
    x, w = bf16_normal(seed, (tokens, in_dim)), bf16_normal(seed + 1, (out_dim, in_dim), 0.02)
    bias = bf16_normal(seed + 2, (out_dim,), 0.02).float()
    dy = bf16_normal(seed + 3, (tokens, out_dim), 1e-3)
    xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=True, decoded_amax=True)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=True)
    xf, wf, ef = x.float().numpy(), w.float().numpy(), dy.float().numpy()
    oxq = oracle.four_six(xf, oracle.row_amax(xf), True)
    owq = oracle.four_six(wf, oracle.tensor_amax(wf)[1], False)
    assert np.array_equal(cpu(xq.bytes), oxq[0]) and np.array_equal(cpu(xq.scales), oracle.scale_pack(oxq[1], tokens, in_dim))
    assert np.array_equal(cpu(wq.bytes), owq[0]) and np.array_equal(cpu(wq.global_scales), owq[2])
    # forward
    y = torch.empty((tokens, out_dim), dtype=torch.bfloat16, device=dev)
    aux = torch.empty_like(y) if epi == 2 else None
    gemm.gemm(xq, wq, bias=bias.to(dev), epilogue=epi, out=y, aux=aux)
    check_rows(oracle, oxq, owq, tokens, in_dim, out_dim, y, bias=bias.numpy(), epi=epi, pre=aux, bf16=True)
    # backward
    sc = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
    side = pkg.SideStream(dev)
    dx, dw, db = bwd.backward_ms_eden(e=dy.to(dev), weight=wq, input=xq, scratch=sc, sign_seed=SIGN, scale_seed=SCALE,
                                      grad_dtype=torch.bfloat16, dweight=torch.empty((out_dim, in_dim), device=dev),
                                      side=side)
    no_timeouts(pkg)
    ok, tk = oracle.padded_k(out_dim), oracle.padded_k(tokens)
    gs_e = oracle.ms_eden_global_scale(float(np.abs(ef).max()))
    e_h = oracle.ms_eden(0, ef, tokens, ok, gs_e, SIGN, SCALE, want_chunk_amax=False)
    e_t = oracle.ms_eden(1, ef, out_dim, tk, gs_e, SIGN, SCALE ^ 0x85EBCA6B, want_chunk_amax=False)
    gs_w = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(*owq, out_dim, in_dim, False)[1][0]))
    w_t = oracle.ms_eden(2, (*owq, out_dim, in_dim), in_dim, ok, gs_w, SIGN, SCALE ^ 0x9E3779B9, want_chunk_amax=False)
    gs_x = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(*oxq, tokens, in_dim, True)[1][0]))
    x_t = oracle.ms_eden(3, (*oxq, tokens, in_dim), in_dim, tk, gs_x, SIGN, SCALE ^ 0xC2B2AE35, want_chunk_amax=False)
    for nm, ref, rows, kk in (("e_h", e_h, tokens, ok), ("e_t_h", e_t, out_dim, tk), ("weight_t_h", w_t, in_dim, ok),
                              ("input_t_h", x_t, in_dim, tk)):
        op = getattr(sc, nm)
        assert np.array_equal(cpu(op["bytes"]), ref[0]), (name, nm)
        assert np.array_equal(cpu(op["scales_packed"]), oracle.scale_pack(ref[1], rows, kk)), (name, nm)
        assert np.array_equal(cpu(op["global_scales"]), ref[2]), (name, nm)
    assert np.array_equal(cpu(db), oracle.bias_grad_tiled(ef))
    check_rows(oracle, e_h[:3], (w_t[0], w_t[1], np.array([gs_w], np.float32)), tokens, ok, in_dim, dx, bf16=True)
    check_rows(oracle, e_t[:3], (x_t[0], x_t[1], np.array([gs_x], np.float32)), out_dim, tk, in_dim, dw)
    # and the quantized gradients approximate the real ones (sampled rows)
    r0, r1 = row_blocks(tokens)[1]
    assert rel_fro(cpu(dx[r0:r1].float()), ef[r0:r1] @ wf) < 0.3


@pytest.mark.parametrize("name,in_dim,out_dim,epi", LAYER_SMALL)
def test_one_layer_at_8192_tokens(pkg, oracle, dev, name, in_dim, out_dim, epi):
    """One GPT-2-small layer's four linears, forward and backward, at 8192 tokens."""
    _layer_case(pkg, oracle, dev, 8192, name, in_dim, out_dim, epi, seed=1000 + in_dim + out_dim)


@pytest.mark.parametrize("name,in_dim,out_dim,epi", LAYER_MEDIUM)
def test_medium_layer_shapes(pkg, oracle, dev, name, in_dim, out_dim, epi):
    """d_model = 1024 / MLP 4096 linears (the 24-layer configuration's shapes) at 4096 tokens."""
    _layer_case(pkg, oracle, dev, 4096, name, in_dim, out_dim, epi, seed=2000 + in_dim + out_dim)


# ------------------------------------------------------------------------------------------ sharding, bit for bit

def test_sharded_backward_reproduces_unsharded_bits(pkg, oracle, dev):
    """Two token shards run back to back with the all-reduced amaxes (dY scale, decoded-X amax), the token
    offset and the unsharded token count: every quantized operand of a shard is the matching slice of the
    unsharded operand, bit for bit, so the shards' dW partial sums add up to the unsharded dW up to f32
    summation order."""
    q, bwd = pkg.Nvfp4QuantModule(), pkg.LinearBackwardModule()
    tokens, in_dim, out_dim = 1024, 256, 384
    x, w = bf16_normal(301, (tokens, in_dim)), bf16_normal(302, (out_dim, in_dim), 0.02)
    dy = bf16_normal(303, (tokens, out_dim), 1e-3).to(dev)
    wq = q.quantize_four_six(w.to(dev), rowwise=False, packed=True)
    xq = q.quantize_four_six(x.to(dev), rowwise=True, packed=True, decoded_amax=True)
    whole = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
    pkg.set_deterministic_reductions(True)
    try:
        dx, dw, db = bwd.backward_ms_eden(e=dy, weight=wq, input=xq, scratch=whole, sign_seed=SIGN, scale_seed=SCALE)
        gs, x_amax = whole.e_h["global_scale"].clone(), xq.decoded_amax.clone()
        half = tokens // 2
        tk = pkg.padded_k(tokens)
        dws, dbs = [], []
        for s in range(2):
            rows = slice(s * half, (s + 1) * half)
            xs = q.quantize_four_six(x[rows].contiguous().to(dev), rowwise=True, packed=True)
            sc = pkg.LinearBackwardScratch(half, in_dim, out_dim, dev)
            dxs, dwsh, dbsh = bwd.backward_ms_eden(e=dy[rows].contiguous(), weight=wq, input=xs, scratch=sc,
                                                   sign_seed=SIGN, scale_seed=SCALE, token_offset=s * half,
                                                   e_global_scale=gs, x_decoded_amax=x_amax, total_token_count=tokens)
            assert torch.equal(sc.e_h["bytes"], whole.e_h["bytes"].view(tokens, -1)[rows].reshape(-1))
            # transposed operands: K = tokens, the shard holds columns [s*half, (s+1)*half) of every row
            for name, nrows in (("e_t_h", out_dim), ("input_t_h", in_dim)):
                w_bytes = getattr(whole, name)["bytes"].view(nrows, tk // 2)[:, s * half // 2:(s + 1) * half // 2]
                assert torch.equal(getattr(sc, name)["bytes"].view(nrows, -1), w_bytes), name
                assert torch.equal(getattr(sc, name)["global_scales"], getattr(whole, name)["global_scales"]), name
            assert torch.equal(sc.weight_t_h["bytes"], whole.weight_t_h["bytes"])
            assert rel_fro(cpu(dxs), cpu(dx[rows])) <= 1e-6
            dws.append(dwsh)
            dbs.append(dbsh)
        assert rel_fro(cpu(dws[0] + dws[1]), cpu(dw)) <= 1e-6
        assert rel_fro(cpu(dbs[0] + dbs[1]), cpu(db)) <= 1e-6
    finally:
        pkg.set_deterministic_reductions(False)
    no_timeouts(pkg)


# ------------------------------------------------------------------------------------------ a wait that runs out

def test_bounded_wait_runs_out_and_kernel_returns(pkg, oracle, dev):
    """The safe form of failure injection: with a 5 ms wait limit, CTA 0 of a GEMM never loads its first k-tile,
    so the waits on that stage run out.  The kernel must return, the status word must name the roles that gave
    up, and tensor memory must have been freed: the next GEMM on the same SMs passes its parity check.  (The
    reference's waits spin without a limit, crates/cuda-kernels/src/utils/nvfp4_tma_matmul/kernels.rs:172-174.)"""
    gemm = pkg.Nvfp4GemmModule()
    m, n, k = 512, 384, 512
    rng = np.random.default_rng(99)
    a, b = rand_nvfp4(rng, m, k, True), rand_nvfp4(rng, n, k, False)
    A, B = to_dev(pkg, dev, a, m, k, True), to_dev(pkg, dev, b, n, k, False)
    assert pkg.read_device_status() == 0
    pkg.set_gemm_wait_timeout_ns(5_000_000)
    pkg.set_gemm_debug_flags(1)
    try:
        for height, width in SHAPES:
            pkg.set_gemm_tile_override(width, height)
            gemm.gemm(A, B)
            torch.cuda.synchronize()  # returns: nothing is left spinning
            status = pkg.read_device_status()
            assert status & 2, f"the MMA / scale-factor warps should have given up, status {status:#x}"
            assert pkg.read_device_status() == 0  # reading clears the word
    finally:
        pkg.set_gemm_debug_flags(0)
        pkg.set_gemm_wait_timeout_ns(0)
        pkg.set_gemm_tile_override(0)
    for height, width in SHAPES:
        pkg.set_gemm_tile_override(width, height)
        out = gemm.gemm(A, B)
        assert rel_fro(cpu(out), oracle.gemm(a, b, m, k, n, 2)) <= GEMM_TOL
    pkg.set_gemm_tile_override(0)
    no_timeouts(pkg)
