"""Pins the CPU oracle against the known-answer cases the reference's own tests hold for the
NVFP4 projection path (crates/cuda-kernels/tests/*.rs), and against independent codecs.
No GPU needed."""
import numpy as np
import pytest

from helpers import set_e2m1_one

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def one_pair_bytes(n):
    return np.full(n // 2, 0x22, np.uint8)  # tests/common/nvfp4.rs:3-8


def one_scales(n):
    return np.full(n // 16, 0x38, np.uint8)  # tests/common/nvfp4.rs:4-12


# ---------------------------------------------------------------------------- codecs

def test_e2m1_decode_table(oracle):
    for code in range(8):
        assert oracle.e2m1_decode(code) == E2M1[code]
        assert oracle.e2m1_decode(code | 8) == -E2M1[code]


def test_codecs_match_ml_dtypes(oracle):
    ml_dtypes = pytest.importorskip("ml_dtypes")
    f8 = np.arange(256, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    for b in range(256):
        d = oracle.e4m3_decode(b)
        assert (np.isnan(d) and np.isnan(f8[b])) or d == f8[b]
    rng = np.random.default_rng(0)
    finite = f8[np.isfinite(f8)]
    finite = np.sort(finite)
    xs = np.concatenate([rng.normal(0, 3, 20000), rng.uniform(-500, 500, 20000),
                         (finite[:-1] + finite[1:]) / 2,  # every E4M3 midpoint (ties)
                         [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.25, -0.1, 0.0, -0.0, 448, 464, 465, 1e6,
                          2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10]]).astype(np.float32)
    want8 = np.clip(xs, -448, 448).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    want4 = np.clip(xs, -6, 6).astype(ml_dtypes.float4_e2m1fn).view(np.uint8) & 0xF
    got8 = np.array([oracle.e4m3_encode(float(x)) for x in xs], np.uint8)
    got4 = np.array([oracle.e2m1_encode(float(x)) for x in xs], np.uint8)
    assert np.array_equal(got8, want8)
    assert np.array_equal(got4, want4)


def test_e4m3_special_values(oracle):
    assert oracle.e4m3_decode(0x38) == 1.0          # tests/common/nvfp4.rs:4
    assert oracle.e4m3_decode(0x7E) == 448.0
    assert np.isnan(oracle.e4m3_decode(0x7F))
    assert oracle.e4m3_encode(1e9) == 0x7E          # satfinite
    assert oracle.e4m3_encode(float("nan")) == 0x7F
    assert oracle.e2m1_encode(float("nan")) == 0x7  # NaN -> +max for a format without NaN
    assert oracle.e2m1_encode(100.0) == 0x7 and oracle.e2m1_encode(-100.0) == 0xF


def test_hash_is_the_two_multiply_xorshift(oracle):
    def ref(v):  # utils/nvfp4/quant/kernels/ms_eden/random.rs:17-23, written out independently
        v &= 0xFFFFFFFF
        v ^= v >> 16
        v = (v * 0x7FEB352D) & 0xFFFFFFFF
        v ^= v >> 15
        v = (v * 0x846CA68B) & 0xFFFFFFFF
        return v ^ (v >> 16)

    for v in [0, 1, 0x12345678, 0x9ABCDEF0, 0xFFFFFFFF, 12345]:
        assert oracle.hash_u32(v) == ref(v)


def test_scale_override_constant(oracle):
    so = np.float32(17.0) / np.float32(16.0) * np.float32(0.93)  # utils/quartet.rs:1
    assert oracle.quartet_scale_override() == float(so)


# ---------------------------------------------------------------------------- decode

def test_decode_transpose_known_answer(oracle):
    """tests/nvfp4_decode.rs:18-51: all-ones payload, scalar scale 3 and rowwise scales (1, 2)."""
    rows, cols = 2, 16
    b, s = one_pair_bytes(rows * cols), one_scales(rows * cols)
    scalar = oracle.decode(b, s, np.array([3.0], np.float32), rows, cols, rowwise=False, transpose=True)
    assert (scalar == 3.0).all()
    rowwise = oracle.decode(b, s, np.array([1.0, 2.0], np.float32), rows, cols, rowwise=True, transpose=True)
    assert np.array_equal(rowwise.reshape(-1), np.tile([1.0, 2.0], cols).astype(np.float32))


# ---------------------------------------------------------------------------- quantizers

def test_four_six_known_answer(oracle):
    """tests/nvfp4_quant.rs:12-41: amax 8 -> global scale 8/(256*6), non-zero buffers."""
    x = np.array([-3.25, -2.0, -1.25, -0.5, -0.125, 0.0, 0.25, 0.75, 1.0, 1.5, 2.25, 3.0, 4.0, 5.0, 6.5, 8.0],
                 np.float32).reshape(1, 16)
    amax = np.array([np.abs(x).max()], np.float32)
    fp4, scales, gs = oracle.four_six(x, amax, rowwise=False)
    assert abs(gs[0] - 8.0 / (256.0 * 6.0)) <= 1e-8
    assert fp4.any() and scales.any()
    # the largest element must decode back to itself: 8 = 6 * scale * gs or 4 * scale * gs
    dec = oracle.decode(fp4, scales, gs, 1, 16, rowwise=False, transpose=False)
    assert dec[0, 15] == pytest.approx(8.0, rel=0.07)
    assert np.abs(dec - x).max() <= 1.0  # half of the coarsest step (2) of the chosen grid


def test_four_six_zero_tensor(oracle):
    x = np.zeros((2, 32), np.float32)
    fp4, scales, gs = oracle.four_six(x, np.zeros(2, np.float32), rowwise=True)
    assert (gs == 1.0).all() and not fp4.any() and not scales.any()


def test_four_six_choice_minimises_error(oracle):
    """The byte written is whichever of the 6- and 4-anchored scales has the smaller squared error."""
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, (64, 64)).astype(np.float32)
    amax = np.array([np.abs(x).max()], np.float32)
    fp4, scales, gs = oracle.four_six(x, amax, rowwise=False)
    dec = oracle.decode(fp4, scales, gs, 64, 64, rowwise=False, transpose=False)
    err = ((dec - x) ** 2).reshape(-1, 16).sum(1)
    g = x.reshape(-1, 16)
    ga = np.abs(g).max(1)
    for anchor in (6.0, 4.0):
        sb = np.array([oracle.e4m3_encode(float(np.float32(a) / (np.float32(anchor) * gs[0] + np.float32(1e-20))))
                       for a in ga], np.uint8)
        sv = np.array([oracle.e4m3_decode(int(b)) for b in sb], np.float32)
        alt = np.empty_like(err)
        for i in range(g.shape[0]):
            inv = np.float32(1.0) / (np.float32(sv[i] if sv[i] != 0 else 1.0) * gs[0] + np.float32(1e-20))
            q = np.array([oracle.e2m1_decode(oracle.e2m1_encode(float(v * inv))) for v in g[i]], np.float32)
            alt[i] = ((g[i] - q * (sv[i] * gs[0])) ** 2).sum()
        assert (err <= alt * (1 + 1e-5) + 1e-12).all()


def test_ms_eden_known_answer(oracle):
    """tests/nvfp4_quant.rs:45-93: 64-value ramp, reference seeds, global scale 1."""
    x = ((np.arange(64, dtype=np.float32) - 31.5) * 0.03125).reshape(2, 32)
    fp4, scales, gss, ca = oracle.ms_eden(0, x, 2, 32, 1.0, 0x12345678, 0x9ABCDEF0)
    assert fp4.any() and scales.any()
    assert (np.abs(gss - 1.0) <= 1e-8).all()
    assert (ca > 0).all() and np.isfinite(ca).all()


def test_ms_eden_rotation_is_orthonormal_and_cancels(oracle):
    """Both GEMM operands share the per-K signs and the Hadamard blocks, so A.B^T is preserved
    (utils/nvfp4/quant/kernels/ms_eden/pack/hadamard.rs; gpt/linear_backward/ms_eden.rs)."""
    rng = np.random.default_rng(5)
    a = rng.normal(0, 1, (8, 128)).astype(np.float32)
    b = rng.normal(0, 1, (8, 128)).astype(np.float32)
    ga = oracle.ms_eden_global_scale(float(np.abs(a).max()))
    gb = oracle.ms_eden_global_scale(float(np.abs(b).max()))
    qa = oracle.ms_eden(0, a, 8, 128, ga, 0x11, 0x22)
    qb = oracle.ms_eden(0, b, 8, 128, gb, 0x11, 0x33)
    da = oracle.decode(qa[0], qa[1], qa[2], 8, 128, rowwise=True, transpose=False)
    db = oracle.decode(qb[0], qb[1], qb[2], 8, 128, rowwise=True, transpose=False)
    exact = a @ b.T
    approx = da @ db.T
    assert np.linalg.norm(approx - exact) / np.linalg.norm(exact) < 0.2


SIGN_SEED, SCALE_SEED, SCALE_OVERRIDE = 0x1C69B3F5, 0x4A7C15D3, 0.25  # tests/ms_eden_transpose/support/mod.rs:9-13


def _transpose_fixture():
    rows, cols = 33, 16  # tests/ms_eden_transpose/support/mod.rs:9-10, fixtures.rs:9-17
    r = np.arange(rows, dtype=np.float32)[:, None]
    c = np.arange(cols, dtype=np.float32)[None, :]
    return ((r - 9.0) * np.float32(0.03125) + (c - 4.0) * np.float32(0.0078125)).astype(np.float32)


def test_fp32_transpose_equals_materialised_transpose(oracle):
    """tests/ms_eden_transpose/fp32.rs:12-68 (bit-exact identity, asserts in support/quant/assert.rs)."""
    x = _transpose_fixture()
    dst = oracle.padded_k(33)
    mat = oracle.ms_eden(0, np.ascontiguousarray(x.T), 16, dst, 0.75, SIGN_SEED, SCALE_SEED, so=SCALE_OVERRIDE)
    direct = oracle.ms_eden(1, x, 16, dst, 0.75, SIGN_SEED, SCALE_SEED, so=SCALE_OVERRIDE)
    for a, b in zip(mat, direct):
        assert np.array_equal(a, b)


def test_nvfp4_transposes_equal_materialised_transpose(oracle):
    """tests/ms_eden_transpose/{nvfp4,rowwise}.rs: decode + transpose + quantize == fused."""
    x = _transpose_fixture()
    dst = oracle.padded_k(33)
    # tensor-scale source
    amax = np.array([np.abs(x).max()], np.float32)
    b, s, g = oracle.four_six(x, amax, rowwise=False)
    dec_t = oracle.decode(b, s, g, 33, 16, rowwise=False, transpose=True)
    gs = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(b, s, g, 33, 16, rowwise=False)[1][0]))
    assert gs == oracle.ms_eden_global_scale(float(np.abs(dec_t).max()))
    mat = oracle.ms_eden(0, dec_t, 16, dst, gs, SIGN_SEED, SCALE_SEED)
    fused = oracle.ms_eden(2, (b, s, g, 33, 16), 16, dst, gs, SIGN_SEED, SCALE_SEED)
    for u, v in zip(mat, fused):
        assert np.array_equal(u, v)
    # rowwise source
    b, s, g = oracle.four_six(x, oracle.row_amax(x), rowwise=True)
    dec_t = oracle.decode(b, s, g, 33, 16, rowwise=True, transpose=True)
    gs = oracle.ms_eden_global_scale(float(np.abs(dec_t).max()))
    mat = oracle.ms_eden(0, dec_t, 16, dst, gs, SIGN_SEED, SCALE_SEED)
    fused = oracle.ms_eden(3, (b, s, g, 33, 16), 16, dst, gs, SIGN_SEED, SCALE_SEED)
    for u, v in zip(mat, fused):
        assert np.array_equal(u, v)


def test_sharded_ms_eden_concatenates_to_the_whole(oracle):
    """Token sharding: with col/group offsets and a shared global scale the shard outputs are the
    slices of the single-device tensor."""
    rng = np.random.default_rng(11)
    x = rng.normal(0, 1e-3, (256, 64)).astype(np.float32)
    gs = oracle.ms_eden_global_scale(float(np.abs(x).max()))
    whole_r = oracle.ms_eden(0, x, 256, 64, gs, 1, 2)
    whole_t = oracle.ms_eden(1, x, 64, 256, gs, 1, 3)
    for shard in range(2):
        xs = x[shard * 128:(shard + 1) * 128]
        r = oracle.ms_eden(0, xs, 128, 64, gs, 1, 2, group_offset=shard * 128 * 4)
        assert np.array_equal(r[0], whole_r[0].reshape(256, -1)[shard * 128:(shard + 1) * 128].reshape(-1))
        assert np.array_equal(r[1], whole_r[1].reshape(256, -1)[shard * 128:(shard + 1) * 128].reshape(-1))
        t = oracle.ms_eden(1, xs, 64, 128, gs, 1, 3, col_offset=shard * 128)
        # transposed operand: K = tokens; nibbles of the shard equal the matching K slice
        assert np.array_equal(t[0].reshape(64, -1), whole_t[0].reshape(64, -1)[:, shard * 64:(shard + 1) * 64])


# ---------------------------------------------------------------------------- scale layout

def test_packed_scale_layout_matches_reference_formula(oracle):
    """utils/nvfp4_tma_matmul/cute.rs:448-467 (block-major byte offset)."""
    k = 256
    k_atoms = k // 64
    seen = set()
    for mn in range(256):
        for g in range(k // 16):
            blk, in_blk = divmod(mn, 128)
            want = blk * k_atoms * 512 + (g // 4) * 512 + (in_blk % 32) * 16 + (in_blk // 32) * 4 + g % 4
            got = oracle.scale_packed_offset(mn, g, k)
            assert got == want
            seen.add(got)
    assert seen == set(range(256 * k // 16))  # a bijection onto the packed plane


def test_scale_pack_pads_with_one(oracle):
    logical = np.arange(130 * 4, dtype=np.uint8)
    packed = oracle.scale_pack(logical, 130, 64)
    assert packed.size == 2 * 512
    assert packed[oracle.scale_packed_offset(129, 3, 64)] == logical[129 * 4 + 3]
    assert packed[oracle.scale_packed_offset(130, 0, 64)] == 0x38  # scale_pack.rs:33-35


# ---------------------------------------------------------------------------- GEMM

def test_lm_head_known_answer(oracle):
    """tests/lm_head.rs:25-72 (exact small integers)."""
    tokens, k, vocab = 2, 64, 16
    a = np.zeros(tokens * k // 2, np.uint8)
    for e in (0, 1, k + 2):
        set_e2m1_one(a, e)
    w = np.zeros(vocab * k // 2, np.uint8)
    for e in (0, k + 1, 2 * k + 2):
        set_e2m1_one(w, e)
    out = oracle.gemm((a, one_scales(tokens * k), np.ones(tokens, np.float32)),
                      (w, one_scales(vocab * k), np.ones(1, np.float32)), tokens, k, vocab, mode=2)
    assert out[0, 0] == 1.0 and out[0, 1] == 1.0 and out[0, 2] == 0.0
    assert out[1, 0] == 0.0 and out[1, 1] == 0.0 and out[1, 2] == 1.0


def test_linear_backward_quartet_known_answer(oracle):
    """tests/linear_backward/quartet.rs:13-76: dinput all ones, dweight row 0 = token count."""
    t = i = o = 64
    first_col = np.zeros(t * o // 2, np.uint8)
    for r in range(t):
        set_e2m1_one(first_col, r * o)
    first_row = np.zeros(o * t // 2, np.uint8)
    for c in range(t):
        set_e2m1_one(first_row, c)
    ones_t = np.ones(t, np.float32)
    dinput = oracle.gemm((first_col, one_scales(t * o), ones_t), (first_col.copy(), one_scales(i * o), np.ones(1, np.float32)),
                         t, o, i, mode=2)
    assert (np.abs(dinput - 1.0) <= 1e-7).all()
    dweight = oracle.gemm((first_row, one_scales(o * t), np.ones(o, np.float32)),
                          (one_pair_bytes(i * t), one_scales(i * t), np.ones(1, np.float32)), o, t, i, mode=2)
    assert (dweight[0] == t).all() and (dweight[1:] == 0).all()


def test_gemm_epilogues(oracle):
    """gpt/projection_postop.rs:97-162 on the patterned fixtures of tests/projection_tma.rs:355-385."""
    rows, k, n = 8, 64, 16
    a = np.zeros(rows * k // 2, np.uint8)
    w = np.zeros(n * k // 2, np.uint8)
    for r in range(rows):
        for c in range(k):
            if (r * 3 + c * 5 + 1) % 17 == 0:
                set_e2m1_one(a, r * k + c)
    for r in range(n):
        for c in range(k):
            if (r * 7 + c * 11 + 3) % 17 == 0:
                set_e2m1_one(w, r * k + c)
    pat = np.array([0x30, 0x34, 0x38, 0x3C, 0x40], np.uint8)
    sa = pat[(np.arange(rows * k // 16) + 0) % 5]
    sw = pat[(np.arange(n * k // 16) + 2) % 5]
    ga = (0.5 + (np.arange(rows) % 7) * 0.125).astype(np.float32)
    gw = np.array([0.75], np.float32)
    bias = (np.arange(n) * 0.25 - 1.0).astype(np.float32)
    raw = oracle.gemm((a, sa, ga), (w, sw, gw), rows, k, n, mode=2)
    with_bias = oracle.gemm((a, sa, ga), (w, sw, gw), rows, k, n, mode=2, bias=bias, epi=1)
    assert np.array_equal(with_bias, raw + bias[None, :])
    relu2, pre = oracle.gemm((a, sa, ga), (w, sw, gw), rows, k, n, mode=2, bias=bias, epi=2, want_pre=True)
    assert np.array_equal(pre, with_bias) and np.array_equal(relu2, np.maximum(pre, 0) ** 2)
    res = ((np.arange(rows * n) % 23) * 0.03125 - 0.25).astype(np.float32).reshape(rows, n)
    added = oracle.gemm((a, sa, ga), (w, sw, gw), rows, k, n, mode=2, bias=bias, epi=3, residual=res)
    assert np.allclose(added, res + with_bias, rtol=0, atol=1e-6)
    # dequantised check against plain numpy
    da = oracle.decode(a, sa, ga, rows, k, rowwise=True, transpose=False)
    dw = oracle.decode(w, sw, gw, n, k, rowwise=False, transpose=False)
    assert np.allclose(raw, da @ dw.T, rtol=1e-6, atol=1e-6)


def test_bias_grad_known_answer(oracle):
    """tests/linear_backward/ms_eden.rs:65-70,83-91: dbias equals the column sums."""
    t, n = 64, 64
    idx = np.arange(t * n)
    e = (((idx // n).astype(np.float32) * 0.5) + ((idx % n).astype(np.float32) - 31.5)) * np.float32(0.015625)
    e = e.reshape(t, n).astype(np.float32)
    db = oracle.bias_grad(e)
    want = np.array([np.float32(sum(e[r, c] for r in range(t))) for c in range(n)], np.float32)
    assert (np.abs(db - want) <= 1e-7 * np.maximum(1, np.abs(want)) + 1e-5).all()


def test_tensor_amax_chunks(oracle):
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, 5000).astype(np.float32)
    chunks, amax = oracle.tensor_amax(x)
    assert chunks.size == 5 and amax[0] == np.abs(x).max()
    assert chunks[4] == np.abs(x[4096:]).max()


def test_schedule_free_value(oracle):
    """gpt/optimizer/schedule_free/value.rs:4-9: each operation rounds to f32 on its own."""
    rng = np.random.default_rng(4)
    z = rng.normal(0, 0.02, 4096).astype(np.float32)
    x = (z + rng.normal(0, 0.003, 4096)).astype(np.float32)
    for beta in (0.0, 0.5, 0.9, 1.0):
        b = np.float32(beta)
        want = (z + (b * (x - z)).astype(np.float32)).astype(np.float32)
        assert np.array_equal(oracle.schedule_free_value(z, x, beta), want)
    assert np.array_equal(oracle.schedule_free_value(z, x, 0.0), z)


def test_relu2_backward(oracle):
    """gpt/mlp/kernels.rs:72-104."""
    pre = np.array([-1.0, -0.0, 0.0, 0.5, 2.0, np.nan], np.float32)
    d = np.array([3.0, 3.0, 3.0, 3.0, -0.25, 1.0], np.float32)
    assert np.array_equal(oracle.relu2_backward(pre, d), np.array([0, 0, 0, 3.0, -1.0, 0], np.float32))


def test_stochastic_scale_integer_identity(oracle):
    """Inside the normal E4M3 range the stochastic rounding of pack/scale.rs:7-30 reduces to integers:
    lower code = (f32 bits >> 20) - 960, p = low 20 mantissa bits / 2^20, draw = 24 hash bits / 2^24.
    The CUDA quantizers use this form; here it is pinned against the restatement of the reference."""
    rng = np.random.default_rng(11)
    values = np.concatenate([rng.uniform(2.0 ** -6, 448.0, 3000), 2.0 ** rng.uniform(-6, 8.8, 3000),
                             [2.0 ** -6, 1.0, 1.125, 447.99, 0.015625 * 1.875]]).astype(np.float32)
    for i, v in enumerate(values):
        if not (np.float32(2.0 ** -6) <= v < np.float32(448.0)):
            continue
        bits = int(v.view(np.uint32))
        seed, group = 0x9ABCDEF0, i * 2654435761 & 0xFFFFFFFF
        draw = oracle.hash_u32(seed ^ group) & 0xFFFFFF
        fast = (bits >> 20) - 960 + (1 if draw < ((bits & 0xFFFFF) << 4) else 0)
        assert fast == oracle.stochastic_e4m3_scale(float(v), seed, group)
