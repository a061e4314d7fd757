"""CPU checks of the oracle: hand-derived known answers, the committed golden
vectors (made by an independent numpy restatement, tests/golden/make_golden.py)
and properties.  The reference ships no vectors of its own, so these are the
pins the oracle has.
"""
import struct

import numpy as np
import pytest

F = np.float32


def f32(x):
    return struct.unpack("f", struct.pack("f", x))[0]


# ---------------------------------------------------------------------------
# scalar helpers
# ---------------------------------------------------------------------------
def test_f16_conversion_matches_ieee(oracle):
    lib = oracle.load()
    rng = np.random.default_rng(1)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(F) * F(100),
        rng.standard_normal(2000).astype(F) * F(1e-5),   # fp16 subnormals
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0**-24, 2.0**-25, 2.0**-25 * 1.0001,
                  np.inf, -np.inf], dtype=F),
    ])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([lib.oracle_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)
    back = np.array([lib.oracle_f16_to_f32(int(h)) for h in range(0, 0x7C01, 37)], dtype=F)
    assert np.array_equal(back, np.arange(0, 0x7C01, 37, dtype=np.uint16).view(np.float16).astype(F))


def test_bf16_conversion_round_half_even(oracle):
    lib = oracle.load()
    # 1 + 2^-8 is exactly half way between two bf16 values: ties to even (down)
    assert lib.oracle_f32_to_bf16(1.0 + 2.0**-8) == 0x3F80
    assert lib.oracle_f32_to_bf16(1.0 + 3 * 2.0**-8) == 0x3F82  # ties up to even
    assert lib.oracle_f32_to_bf16(f32(1.0 + 2.0**-8 + 2.0**-20)) == 0x3F81
    assert lib.oracle_bf16_to_f32(0x3F80) == 1.0


def test_two_step_narrowing_known_answers(oracle):
    lib = oracle.load()
    AW, DI = oracle.ROUND_AS_WRITTEN, oracle.ROUND_DIRECT
    # 64.51 -> fp16 grid near 64 has spacing 1/16: 64.5 -> ties to even 64; direct gives 65
    assert lib.oracle_narrow_i8(64.51, AW) == 64
    assert lib.oracle_narrow_i8(64.51, DI) == 65
    # 0.50001 -> fp16 0.5 -> 0 ; direct 1
    assert lib.oracle_narrow_i8(0.50001, AW) == 0
    assert lib.oracle_narrow_i8(0.50001, DI) == 1
    for v, want in [(0.5, 0), (1.5, 2), (2.5, 2), (-0.5, 0), (-1.5, -2), (-2.5, -2), (126.5, 126), (127.0, 127),
                    (127.49, 127), (-127.5, -128), (300.0, 127), (-300.0, -128), (float("inf"), 127),
                    (float("-inf"), -128), (float("nan"), 0)]:
        assert lib.oracle_narrow_i8(v, AW) == want, v
    for v, want in [(0.5, 0), (1.5, 2), (2.5, 2), (127.6, 127), (-128.6, -128), (float("nan"), 0)]:
        assert lib.oracle_narrow_i8(v, DI) == want, v


def test_canonical_exp_accuracy_and_edges(oracle):
    lib = oracle.load()
    xs = np.linspace(-87, 88, 20001).astype(F)
    got = np.array([lib.oracle_expf(float(v)) for v in xs], dtype=F)
    ref = np.exp(xs.astype(np.float64))
    ulp = np.abs(got.astype(np.float64) - ref) / np.spacing(ref.astype(F)).astype(np.float64)
    assert ulp.max() < 1.5
    assert lib.oracle_expf(0.0) == 1.0
    assert lib.oracle_expf(1000.0) == float("inf")
    assert lib.oracle_expf(-1000.0) == 0.0
    assert np.isnan(lib.oracle_expf(float("nan")))
    # silu: gate far negative -> -0, far positive -> identity, zero -> 0
    assert lib.oracle_silu(-200.0, oracle.EXP_CANONICAL) == 0.0
    assert lib.oracle_silu(50.0, oracle.EXP_CANONICAL) == 50.0
    assert lib.oracle_silu(0.0, oracle.EXP_CANONICAL) == 0.0


# ---------------------------------------------------------------------------
# DynamicQuant
# ---------------------------------------------------------------------------
def test_dq_hand_derived(oracle):
    # row: max |x| = 2.0 -> scale = 2*(1/127), inv = 0.5*127 = 63.5
    x = np.array([[2.0, -2.0, 1.0, 0.0, 0.0078125, -1.0, 0.5, 1.9921875]], dtype=F)
    y, s = oracle.dynamic_quant(oracle.f32_to_bf16_bits(x), oracle.DT_BF16)
    assert s[0] == F(2.0) * F(1.0 / 127.0)
    # 63.5 -> 64 (tie to even), 0.49609375 -> 0, 31.75 -> 32, 1.9921875*63.5 = 126.50390625 -> fp16 126.5 -> 126
    assert y.tolist() == [[127, -127, 64, 0, 0, -64, 32, 126]]
    yd, _ = oracle.dynamic_quant(oracle.f32_to_bf16_bits(x), oracle.DT_BF16, oracle.ROUND_DIRECT)
    assert yd.tolist() == [[127, -127, 64, 0, 0, -64, 32, 127]]  # the double rounding shows in the last element


def test_dq_zero_row_and_specials(oracle):
    x = np.zeros((3, 16), dtype=F)
    x[1, 2] = np.inf
    x[1, 3] = 1.0
    x[2, 4] = np.nan
    x[2, 5] = 1.0
    y, s = oracle.dynamic_quant(oracle.f32_to_bf16_bits(x), oracle.DT_BF16)
    assert s[0] == F(1e-12) * F(1.0 / 127.0)
    assert np.isinf(s[1]) and np.isnan(s[2])
    assert not y.any()


@pytest.mark.parametrize("kind", ["bf16", "f16"])
def test_dq_golden(oracle, golden, kind):
    dt = oracle.DT_BF16 if kind == "bf16" else oracle.DT_F16
    y, s = oracle.dynamic_quant(golden[f"dq_{kind}_x"], dt)
    assert np.array_equal(y, golden[f"dq_{kind}_y"])
    assert np.array_equal(s.view(np.uint32), golden[f"dq_{kind}_scale"].view(np.uint32))
    yd, _ = oracle.dynamic_quant(golden[f"dq_{kind}_x"], dt, oracle.ROUND_DIRECT)
    assert np.array_equal(yd, golden[f"dq_{kind}_y_direct"])


def test_dq_properties(oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((64, 333)).astype(F)
    xb = oracle.f32_to_bf16_bits(x)
    y, s = oracle.dynamic_quant(xb, oracle.DT_BF16)
    xf = oracle.bf16_bits_to_f32(xb)
    assert np.abs(y.astype(np.int32)).max() <= 127
    # dequantised value within half a step (+ the fp16 grid's 1/32) of the input
    err = np.abs(y.astype(F) * s[:, None] - xf)
    assert (err <= s[:, None] * 0.54).all()
    # each row attains +-127 at its absolute maximum
    assert (np.abs(y).max(axis=1) == 127).all()
    # row permutation invariance
    perm = rng.permutation(64)
    y2, s2 = oracle.dynamic_quant(xb[perm], oracle.DT_BF16)
    assert np.array_equal(y2, y[perm]) and np.array_equal(s2, s[perm])
    # empty input
    y0, s0 = oracle.dynamic_quant(np.zeros((0, 16), np.uint16), oracle.DT_BF16)
    assert y0.shape == (0, 16) and s0.shape == (0,)


# ---------------------------------------------------------------------------
# AddRmsNormDynamicQuant
# ---------------------------------------------------------------------------
def test_ardq_hand_derived(oracle):
    # x1 + x2 = [3, -4, 0, 0]; gamma = 1; eps = 0: sum sq = 25, mean = 6.25, rms = 2.5 (all exact)
    x1 = np.array([[1.0, -1.0, 0.0, 0.0]], dtype=F)
    x2 = np.array([[2.0, -3.0, 0.0, 0.0]], dtype=F)
    g = np.ones(4, dtype=F)
    b = oracle.f32_to_bf16_bits
    for order in (oracle.SUM_CANONICAL, oracle.SUM_FP64):
        y, xo, sc = oracle.add_rms_norm_dynamic_quant(b(x1), b(x2), b(g), 0.0, oracle.DT_BF16, sum_order=order)
        assert oracle.bf16_bits_to_f32(xo).tolist() == [[3.0, -4.0, 0.0, 0.0]]
        rstd = F(1.0) / F(2.5)
        m = F(4.0) * rstd
        want_scale = m * F(1.0 / 127.0)
        assert sc[0] == want_scale
        k = rstd / want_scale
        assert y.tolist() == [[int(np.rint(np.float16(F(3.0) * k))), -127, 0, 0]]


def test_ardq_zero_row_scale_is_clamp_constant(oracle):
    z = np.zeros((1, 64), np.uint16)
    g = oracle.f32_to_bf16_bits(np.ones(64, F))
    y, xo, sc = oracle.add_rms_norm_dynamic_quant(z, z, g, 1e-6, oracle.DT_BF16)
    assert sc[0] == F(1e-12) * F(1.0 / 127.0)
    assert not y.any() and not xo.any()
    # eps = 0 on an all-zero row: rms = 0, rstd = inf, m = NaN -> NaN scale, zero output
    y, xo, sc = oracle.add_rms_norm_dynamic_quant(z, z, g, 0.0, oracle.DT_BF16)
    assert np.isnan(sc[0]) and not y.any()


@pytest.mark.parametrize("kind", ["bf16", "f16"])
def test_ardq_golden(oracle, golden, kind):
    dt = oracle.DT_BF16 if kind == "bf16" else oracle.DT_F16
    y, xo, sc = oracle.add_rms_norm_dynamic_quant(golden[f"ardq_{kind}_x1"], golden[f"ardq_{kind}_x2"],
                                                  golden[f"ardq_{kind}_gamma"], 1e-6, dt,
                                                  sum_order=oracle.SUM_FP64)
    assert np.array_equal(y, golden[f"ardq_{kind}_y"])
    nan = np.isnan(oracle.bits_to_f32(xo, dt))
    assert np.array_equal(xo[~nan], golden[f"ardq_{kind}_xout"][~nan])
    want = golden[f"ardq_{kind}_scale"]
    assert np.array_equal(np.isnan(sc), np.isnan(want))
    assert np.array_equal(sc[~np.isnan(sc)], want[~np.isnan(want)])


def test_ardq_canonical_order_within_tolerance_of_fp64(oracle):
    rng = np.random.default_rng(3)
    rows, n = 256, 7168
    b = oracle.f32_to_bf16_bits
    x1, x2 = b(rng.standard_normal((rows, n)).astype(F)), b(rng.standard_normal((rows, n)).astype(F))
    g = b((1 + 0.1 * rng.standard_normal(n)).astype(F))
    ya, xa, sa = oracle.add_rms_norm_dynamic_quant(x1, x2, g, 1e-6, oracle.DT_BF16, sum_order=oracle.SUM_CANONICAL)
    yb, xb, sb = oracle.add_rms_norm_dynamic_quant(x1, x2, g, 1e-6, oracle.DT_BF16, sum_order=oracle.SUM_FP64)
    assert np.array_equal(xa, xb)
    # tolerance of the summation order: a few fp32 ulp on the scale, +-1 LSB on <= 1e-4 of the elements
    assert (np.abs(sa - sb) <= 4 * np.spacing(sb)).all()
    d = np.abs(ya.astype(np.int32) - yb.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= 1e-4


def test_ardq_rejects_long_rows(oracle):
    z = np.zeros((1, 16392), np.uint16)
    with pytest.raises(ValueError):
        oracle.add_rms_norm_dynamic_quant(z, z, z[0], 1e-6, oracle.DT_BF16)


# ---------------------------------------------------------------------------
# QuantMatmul
# ---------------------------------------------------------------------------
def test_qm_golden_all_epilogue_forms(oracle, golden):
    O = oracle
    g = golden
    fl = O.QM_SCALE_PERCHAN | O.QM_HAS_PT
    out, acc = O.quant_matmul(g["qm_x1"], g["qm_x2"], g["qm_scale"], pertoken=g["qm_pt"], flags=fl,
                              out_dtype=O.DT_BF16, want_acc=True)
    assert np.array_equal(acc, g["qm_acc"]) and np.array_equal(out, g["qm_out_pt_bf16"])
    fl = (O.QM_SCALE_PERCHAN | O.QM_HAS_PT | O.QM_HAS_OFFSET | O.QM_OFFSET_PERCHAN |
          (O.QM_BIAS_BF16 << O.QM_BIAS_SHIFT) | O.QM_BIAS_PERCHAN)
    out = O.quant_matmul(g["qm_x1"], g["qm_x2"], g["qm_scale"], offset=g["qm_offset"], pertoken=g["qm_pt"],
                         bias=g["qm_bias_bf16"], flags=fl, out_dtype=O.DT_BF16)
    assert np.array_equal(out, g["qm_out_full_bf16"])
    fl = (O.QM_SCALE_PERCHAN | O.QM_HAS_OFFSET | O.QM_OFFSET_PERCHAN | (O.QM_BIAS_I32 << O.QM_BIAS_SHIFT) |
          O.QM_BIAS_PERCHAN)
    out = O.quant_matmul(g["qm_x1"], g["qm_x2"], g["qm_scale"], offset=g["qm_offset"], bias=g["qm_bias_i32"],
                         flags=fl, out_dtype=O.DT_F16)
    assert np.array_equal(out, g["qm_out_i32bias_f16"])
    out = O.quant_matmul(g["qm_x1"], g["qm_x2"], g["qm_scale"][:1].copy(), flags=0, out_dtype=O.DT_F16)
    assert np.array_equal(out, g["qm_out_scalar_f16"])
    x2t = np.ascontiguousarray(g["qm_x2"].T)
    out_t = O.quant_matmul(g["qm_x1"], x2t, g["qm_scale"][:1].copy(), flags=0, out_dtype=O.DT_F16,
                           x2_transposed=True)
    assert np.array_equal(out, out_t)


def test_qm_order_of_operations_hand_derived(oracle):
    O = oracle
    # acc = 3; ((3 + 2) * 0.5 + 0.25) * 4 + 1 = 12.0
    x1 = np.array([[1, 1, 1] + [0] * 13], np.int8)
    x2 = np.zeros((16, 16), np.int8)
    x2[:3, 0] = 1
    fl = O.QM_HAS_OFFSET | O.QM_HAS_PT | (O.QM_BIAS_I32 << O.QM_BIAS_SHIFT)
    out = O.quant_matmul(x1, x2, np.array([0.5], F), offset=np.array([0.25], F), pertoken=np.array([4.0], F),
                         bias=np.array([2], np.int32), flags=fl, out_dtype=O.DT_F16)
    assert O.f16_bits_to_f32(out)[0, 0] == 11.0  # int32 bias is added before the scale
    fl = O.QM_HAS_OFFSET | O.QM_HAS_PT | (O.QM_BIAS_F32 << O.QM_BIAS_SHIFT)
    out = O.quant_matmul(x1, x2, np.array([0.5], F), offset=np.array([0.25], F), pertoken=np.array([4.0], F),
                         bias=np.array([1.0], F), flags=fl, out_dtype=O.DT_F16)
    assert O.f16_bits_to_f32(out)[0, 0] == 8.0   # (3*0.5 + 0.25) * 4 + 1


def test_qm_cfg1_chain_runs_on_cpu(oracle):
    """Benchmark configuration 1: DynamicQuant -> QuantMatmul, seed 0, M=128 K=1024 N=1024."""
    O = oracle
    rng = np.random.default_rng(0)
    x = rng.standard_normal((128, 1024)).astype(F)
    w = rng.integers(-127, 128, (1024, 1024)).astype(np.int8)
    ws = rng.uniform(1e-3, 1e-2, 1024).astype(F)
    xq, xs = O.dynamic_quant(O.f32_to_bf16_bits(x), O.DT_BF16)
    out, acc = O.quant_matmul(xq, w, ws, pertoken=xs, flags=O.QM_SCALE_PERCHAN | O.QM_HAS_PT, out_dtype=O.DT_BF16,
                              want_acc=True)
    ref_acc = xq.astype(np.int64) @ w.astype(np.int64)
    assert np.array_equal(acc, ref_acc.astype(np.int32))
    approx = (O.bf16_bits_to_f32(O.f32_to_bf16_bits(x)).astype(np.float64) @ (w.astype(np.float64) * ws[None, :]))
    got = O.bf16_bits_to_f32(out).astype(np.float64)
    # quantisation noise only: relative Frobenius error around 1 %
    assert np.linalg.norm(got - approx) / np.linalg.norm(approx) < 0.02


# ---------------------------------------------------------------------------
# GroupedMatmulSwigluQuant / GroupedMatmul
# ---------------------------------------------------------------------------
def test_gmsq_golden(oracle, golden):
    g = golden
    y, ys, act = oracle.grouped_matmul_swiglu_quant(g["gmsq_x"], g["gmsq_w"], g["gmsq_ws"], g["gmsq_xs"], g["gmsq_gl"],
                                                    exp_kind=oracle.EXP_LIBM, want_act=True)
    assert np.array_equal(act.view(np.uint32), g["gmsq_act"].view(np.uint32))
    assert np.array_equal(y, g["gmsq_y"]) and np.array_equal(ys, g["gmsq_yscale"])
    # the all-zero row clamps to FLT_MIN: scale FLT_MIN/127 (a denormal), output zeros
    assert ys[4] == F(1.1754944e-38) * F(1.0 / 127.0) and not y[4].any()
    # canonical exp agrees within the stated tolerance (here: exactly)
    y2, ys2 = oracle.grouped_matmul_swiglu_quant(g["gmsq_x"], g["gmsq_w"], g["gmsq_ws"], g["gmsq_xs"], g["gmsq_gl"])
    assert np.abs(y2.astype(np.int32) - y.astype(np.int32)).max() <= 1
    assert np.allclose(ys2, ys, rtol=1e-6, atol=0)


def test_gmsq_group_split_invariance_and_layouts(oracle):
    rng = np.random.default_rng(4)
    m, k, n = 40, 64, 96
    x = rng.integers(-127, 128, (m, k)).astype(np.int8)
    w1 = rng.integers(-127, 128, (1, k, n)).astype(np.int8)
    ws1 = rng.uniform(1e-3, 1e-2, (1, n)).astype(F)
    xs = rng.uniform(1e-3, 5e-2, m).astype(F)
    y1, s1 = oracle.grouped_matmul_swiglu_quant(x, w1, ws1, xs, [m])
    # the same weights repeated as 5 experts, arbitrary split (with an empty group)
    w5, ws5 = np.repeat(w1, 5, 0), np.repeat(ws1, 5, 0)
    y5, s5 = oracle.grouped_matmul_swiglu_quant(x, w5, ws5, xs, [7, 7, 20, 39, 40])
    assert np.array_equal(y1, y5) and np.array_equal(s1, s5)
    # [E, N, K] layout gives the same result
    yt, st = oracle.grouped_matmul_swiglu_quant(x, np.ascontiguousarray(w5.transpose(0, 2, 1)), ws5, xs,
                                                [7, 7, 20, 39, 40], w_transposed=True)
    assert np.array_equal(yt, y5) and np.array_equal(st, s5)
    assert np.abs(y1.astype(np.int32)).max() <= 127
    with pytest.raises(ValueError):
        oracle.grouped_matmul_swiglu_quant(x, w5, ws5, xs, [7, 6, 20, 39, 40])   # not monotone
    with pytest.raises(ValueError):
        oracle.grouped_matmul_swiglu_quant(x, w5, ws5, xs, [7, 7, 20, 39, 39])   # last != M


def test_gmsq_gate_is_left_half(oracle):
    # one row, K = 16: acc_left = 16, acc_right = 32 with unit scales: act = silu(16) * 32
    x = np.ones((1, 16), np.int8)
    w = np.zeros((1, 16, 32), np.int8)
    w[0, :, 0] = 1
    w[0, :, 16] = 2
    y, ys, act = oracle.grouped_matmul_swiglu_quant(x, w, np.ones((1, 32), F), np.ones(1, F), [1], want_act=True)
    lib = oracle.load()
    assert act[0, 0] == F(lib.oracle_silu(16.0, oracle.EXP_CANONICAL)) * F(32.0)
    assert y[0, 0] == 127 and not y[0, 1:].any()


def test_gmm_int8_golden_and_equals_quant_matmul_per_group(oracle, golden):
    g = golden
    O = oracle
    out = O.grouped_matmul(g["gmm_x"], g["gmm_w"], g["gmm_gl"], dtype=O.DT_I8, x_scale=g["gmm_xs"],
                           w_scale=g["gmm_ws"])
    assert np.array_equal(out, g["gmm_out"])
    # each group equals a quant_matmul call with that expert's weights
    start = 0
    for e, end in enumerate(g["gmm_gl"]):
        end = int(end)
        if end > start:
            ref = O.quant_matmul(g["gmm_x"][start:end], g["gmm_w"][e], g["gmm_ws"][e].copy(),
                                 pertoken=g["gmm_xs"][start:end].copy(), flags=O.QM_SCALE_PERCHAN | O.QM_HAS_PT,
                                 out_dtype=O.DT_BF16)
            assert np.array_equal(out[start:end], ref)
        start = end


def test_gmm_float_path_against_fp64(oracle):
    rng = np.random.default_rng(5)
    m, k, n, e = 24, 48, 40, 3
    gl = [10, 10, 24]
    x = (rng.standard_normal((m, k))).astype(F)
    w = (rng.standard_normal((e, k, n)) * 0.1).astype(F)
    bias = rng.standard_normal((e, n)).astype(F)
    xb, wb = oracle.f32_to_bf16_bits(x), oracle.f32_to_bf16_bits(w)
    out = oracle.grouped_matmul(xb, wb, gl, dtype=oracle.DT_BF16, bias=bias, bias_dtype=oracle.DT_F32)
    xf, wf = oracle.bf16_bits_to_f32(xb).astype(np.float64), oracle.bf16_bits_to_f32(wb).astype(np.float64)
    ref = np.zeros((m, n))
    ref[:10] = xf[:10] @ wf[0] + bias[0]
    ref[10:] = xf[10:] @ wf[2] + bias[2]
    got = oracle.bf16_bits_to_f32(out).astype(np.float64)
    assert np.abs(got - ref).max() <= np.abs(ref).max() * 2.0**-7


# ---------------------------------------------------------------------------
# expert-parallel bookkeeping
# ---------------------------------------------------------------------------
def test_route_count_is_stable_sort(oracle):
    rng = np.random.default_rng(6)
    t, topk, e = 50, 4, 8
    idx = rng.integers(0, e, (t, topk)).astype(np.int32)
    cnt, cum, pos = oracle.route_count(idx, e)
    flat = idx.reshape(-1)
    order = np.argsort(flat, kind="stable")
    want_pos = np.empty(t * topk, np.int64)
    want_pos[order] = np.arange(t * topk)
    assert np.array_equal(pos.reshape(-1), want_pos)
    assert np.array_equal(cnt, np.bincount(flat, minlength=e))
    assert np.array_equal(cum, np.cumsum(cnt))


def test_combine_hand_derived(oracle):
    rows = oracle.f32_to_bf16_bits(np.array([[1.0, 2.0], [4.0, 8.0], [100.0, 100.0]], F))
    probs = np.array([[0.5, 0.25]], F)
    pos = np.array([[1, 0]], np.int64)
    out = oracle.combine(rows, probs, pos, oracle.DT_BF16)
    assert oracle.bf16_bits_to_f32(out).tolist() == [[2.25, 4.5]]
    out = oracle.combine(rows, probs, np.array([[1, -1]], np.int64), oracle.DT_BF16)
    assert oracle.bf16_bits_to_f32(out).tolist() == [[2.0, 4.0]]


def test_moe_re_routing_hand_derived_and_against_regroup_index(oracle):
    """Rank 0 sends 2 rows to expert 0 and 1 to expert 2; rank 1 sends 1 row to expert 0 and 3 to expert 1.
    Source order is rank-major (rows 0-2 from rank 0, 3-6 from rank 1); the expert-major order is therefore
    e0: [0, 1, 3], e1: [4, 5, 6], e2: [2]."""
    cnt = np.array([[2, 0, 1], [1, 3, 0]])
    tok = np.arange(7 * 4, dtype=np.int8).reshape(7, 4)
    scl = np.arange(7, dtype=F) + 0.5
    out, out_s, idx, num = oracle.moe_re_routing(tok, cnt, scl)
    assert idx.tolist() == [0, 1, 3, 4, 5, 6, 2]
    assert num.tolist() == [3, 3, 1]
    assert np.array_equal(out, tok[idx]) and np.array_equal(out_s, scl[idx])
    # the host-side index the expert-parallel chain uses is the same permutation
    from cannbench_operator_solutions_b200.ep import regroup_index

    rng = np.random.default_rng(12)
    cnt = rng.integers(0, 5, (4, 6))
    cnt[1, :] = 0
    cnt[:, 2] = 0
    a = int(cnt.sum())
    tok = rng.integers(-128, 128, (a + 3, 16)).astype(np.int8)  # three rows past the routed total
    out, _, idx, num = oracle.moe_re_routing(tok, cnt)
    src_of_dst, cumsum = regroup_index(cnt)
    assert np.array_equal(idx[:a], src_of_dst) and np.array_equal(np.cumsum(num), cumsum)
    assert np.array_equal(out[:a], tok[idx[:a]]) and not out[a:].any()
    assert np.array_equal(num, cnt.sum(axis=0))
    with pytest.raises(ValueError):
        oracle.moe_re_routing(tok[:2], cnt)


def test_moe_finalize_routing_hand_derived(oracle):
    """Two output rows, K = 2, H = 2, fp32 so that every step is exact.
    rows = [[1, 2], [10, 20], [100, 200]], bias = [[0.5, 0.5], [-1, -1]], scales = [[2, 3], [4, 5]],
    expert = [[0, 1], [1, 7]] (7 is out of range: its bias is dropped), skip1 = 1000, skip2 = 0.25.
    Column arrangement (mode 0): esdr = [p(0,0), p(1,0), p(0,1), p(1,1)] = [2, 0, 1, -1].
      out[0] = 1000.25 + 2*(rows[2] + bias[0]) + 3*(rows[1] + bias[1]) = 1000.25 + [201, 401] + [27, 57]
      out[1] = 1000.25 + 4*(rows[0] + bias[1]) + (term dropped)       = 1000.25 + [0, 4]"""
    rows = np.array([[1, 2], [10, 20], [100, 200]], F)
    bias = np.array([[0.5, 0.5], [-1, -1]], F)
    scales = np.array([[2, 3], [4, 5]], F)
    expert = np.array([[0, 1], [1, 7]], np.int32)
    skip1 = np.full((2, 2), 1000.0, F)
    skip2 = np.full((2, 2), 0.25, F)
    out = oracle.moe_finalize_routing(rows, np.array([2, 0, 1, -1], np.int32), oracle.DT_F32, skip1=skip1, skip2=skip2,
                                      bias=bias, scales=scales, expert=expert, drop_pad_mode=0)
    assert out.tolist() == [[1228.25, 1458.25], [1000.25, 1004.25]]
    # row arrangement (mode 2) of the same mapping
    out2 = oracle.moe_finalize_routing(rows, np.array([2, 1, 0, -1], np.int32), oracle.DT_F32, skip1=skip1,
                                       skip2=skip2, bias=bias, scales=scales, expert=expert, drop_pad_mode=2)
    assert np.array_equal(out, out2)
    # bias without expert ids is ignored; no scales means K = 1 and unit weights
    out3 = oracle.moe_finalize_routing(rows, np.array([1, 5], np.int32), oracle.DT_F32, bias=bias)
    assert out3.tolist() == [[10.0, 20.0], [0.0, 0.0]]
    # the expert-parallel combine is the scales-only, row-arranged special case
    rng = np.random.default_rng(3)
    r16 = oracle.f32_to_bf16_bits(rng.standard_normal((12, 16)).astype(F))
    probs = rng.random((5, 3)).astype(F)
    pos = rng.integers(-1, 12, (5, 3))
    a = oracle.combine(r16, probs, pos.astype(np.int64), oracle.DT_BF16)
    b = oracle.moe_finalize_routing(r16, pos.astype(np.int32).reshape(-1), oracle.DT_BF16, scales=probs,
                                    drop_pad_mode=2)
    assert np.array_equal(a, b)


def test_moe_finalize_routing_rounds_each_step_in_fp32(oracle):
    """(row + bias) is rounded to fp32 before the multiplication, and the product before the addition:
    row = 1, bias = 2^-24 -> 1 (the half-ulp tie rounds to even); scale 3 -> 3; a fused or reordered evaluation,
    scale*row + scale*bias, would give 3 + 3*2^-24, which rounds to the next fp32 above 3."""
    rows = np.array([[1.0]], F)
    bias = np.array([[2.0**-24]], F)
    out = oracle.moe_finalize_routing(rows, np.array([0], np.int32), oracle.DT_F32, bias=bias,
                                      scales=np.array([[3.0]], F), expert=np.array([[0]], np.int32))
    assert out[0, 0] == np.float32(3.0)


def test_moe_gating_top_k_softmax_hand_derived_and_against_fp64(oracle):
    # equal logits: every probability is exactly 1/4; ties go to the lower column; row_idx = j * rows + r
    x = np.zeros((3, 4), F)
    y, ei, ri = oracle.moe_gating_top_k_softmax(x, oracle.DT_F32, 2, finished=np.array([0, 1, 0], np.uint8))
    assert y.tolist() == [[0.25, 0.25]] * 3
    assert ei.tolist() == [[0, 1], [4, 4], [0, 1]]          # the finished row reports inner = 4
    assert ri.tolist() == [[0, 3], [1, 4], [2, 5]]
    # separated logits against an fp64 softmax: same columns, probabilities within 4 fp32 ulp
    rng = np.random.default_rng(21)
    x = rng.standard_normal((64, 256)).astype(F) * 3
    y, ei, _ = oracle.moe_gating_top_k_softmax(x, oracle.DT_F32, 8)
    p = np.exp(x.astype(np.float64) - x.max(1, keepdims=True).astype(np.float64))
    p /= p.sum(1, keepdims=True)
    order = np.argsort(-p, axis=1, kind="stable")[:, :8]
    assert np.array_equal(ei, order)
    want = np.take_along_axis(p, order, 1)
    assert np.abs(y - want).max() <= 4 * np.spacing(want.astype(F)).max()
    # 16-bit inputs: probabilities are rounded to the input type
    xb = oracle.f32_to_bf16_bits(x)
    yb, eib, _ = oracle.moe_gating_top_k_softmax(xb, oracle.DT_BF16, 4)
    xf = oracle.bf16_bits_to_f32(xb).astype(np.float64)
    pb = np.exp(xf - xf.max(1, keepdims=True))
    pb /= pb.sum(1, keepdims=True)
    got = oracle.bf16_bits_to_f32(yb)
    want = np.take_along_axis(pb, eib.astype(np.int64), 1)
    assert np.abs(got - want).max() <= 2.0**-8 * want.max()
    with pytest.raises(ValueError):
        oracle.moe_gating_top_k_softmax(x, oracle.DT_F32, 257)


def test_dequant_swiglu_quant_hand_derived(oracle):
    """One row, H = 2, int32 input.  x = [4, -8 | 0, 0] with unit weight scales and activation scale 0.5:
    a = [2, -4], b = [0, 0].  activate_left = 0 gates on b: out = (a*b)/(1+exp(0)) = [0, -0] -> scale clamps to
    1e-12, y = 0.  activate_left = 1 gates on a with b = [1, 1] (x = [4, -8 | 2, 2]):
    out = a*b/(1+exp(-a)) = [2/(1+e^-2), -4/(1+e^4)]."""
    x = np.array([[4, -8, 0, 0]], np.int32)
    ws = np.ones(4, F)
    a_s = np.array([0.5], F)
    y, s = oracle.dequant_swiglu_quant(x, oracle.DT_I32, weight_scale=ws, activation_scale=a_s)
    assert y.tolist() == [[0, 0]] and s[0] == np.float32(1e-12)
    x = np.array([[4, -8, 2, 2]], np.int32)
    y, s, out = oracle.dequant_swiglu_quant(x, oracle.DT_I32, weight_scale=ws, activation_scale=a_s,
                                            activate_left=True, want_out=True)
    want = np.array([2.0 / (1.0 + np.exp(-2.0)), -4.0 / (1.0 + np.exp(4.0))])
    assert np.abs(out[0] - want).max() < 1e-6
    assert abs(s[0] - want[0] / 127.0) < 1e-8 and y[0, 0] == 127 and y[0, 1] == round(want[1] / (want[0] / 127.0))
    # quant_scale multiplies the half that is not the gate input: gating on a, it scales b
    y2, s2, out2 = oracle.dequant_swiglu_quant(x, oracle.DT_I32, weight_scale=ws, activation_scale=a_s,
                                               quant_scale=np.array([2.0, 0.5], F), activate_left=True,
                                               want_out=True)
    assert np.allclose(out2[0], want * np.array([2.0, 0.5]), rtol=1e-6)
    # 16-bit input takes no scales; activate_left = 0 gates on the right half
    xb = oracle.f32_to_bf16_bits(np.array([[3.0, 1.0, 2.0, -1.0]], F))
    _, _, out3 = oracle.dequant_swiglu_quant(xb, oracle.DT_BF16, want_out=True)
    want3 = np.array([3.0 * 2.0 / (1.0 + np.exp(-2.0)), 1.0 * -1.0 / (1.0 + np.exp(1.0))])
    assert np.abs(out3[0] - want3).max() < 1e-6
    with pytest.raises(ValueError):
        oracle.dequant_swiglu_quant(xb, oracle.DT_BF16, weight_scale=ws)
    with pytest.raises(ValueError):
        oracle.dequant_swiglu_quant(x, oracle.DT_I32, weight_scale=ws)


# ---------------------------------------------------------------------------
# The operators either side of the path against the independent numpy restatement (tests/golden/make_golden.py)
# ---------------------------------------------------------------------------
def _dt(oracle, kind):
    return {"bf16": oracle.DT_BF16, "f16": oracle.DT_F16, "f32": oracle.DT_F32, "i32": oracle.DT_I32}[kind]


def _same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.dtype == b.dtype and a.shape == b.shape and a.tobytes() == b.tobytes()


def test_moe_re_routing_golden(oracle, golden):
    g = golden
    out, out_s, idx, num = oracle.moe_re_routing(g["mrr_tokens"], g["mrr_counts"], g["mrr_scales"])
    total = int(g["mrr_counts"].sum())
    assert _same_bits(out[:total], g["mrr_out"]) and _same_bits(out_s[:total], g["mrr_out_scales"])
    assert _same_bits(idx[:total], g["mrr_idx"]) and _same_bits(num, g["mrr_num"])


@pytest.mark.parametrize("kind", ["bf16", "f16", "f32"])
def test_moe_finalize_routing_golden(oracle, golden, kind):
    g, dt = golden, _dt(oracle, kind)
    p = f"mfr_{kind}_"
    full = oracle.moe_finalize_routing(g[p + "rows"], g[p + "esdr"], dt, skip1=g[p + "skip1"], skip2=g[p + "skip2"],
                                       bias=g[p + "bias"], scales=g[p + "scales"], expert=g[p + "expert"],
                                       drop_pad_mode=0)
    assert _same_bits(full, g[p + "out_mode0"])
    rowwise = oracle.moe_finalize_routing(g[p + "rows"], g[p + "esdr"], dt, skip1=g[p + "skip1"],
                                          scales=g[p + "scales"], drop_pad_mode=2)
    assert _same_bits(rowwise, g[p + "out_mode2"])
    r = g[p + "scales"].shape[0]
    plain = oracle.moe_finalize_routing(g[p + "rows"], g[p + "esdr"][:r], dt)
    assert _same_bits(plain, g[p + "out_plain"])


@pytest.mark.parametrize("kind", ["bf16", "f16", "f32"])
def test_moe_gating_golden(oracle, golden, kind):
    g, dt = golden, _dt(oracle, kind)
    y, ei, ri = oracle.moe_gating_top_k_softmax(g[f"gate_{kind}_x"], dt, 8, finished=g[f"gate_{kind}_finished"])
    assert _same_bits(y, g[f"gate_{kind}_y"])
    assert _same_bits(ei, g[f"gate_{kind}_idx"]) and _same_bits(ri, g[f"gate_{kind}_row_idx"])
    # the tie in row 1 resolves to ascending columns, the all-equal row 2 is finished (index = row length)
    assert (ei[2] == 70).all()


def test_moe_gating_golden_k_equals_row_length(oracle, golden):
    g = golden
    y, ei, ri = oracle.moe_gating_top_k_softmax(g["gate_small_x"], oracle.DT_F32, 5)
    assert _same_bits(y, g["gate_small_y"]) and _same_bits(ei, g["gate_small_idx"])
    assert _same_bits(ri, g["gate_small_row_idx"])


@pytest.mark.parametrize("tag,kind", [("dqsq_i32_short", "i32"), ("dqsq_i32_long", "i32"), ("dqsq_bf16_short", "bf16"),
                                      ("dqsq_f16_long", "f16")])
def test_dequant_swiglu_quant_golden(oracle, golden, tag, kind):
    """Both scaling forms (division for short rows, reciprocal for long ones), both gate sides, with and without
    the smooth scale, both rounding modes."""
    g, dt = golden, _dt(oracle, kind)
    ws = g[tag + "_ws"] if kind == "i32" else None
    a_s = g[tag + "_as"] if kind == "i32" else None
    for left in (0, 1):
        y, s, act = oracle.dequant_swiglu_quant(g[tag + "_x"], dt, weight_scale=ws, activation_scale=a_s,
                                                quant_scale=g[tag + "_qs"], activate_left=bool(left), want_out=True)
        want_act = g[f"{tag}_act_left{left}"]
        nan = np.isnan(want_act)
        assert np.array_equal(np.isnan(act), nan)
        assert np.array_equal(act.view(np.uint32)[~nan], want_act.view(np.uint32)[~nan])
        assert _same_bits(y, g[f"{tag}_y_left{left}"]) and _same_bits(s, g[f"{tag}_scale_left{left}"])
    y, s = oracle.dequant_swiglu_quant(g[tag + "_x"], dt, weight_scale=ws, activation_scale=a_s, activate_left=True,
                                       round_mode=oracle.ROUND_DIRECT)
    assert _same_bits(y, g[tag + "_y_noq_direct"]) and _same_bits(s, g[tag + "_scale_noq"])
