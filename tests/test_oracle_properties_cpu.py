"""Property tests of the CPU oracle over generated shapes and values (hypothesis): the invariants every operator
of the path has to keep whatever the input, checked on the restatement the CUDA kernels are compared with."""
import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

F = np.float32
SET = dict(max_examples=40, deadline=None)


def _rows(draw, max_rows=12, max_cols=96):
    rows = draw(st.integers(1, max_rows))
    cols = draw(st.integers(1, max_cols))
    seed = draw(st.integers(0, 2**31 - 1))
    scale = draw(st.sampled_from([1e-6, 1e-2, 1.0, 300.0, 6e4]))
    return np.random.default_rng(seed).standard_normal((rows, cols)).astype(F) * F(scale)


@settings(**SET)
@given(st.data())
def test_dynamic_quant_invariants(oracle, data):
    x = _rows(data.draw)
    dt = data.draw(st.sampled_from([oracle.DT_BF16, oracle.DT_F16]))
    xb = oracle.f32_to_bits(x, dt)
    xf = oracle.bits_to_f32(xb, dt)
    finite = np.isfinite(xf).all(axis=1)
    y, s = oracle.dynamic_quant(xb, dt)
    assert np.abs(y.astype(np.int32)).max() <= 127
    amax = np.abs(xf).max(axis=1)
    want = np.maximum(amax, F(1e-12)) * F(1.0 / 127.0)
    assert np.array_equal(s[finite], want[finite])                       # scale = max(amax, 1e-12) * (1/127)
    big = finite & (amax > 1e-6)
    assert (np.abs(y[big]).max(axis=1) == 127).all()                     # the row maximum lands on +-127
    err = np.abs(y[big].astype(F) * s[big, None] - xf[big])
    assert (err <= s[big, None] * 0.54).all()                            # half a step + the fp16 grid
    # rows are independent: any row alone gives the same bytes
    r = data.draw(st.integers(0, x.shape[0] - 1))
    y1, s1 = oracle.dynamic_quant(xb[r:r + 1], dt)
    assert np.array_equal(y1[0], y[r]) and s1[0].tobytes() == s[r].tobytes()


@settings(**SET)
@given(st.data())
def test_add_rms_norm_dynamic_quant_invariants(oracle, data):
    x1 = _rows(data.draw)
    x2 = np.random.default_rng(data.draw(st.integers(0, 2**31 - 1))).standard_normal(x1.shape).astype(F)
    gamma = (1 + 0.1 * np.random.default_rng(1).standard_normal(x1.shape[1])).astype(F)
    dt = oracle.DT_BF16
    b1, b2, bg = (oracle.f32_to_bits(a, dt) for a in (x1, x2, gamma))
    y, x_out, s = oracle.add_rms_norm_dynamic_quant(b1, b2, bg, 1e-6, dt)
    # the residual output is the fp32 sum rounded once
    want_out = oracle.f32_to_bits(oracle.bits_to_f32(b1, dt) + oracle.bits_to_f32(b2, dt), dt)
    assert np.array_equal(x_out, want_out)
    assert np.abs(y.astype(np.int32)).max() <= 127 and (s > 0).all()
    # scaling both inputs by a power of two leaves the int8 result unchanged (the norm cancels it) unless eps bites
    big = np.abs(oracle.bits_to_f32(x_out, dt)).max(axis=1) > 1e-2
    y2, _, _ = oracle.add_rms_norm_dynamic_quant(oracle.f32_to_bits(oracle.bits_to_f32(b1, dt) * 4, dt),
                                                 oracle.f32_to_bits(oracle.bits_to_f32(b2, dt) * 4, dt), bg, 0.0, dt)
    y0, _, _ = oracle.add_rms_norm_dynamic_quant(b1, b2, bg, 0.0, dt)
    assert (np.abs(y2[big].astype(np.int32) - y0[big].astype(np.int32)) <= 1).all()


@settings(**SET)
@given(st.data())
def test_grouped_matmul_swiglu_quant_group_split_invariance(oracle, data):
    """One group of M rows equals any split of the same rows into groups that share the weights."""
    seed = data.draw(st.integers(0, 2**31 - 1))
    rng = np.random.default_rng(seed)
    m = data.draw(st.integers(1, 24))
    k, n = 32, 16
    x = rng.integers(-127, 128, (m, k)).astype(np.int8)
    w1 = rng.integers(-127, 128, (1, k, n)).astype(np.int8)
    ws1 = rng.uniform(1e-3, 1e-2, (1, n)).astype(F)
    xs = rng.uniform(1e-3, 5e-2, m).astype(F)
    cuts = sorted(data.draw(st.lists(st.integers(0, m), min_size=0, max_size=4)))
    ends = cuts + [m]
    e = len(ends)
    y_one, s_one = oracle.grouped_matmul_swiglu_quant(x, w1, ws1, xs, [m])
    y_split, s_split = oracle.grouped_matmul_swiglu_quant(x, np.repeat(w1, e, 0), np.repeat(ws1, e, 0), xs, ends)
    assert np.array_equal(y_one, y_split) and s_one.tobytes() == s_split.tobytes()
    assert np.abs(y_one.astype(np.int32)).max() <= 127


@settings(**SET)
@given(st.data())
def test_quant_matmul_is_linear_in_the_channel_scale(oracle, data):
    """Doubling the per-channel scale doubles every finite output exactly (a power of two commutes with every
    rounding of the epilogue), and the int32 accumulator does not depend on the epilogue at all."""
    rng = np.random.default_rng(data.draw(st.integers(0, 2**31 - 1)))
    m, k, n = data.draw(st.integers(1, 9)), 16 * data.draw(st.integers(1, 4)), 16 * data.draw(st.integers(1, 3))
    x1 = rng.integers(-127, 128, (m, k)).astype(np.int8)
    x2 = rng.integers(-127, 128, (k, n)).astype(np.int8)
    sc = rng.uniform(1e-3, 1e-2, n).astype(F)
    pt = rng.uniform(1e-3, 5e-2, m).astype(F)
    fl = oracle.QM_SCALE_PERCHAN | oracle.QM_HAS_PT
    a, acc_a = oracle.quant_matmul(x1, x2, sc, pertoken=pt, flags=fl, out_dtype=oracle.DT_BF16, want_acc=True)
    b, acc_b = oracle.quant_matmul(x1, x2, sc * 2, pertoken=pt, flags=fl, out_dtype=oracle.DT_BF16, want_acc=True)
    assert np.array_equal(acc_a, acc_b)
    assert np.array_equal(acc_a, x1.astype(np.int64) @ x2.astype(np.int64))
    assert np.array_equal(oracle.bf16_bits_to_f32(a) * 2, oracle.bf16_bits_to_f32(b))


@settings(**SET)
@given(st.data())
def test_moe_re_routing_is_a_permutation_and_finalize_inverts_it(oracle, data):
    rng = np.random.default_rng(data.draw(st.integers(0, 2**31 - 1)))
    n, e = data.draw(st.integers(1, 5)), data.draw(st.integers(1, 6))
    cnt = rng.integers(0, 4, (n, e))
    a = int(cnt.sum())
    if a == 0:
        cnt[0, 0] = 1
        a = 1
    tok = rng.standard_normal((a, 8)).astype(F)
    out, _, idx, num = oracle.moe_re_routing(tok, cnt)
    assert sorted(idx.tolist()) == list(range(a)) and np.array_equal(out, tok[idx])
    assert np.array_equal(num, cnt.sum(0))
    # MoeFinalizeRouting with K = 1, unit scales and the inverse index undoes the regroup
    inv = np.empty(a, np.int32)
    inv[idx] = np.arange(a, dtype=np.int32)
    back = oracle.moe_finalize_routing(out, inv, oracle.DT_F32)
    assert np.array_equal(back, tok)
