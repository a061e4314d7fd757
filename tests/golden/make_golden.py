"""Generates tests/golden/golden.npz: small seeded inputs with expected outputs.

The reference catalog ships no golden vectors and cannot run outside the
Ascend toolchain, so these vectors come from an INDEPENDENT restatement of the
reference formulas in numpy float32 arithmetic (this file), written separately
from the C oracle.  They pin the oracle (and through it the CUDA kernels)
against regressions and against transcription mistakes that the two
restatements do not share.

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import os

import numpy as np

F = np.float32
HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=F).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_f32(b):
    return (b.astype(np.uint32) << 16).view(F)


def to_bits(a, kind):
    if kind == "bf16":
        return bf16_round(a)
    with np.errstate(over="ignore"):
        return np.asarray(a, dtype=F).astype(np.float16).view(np.uint16)


def from_bits(b, kind):
    return bf16_f32(b) if kind == "bf16" else b.view(np.float16).astype(F)


def narrow(v, direct=False):
    """fp32 -> (fp16 ->) int8, round half even, saturate, NaN -> 0."""
    v = np.asarray(v, dtype=F)
    if not direct:
        with np.errstate(over="ignore"):
            v = v.astype(np.float16).astype(F)
    r = np.rint(v)
    r = np.where(np.isnan(r), F(0), r)
    return np.clip(r, -128, 127).astype(np.int8)


def nanmax_propagating(a, axis=-1):
    return np.max(a, axis=axis)  # numpy max propagates NaN


def dq(xb, kind, direct=False):
    x = from_bits(xb, kind)
    amax = nanmax_propagating(np.abs(x))
    amax = np.where(amax < F(1e-12), F(1e-12), amax).astype(F)
    scale = (amax * F(1.0 / 127.0)).astype(F)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = ((F(1.0) / amax).astype(F) * F(127.0)).astype(F)
        v = (x * inv[:, None]).astype(F)
    return narrow(v, direct), scale


def ardq(x1b, x2b, gb, eps, kind, direct=False):
    x1, x2, g = from_bits(x1b, kind), from_bits(x2b, kind), from_bits(gb, kind)
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        xo = (x1 + x2).astype(F)
        xout = to_bits(xo, kind)
        z = (xo * g[None, :]).astype(F)
        ssum = np.sum(xo.astype(np.float64) ** 2, axis=-1).astype(F)  # fp64 sequential-equivalent
        n = xo.shape[-1]
        mean = (ssum * F(F(1.0) / F(n))).astype(F)
        rms = np.sqrt((mean + F(eps)).astype(F)).astype(F)
        maxabs = nanmax_propagating(np.abs(z))
        rstd = (F(1.0) / rms).astype(F)
        m = (maxabs * rstd).astype(F)
        sm = np.where(m < F(1e-12), F(1e-12), m).astype(F)
        sc = (sm * F(1.0 / 127.0)).astype(F)
        k = (rstd / sc).astype(F)
        v = (z * k[:, None]).astype(F)
    return narrow(v, direct), xout, sc


def qmm(x1, x2, scale, offset, pertoken, bias, bias_kind, out_kind):
    acc = x1.astype(np.int64) @ x2.astype(np.int64)
    assert np.abs(acc).max() < 2**31
    v = acc.astype(np.int32).astype(F)
    if bias_kind == "i32":
        v = (v + bias.astype(F)).astype(F)
    v = (v * scale.astype(F)).astype(F)
    if offset is not None:
        v = (v + offset).astype(F)
    if pertoken is not None:
        v = (v * pertoken[:, None]).astype(F)
    if bias_kind in ("f32", "bf16", "f16"):
        v = (v + bias.astype(F)).astype(F)
    return to_bits(v, out_kind), acc.astype(np.int32)


def gmsq(x, w, ws, xs, gl, direct=False):
    m, k = x.shape
    e, _, n = w.shape
    h = n // 2
    y = np.zeros((m, h), np.int8)
    ysc = np.zeros((m,), F)
    act_all = np.zeros((m, h), F)
    start = 0
    for g in range(e):
        end = int(gl[g])
        if end > start:
            acc = (x[start:end].astype(np.int64) @ w[g].astype(np.int64)).astype(np.int32).astype(F)
            d = ((acc * xs[start:end, None]).astype(F) * ws[g][None, :]).astype(F)
            l, u = d[:, :h], d[:, h:]
            ex = np.exp(-(l.astype(np.float64))).astype(F)  # correctly rounded fp32 exp
            silu = (l / (ex + F(1.0)).astype(F)).astype(F)
            act = (silu * u).astype(F)
            act_all[start:end] = act
            amax = np.max(np.abs(act), axis=-1)
            amax = np.where(amax > F(1.1754944e-38), amax, F(1.1754944e-38)).astype(F)
            ysc[start:end] = (amax * F(1.0 / 127.0)).astype(F)
            inv = (F(127.0) / amax).astype(F)
            v = np.clip((act * inv[:, None]).astype(F), F(-128), F(127))
            y[start:end] = narrow(v, direct)
        start = end
    return y, ysc, act_all


def gmm_i8(x, w, ws, xs, gl, bias):
    m, k = x.shape
    e, _, n = w.shape
    out = np.zeros((m, n), np.uint16)
    start = 0
    for g in range(e):
        end = int(gl[g])
        if end > start:
            acc = (x[start:end].astype(np.int64) @ w[g].astype(np.int64)).astype(np.int32).astype(F)
            v = ((acc * ws[g][None, :]).astype(F) * xs[start:end, None]).astype(F)
            if bias is not None:
                v = (v + bias[g][None, :]).astype(F)
            out[start:end] = to_bits(v, "bf16")
        start = end
    return out


# ---------------------------------------------------------------------------
# The four operators either side of the path.  exp is the project's fixed
# fp32 exp (range reduction by ln2 in two pieces, degree-5 polynomial, two-step
# scaling); here it is restated with each fused multiply-add evaluated in
# float64 and rounded once to float32 (a 24 x 24 bit product is exact in
# float64, and the sum is then rounded to 53 bits before the final rounding: a
# double rounding that could only show on a near-tie of the 53-bit sum).
# ---------------------------------------------------------------------------
def fma32(a, b, c):
    return (np.asarray(a, F).astype(np.float64) * np.asarray(b, F).astype(np.float64)
            + np.asarray(c, F).astype(np.float64)).astype(F)


def canon_exp(x):
    x = np.asarray(x, F)
    nan = np.isnan(x)
    t = np.clip(np.where(nan, F(0), x), F(-104.0), F(89.0)).astype(F)
    n = np.rint((t * F(1.44269504088896341)).astype(F)).astype(F)
    r = fma32(n, F(-0.693359375), t)
    r = fma32(n, F(2.12194440e-4), r)
    p = np.full_like(r, F(1.9875691500e-4))
    for c in (1.3981999507e-3, 8.3334519073e-3, 4.1665795894e-2, 1.6666665459e-1, 5.0000001201e-1):
        p = fma32(p, r, F(c))
    e = (fma32(p, (r * r).astype(F), r) + F(1.0)).astype(F)
    ni = n.astype(np.int64)
    n1 = ni >> 1
    n2 = ni - n1
    s1 = ((n1 + 127).astype(np.uint32) << np.uint32(23)).view(F)
    s2 = ((n2 + 127).astype(np.uint32) << np.uint32(23)).view(F)
    out = ((e * s1).astype(F) * s2).astype(F)
    return np.where(nan, x, out).astype(F)


def mrr(tokens, counts, scales):
    """Rank-major / expert-minor rows -> expert-major rows (the layout after an expert-parallel all-to-all)."""
    n, e = counts.shape
    a = tokens.shape[0]
    # source order: for rank i, for expert j; destination order: for expert j, for rank i
    src_start = np.zeros((n, e), np.int64)
    run = 0
    for i in range(n):
        for j in range(e):
            src_start[i, j] = run
            run += counts[i, j]
    out = np.zeros_like(tokens)
    out_s = np.zeros((a,), F)
    idx = np.zeros((a,), np.int32)
    d = 0
    for j in range(e):
        for i in range(n):
            c = int(counts[i, j])
            s = int(src_start[i, j])
            out[d:d + c] = tokens[s:s + c]
            if scales is not None:
                out_s[d:d + c] = scales[s:s + c]
            idx[d:d + c] = np.arange(s, s + c)
            d += c
    return out, out_s, idx, counts.sum(axis=0).astype(np.int64)


def mfr(rows_b, kind, esdr, skip1_b, skip2_b, bias_b, scales, expert, mode):
    """out[i] = skip1[i] + skip2[i] + sum_k (rows[p(i,k)] + bias[expert[i,k]]) * scales[i,k], fp32, ascending k."""
    conv = (lambda b: b.astype(F)) if kind == "f32" else (lambda b: from_bits(b, kind))
    rows = conv(rows_b)
    num_dst, h = rows.shape
    kk = 1 if scales is None else scales.shape[1]
    r = esdr.size // kk
    acc = np.zeros((r, h), F)
    if skip1_b is not None:
        acc = conv(skip1_b).copy()
    if skip2_b is not None:
        acc = (acc + conv(skip2_b)).astype(F)
    for i in range(r):
        for k in range(kk):
            p = int(esdr[k * r + i] if mode <= 1 else esdr[i * kk + k])
            if p < 0 or p >= num_dst:
                continue
            term = rows[p].copy()
            if bias_b is not None and expert is not None:
                eid = int(expert[i, k])
                if 0 <= eid < bias_b.shape[0]:
                    term = (term + conv(bias_b)[eid]).astype(F)
            if scales is not None:
                term = (term * F(scales[i, k])).astype(F)
            acc[i] = (acc[i] + term).astype(F)
    return acc if kind == "f32" else to_bits(acc, kind)


def gating(xb, kind, k, finished):
    x = xb.astype(F) if kind == "f32" else from_bits(xb, kind)
    rows, inner = x.shape
    e = canon_exp((x - np.max(x, axis=1, keepdims=True)).astype(F))
    # the row sum in the project's fixed order: 32 lanes, lane t adds columns t, t+32, ...; then a butterfly
    lanes = np.zeros((rows, 32), F)
    for c in range(inner):
        lanes[:, c & 31] = (lanes[:, c & 31] + e[:, c]).astype(F)
    for off in (16, 8, 4, 2, 1):
        lanes = (lanes + lanes[:, np.arange(32) ^ off]).astype(F)
    total = lanes[:, 0]
    # stable sort of (-value, column): equal probabilities keep ascending column order
    order = np.argsort(-e, axis=1, kind="stable")[:, :k]
    top = np.take_along_axis(e, order, axis=1)
    y = (top / total[:, None]).astype(F)
    idx = order.astype(np.int32)
    if finished is not None:
        idx = np.where(finished[:, None] != 0, np.int32(inner), idx).astype(np.int32)
    row_idx = (np.arange(k, dtype=np.int64)[None, :] * rows + np.arange(rows, dtype=np.int64)[:, None]).astype(np.int32)
    return (y if kind == "f32" else to_bits(y, kind)), idx, row_idx


def dqsq(x, kind, wscale, ascale, qscale, activate_left, direct=False):
    m, n2 = x.shape
    h = n2 // 2
    if kind == "i32":
        a = (x[:, :h].astype(F) * wscale[None, :h]).astype(F)
        b = (x[:, h:].astype(F) * wscale[None, h:]).astype(F)
    else:
        v = from_bits(x, kind)
        a, b = v[:, :h].copy(), v[:, h:].copy()
    if qscale is not None:
        if activate_left:
            b = (b * qscale[None, :]).astype(F)
        else:
            a = (a * qscale[None, :]).astype(F)
    if kind == "i32":
        a = (a * ascale[:, None]).astype(F)
        b = (b * ascale[:, None]).astype(F)
    gate = a if activate_left else b
    den = (canon_exp((gate * F(-1.0)).astype(F)) + F(1.0)).astype(F)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        out = ((a * b).astype(F) / den).astype(F)
        mx = np.fmax.reduce(np.abs(out), axis=1, initial=F(0))  # NaN ignored, as fmaxf does
        s = np.maximum((mx * F(1.0 / 127.0)).astype(F), F(1e-12)).astype(F)
        pad = 8 if kind == "i32" else 16
        if -(-h // pad) * pad <= 1984:
            q = (out / s[:, None]).astype(F)
        else:
            q = (out * (F(1.0) / s).astype(F)[:, None]).astype(F)
    y = narrow(np.clip(q, F(-128), F(127)), direct)
    y = np.where(np.isnan(q), np.int8(0), y).astype(np.int8)
    return y, s, out


def main():
    rng = np.random.default_rng(20260101)
    out = {}

    # ---- DynamicQuant -----------------------------------------------------
    for kind in ("bf16", "f16"):
        x = rng.standard_normal((8, 40)).astype(F)
        x[1] = 0.0                       # all-zero row -> scale 1e-12/127
        x[2, :] = np.linspace(-2, 2, 40)  # regular ramp (ties after scaling)
        x[3, 5] = np.inf                 # inf row -> zeros, scale inf
        x[4, 7] = np.nan                 # NaN row -> zeros, scale NaN
        x[5] *= 1e-20                    # below the 1e-12 clamp
        x[6] *= 3e4                      # large magnitudes
        xb = to_bits(x, kind)
        y, s = dq(xb, kind)
        yd, _ = dq(xb, kind, direct=True)
        out[f"dq_{kind}_x"] = xb
        out[f"dq_{kind}_y"] = y
        out[f"dq_{kind}_y_direct"] = yd
        out[f"dq_{kind}_scale"] = s

    # ---- AddRmsNormDynamicQuant --------------------------------------------
    for kind in ("bf16", "f16"):
        x1 = rng.standard_normal((6, 72)).astype(F)
        x2 = rng.standard_normal((6, 72)).astype(F)
        g = (1.0 + 0.1 * rng.standard_normal(72)).astype(F)
        x1[1] = 0.0
        x2[1] = 0.0                      # all-zero row -> scale 1e-12/127, y = 0
        x1[2, 3] = np.inf                # inf row
        x2[3, 4] = np.nan                # NaN row
        x1b, x2b, gb = to_bits(x1, kind), to_bits(x2, kind), to_bits(g, kind)
        y, xo, sc = ardq(x1b, x2b, gb, 1e-6, kind)
        out[f"ardq_{kind}_x1"] = x1b
        out[f"ardq_{kind}_x2"] = x2b
        out[f"ardq_{kind}_gamma"] = gb
        out[f"ardq_{kind}_y"] = y
        out[f"ardq_{kind}_xout"] = xo
        out[f"ardq_{kind}_scale"] = sc

    # ---- QuantMatmul --------------------------------------------------------
    m, k, n = 5, 48, 32
    x1 = rng.integers(-127, 128, (m, k)).astype(np.int8)
    x2 = rng.integers(-127, 128, (k, n)).astype(np.int8)
    scale = rng.uniform(1e-3, 1e-2, n).astype(F)
    offset = rng.uniform(-1, 1, n).astype(F)
    pt = rng.uniform(1e-3, 5e-2, m).astype(F)
    bias_f = (0.02 * rng.standard_normal(n)).astype(F)
    bias_bf = bf16_f32(bf16_round(bias_f))
    bias_i = rng.integers(-1000, 1000, n).astype(np.int32)
    out["qm_x1"], out["qm_x2"], out["qm_scale"], out["qm_offset"], out["qm_pt"] = x1, x2, scale, offset, pt
    out["qm_bias_bf16"] = bf16_round(bias_f)
    out["qm_bias_i32"] = bias_i
    o1, acc = qmm(x1, x2, scale, None, pt, None, None, "bf16")
    out["qm_acc"] = acc
    out["qm_out_pt_bf16"] = o1
    out["qm_out_full_bf16"] = qmm(x1, x2, scale, offset, pt, bias_bf, "bf16", "bf16")[0]
    out["qm_out_i32bias_f16"] = qmm(x1, x2, scale, offset, None, bias_i, "i32", "f16")[0]
    out["qm_out_scalar_f16"] = qmm(x1, x2, scale[:1], None, None, None, None, "f16")[0]

    # ---- GroupedMatmulSwigluQuant -------------------------------------------
    m, k, n, e = 9, 32, 64, 4
    gl = np.array([3, 3, 8, 9], np.int64)  # expert 1 is empty, expert 3 has one row
    x = rng.integers(-127, 128, (m, k)).astype(np.int8)
    w = rng.integers(-127, 128, (e, k, n)).astype(np.int8)
    ws = rng.uniform(1e-3, 1e-2, (e, n)).astype(F)
    xs = rng.uniform(1e-3, 5e-2, m).astype(F)
    x[4] = 0  # all-zero row -> amax clamps to FLT_MIN
    y, ysc, act = gmsq(x, w, ws, xs, gl)
    out["gmsq_x"], out["gmsq_w"], out["gmsq_ws"], out["gmsq_xs"], out["gmsq_gl"] = x, w, ws, xs, gl
    out["gmsq_y"], out["gmsq_yscale"], out["gmsq_act"] = y, ysc, act

    # ---- GroupedMatmul int8 down projection ---------------------------------
    m, k, n, e = 9, 32, 48, 4
    x = rng.integers(-127, 128, (m, k)).astype(np.int8)
    w = rng.integers(-127, 128, (e, k, n)).astype(np.int8)
    ws = rng.uniform(1e-3, 1e-2, (e, n)).astype(F)
    xs = rng.uniform(1e-3, 5e-2, m).astype(F)
    out["gmm_x"], out["gmm_w"], out["gmm_ws"], out["gmm_xs"], out["gmm_gl"] = x, w, ws, xs, gl
    out["gmm_out"] = gmm_i8(x, w, ws, xs, gl, None)

    # ---- the operators either side of the path (their own generator: the arrays above stay as they were) ------
    rng = np.random.default_rng(20260202)

    # MoeReRouting: 3 ranks x 4 local experts, an empty cell, an empty expert column, spare rows at the end
    counts = np.array([[2, 0, 3, 0], [1, 4, 0, 0], [0, 2, 5, 0]], np.int64)
    a = int(counts.sum()) + 3
    tok = rng.integers(-128, 128, (a, 24)).astype(np.int8)
    scl = rng.random(a).astype(F)
    o, os_, idx, num = mrr(tok, counts, scl)
    total = int(counts.sum())
    out["mrr_tokens"], out["mrr_counts"], out["mrr_scales"] = tok, counts, scl
    out["mrr_out"], out["mrr_out_scales"], out["mrr_idx"], out["mrr_num"] = o[:total], os_[:total], idx[:total], num

    # MoeFinalizeRouting: every optional operand, both index layouts, dropped rows and out-of-range expert ids
    r, k, h, e = 7, 3, 40, 5
    for kind in ("bf16", "f16", "f32"):
        enc = (lambda v: v.astype(F)) if kind == "f32" else (lambda v, kind=kind: to_bits(v, kind))
        rows = enc(rng.standard_normal((r * k + 2, h)).astype(F))
        s1 = enc(rng.standard_normal((r, h)).astype(F))
        s2 = enc(rng.standard_normal((r, h)).astype(F))
        bias = enc(rng.standard_normal((e, h)).astype(F))
        scales = rng.random((r, k)).astype(F)
        esdr = rng.permutation(r * k).astype(np.int32)
        esdr[4] = -1               # dropped
        esdr[9] = r * k + 5        # past the rows: dropped
        expert = rng.integers(0, e, (r, k)).astype(np.int32)
        expert[2, 1] = e + 3       # bias dropped, term kept
        expert[5, 0] = -2
        out[f"mfr_{kind}_rows"], out[f"mfr_{kind}_skip1"], out[f"mfr_{kind}_skip2"] = rows, s1, s2
        out[f"mfr_{kind}_bias"], out[f"mfr_{kind}_scales"] = bias, scales
        out[f"mfr_{kind}_esdr"], out[f"mfr_{kind}_expert"] = esdr, expert
        out[f"mfr_{kind}_out_mode0"] = mfr(rows, kind, esdr, s1, s2, bias, scales, expert, 0)
        out[f"mfr_{kind}_out_mode2"] = mfr(rows, kind, esdr, s1, None, None, scales, None, 2)
        out[f"mfr_{kind}_out_plain"] = mfr(rows, kind, esdr[:r], None, None, None, None, None, 0)

    # MoeGatingTopKSoftmax: ties (repeated logits), a dominant logit, finished rows, k up to the row length
    for kind in ("bf16", "f16", "f32"):
        x = rng.standard_normal((6, 70)).astype(F)
        x[1, 10] = x[1, 3]          # equal values: the lower column comes first
        x[1, 50] = x[1, 3]
        x[2] = 0.25                 # every probability equal
        x[3, 7] = 60.0              # one expert takes nearly everything
        xb = x if kind == "f32" else to_bits(x, kind)
        fin = np.array([0, 0, 1, 0, 1, 0], np.uint8)
        y, ei, ri = gating(xb, kind, 8, fin)
        out[f"gate_{kind}_x"], out[f"gate_{kind}_finished"] = xb, fin
        out[f"gate_{kind}_y"], out[f"gate_{kind}_idx"], out[f"gate_{kind}_row_idx"] = y, ei, ri
    xs = rng.standard_normal((3, 5)).astype(F)
    y, ei, ri = gating(xs, "f32", 5, None)
    out["gate_small_x"], out["gate_small_y"], out["gate_small_idx"], out["gate_small_row_idx"] = xs, y, ei, ri

    # DequantSwigluQuant: int32 / 16-bit input, either gate side, smooth scale, the short-row (division) and
    # long-row (reciprocal) scaling forms, an all-zero row, a NaN element
    for name, h, kind in (("short", 48, "i32"), ("long", 2000, "i32"), ("short", 40, "bf16"), ("long", 1992, "f16")):
        m = 5
        tag = f"dqsq_{kind}_{name}"
        if kind == "i32":
            x = rng.integers(-300000, 300000, (m, 2 * h)).astype(np.int32)
            x[2] = 0
            ws = rng.uniform(1e-3, 1e-2, 2 * h).astype(F)
            a_s = rng.uniform(1e-3, 5e-2, m).astype(F)
        else:
            xv = (3.0 * rng.standard_normal((m, 2 * h))).astype(F)
            xv[2] = 0.0
            xv[3, 5] = np.nan
            x = to_bits(xv, kind)
            ws = a_s = None
        qs = rng.uniform(0.5, 1.5, h).astype(F)
        out[f"{tag}_x"], out[f"{tag}_qs"] = x, qs
        if ws is not None:
            out[f"{tag}_ws"], out[f"{tag}_as"] = ws, a_s
        for left in (0, 1):
            y, s, act = dqsq(x, kind, ws, a_s, qs, bool(left))
            out[f"{tag}_y_left{left}"], out[f"{tag}_scale_left{left}"], out[f"{tag}_act_left{left}"] = y, s, act
        y, s, _ = dqsq(x, kind, ws, a_s, None, True, direct=True)
        out[f"{tag}_y_noq_direct"], out[f"{tag}_scale_noq"] = y, s

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", os.path.join(HERE, "golden.npz"), "with", len(out), "arrays")


if __name__ == "__main__":
    main()
