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

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", os.path.join(HERE, "golden.npz"), "with", len(out), "arrays")


if __name__ == "__main__":
    main()
