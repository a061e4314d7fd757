"""Seeded random sweep of the grouped operators against the oracle: expert counts, group sizes around every tile
boundary (0, 1, 127-130, 255-257, 383-385, 511-513 rows, sometimes one large group so that the two-launch form
runs), K, N, both weight layouts, host and device group lists.  Bit-exact int8 / scale / bf16 comparison."""
import numpy as np
import pytest
import torch

from helpers import bits

pytestmark = pytest.mark.gpu

@pytest.fixture
def force_shape():
    """Forces a kernel shape for the duration of a test ("auto" = the library's own choice)."""
    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()

    def _set(shape, epilogue_warps=16, fused_requant=0):
        assert lib.w8a8_set_gemm_shape(0 if shape == "auto" else int(shape)) >= 0
        assert lib.w8a8_set_gmsq_epilogue_warps(epilogue_warps) in (8, 16)
        lib.w8a8_set_gmsq_fused_requant(fused_requant)

    yield _set
    lib.w8a8_set_gemm_shape(0)
    lib.w8a8_set_gmsq_epilogue_warps(16)
    lib.w8a8_set_gmsq_fused_requant(0)


SPECIAL = [0, 0, 1, 2, 7, 63, 64, 65, 127, 128, 129, 130, 200, 255, 256, 257, 300, 383, 384, 385, 511, 512, 513, 700]


@pytest.mark.parametrize("shape", ["auto", "1", "2", "3"])
@pytest.mark.parametrize("seed", [11, 12])
def test_random_grouped_problems_match_the_oracle(ops, oracle, force_shape, shape, seed):
    # the second seed also runs the SwiGLU kernels' other forms: eight epilogue warps, requantisation in the kernel
    force_shape(shape, epilogue_warps=16 if seed == 11 else 8, fused_requant=0 if seed == 11 else 1)
    rng = np.random.default_rng(seed)
    for case in range(12):
        e = int(rng.integers(1, 24))
        counts = np.array([SPECIAL[rng.integers(0, len(SPECIAL))] for _ in range(e)])
        if rng.random() < 0.3:
            counts[rng.integers(0, e)] += int(rng.integers(1000, 3000))
        if counts.sum() == 0:
            counts[0] = 5
        m = int(counts.sum())
        gl = np.cumsum(counts).tolist()
        k = int(rng.integers(1, 17)) * 16
        n = int(rng.integers(1, 13)) * 32
        nk = bool(rng.integers(0, 2))
        x = torch.from_numpy(rng.integers(-127, 128, (m, k)).astype(np.int8)).cuda()
        w_kn = rng.integers(-127, 128, (e, k, n)).astype(np.int8)
        w = torch.from_numpy(np.ascontiguousarray(w_kn.transpose(0, 2, 1)) if nk else w_kn).cuda()
        ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(np.float32)).cuda()
        xs = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(np.float32)).cuda()
        glarg = torch.tensor(gl, dtype=torch.int64, device="cuda") if rng.integers(0, 2) else gl
        what = f"case {case}: counts {counts.tolist()} k {k} n {n} nk {nk}"
        y, ysc = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, glarg, transpose_weight=nk)
        wy, wsc = oracle.grouped_matmul_swiglu_quant(x.cpu().numpy(), w_kn, ws.cpu().numpy(), xs.cpu().numpy(), gl)
        assert np.array_equal(y.cpu().numpy(), wy), what
        assert ysc.cpu().numpy().tobytes() == wsc.tobytes(), what
        k2, n2 = n // 2, int(rng.integers(1, 9)) * 32
        w2_kn = rng.integers(-127, 128, (e, k2, n2)).astype(np.int8)
        ws2 = rng.uniform(1e-3, 1e-2, (e, n2)).astype(np.float32)
        out = ops.grouped_matmul(y, torch.from_numpy(w2_kn).cuda(), glarg, None, 3, False, x_scale=ysc,
                                 weight_scale=torch.from_numpy(ws2).cuda())[0]
        want = oracle.grouped_matmul(wy, w2_kn, gl, dtype=oracle.DT_I8, x_scale=wsc, w_scale=ws2,
                                     out_dtype=oracle.DT_BF16)
        assert np.array_equal(bits(out), want), what


@pytest.mark.parametrize("shape", ["auto", "1", "2"])
def test_random_quant_matmul_epilogues_match_the_oracle(ops, oracle, force_shape, shape):
    """Random M (1 .. 700, around the 128 / 256 tile edges), K, N, weight layout and every combination of the
    epilogue's optional terms: scale scalar / per channel, fp32 / bf16; offset none / scalar / per channel;
    per-token scale; bias none / int32 / fp16 / bf16 / fp32, scalar or per channel; fp16 or bf16 output."""
    force_shape(shape)
    O = oracle
    rng = np.random.default_rng(21)
    rows = [1, 3, 16, 64, 127, 128, 129, 255, 256, 257, 300, 511, 513, 700]
    for case in range(30):
        m = rows[rng.integers(0, len(rows))]
        k = int(rng.integers(1, 17)) * 16
        n = int(rng.integers(1, 25)) * 16
        nk = bool(rng.integers(0, 2))
        x1 = rng.integers(-127, 128, (m, k)).astype(np.int8)
        w = rng.integers(-127, 128, (k, n)).astype(np.int8)
        flags, kw, okw = 0, {}, {}
        perchan = bool(rng.integers(0, 2))
        sc = rng.uniform(1e-3, 1e-2, n if perchan else 1).astype(np.float32)
        flags |= O.QM_SCALE_PERCHAN if perchan else 0
        if rng.integers(0, 2):
            sc_t = torch.from_numpy(sc).to(torch.bfloat16).cuda()
            flags |= O.QM_SCALE_BF16
            sc_o = bits(sc_t)
        else:
            sc_t, sc_o = torch.from_numpy(sc).cuda(), sc
        off_kind = int(rng.integers(0, 3))
        if off_kind:
            off = rng.standard_normal(n if off_kind == 2 else 1).astype(np.float32)
            kw["offset"], okw["offset"] = torch.from_numpy(off).cuda(), off
            flags |= O.QM_HAS_OFFSET | (O.QM_OFFSET_PERCHAN if off_kind == 2 else 0)
        if rng.integers(0, 2):
            pt = rng.uniform(1e-3, 5e-2, m).astype(np.float32)
            kw["pertoken_scale"], okw["pertoken"] = torch.from_numpy(pt).cuda(), pt
            flags |= O.QM_HAS_PT
        bias_kind = int(rng.integers(0, 5))
        if bias_kind:
            bn = n if rng.integers(0, 2) else 1
            if bias_kind == O.QM_BIAS_I32:
                b = rng.integers(-50000, 50000, bn).astype(np.int32)
                bt, bo = torch.from_numpy(b).cuda(), b
            elif bias_kind == O.QM_BIAS_F32:
                b = rng.standard_normal(bn).astype(np.float32)
                bt, bo = torch.from_numpy(b).cuda(), b
            else:
                dt = torch.float16 if bias_kind == O.QM_BIAS_F16 else torch.bfloat16
                bt = torch.from_numpy(rng.standard_normal(bn).astype(np.float32)).to(dt).cuda()
                bo = bits(bt)
            kw["bias"], okw["bias"] = bt, bo
            flags |= (bias_kind << O.QM_BIAS_SHIFT) | (O.QM_BIAS_PERCHAN if bn > 1 else 0)
        out_bf = bool(rng.integers(0, 2))
        x2 = torch.from_numpy(np.ascontiguousarray(w.T) if nk else w).cuda()
        got = ops.quant_matmul(torch.from_numpy(x1).cuda(), x2, sc_t, output_dtype="bfloat16" if out_bf else None,
                               transpose_x2=nk, **kw)
        want = O.quant_matmul(x1, w, sc_o, flags=flags, out_dtype=O.DT_BF16 if out_bf else O.DT_F16, **okw)
        assert np.array_equal(bits(got), want), f"case {case}: m {m} k {k} n {n} nk {nk} flags {flags:#x}"
