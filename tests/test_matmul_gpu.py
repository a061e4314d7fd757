"""GPU parity of the tensor-core operators through the C-ABI vs the CPU oracle:
raw int32 accumulators, quant_matmul, grouped_matmul_swiglu_quant and
grouped_matmul.  int32 accumulators and int8 outputs are bit-exact; 16-bit
float outputs of the int8 paths are bit-exact too (same fp32 chain, one
rounding); only the float grouped_matmul, whose accumulation order the
reference leaves to its matmul library, is compared with a tolerance."""

import numpy as np
import pytest
import torch

from helpers import assert_same_f32, bits, from_bits, seed_of, zipf_group_list

pytestmark = pytest.mark.gpu

F = np.float32


@pytest.fixture(autouse=True, params=["auto", "single", "pair", "hybrid"])
def cta_group(request):
    """Every test runs with the library's own choice of kernel shape, with single-CTA tiles forced, with CTA-pair
    (cta_group::2) tiles forced, and with the two-launch form of grouped problems forced (pairs on whole 256-row
    blocks, single CTAs on the leftovers; dense problems ignore it): all must give identical results."""
    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()
    prev = lib.w8a8_set_gemm_shape({"auto": 0, "single": 1, "pair": 2, "hybrid": 3}[request.param])
    assert prev >= 0
    yield request.param
    lib.w8a8_set_gemm_shape(0)


def _i8(rng, shape):
    return torch.from_numpy(rng.integers(-127, 128, shape).astype(np.int8)).cuda()


def _raw_matmul(x1, x2, layout_nk=False):
    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()
    batch = 1
    for d in x1.shape[:-2]:
        batch *= d
    m, k = x1.shape[-2], x1.shape[-1]
    n = x2.shape[-2] if layout_nk else x2.shape[-1]
    c = torch.full(tuple(x1.shape[:-1]) + (n,), -7, dtype=torch.int32, device="cuda")
    rc = lib.w8a8_matmul_i8_i32(x1.data_ptr(), x2.data_ptr(), c.data_ptr(), batch, m, n, k,
                                L.W_NK if layout_nk else L.W_KN, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.status_string(rc)
    torch.cuda.synchronize()
    return c


@pytest.mark.parametrize("layout_nk", [False, True])
@pytest.mark.parametrize("m,k,n", [(128, 128, 256), (128, 1024, 1024), (16, 7168, 512), (300, 1040, 400),
                                   (1, 16, 16), (129, 144, 272), (2048, 512, 768)])
def test_int32_accumulators_bit_exact(layout_nk, m, k, n):
    rng = np.random.default_rng(seed_of("acc", m, k, n))
    x1 = _i8(rng, (m, k))
    w = _i8(rng, (k, n))
    x2 = w.t().contiguous() if layout_nk else w
    c = _raw_matmul(x1, x2, layout_nk)
    ref = (x1.cpu().numpy().astype(np.int64) @ w.cpu().numpy().astype(np.int64)).astype(np.int32)
    got = c.cpu().numpy()
    bad = np.argwhere(got != ref)
    assert bad.size == 0, f"{len(bad)} of {ref.size} accumulators differ; first at {bad[:4].tolist()}: " \
                          f"got {got[tuple(bad[0])]}, want {ref[tuple(bad[0])]}"


def test_int32_accumulators_batched_and_extremes():
    rng = np.random.default_rng(11)
    x1 = _i8(rng, (3, 70, 256))
    x2 = _i8(rng, (3, 256, 144))
    c = _raw_matmul(x1, x2)
    ref = np.einsum("bmk,bkn->bmn", x1.cpu().numpy().astype(np.int64), x2.cpu().numpy().astype(np.int64))
    assert np.array_equal(c.cpu().numpy(), ref.astype(np.int32))
    # saturating magnitudes: all -128 x all -128 over K = 7168 stays exact in int32
    a = torch.full((128, 7168), -128, dtype=torch.int8, device="cuda")
    b = torch.full((7168, 256), -128, dtype=torch.int8, device="cuda")
    c = _raw_matmul(a, b)
    assert bool((c == 128 * 128 * 7168).all())


def _qm_oracle(oracle, x1, x2, scale, **kw):
    return oracle.quant_matmul(x1.cpu().numpy(), x2.cpu().numpy(), scale, **kw)


@pytest.mark.parametrize("layout_nk", [False, True])
@pytest.mark.parametrize("m,k,n,out", [(128, 1024, 1024, "bfloat16"), (16, 7168, 512, "bfloat16"),
                                       (200, 512, 272, None), (2048, 1024, 512, "bfloat16")])
def test_quant_matmul_pertoken_perchannel(ops, oracle, layout_nk, m, k, n, out):
    rng = np.random.default_rng(seed_of("qm", m, k, n))
    x1 = _i8(rng, (m, k))
    w = _i8(rng, (k, n))
    x2 = w.t().contiguous() if layout_nk else w
    scale = torch.from_numpy(rng.uniform(1e-3, 1e-2, n).astype(F)).cuda()
    pt = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(F)).cuda()
    got = ops.quant_matmul(x1, x2, scale, pertoken_scale=pt, output_dtype=out, transpose_x2=layout_nk)
    assert got.dtype == (torch.bfloat16 if out == "bfloat16" else torch.float16) and got.shape == (m, n)
    O = oracle
    ref = O.quant_matmul(x1.cpu().numpy(), w.cpu().numpy(), scale.cpu().numpy(), pertoken=pt.cpu().numpy(),
                         flags=O.QM_SCALE_PERCHAN | O.QM_HAS_PT,
                         out_dtype=O.DT_BF16 if out == "bfloat16" else O.DT_F16)
    assert np.array_equal(bits(got), ref)


def test_quant_matmul_every_epilogue_term(ops, oracle, golden):
    g = golden
    O = oracle
    x1 = torch.from_numpy(g["qm_x1"]).cuda()
    x2 = torch.from_numpy(g["qm_x2"]).cuda()
    scale = torch.from_numpy(g["qm_scale"]).cuda()
    offset = torch.from_numpy(g["qm_offset"]).cuda()
    pt = torch.from_numpy(g["qm_pt"]).cuda()
    bias_bf = from_bits(g["qm_bias_bf16"], torch.bfloat16)
    bias_i = torch.from_numpy(g["qm_bias_i32"]).cuda()
    assert np.array_equal(bits(ops.quant_matmul(x1, x2, scale, pertoken_scale=pt, output_dtype="bfloat16")),
                          g["qm_out_pt_bf16"])
    assert np.array_equal(bits(ops.quant_matmul(x1, x2, scale, offset=offset, pertoken_scale=pt, bias=bias_bf,
                                                output_dtype="bfloat16")), g["qm_out_full_bf16"])
    assert np.array_equal(bits(ops.quant_matmul(x1, x2, scale, offset=offset, bias=bias_i)), g["qm_out_i32bias_f16"])
    assert np.array_equal(bits(ops.quant_matmul(x1, x2, scale[:1].contiguous())), g["qm_out_scalar_f16"])
    # bf16 scale, scalar offset, scalar fp32 bias, fp16 bias
    rng = np.random.default_rng(12)
    sc_bf = torch.from_numpy(rng.uniform(1e-3, 1e-2, 32).astype(F)).to(torch.bfloat16).cuda()
    off1 = torch.tensor([0.125], dtype=torch.float32, device="cuda")
    b1 = torch.tensor([-0.5], dtype=torch.float32, device="cuda")
    got = ops.quant_matmul(x1, x2, sc_bf, offset=off1, bias=b1, output_dtype="bfloat16")
    fl = O.QM_SCALE_PERCHAN | O.QM_SCALE_BF16 | O.QM_HAS_OFFSET | (O.QM_BIAS_F32 << O.QM_BIAS_SHIFT)
    ref = O.quant_matmul(g["qm_x1"], g["qm_x2"], bits(sc_bf), offset=off1.cpu().numpy(), bias=b1.cpu().numpy(),
                         flags=fl, out_dtype=O.DT_BF16)
    assert np.array_equal(bits(got), ref)
    b16 = torch.from_numpy(rng.standard_normal(32).astype(F)).to(torch.float16).cuda()
    got = ops.quant_matmul(x1, x2, scale, bias=b16)
    fl = O.QM_SCALE_PERCHAN | (O.QM_BIAS_F16 << O.QM_BIAS_SHIFT) | O.QM_BIAS_PERCHAN
    ref = O.quant_matmul(g["qm_x1"], g["qm_x2"], g["qm_scale"], bias=bits(b16), flags=fl, out_dtype=O.DT_F16)
    assert np.array_equal(bits(got), ref)


def test_quant_matmul_batched(ops, oracle):
    O = oracle
    rng = np.random.default_rng(13)
    b, m, k, n = 3, 40, 128, 96
    x1, x2 = _i8(rng, (b, m, k)), _i8(rng, (b, k, n))
    scale = torch.from_numpy(rng.uniform(1e-3, 1e-2, n).astype(F)).cuda()
    pt = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(F)).cuda()
    bias = torch.from_numpy(rng.standard_normal((b, 1, n)).astype(F)).cuda()
    got = ops.quant_matmul(x1, x2, scale, pertoken_scale=pt, bias=bias, output_dtype="bfloat16")
    assert got.shape == (b, m, n)
    for i in range(b):  # a batched bias is one epilogue per batch in the reference
        fl = O.QM_SCALE_PERCHAN | O.QM_HAS_PT | (O.QM_BIAS_F32 << O.QM_BIAS_SHIFT) | O.QM_BIAS_PERCHAN
        ref = O.quant_matmul(x1[i].cpu().numpy(), x2[i].cpu().numpy(), scale.cpu().numpy(), pertoken=pt.cpu().numpy(),
                             bias=bias[i, 0].cpu().numpy().copy(), flags=fl, out_dtype=O.DT_BF16)
        assert np.array_equal(bits(got[i]), ref)


def test_cfg1_chain_dynamic_quant_then_quant_matmul(ops, oracle):
    """Benchmark configuration 1, seed 0: the GPU chain equals the CPU chain bit for bit."""
    O = oracle
    rng = np.random.default_rng(0)
    x = rng.standard_normal((128, 1024)).astype(F)
    w = rng.integers(-127, 128, (1024, 1024)).astype(np.int8)
    ws = rng.uniform(1e-3, 1e-2, 1024).astype(F)
    xq, xs = ops.dynamic_quant(torch.from_numpy(x).to(torch.bfloat16).cuda())
    out = ops.quant_matmul(xq, torch.from_numpy(w).cuda(), torch.from_numpy(ws).cuda(), pertoken_scale=xs,
                           output_dtype="bfloat16")
    xq_o, xs_o = O.dynamic_quant(O.f32_to_bf16_bits(x), O.DT_BF16)
    ref = O.quant_matmul(xq_o, w, ws, pertoken=xs_o, flags=O.QM_SCALE_PERCHAN | O.QM_HAS_PT, out_dtype=O.DT_BF16)
    assert np.array_equal(xq.cpu().numpy(), xq_o)
    assert np.array_equal(bits(out), ref)


def _gmsq_case(rng, m, k, n, e, gl):
    x = _i8(rng, (m, k))
    w = _i8(rng, (e, k, n))
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(F)).cuda()
    xs = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(F)).cuda()
    return x, w, ws, xs, [int(v) for v in gl]


@pytest.mark.parametrize("layout_nk", [False, True])
@pytest.mark.parametrize("m,k,n,e,gl", [
    (9, 32, 64, 4, [3, 3, 8, 9]),
    (300, 256, 512, 5, [0, 130, 130, 299, 300]),
    (513, 1024, 4096, 3, [128, 385, 513]),
    (260, 7168, 256, 2, [4, 260]),
    (64, 128, 96, 1, [64]),
])
def test_gmsq_matches_oracle(ops, oracle, layout_nk, m, k, n, e, gl):
    rng = np.random.default_rng(seed_of("gmsq", m, k, n, e))
    x, w, ws, xs, gl = _gmsq_case(rng, m, k, n, e, gl)
    wt = w.transpose(1, 2).contiguous() if layout_nk else w
    y, ysc = ops.grouped_matmul_swiglu_quant(x, wt, ws, xs, gl, transpose_weight=layout_nk)
    assert y.shape == (m, n // 2) and y.dtype == torch.int8 and ysc.shape == (m,)
    yo, yso = oracle.grouped_matmul_swiglu_quant(x.cpu().numpy(), w.cpu().numpy(), ws.cpu().numpy(), xs.cpu().numpy(),
                                                 gl)
    assert_same_f32(ysc, yso, "y_scale")
    d = y.cpu().numpy() != yo
    assert not d.any(), f"{d.sum()} of {d.size} int8 outputs differ"


def test_gmsq_golden_and_device_group_list(ops, oracle, golden):
    g = golden
    x, w = torch.from_numpy(g["gmsq_x"]).cuda(), torch.from_numpy(g["gmsq_w"]).cuda()
    ws, xs = torch.from_numpy(g["gmsq_ws"]).cuda(), torch.from_numpy(g["gmsq_xs"]).cuda()
    gl = [int(v) for v in g["gmsq_gl"]]
    y, ysc = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, gl)
    # golden used a correctly rounded exp; the canonical exp is allowed +-1 LSB on rare elements
    assert np.abs(y.cpu().numpy().astype(np.int32) - g["gmsq_y"].astype(np.int32)).max() <= 1
    assert np.allclose(ysc.cpu().numpy(), g["gmsq_yscale"], rtol=1e-6, atol=0)
    assert ysc[4].item() == F(1.1754944e-38) * F(1.0 / 127.0)  # all-zero row: FLT_MIN clamp
    # the same call with the list in device memory (validated on the device)
    gl_dev = torch.tensor(gl, dtype=torch.int64, device="cuda")
    y2, ysc2 = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, gl_dev)
    assert torch.equal(y, y2) and torch.equal(ysc, ysc2)
    # an invalid device list is reported through the workspace error word and writes nothing
    from cannbench_operator_solutions_b200 import _lib as L
    lib = L.load()
    need = lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(9, 32, 64, 4)
    wsb = torch.zeros((need,), dtype=torch.uint8, device="cuda")
    bad = torch.tensor([3, 2, 8, 9], dtype=torch.int64, device="cuda")
    y3 = torch.full_like(y, 55)
    ys3 = torch.zeros_like(ysc)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.w8a8_grouped_matmul_swiglu_quant(x.data_ptr(), w.data_ptr(), ws.data_ptr(), xs.data_ptr(), y3.data_ptr(),
                                              ys3.data_ptr(), 9, 32, 64, 4, bad.data_ptr(), 1, L.W_KN, 0,
                                              wsb.data_ptr(), need, st)
    assert rc == 0
    assert lib.w8a8_workspace_error(wsb.data_ptr(), st) == 1
    assert bool((y3 == 55).all())
    with pytest.raises(RuntimeError, match="cumsum"):
        ops.grouped_matmul_swiglu_quant(x, w, ws, xs, [3, 2, 8, 9])


def test_gmsq_zipf_groups_256_experts(ops, oracle):
    """Config-4-like skew (E = 256, Zipf 1.1, many experts below one tile, some empty) at a CPU-checkable size."""
    rng = np.random.default_rng(14)
    m, k, n, e = 2048, 512, 512, 256
    gl = zipf_group_list(rng, m, e)
    x, w, ws, xs, gl = _gmsq_case(rng, m, k, n, e, gl)
    y, ysc = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, gl)
    yo, yso = oracle.grouped_matmul_swiglu_quant(x.cpu().numpy(), w.cpu().numpy(), ws.cpu().numpy(), xs.cpu().numpy(),
                                                 gl)
    assert_same_f32(ysc, yso, "y_scale")
    assert np.array_equal(y.cpu().numpy(), yo)
    # group-split invariance on the device: same weights for every expert, two different splits
    w1 = w[:1].expand(e, k, n).contiguous()
    ws1 = ws[:1].expand(e, n).contiguous()
    ya, sa = ops.grouped_matmul_swiglu_quant(x, w1, ws1, xs, gl)
    yb, sb = ops.grouped_matmul_swiglu_quant(x, w1[:1].contiguous(), ws1[:1].contiguous(), xs, [m])
    assert torch.equal(ya, yb) and torch.equal(sa, sb)


@pytest.mark.parametrize("layout_nk", [False, True])
def test_grouped_matmul_int8_down_projection(ops, oracle, layout_nk):
    O = oracle
    rng = np.random.default_rng(15)
    m, k, n, e = 700, 2048, 1024, 6
    gl = [100, 100, 356, 357, 699, 700]
    x, w = _i8(rng, (m, k)), _i8(rng, (e, k, n))
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(F)).cuda()
    xs = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(F)).cuda()
    wt = w.transpose(1, 2).contiguous() if layout_nk else w
    outs = ops.grouped_matmul(x, wt, gl, None, 0, layout_nk, x_scale=xs, weight_scale=ws)
    assert len(outs) == e and [o.shape[0] for o in outs] == [100, 0, 256, 1, 342, 1]
    joined = ops.grouped_matmul(x, wt, gl, None, 3, layout_nk, x_scale=xs, weight_scale=ws)
    assert len(joined) == 1 and torch.equal(torch.cat(outs, 0), joined[0])
    ref = O.grouped_matmul(x.cpu().numpy(), w.cpu().numpy(), gl, dtype=O.DT_I8, x_scale=xs.cpu().numpy(),
                           w_scale=ws.cpu().numpy())
    assert np.array_equal(bits(joined[0]), ref)
    bias = torch.from_numpy(rng.standard_normal((e, n)).astype(F)).cuda()
    jb = ops.grouped_matmul(x, wt, gl, bias, 2, layout_nk, x_scale=xs, weight_scale=ws)[0]
    refb = O.grouped_matmul(x.cpu().numpy(), w.cpu().numpy(), gl, dtype=O.DT_I8, x_scale=xs.cpu().numpy(),
                            w_scale=ws.cpu().numpy(), bias=bias.cpu().numpy(), bias_dtype=O.DT_F32)
    assert np.array_equal(bits(jb), refb)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layout_nk", [False, True])
def test_grouped_matmul_float_path(ops, oracle, dtype, layout_nk):
    """The reference's own (float) grouped_matmul: fp32 accumulation in an order its matmul library does not
    document, so the comparison is against an fp64 product with a relative tolerance of 2^-7 of the row scale."""
    rng = np.random.default_rng(16)
    m, k, n, e = 260, 320, 272, 3
    gl = [130, 130, 260]
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(F)).to(dtype).cuda()
    w = torch.from_numpy((rng.standard_normal((e, k, n)) * 0.1).astype(F)).to(dtype).cuda()
    bias = torch.from_numpy(rng.standard_normal((e, n)).astype(F)).to(dtype).cuda()
    wt = w.transpose(1, 2).contiguous() if layout_nk else w
    out = ops.grouped_matmul(x, wt, gl, bias, 2, layout_nk)[0]
    assert out.dtype == dtype and out.shape == (m, n)
    xf, wf, bf = x.double().cpu(), w.double().cpu(), bias.double().cpu()
    ref = torch.empty((m, n), dtype=torch.float64)
    ref[:130] = xf[:130] @ wf[0] + bf[0]
    ref[130:] = xf[130:] @ wf[2] + bf[2]
    err = (out.double().cpu() - ref).abs().max().item()
    assert err <= ref.abs().max().item() * 2.0**-7, err


def test_gmsq_fused_and_two_kernel_requantisation_agree(ops, oracle, cta_group):
    """The requantisation runs as a second kernel over the stored activations by default, inside the matmul kernels
    when switched on (the CTA that finishes the last column tile of a row block quantises it), and as a call of
    its own when the caller runs the operator's two stages separately: all forms give the oracle's bits."""
    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()
    rng = np.random.default_rng(31)
    counts = [700, 0, 129, 5, 256, 300, 1, 127]
    gl = np.cumsum(counts).tolist()
    m, k, n, e = gl[-1], 256, 1280, len(counts)   # 5 column tiles per row block
    x = _i8(rng, (m, k))
    w = _i8(rng, (e, k, n))
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(F)).cuda()
    xs = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(F)).cuda()
    want_y, want_s = oracle.grouped_matmul_swiglu_quant(x.cpu().numpy(), w.cpu().numpy(), ws.cpu().numpy(),
                                                        xs.cpu().numpy(), gl)
    try:
        for epilogue_warps in (8, 16):   # both widths of the SwiGLU epilogue
            assert lib.w8a8_set_gmsq_epilogue_warps(epilogue_warps) in (8, 16)
            for fused in (1, 0):
                lib.w8a8_set_gmsq_fused_requant(fused)
                for glarg in (gl, torch.tensor(gl, dtype=torch.int64, device="cuda")):
                    y, ysc = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, glarg)
                    assert np.array_equal(y.cpu().numpy(), want_y), (epilogue_warps, fused)
                    assert ysc.cpu().numpy().tobytes() == want_s.tobytes(), (epilogue_warps, fused)
        assert lib.w8a8_set_gmsq_epilogue_warps(12) == L.ERR_INVALID
    finally:
        lib.w8a8_set_gmsq_fused_requant(0)
        lib.w8a8_set_gmsq_epilogue_warps(16)
    # the two stages as two calls (the reference's two launchers)
    need = lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(m, k, n, e)
    wsb = torch.empty((need,), dtype=torch.uint8, device="cuda")
    y = torch.zeros((m, n // 2), dtype=torch.int8, device="cuda")
    ysc = torch.zeros((m,), dtype=torch.float32, device="cuda")
    glt = torch.tensor(gl, dtype=torch.int64)
    for stage in (L.F_STAGE_MATMUL, L.F_STAGE_REQUANT):
        rc = lib.w8a8_grouped_matmul_swiglu_quant(x.data_ptr(), w.data_ptr(), ws.data_ptr(), xs.data_ptr(),
                                                  y.data_ptr(), ysc.data_ptr(), m, k, n, e, glt.data_ptr(), 0, L.W_KN,
                                                  stage, wsb.data_ptr(), need, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, L.status_string(rc)
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), want_y) and ysc.cpu().numpy().tobytes() == want_s.tobytes()


@pytest.mark.parametrize("layout_nk", [False, True])
def test_grouped_matmul_fp32_operands(ops, layout_nk):
    """fp32 x and weight (the reference's GMM_DT_FLOAT dispatch): three-piece bf16 split of both operands on the
    tensor cores, fp32 accumulation.  Against the fp64 product the error stays within 2^-20 of the largest output
    (fp32 rounding of a 320-term sum; a plain bf16 or tf32 product would miss this bound by orders of magnitude)."""
    rng = np.random.default_rng(17)
    m, k, n, e = 300, 320, 272, 4
    gl = [130, 130, 171, 300]
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(F)).cuda()
    w = torch.from_numpy((rng.standard_normal((e, k, n)) * 0.1).astype(F)).cuda()
    bias = torch.from_numpy(rng.standard_normal((e, n)).astype(F)).cuda()
    wt = w.transpose(1, 2).contiguous() if layout_nk else w
    out = ops.grouped_matmul(x, wt, gl, bias, 2, layout_nk)[0]
    assert out.dtype == torch.float32 and out.shape == (m, n)
    xf, wf, bf = x.double().cpu(), w.double().cpu(), bias.double().cpu()
    ref = torch.empty((m, n), dtype=torch.float64)
    start = 0
    for g, end in enumerate(gl):
        ref[start:end] = xf[start:end] @ wf[g] + bf[g]
        start = end
    err = (out.double().cpu() - ref).abs().max().item()
    assert err <= ref.abs().max().item() * 2.0**-20, err
    views = ops.grouped_matmul(x, wt, gl, None, 0, layout_nk)
    assert [v.shape[0] for v in views] == [130, 0, 41, 129]


def test_grouped_matmul_float_rejects_partial_column_chunks(ops):
    """The epilogue moves per-channel operands and outputs in 16-column pieces: N must be a multiple of 16 for
    every operand type (N = 24 used to slip through for 16-bit operands and lose the bias of its last columns)."""
    from cannbench_operator_solutions_b200 import _lib as L

    x = torch.zeros((8, 32), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((1, 32, 24), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="not supported"):
        ops.grouped_matmul(x, w, [8], None, 2, False)
    assert L.ERR_UNSUPPORTED == -6


def test_quant_matmul_full_size_sampled_rows(ops, oracle, cta_group):
    """Benchmark configuration 3 at full size (M=8192, K=7168, N=18432): rows sampled across all row tiles are
    compared bit for bit with the oracle, and the remaining rows through linearity in the per-token scale."""
    if cta_group == "single":
        pytest.skip("full-size case runs on the library's own kernel choice and on forced pairs")
    O = oracle
    g = torch.Generator(device="cuda").manual_seed(3)
    m, k, n = 8192, 7168, 18432
    x = torch.randint(-127, 128, (m, k), generator=g, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (k, n), generator=g, device="cuda", dtype=torch.int8)
    sc = torch.empty((n,), device="cuda").uniform_(1e-3, 1e-2, generator=g)
    pt = torch.empty((m,), device="cuda").uniform_(1e-3, 5e-2, generator=g)
    out = ops.quant_matmul(x, w, sc, pertoken_scale=pt, output_dtype="bfloat16")
    rows = torch.arange(5, m, 257, device="cuda")  # 32 rows, every 256-row tile boundary region gets hit
    ref = O.quant_matmul(x[rows].cpu().numpy(), w.cpu().numpy(), sc.cpu().numpy(), pertoken=pt[rows].cpu().numpy(),
                         flags=O.QM_SCALE_PERCHAN | O.QM_HAS_PT, out_dtype=O.DT_BF16)
    assert np.array_equal(bits(out[rows]), ref)
    # doubling every per-token scale doubles every output exactly (power-of-two scaling commutes with rounding)
    out2 = ops.quant_matmul(x, w, sc, pertoken_scale=pt * 2, output_dtype="bfloat16")
    assert torch.equal(out2.float(), out.float() * 2)


def test_gmsq_full_size_sampled_rows(ops, oracle, cta_group):
    """Benchmark configuration 4 at full size (E=256, 131072 rows, Zipf 1.1, K=7168, N=4096): every row of a few
    experts (a large one, a one-tile one, tiny ones, the neighbours of an empty one) is compared bit for bit with
    the oracle; all rows must use the full int8 range."""
    if cta_group == "single":
        pytest.skip("full-size case runs on the library's own kernel choice and on forced pairs")
    rng = np.random.default_rng(0)
    e, m, k, n = 256, 131072, 7168, 4096
    gl = zipf_group_list(rng, m, e)
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randint(-127, 128, (m, k), generator=g, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (e, k, n), generator=g, device="cuda", dtype=torch.int8)
    ws = torch.empty((e, n), device="cuda").uniform_(1e-3, 1e-2, generator=g)
    xs = torch.empty((m,), device="cuda").uniform_(1e-3, 5e-2, generator=g)
    y, ysc = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, [int(v) for v in gl])
    assert bool((y.to(torch.int32).abs().amax(-1) == 127).all())
    starts = np.concatenate([[0], gl[:-1]])
    sizes = gl - starts
    picks = [int(np.argmax(sizes >= 1)), 40, 100, 200, 255]
    picks += [int(i) for i in np.flatnonzero(sizes == 0)[:1]]
    for ex in picks:
        lo, hi = int(starts[ex]), int(gl[ex])
        if hi == lo:
            continue
        hi = min(hi, lo + 300)  # a slice of the largest expert is enough
        yo, yso = oracle.grouped_matmul_swiglu_quant(x[lo:hi].cpu().numpy(), w[ex:ex + 1].cpu().numpy(),
                                                     ws[ex:ex + 1].cpu().numpy(), xs[lo:hi].cpu().numpy(), [hi - lo])
        assert_same_f32(ysc[lo:hi], yso, f"y_scale of expert {ex}")
        assert np.array_equal(y[lo:hi].cpu().numpy(), yo), f"expert {ex}"


@pytest.mark.parametrize("chunk", [96, 1000, 5000])
def test_host_front_end_equals_the_whole_tensor_operator(ops, chunk, cta_group):
    """Rows pipelined through the host-buffer front end in chunks (which start and end inside experts) give the
    same bytes as one call on the whole tensor."""
    from cannbench_operator_solutions_b200.host_io import GroupedSwigluQuantFromHost

    if cta_group != "auto":
        pytest.skip("kernel shape does not matter here")
    rng = np.random.default_rng(seed_of("front", chunk))
    e, k, n = 7, 256, 512
    counts = np.array([300, 0, 1, 700, 129, 0, 1270])
    m = int(counts.sum())
    gl = np.cumsum(counts).tolist()
    x = _i8(rng, (m, k))
    w = _i8(rng, (e, k, n))
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(F)).cuda()
    xs = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(F)).cuda()
    want_y, want_s = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, gl)
    front = GroupedSwigluQuantFromHost(w, ws, chunk_rows=chunk)
    got_y, got_s = front(x.cpu().pin_memory(), xs.cpu().pin_memory(), gl)
    torch.cuda.synchronize()
    assert torch.equal(got_y, want_y.cpu()) and torch.equal(got_s, want_s.cpu())
    got_y2, got_s2 = front(x.cpu().pin_memory(), xs.cpu().pin_memory(), gl)      # buffers are reusable
    torch.cuda.synchronize()
    assert torch.equal(got_y2, want_y.cpu()) and torch.equal(got_s2, want_s.cpu())
    with pytest.raises(RuntimeError, match="cumsum"):
        front(x.cpu(), xs.cpu(), [5, 3] + gl[2:])


def test_grouped_operators_capture_into_a_cuda_graph(oracle):
    """With the group list in device memory the grouped operators read nothing back and allocate nothing, so the up
    projection and the down projection can be captured into one CUDA graph; a replay after the inputs AND the group
    list have been overwritten in place gives the oracle's bits for the new problem (the tile tables are rebuilt on
    the device inside the graph)."""
    from cannbench_operator_solutions_b200 import _lib as L

    O = oracle
    lib = L.load()
    rng = np.random.default_rng(77)
    m, k, n, e, n2 = 900, 256, 512, 5, 384
    x = torch.empty((m, k), dtype=torch.int8, device="cuda")
    xs = torch.empty((m,), dtype=torch.float32, device="cuda")
    gl = torch.empty((e,), dtype=torch.int64, device="cuda")
    w = _i8(rng, (e, k, n))
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(F)).cuda()
    w2 = _i8(rng, (e, n // 2, n2))
    ws2 = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n2)).astype(F)).cuda()
    y = torch.zeros((m, n // 2), dtype=torch.int8, device="cuda")
    ys = torch.zeros((m,), dtype=torch.float32, device="cuda")
    out = torch.zeros((m, n2), dtype=torch.bfloat16, device="cuda")
    need1 = lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(m, k, n, e)
    need2 = lib.w8a8_grouped_matmul_workspace_size(m, n2, n // 2, e)
    wsb1 = torch.empty((need1,), dtype=torch.uint8, device="cuda")
    wsb2 = torch.empty((need2,), dtype=torch.uint8, device="cuda")

    def fill(counts, seed):
        r = np.random.default_rng(seed)
        x.copy_(torch.from_numpy(r.integers(-127, 128, (m, k)).astype(np.int8)))
        xs.copy_(torch.from_numpy(r.uniform(1e-3, 5e-2, m).astype(F)))
        gl.copy_(torch.from_numpy(np.cumsum(counts).astype(np.int64)))

    def enqueue():
        st = torch.cuda.current_stream().cuda_stream
        rc = lib.w8a8_grouped_matmul_swiglu_quant(x.data_ptr(), w.data_ptr(), ws.data_ptr(), xs.data_ptr(),
                                                  y.data_ptr(), ys.data_ptr(), m, k, n, e, gl.data_ptr(), 1, L.W_KN, 0,
                                                  wsb1.data_ptr(), need1, st)
        assert rc == 0, L.status_string(rc)
        rc = lib.w8a8_grouped_matmul(y.data_ptr(), w2.data_ptr(), None, out.data_ptr(), ys.data_ptr(), ws2.data_ptr(),
                                     m, n2, n // 2, e, gl.data_ptr(), 1, L.DT_I8, L.DT_F32, L.DT_BF16, L.W_KN,
                                     wsb2.data_ptr(), need2, st)
        assert rc == 0, L.status_string(rc)

    first, second = [300, 0, 257, 43, 300], [1, 640, 0, 130, 129]
    fill(first, 1)
    enqueue()  # warm-up outside the capture (function attributes, first-use initialisation)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        enqueue()
    for counts, seed in ((first, 1), (second, 2), (first, 3)):
        fill(counts, seed)
        y.zero_(), ys.zero_(), out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        gl_host = np.cumsum(counts).tolist()
        want_y, want_s = O.grouped_matmul_swiglu_quant(x.cpu().numpy(), w.cpu().numpy(), ws.cpu().numpy(),
                                                       xs.cpu().numpy(), gl_host)
        assert np.array_equal(y.cpu().numpy(), want_y), counts
        assert ys.cpu().numpy().tobytes() == want_s.tobytes(), counts
        want_out = O.grouped_matmul(want_y, w2.cpu().numpy(), gl_host, dtype=O.DT_I8, x_scale=want_s,
                                    w_scale=ws2.cpu().numpy())
        assert np.array_equal(bits(out), want_out), counts
        assert lib.w8a8_workspace_error(wsb1.data_ptr(), None) == 0
