"""The torch plugin (torch.ops.cann_bench.*, C++ host code over the C-ABI) gives the
same results as the ctypes operator functions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cb(ops):
    import cannbench_operator_solutions_b200 as pkg

    pkg.load_torch_plugin()
    return torch.ops.cann_bench


def test_plugin_matches_ctypes_operators(cb, ops):
    rng = np.random.default_rng(21)
    x1 = torch.from_numpy(rng.standard_normal((130, 512)).astype(np.float32)).to(torch.bfloat16).cuda()
    x2 = torch.from_numpy(rng.standard_normal((130, 512)).astype(np.float32)).to(torch.bfloat16).cuda()
    gamma = torch.ones(512, dtype=torch.bfloat16, device="cuda")
    for a, b in zip(cb.dynamic_quant(x1), ops.dynamic_quant(x1)):
        assert torch.equal(a, b)
    q = cb.add_rms_norm_dynamic_quant(x1, x2, gamma, 1e-6)
    for a, b in zip(q, ops.add_rms_norm_dynamic_quant(x1, x2, gamma, 1e-6)):
        assert torch.equal(a, b)
    w = torch.from_numpy(rng.integers(-127, 128, (512, 256)).astype(np.int8)).cuda()
    sc = torch.from_numpy(rng.uniform(1e-3, 1e-2, 256).astype(np.float32)).cuda()
    a = cb.quant_matmul(q[0], w, sc, pertoken_scale=q[2], output_dtype="bfloat16")
    b = ops.quant_matmul(q[0], w, sc, pertoken_scale=q[2], output_dtype="bfloat16")
    assert a.dtype == torch.bfloat16 and torch.equal(a, b)
    assert cb.quant_matmul(q[0], w, sc).dtype == torch.float16
    we = torch.from_numpy(rng.integers(-127, 128, (3, 512, 256)).astype(np.int8)).cuda()
    se = torch.from_numpy(rng.uniform(1e-3, 1e-2, (3, 256)).astype(np.float32)).cuda()
    gl = [60, 60, 130]
    h = cb.grouped_matmul_swiglu_quant(q[0], we, se, q[2], gl)
    for a, b in zip(h, ops.grouped_matmul_swiglu_quant(q[0], we, se, q[2], gl)):
        assert torch.equal(a, b)
    wd = torch.from_numpy(rng.integers(-127, 128, (3, 128, 512)).astype(np.int8)).cuda()
    sd = torch.from_numpy(rng.uniform(1e-3, 1e-2, (3, 512)).astype(np.float32)).cuda()
    outs = cb.grouped_matmul(h[0], wd, gl, None, 0, False, h[1], sd)
    ref = ops.grouped_matmul(h[0], wd, gl, None, 0, False, x_scale=h[1], weight_scale=sd)
    assert len(outs) == 3 and all(torch.equal(a, b) for a, b in zip(outs, ref))
    xb = torch.from_numpy(rng.standard_normal((130, 128)).astype(np.float32)).to(torch.bfloat16).cuda()
    wb = torch.from_numpy(rng.standard_normal((3, 128, 64)).astype(np.float32)).to(torch.bfloat16).cuda()
    assert torch.equal(cb.grouped_matmul(xb, wb, gl, None, 2)[0], ops.grouped_matmul(xb, wb, gl, None, 2)[0])


def test_plugin_errors_are_torch_checks(cb):
    x = torch.zeros((4, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="float16 / bfloat16"):
        cb.dynamic_quant(x)
    with pytest.raises(RuntimeError, match="must equal M"):
        cb.grouped_matmul(torch.zeros((8, 32), dtype=torch.bfloat16, device="cuda"),
                          torch.zeros((2, 32, 16), dtype=torch.bfloat16, device="cuda"), [3, 7])
    y, s = cb.dynamic_quant(torch.empty((0, 64), dtype=torch.bfloat16, device="cuda"))
    assert y.shape == (0, 64)


def test_plugin_moe_re_routing_matches_ctypes_operator(cb, ops):
    g = torch.Generator(device="cuda").manual_seed(5)
    cnt = torch.randint(0, 9, (4, 16), generator=g, device="cuda", dtype=torch.int64)
    a = int(cnt.sum())
    tok = torch.randint(-128, 128, (a, 256), generator=g, device="cuda", dtype=torch.int8)
    scl = torch.rand((a,), generator=g, device="cuda")
    got = cb.moe_re_routing(tok, cnt, scl)
    want = ops.moe_re_routing(tok, cnt, scl)
    for x, y in zip(got, want):
        assert torch.equal(x, y)
    got = cb.moe_re_routing(tok, cnt.to(torch.int32), None, 1, 0)
    assert torch.equal(got[0], want[0]) and got[3].dtype == torch.int32
    with pytest.raises(RuntimeError, match="idx_type == 0"):
        cb.moe_re_routing(tok, cnt, None, 1, 1)


def test_plugin_moe_finalize_routing_matches_ctypes_operator(cb, ops):
    g = torch.Generator(device="cuda").manual_seed(9)
    r, k, h, e = 50, 4, 1024, 8
    rows = torch.randn((r * k, h), generator=g, device="cuda").to(torch.bfloat16)
    skip = torch.randn((r, h), generator=g, device="cuda").to(torch.bfloat16)
    bias = torch.randn((e, h), generator=g, device="cuda").to(torch.bfloat16)
    scales = torch.rand((r, k), generator=g, device="cuda").to(torch.bfloat16)
    esdr = torch.randperm(r * k, generator=g, device="cuda").to(torch.int32)
    expert = torch.randint(0, e, (r, k), generator=g, device="cuda", dtype=torch.int32)
    got = cb.moe_finalize_routing(rows, esdr, skip, None, bias, scales, expert, 0)
    want = ops.moe_finalize_routing(rows, esdr, skip, None, bias, scales, expert, 0)
    assert torch.equal(got, want)
    assert torch.equal(cb.moe_finalize_routing(rows, esdr[:r]), ops.moe_finalize_routing(rows, esdr[:r]))
    assert torch.equal(cb.moe_finalize_routing(rows, esdr, scales=scales, drop_pad_mode=9),     # clamped to 3
                       ops.moe_finalize_routing(rows, esdr, scales=scales, drop_pad_mode=3))
    with pytest.raises(RuntimeError, match="must be int32"):
        cb.moe_finalize_routing(rows, esdr.to(torch.int64))
    with pytest.raises(RuntimeError, match="K\\*NUM_ROWS"):
        cb.moe_finalize_routing(rows, esdr[:7], scales=scales)


def test_plugin_moe_gating_matches_ctypes_operator(cb, ops):
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn((300, 256), generator=g, device="cuda").to(torch.bfloat16)
    fin = torch.rand((300,), generator=g, device="cuda") < 0.5
    for a, b in zip(cb.moe_gating_top_k_softmax(x, fin, 8), ops.moe_gating_top_k_softmax(x, fin, 8)):
        assert torch.equal(a, b)
    for a, b in zip(cb.moe_gating_top_k_softmax(x), ops.moe_gating_top_k_softmax(x)):
        assert torch.equal(a, b)
    with pytest.raises(RuntimeError, match="0 < k <= x.size"):
        cb.moe_gating_top_k_softmax(x, None, 0)
    with pytest.raises(RuntimeError, match="bool 'finished'"):
        cb.moe_gating_top_k_softmax(x, fin.to(torch.int32), 2)


def test_plugin_dequant_swiglu_quant_matches_ctypes_operator(cb, ops):
    g = torch.Generator(device="cuda").manual_seed(13)
    x = torch.randint(-100000, 100000, (50, 512), generator=g, device="cuda", dtype=torch.int32)
    ws = torch.rand((512,), generator=g, device="cuda") * 1e-2
    a_s = torch.rand((50,), generator=g, device="cuda") * 1e-2
    qs = torch.rand((256,), generator=g, device="cuda") + 0.5
    for a, b in zip(cb.dequant_swiglu_quant(x, ws, a_s, qs, True), ops.dequant_swiglu_quant(x, ws, a_s, qs, True)):
        assert torch.equal(a, b)
    xb = torch.randn((20, 128), generator=g, device="cuda").to(torch.bfloat16)
    for a, b in zip(cb.dequant_swiglu_quant(xb), ops.dequant_swiglu_quant(xb)):
        assert torch.equal(a, b)
    with pytest.raises(RuntimeError, match="weight_scale is required"):
        cb.dequant_swiglu_quant(x)
    with pytest.raises(RuntimeError, match="must be None for float16"):
        cb.dequant_swiglu_quant(xb, ws[:128])


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _i8(rng, shape):
    return torch.from_numpy(rng.integers(-127, 128, shape).astype(np.int8)).cuda()


@pytest.mark.parametrize("m,k,n", [(37, 40, 24), (130, 100, 250), (5, 17, 1)])
def test_plugin_quant_matmul_any_k_and_n(cb, oracle, m, k, n):
    """The schema takes any K and N; the kernels take multiples of 16.  The plugin runs shapes in between on
    zero-padded copies and cuts the result back: the returned elements are the oracle's on the unpadded problem."""
    O = oracle
    rng = np.random.default_rng(100 + k)
    x1, x2 = _i8(rng, (m, k)), _i8(rng, (k, n))
    scale = torch.from_numpy(rng.uniform(1e-3, 1e-2, n).astype(np.float32)).cuda()
    offset = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).cuda()
    pt = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    per = O.QM_SCALE_PERCHAN | O.QM_OFFSET_PERCHAN | O.QM_BIAS_PERCHAN if n > 1 else 0
    got = cb.quant_matmul(x1, x2, scale, offset=offset, pertoken_scale=pt, bias=bias, output_dtype="bfloat16")
    assert got.shape == (m, n)
    ref = O.quant_matmul(x1.cpu().numpy(), x2.cpu().numpy(), scale.cpu().numpy(), offset=offset.cpu().numpy(),
                         pertoken=pt.cpu().numpy(), bias=bias.cpu().numpy(),
                         flags=per | O.QM_HAS_OFFSET | O.QM_HAS_PT | (O.QM_BIAS_F32 << O.QM_BIAS_SHIFT),
                         out_dtype=O.DT_BF16)
    assert np.array_equal(_bits(got), ref)
    # batched, one bias row per batch entry
    xb, wb = _i8(rng, (2, m, k)), _i8(rng, (2, k, n))
    bb = torch.from_numpy(rng.standard_normal((2, 1, n)).astype(np.float32)).cuda()
    got = cb.quant_matmul(xb, wb, scale, bias=bb)
    assert got.shape == (2, m, n)
    for i in range(2):
        ref = O.quant_matmul(xb[i].cpu().numpy(), wb[i].cpu().numpy(), scale.cpu().numpy(),
                             bias=bb[i, 0].cpu().numpy(),
                             flags=(O.QM_SCALE_PERCHAN | O.QM_BIAS_PERCHAN if n > 1 else 0)
                             | (O.QM_BIAS_F32 << O.QM_BIAS_SHIFT), out_dtype=O.DT_F16)
        assert np.array_equal(_bits(got[i]), ref)


@pytest.mark.parametrize("k,half", [(72, 40), (100, 129), (256, 8)])
def test_plugin_gmsq_any_k_and_n(cb, oracle, k, half):
    rng = np.random.default_rng(200 + half)
    counts = [33, 0, 140, 7]
    gl = np.cumsum(counts).tolist()
    m, e, n = gl[-1], len(counts), 2 * half
    x, w = _i8(rng, (m, k)), _i8(rng, (e, k, n))
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(np.float32)).cuda()
    xs = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(np.float32)).cuda()
    y, ys = cb.grouped_matmul_swiglu_quant(x, w, ws, xs, gl)
    want_y, want_s = oracle.grouped_matmul_swiglu_quant(x.cpu().numpy(), w.cpu().numpy(), ws.cpu().numpy(),
                                                        xs.cpu().numpy(), gl)
    assert y.shape == (m, half)
    assert np.array_equal(y.cpu().numpy(), want_y)
    assert ys.cpu().numpy().tobytes() == want_s.tobytes()


@pytest.mark.parametrize("transpose", [False, True])
def test_plugin_grouped_matmul_any_k_and_n(cb, oracle, transpose):
    O = oracle
    rng = np.random.default_rng(300)
    gl = [50, 50, 131]
    m, k, n, e = 131, 100, 40, 3
    x, w = _i8(rng, (m, k)), _i8(rng, (e, k, n))
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(np.float32)).cuda()
    xs = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal((e, n)).astype(np.float32)).cuda()
    wt = w.transpose(1, 2).contiguous() if transpose else w
    got = cb.grouped_matmul(x, wt, gl, bias, 2, transpose, xs, ws)[0]
    ref = O.grouped_matmul(x.cpu().numpy(), w.cpu().numpy(), gl, dtype=O.DT_I8, x_scale=xs.cpu().numpy(),
                           w_scale=ws.cpu().numpy(), bias=bias.cpu().numpy(), bias_dtype=O.DT_F32)
    assert got.shape == (m, n) and np.array_equal(_bits(got), ref)
    # the float form: K = 100 is not a multiple of 8 for fp32 either; fp64 product as the yardstick
    xf = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
    wf = torch.from_numpy((rng.standard_normal((e, k, n)) * 0.1).astype(np.float32)).cuda()
    for dtype, tol in ((torch.float32, 2.0**-18), (torch.bfloat16, 2.0**-7)):
        xd, wd = xf.to(dtype), wf.to(dtype)
        wdt = wd.transpose(1, 2).contiguous() if transpose else wd
        outs = cb.grouped_matmul(xd, wdt, gl, None, 0, transpose)
        assert [o.shape for o in outs] == [(50, n), (0, n), (81, n)]
        ref = torch.cat([xd[:50].double() @ wd[0].double(), xd[50:].double() @ wd[2].double()]).cpu()
        err = (torch.cat(list(outs)).double().cpu() - ref).abs().max().item()
        assert err <= ref.abs().max().item() * tol, (dtype, err)
