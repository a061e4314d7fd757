"""GPU parity: DynamicQuant and AddRmsNormDynamicQuant through the C-ABI vs the
CPU oracle.  int8 outputs, fp32 scales and 16-bit xOut are compared bit for
bit (the kernel and the oracle share the reduction order)."""
import numpy as np
import pytest
import torch

from helpers import assert_same_16, assert_same_f32, bits, dt_code, from_bits, seed_of

pytestmark = pytest.mark.gpu


def _rand16(rng, shape, dtype, scale=1.0):
    return torch.from_numpy((rng.standard_normal(shape) * scale).astype(np.float32)).to(dtype).cuda()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 1024), (37, 7168), (5, 3, 512), (3, 40), (2, 8), (9, 333), (4, 16384),
                                   (2, 20000), (2, 70000)])
def test_dynamic_quant_matches_oracle(ops, oracle, dtype, shape):
    rng = np.random.default_rng(seed_of(dtype, shape))
    x = _rand16(rng, shape, dtype)
    y, s = ops.dynamic_quant(x)
    assert y.shape == x.shape and y.dtype == torch.int8 and s.shape == x.shape[:-1] and s.dtype == torch.float32
    yo, so = oracle.dynamic_quant(bits(x), dt_code(dtype))
    assert np.array_equal(y.cpu().numpy(), yo)
    assert_same_f32(s, so, "scale")
    yd, _ = ops.dynamic_quant(x, round_direct=True)
    ydo, _ = oracle.dynamic_quant(bits(x), dt_code(dtype), oracle.ROUND_DIRECT)
    assert np.array_equal(yd.cpu().numpy(), ydo)


@pytest.mark.parametrize("kind,dtype", [("bf16", torch.bfloat16), ("f16", torch.float16)])
def test_dynamic_quant_golden_specials(ops, golden, kind, dtype):
    x = from_bits(golden[f"dq_{kind}_x"], dtype)
    y, s = ops.dynamic_quant(x)
    assert np.array_equal(y.cpu().numpy(), golden[f"dq_{kind}_y"])
    assert_same_f32(s, golden[f"dq_{kind}_scale"], "scale")
    yd, _ = ops.dynamic_quant(x, round_direct=True)
    assert np.array_equal(yd.cpu().numpy(), golden[f"dq_{kind}_y_direct"])


def test_dynamic_quant_non_contiguous_and_empty(ops, oracle):
    rng = np.random.default_rng(7)
    base = _rand16(rng, (16, 96), torch.bfloat16)
    x = base[:, ::2]  # the wrapper makes it contiguous, like the reference plugin
    y, s = ops.dynamic_quant(x)
    yo, so = oracle.dynamic_quant(bits(x.contiguous()), oracle.DT_BF16)
    assert np.array_equal(y.cpu().numpy(), yo)
    y0, s0 = ops.dynamic_quant(torch.empty((0, 64), dtype=torch.bfloat16, device="cuda"))
    assert y0.shape == (0, 64) and s0.shape == (0,)


def test_dynamic_quant_full_size_properties(ops):
    """Benchmark configuration 2 shape: size-independent properties instead of a full CPU comparison."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((8192, 7168), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    y, s = ops.dynamic_quant(x)
    xf = x.float()
    amax = xf.abs().amax(-1)
    inv127 = torch.tensor(np.float32(1.0) / np.float32(127.0), device="cuda")
    assert torch.equal(s, amax * inv127)
    assert int(y.abs().amax()) == 127 and bool((y.to(torch.int32).abs().amax(-1) == 127).all())
    err = (y.float() * s[:, None] - xf).abs()
    assert bool((err <= s[:, None] * 0.54).all())
    # idempotence of the grid: re-quantising the dequantised tensor reproduces y
    y2, _ = ops.dynamic_quant((y.float() * s[:, None]).to(torch.bfloat16))
    assert (y2 != y).float().mean().item() < 0.02


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(64, 7168), (33, 1024), (3, 5, 2048), (7, 72), (4, 8), (5, 333), (3, 16384),
                                   (300, 4096)])
def test_add_rms_norm_dynamic_quant_matches_oracle(ops, oracle, dtype, shape):
    rng = np.random.default_rng(seed_of(dtype, shape, 1))
    x1, x2 = _rand16(rng, shape, dtype), _rand16(rng, shape, dtype)
    gamma = torch.from_numpy((1 + 0.1 * rng.standard_normal(shape[-1])).astype(np.float32)).to(dtype).cuda()
    y, xo, sc = ops.add_rms_norm_dynamic_quant(x1, x2, gamma, 1e-6)
    assert y.shape == x1.shape and xo.shape == x1.shape and xo.dtype == dtype and sc.shape == x1.shape[:-1]
    code = dt_code(dtype)
    yo, xoo, sco = oracle.add_rms_norm_dynamic_quant(bits(x1), bits(x2), bits(gamma), 1e-6, code)
    assert_same_16(bits(xo), xoo, code, "xOut")
    assert_same_f32(sc, sco, "scaleOut")
    assert np.array_equal(y.cpu().numpy(), yo)
    # against the fp64-sum oracle: the tolerance the summation order is allowed
    yb, _, scb = oracle.add_rms_norm_dynamic_quant(bits(x1), bits(x2), bits(gamma), 1e-6, code,
                                                   sum_order=oracle.SUM_FP64)
    d = np.abs(y.cpu().numpy().astype(np.int32) - yb.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= 1e-4
    assert (np.abs(sc.cpu().numpy() - scb) <= 4 * np.spacing(scb)).all()


@pytest.mark.parametrize("kind,dtype", [("bf16", torch.bfloat16), ("f16", torch.float16)])
def test_add_rms_norm_dynamic_quant_golden_specials(ops, golden, kind, dtype):
    x1, x2 = from_bits(golden[f"ardq_{kind}_x1"], dtype), from_bits(golden[f"ardq_{kind}_x2"], dtype)
    gamma = from_bits(golden[f"ardq_{kind}_gamma"], dtype)
    y, xo, sc = ops.add_rms_norm_dynamic_quant(x1, x2, gamma, 1e-6)
    assert_same_16(bits(xo), golden[f"ardq_{kind}_xout"], dt_code(dtype), "xOut")
    # the golden vectors sum the squares in fp64; the kernel's fp32 order is allowed a few ulp on the scale
    # and +-1 LSB on rare elements (here: none expected on 6 short rows)
    want_s, got_s = golden[f"ardq_{kind}_scale"], sc.cpu().numpy()
    assert np.array_equal(np.isnan(got_s), np.isnan(want_s))
    fin = ~np.isnan(want_s)
    assert (np.abs(got_s[fin] - want_s[fin]) <= 4 * np.spacing(want_s[fin])).all()
    assert np.abs(y.cpu().numpy().astype(np.int32) - golden[f"ardq_{kind}_y"].astype(np.int32)).max() <= 1


def test_add_rms_norm_dynamic_quant_edge_rows(ops, oracle):
    z = torch.zeros((2, 64), dtype=torch.bfloat16, device="cuda")
    g = torch.ones((64,), dtype=torch.bfloat16, device="cuda")
    y, xo, sc = ops.add_rms_norm_dynamic_quant(z, z, g, 1e-6)
    assert sc[0].item() == np.float32(1e-12) * np.float32(1.0 / 127.0) and not y.any()
    y, xo, sc = ops.add_rms_norm_dynamic_quant(z, z, g, 0.0)  # rms = 0: NaN scale, zero output
    assert torch.isnan(sc).all() and not y.any()
    with pytest.raises(RuntimeError, match="16384"):
        big = torch.zeros((1, 16392), dtype=torch.bfloat16, device="cuda")
        ops.add_rms_norm_dynamic_quant(big, big, big[0], 1e-6)
    e = torch.empty((0, 64), dtype=torch.bfloat16, device="cuda")
    y0, x0, s0 = ops.add_rms_norm_dynamic_quant(e, e, g, 1e-6)
    assert y0.shape == (0, 64) and s0.shape == (0,)


def test_add_rms_norm_dynamic_quant_full_size_properties(ops, oracle):
    """Benchmark configuration 2: [8192, 7168] bf16; a 64-row sample is compared with the oracle, the rest by properties."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x1 = torch.randn((8192, 7168), generator=g, device="cuda").to(torch.bfloat16)
    x2 = torch.randn((8192, 7168), generator=g, device="cuda").to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn((7168,), generator=g, device="cuda")).to(torch.bfloat16)
    y, xo, sc = ops.add_rms_norm_dynamic_quant(x1, x2, gamma, 1e-6)
    assert torch.equal(xo, (x1.float() + x2.float()).to(torch.bfloat16))
    assert bool((y.to(torch.int32).abs().amax(-1) == 127).all())
    s = x1.float() + x2.float()
    norm = s * torch.rsqrt((s * s).mean(-1, keepdim=True) + 1e-6) * gamma.float()
    err = (y.float() * sc[:, None] - norm).abs()
    assert bool((err <= sc[:, None] * 0.55 + 1e-5).all())
    idx = torch.arange(0, 8192, 128, device="cuda")
    yo, xoo, sco = oracle.add_rms_norm_dynamic_quant(bits(x1[idx]), bits(x2[idx]), bits(gamma), 1e-6, oracle.DT_BF16)
    assert np.array_equal(y[idx].cpu().numpy(), yo)
    assert_same_f32(sc[idx], sco, "scaleOut sample")


@pytest.mark.parametrize("xdtype", [torch.int32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,h", [(64, 2048), (7, 24), (3, 4096), (5, 20480), (130, 256), (2, 7), (9, 9000)])
@pytest.mark.parametrize("left", [False, True])
def test_dequant_swiglu_quant_matches_oracle(ops, oracle, xdtype, m, h, left):
    from helpers import assert_same_f32, bits, seed_of
    g = torch.Generator(device="cuda").manual_seed(seed_of("dqsq", str(xdtype), m, h, left))
    if xdtype == torch.int32:
        x = torch.randint(-200000, 200000, (m, 2 * h), generator=g, device="cuda", dtype=torch.int32)
        ws = torch.empty((2 * h,), device="cuda").uniform_(1e-3, 1e-2, generator=g)
        a_s = torch.empty((m,), device="cuda").uniform_(1e-3, 5e-2, generator=g)
        x[0, :] = 0                                          # an all-zero row: scale clamps to 1e-12
        kw = dict(weight_scale=ws, activation_scale=a_s)
        okw = dict(weight_scale=ws.cpu().numpy(), activation_scale=a_s.cpu().numpy())
        ox = x.cpu().numpy()
        code = oracle.DT_I32
    else:
        x = (torch.randn((m, 2 * h), generator=g, device="cuda") * 3).to(xdtype)
        if m > 1:
            x[1, 3] = float("nan")                           # a NaN activation quantises to 0
        kw, okw, ox = {}, {}, bits(x)
        code = oracle.DT_BF16 if xdtype == torch.bfloat16 else oracle.DT_F16
    qs = torch.empty((h,), device="cuda").uniform_(0.5, 2.0, generator=g)
    for quant_scale in (None, qs):
        y, sc = ops.dequant_swiglu_quant(x, quant_scale=quant_scale, activate_left=left, **kw)
        wy, wsc = oracle.dequant_swiglu_quant(ox, code, quant_scale=None if quant_scale is None else qs.cpu().numpy(),
                                              activate_left=left, **okw)
        assert y.shape == (m, h) and y.dtype == torch.int8 and sc.shape == (m,)
        assert_same_f32(sc, wsc, "dqsq scale")
        assert np.array_equal(y.cpu().numpy(), wy)
    y, _ = ops.dequant_swiglu_quant(x, activate_left=left, round_direct=True, **kw)
    wy, _ = oracle.dequant_swiglu_quant(ox, code, activate_left=left, round_mode=oracle.ROUND_DIRECT, **okw)
    assert np.array_equal(y.cpu().numpy(), wy)


def test_dequant_swiglu_quant_is_the_unfused_form_of_the_grouped_epilogue(ops, oracle):
    """int32 accumulators -> dequant_swiglu_quant(activate_left=True) against grouped_matmul_swiglu_quant on the
    same operands: the fused operator gates on the left half too; its dequantisation multiplies by the token scale
    first and its quantisation multiplies by 127/amax, so the int8 results may differ by one step on a few elements
    and the scales by an ulp."""
    g = torch.Generator(device="cuda").manual_seed(99)
    m, k, n = 256, 512, 1024
    x = torch.randint(-127, 128, (m, k), generator=g, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (1, k, n), generator=g, device="cuda", dtype=torch.int8)
    ws = torch.empty((1, n), device="cuda").uniform_(1e-3, 1e-2, generator=g)
    xs = torch.empty((m,), device="cuda").uniform_(1e-3, 5e-2, generator=g)
    y_fused, s_fused = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, [m])
    acc = (x.double() @ w[0].double()).to(torch.int32)
    y, s = ops.dequant_swiglu_quant(acc, ws.view(-1), xs, None, True)
    assert torch.allclose(s, s_fused, rtol=1e-5)
    diff = (y.int() - y_fused.int()).abs()
    assert int(diff.max()) <= 1 and float((diff > 0).float().mean()) < 2e-2


@pytest.mark.parametrize("fused", [False, True])
def test_host_front_end_equals_the_whole_tensor_operators(ops, fused):
    """Rows pipelined through the host-buffer front end in chunks give the same bytes as one call."""
    from cannbench_operator_solutions_b200.host_io import RowQuantFromHost

    g = torch.Generator(device="cuda").manual_seed(31)
    rows, n = 1000, 1536
    x1 = torch.randn((rows, n), generator=g, device="cuda").to(torch.bfloat16)
    x2 = torch.randn((rows, n), generator=g, device="cuda").to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn((n,), generator=g, device="cuda")).to(torch.bfloat16)
    front = RowQuantFromHost(n, torch.bfloat16, "cuda", fused=fused, gamma=gamma if fused else None, chunk_rows=96)
    for _ in range(2):   # staging buffers are reusable
        if fused:
            want = ops.add_rms_norm_dynamic_quant(x1, x2, gamma, 1e-6)
            got = front(x1.cpu().pin_memory(), x2.cpu().pin_memory())
        else:
            want = ops.dynamic_quant(x1)
            got = front(x1.cpu().pin_memory())
        torch.cuda.synchronize()
        assert len(got) == len(want)
        for a, b in zip(got, want):
            assert torch.equal(a.view(torch.uint8), b.cpu().view(torch.uint8))
