"""GPU parity of the expert-parallel helper kernels (routing plan, scatter, permute, combine) and of the
whole chain on one GPU, against the CPU oracle."""
import numpy as np
import pytest
import torch

from helpers import bits, seed_of

pytestmark = pytest.mark.gpu
F = np.float32


@pytest.fixture(scope="module")
def backend(ops):
    from cannbench_operator_solutions_b200.ep import CudaBackend

    return CudaBackend()


@pytest.mark.parametrize("t,topk,e", [(50, 4, 8), (1000, 8, 256), (3, 1, 5), (257, 2, 64)])
def test_route_plan_is_stable_counting_sort(backend, oracle, t, topk, e):
    rng = np.random.default_rng(t * 31 + e)
    idx = rng.integers(0, e, (t, topk)).astype(np.int32)
    cnt, cum, pos = backend.route_plan(torch.from_numpy(idx).cuda(), e)
    c0, u0, p0 = oracle.route_count(idx, e)
    assert np.array_equal(cnt.cpu().numpy(), c0)
    assert np.array_equal(cum.cpu().numpy(), u0)
    assert np.array_equal(pos.cpu().numpy(), p0)


def test_scatter_permute_combine_match_oracle(backend, oracle):
    rng = np.random.default_rng(31)
    t, topk, e, h = 300, 8, 32, 7168
    idx = rng.integers(0, e, (t, topk)).astype(np.int32)
    _, _, pos = backend.route_plan(torch.from_numpy(idx).cuda(), e)
    rows = torch.from_numpy(rng.integers(-127, 128, (t, h)).astype(np.int8)).cuda()
    sc = torch.from_numpy(rng.uniform(0.1, 1, t).astype(F)).cuda()
    dst, dsc = backend.scatter_rows(rows, sc, pos, t * topk)
    p = pos.cpu().numpy()
    want = np.empty((t * topk, h), np.int8)
    want_s = np.empty((t * topk,), F)
    for k in range(topk):
        want[p[:, k]] = rows.cpu().numpy()
        want_s[p[:, k]] = sc.cpu().numpy()
    assert np.array_equal(dst.cpu().numpy(), want) and np.array_equal(dsc.cpu().numpy(), want_s)
    perm = torch.from_numpy(rng.permutation(t * topk).astype(np.int64)).cuda()
    g, gs = backend.permute_rows(dst, dsc, perm)
    assert np.array_equal(g.cpu().numpy(), want[perm.cpu().numpy()])
    assert np.array_equal(gs.cpu().numpy(), want_s[perm.cpu().numpy()])
    # combine: bf16 rows, fp32 probabilities, ascending k
    y = torch.from_numpy(rng.standard_normal((t * topk, h)).astype(F)).to(torch.bfloat16).cuda()
    probs = torch.from_numpy(rng.uniform(0, 1, (t, topk)).astype(F)).cuda()
    out = backend.combine(y, probs, pos)
    ref = oracle.combine(bits(y), probs.cpu().numpy(), p, oracle.DT_BF16)
    assert np.array_equal(bits(out), ref)
    # a dropped pair (negative position) contributes nothing
    pos2 = pos.clone()
    pos2[:, 3] = -1
    out2 = backend.combine(y, probs, pos2)
    p2 = p.copy()
    p2[:, 3] = -1
    assert np.array_equal(bits(out2), oracle.combine(bits(y), probs.cpu().numpy(), p2, oracle.DT_BF16))


def test_single_gpu_chain_matches_oracle_chain(ops, oracle):
    """The full chain on one GPU (all experts local) against the same chain computed by the CPU oracle."""
    from test_ep_cpu import OracleBackend, _problem

    from cannbench_operator_solutions_b200.ep import ExpertShard, MoeFfnChain

    experts = 8
    x, res, gamma, idx, probs, w_up, s_up, w_dn, s_dn = _problem(seed=3, tokens=200, hidden=512, inter=256,
                                                                 experts=experts, topk=4)
    cpu_chain = MoeFfnChain(experts, ExpertShard(w_up, s_up, w_dn, s_dn), backend=OracleBackend())
    want, want_x = cpu_chain.forward(x, res, gamma, 1e-6, idx, probs)
    dev = "cuda"
    gpu_chain = MoeFfnChain(experts, ExpertShard(w_up.to(dev), s_up.to(dev), w_dn.to(dev), s_dn.to(dev)))
    got, got_x = gpu_chain.forward(x.to(dev), res.to(dev), gamma.to(dev), 1e-6, idx.to(dev), probs.to(dev))
    assert np.array_equal(bits(got_x), bits(want_x))
    assert np.array_equal(bits(got), bits(want))


def test_single_gpu_chain_peer_transport_equals_collective_transport(ops):
    """The fused transport (dispatch kernel and down-projection epilogue store rows at their final positions)
    gives the same bits as pack / all-to-all / regroup; with one rank the 'peer' buffers are this GPU's own."""
    from test_ep_cpu import _problem

    from cannbench_operator_solutions_b200.ep import ExpertShard, MoeFfnChain

    experts = 16
    x, res, gamma, idx, probs, w_up, s_up, w_dn, s_dn = _problem(seed=5, tokens=300, hidden=512, inter=256,
                                                                 experts=experts, topk=4)
    dev = "cuda"
    shard = ExpertShard(w_up.to(dev), s_up.to(dev), w_dn.to(dev), s_dn.to(dev))
    args = (x.to(dev), res.to(dev), gamma.to(dev), 1e-6, idx.to(dev), probs.to(dev))
    a, ax = MoeFfnChain(experts, shard, transport="nccl").forward(*args)
    chain = MoeFfnChain(experts, shard, transport="p2p")
    for _ in range(2):  # the second pass reuses the buffers of the first
        b, bx = chain.forward(*args)
        assert torch.equal(a, b) and torch.equal(ax, bx)
    # the same transport with the address tables built on the device (no host readback in the step)
    chain = MoeFfnChain(experts, shard, transport="p2p", device_tables=True)
    for _ in range(2):
        b, bx = chain.forward(*args)
        assert torch.equal(a, b) and torch.equal(ax, bx)
    chain.check()
    assert chain._native is not None  # that was the library's C++ step function (one call per step)
    # ... and as the Python sequence of the same library calls
    chain = MoeFfnChain(experts, shard, transport="p2p", device_tables=True, native_step=False)
    for _ in range(2):
        b, bx = chain.forward(*args)
        assert torch.equal(a, b) and torch.equal(ax, bx)
    chain.check()
    assert chain._native is None
    for native in (True, False):
        tight = MoeFfnChain(experts, shard, transport="p2p", device_tables=True, capacity_rows=256,
                            native_step=native)   # 1200 rows routed
        tight.forward(*args)
        with pytest.raises(RuntimeError, match="too small"):
            tight.check()
        tight.check()  # the flag was cleared by the read
        # an overflow is not forgotten when a later step fits (the flag is sticky until it is read)
        tight.forward(*args)
        small = tuple(t[:40].contiguous() if i in (0, 1, 4, 5) else t for i, t in enumerate(args))
        if not native:  # the C++ step is built for one token count; the Python sequence takes any
            tight.forward(*small)
        with pytest.raises(RuntimeError, match="too small"):
            tight.check()


def test_native_step_captures_into_a_cuda_graph(ops):
    """The C++ step enqueues everything on the caller's stream and on a second stream forked from and joined to it by
    events, reads nothing back and allocates nothing: a stream capture follows both streams, and replaying the graph
    after the inputs have been overwritten in place gives the result of an eager step on the new inputs."""
    from test_ep_cpu import _problem

    from cannbench_operator_solutions_b200.ep import ExpertShard, MoeFfnChain

    experts, dev = 16, "cuda"
    first = _problem(seed=7, tokens=256, hidden=512, inter=256, experts=experts, topk=4)
    second = _problem(seed=8, tokens=256, hidden=512, inter=256, experts=experts, topk=4)
    shard = ExpertShard(*(t.to(dev) for t in first[5:]))

    def step_args(problem):
        x, res, gamma, idx, probs = problem[:5]
        return [x.to(dev), res.to(dev), gamma.to(dev), idx.to(dev), probs.to(dev)]

    eager = MoeFfnChain(experts, shard, transport="p2p", device_tables=True)
    want = []
    for problem in (first, second):
        x, res, gamma, idx, probs = step_args(problem)
        out, x_out = eager.forward(x, res, gamma, 1e-6, idx, probs)
        want.append((out.clone(), x_out.clone()))
    eager.check()

    chain = MoeFfnChain(experts, shard, transport="p2p", device_tables=True)
    static = step_args(first)
    chain.forward(static[0], static[1], static[2], 1e-6, static[3], static[4])  # first-use set-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out, x_out = chain.forward(static[0], static[1], static[2], 1e-6, static[3], static[4])
    assert chain._native is not None
    for problem, (want_out, want_x) in ((first, want[0]), (second, want[1]), (first, want[0])):
        for dst, src in zip(static, step_args(problem)):
            dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want_out) and torch.equal(x_out, want_x)
    chain.check()


def test_chain_with_requantisation_inside_the_matmul_kernels(ops):
    """The optional in-kernel requantisation of grouped_matmul_swiglu_quant on the chain's capacity-sized buffers (a
    device group list that ends below the row capacity): same bits as the default two-kernel form."""
    from test_ep_cpu import _problem

    from cannbench_operator_solutions_b200 import _lib as L
    from cannbench_operator_solutions_b200.ep import ExpertShard, MoeFfnChain

    experts, dev = 8, "cuda"
    problem = _problem(seed=11, tokens=700, hidden=512, inter=384, experts=experts, topk=4)   # 2800 routed rows
    shard = ExpertShard(*(t.to(dev) for t in problem[5:]))
    x, res, gamma, idx, probs = (t.to(dev) for t in problem[:5])
    lib = L.load()
    results = []
    try:
        for fused in (0, 1):
            lib.w8a8_set_gmsq_fused_requant(fused)
            chain = MoeFfnChain(experts, shard, transport="p2p", device_tables=True)
            out, x_out = chain.forward(x, res, gamma, 1e-6, idx, probs)
            chain.check()
            results.append((out.clone(), x_out.clone()))
    finally:
        lib.w8a8_set_gmsq_fused_requant(0)
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    assert lib.w8a8_pipeline_error(None) == 0


def test_moe_ffn_step_argument_checks(ops):
    """The C++ step function validates its description before it touches the GPU."""
    import ctypes

    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()
    step = L.MoeFfnStep()
    assert lib.w8a8_moe_ffn_step_workspace_size(ctypes.byref(step)) == 0
    step.world, step.rank, step.num_experts, step.topk, step.dtype = 1, 0, 8, 2, L.DT_BF16
    step.tokens, step.hidden, step.inter, step.cap_rows, step.home_rows = 16, 64, 32, 64, 32
    need = lib.w8a8_moe_ffn_step_workspace_size(ctypes.byref(step))
    assert need > 16 * 64
    p = 4096
    assert lib.w8a8_moe_ffn_step(ctypes.byref(step), p, p, p, 1e-6, p, p, p, p, None) == L.ERR_INVALID  # no buffers
    step.num_experts = 7
    step.world = 2
    assert lib.w8a8_moe_ffn_step_workspace_size(ctypes.byref(step)) == 0  # experts not divisible by ranks
    assert lib.w8a8_ep_comm_create(None, 2, 0, None) == L.ERR_INVALID
    assert lib.w8a8_ep_comm_destroy(None) == L.OK


@pytest.mark.parametrize("tok_dtype", [torch.int8, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cnt_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("n,e,h,spare", [(4, 6, 64, 0), (8, 32, 7168, 5), (1, 1, 24, 0), (3, 300, 10, 2)])
def test_moe_re_routing_matches_oracle(ops, oracle, tok_dtype, cnt_dtype, n, e, h, spare):
    rng = np.random.default_rng(seed_of(n, e, h, str(tok_dtype), str(cnt_dtype)))
    cnt = rng.integers(0, 6, (n, e))
    if n > 1:
        cnt[rng.integers(0, n), :] = 0      # a rank that sent nothing
    if e > 1:
        cnt[:, rng.integers(0, e)] = 0      # an expert that received nothing
    cnt[0, 0] += 1
    a = int(cnt.sum()) + spare
    if tok_dtype == torch.int8:
        tok = rng.integers(-128, 128, (a, h)).astype(np.int8)
    else:
        tok = rng.integers(0, 1 << 16, (a, h)).astype(np.uint16)   # any bit pattern, NaNs included
    scl = rng.standard_normal(a).astype(np.float32)
    want_tok, want_scl, want_idx, want_num = oracle.moe_re_routing(tok, cnt, scl)
    t_tok = torch.from_numpy(tok.view(np.int16) if tok.dtype == np.uint16 else tok).cuda()
    if tok_dtype != torch.int8:
        t_tok = t_tok.view(tok_dtype)
    t_cnt = torch.from_numpy(cnt).to(cnt_dtype).cuda()
    routed = a - spare
    for with_scales in (True, False):
        got_tok, got_scl, got_idx, got_num = ops.moe_re_routing(t_tok, t_cnt, torch.from_numpy(scl).cuda()
                                                                if with_scales else None)
        assert got_tok.dtype == tok_dtype and got_idx.dtype == torch.int32 and got_num.dtype == cnt_dtype
        raw = got_tok.view(torch.int16) if tok_dtype != torch.int8 else got_tok
        assert np.array_equal(raw.cpu().numpy().view(tok.dtype)[:routed], want_tok[:routed])
        assert np.array_equal(got_idx.cpu().numpy()[:routed], want_idx[:routed])
        assert np.array_equal(got_num.cpu().numpy(), want_num)
        if with_scales:
            assert np.array_equal(got_scl.cpu().numpy()[:routed].view(np.uint32), want_scl[:routed].view(np.uint32))


def test_moe_re_routing_flags_bad_counts_and_empty_inputs(ops):
    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()
    tok = torch.full((8, 32), 7, dtype=torch.int8, device="cuda")
    out = torch.zeros_like(tok)
    idx = torch.full((8,), -5, dtype=torch.int32, device="cuda")
    num = torch.zeros((2,), dtype=torch.int32, device="cuda")
    ws = torch.empty((lib.w8a8_moe_re_routing_workspace_size(8, 2, 2),), dtype=torch.uint8, device="cuda")
    for bad in ([[5, 4], [0, 0]], [[1, -1], [2, 2]]):       # more rows than A; a negative count
        cnt = torch.tensor(bad, dtype=torch.int32, device="cuda")
        rc = lib.w8a8_moe_re_routing(tok.data_ptr(), cnt.data_ptr(), None, out.data_ptr(), None, idx.data_ptr(),
                                     num.data_ptr(), 8, 32, 2, 2, 4, ws.data_ptr(), ws.numel(), None)
        assert rc == L.OK
        assert lib.w8a8_workspace_error(ws.data_ptr(), None) == 1
        assert not out.any() and (idx == -5).all()
    cnt = torch.tensor([[1, 2], [3, 2]], dtype=torch.int32, device="cuda")
    rc = lib.w8a8_moe_re_routing(tok.data_ptr(), cnt.data_ptr(), None, out.data_ptr(), None, idx.data_ptr(),
                                 num.data_ptr(), 8, 32, 2, 2, 4, ws.data_ptr(), ws.numel(), None)
    assert rc == L.OK and lib.w8a8_workspace_error(ws.data_ptr(), None) == 0
    assert (out == 7).all() and num.tolist() == [4, 4]
    # empty token buffer: outputs come back with the reference's shapes and nothing is launched
    e_tok, e_scl, e_idx, e_num = ops.moe_re_routing(tok[:0], torch.zeros((2, 3), dtype=torch.int64, device="cuda"))
    assert e_tok.shape == (0, 32) and e_scl.shape == (0,) and e_idx.shape == (0,) and e_num.shape == (3,)


_T = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}


def _to_oracle(t: torch.Tensor):
    return t.cpu().numpy() if t.dtype == torch.float32 else bits(t)


def _code(oracle, dt):
    return {torch.float16: oracle.DT_F16, torch.bfloat16: oracle.DT_BF16, torch.float32: oracle.DT_F32}[dt]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("scale_dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mode", [0, 2])
@pytest.mark.parametrize("r,k,h,e", [(33, 8, 7168, 16), (7, 3, 100, 4), (5, 1, 8, 2), (64, 20, 256, 300)])
def test_moe_finalize_routing_matches_oracle(ops, oracle, dtype, scale_dtype, mode, r, k, h, e):
    g = torch.Generator(device="cuda").manual_seed(seed_of(_T[dtype], _T[scale_dtype], mode, r, k, h, e))
    num_dst = r * k + 3
    rows = torch.randn((num_dst, h), generator=g, device="cuda").to(dtype)
    skip1 = torch.randn((r, h), generator=g, device="cuda").to(dtype)
    skip2 = torch.randn((r, h), generator=g, device="cuda").to(dtype)
    bias = torch.randn((e, h), generator=g, device="cuda").to(dtype)
    scales = torch.rand((r, k), generator=g, device="cuda").to(scale_dtype)
    esdr = torch.randint(-2, num_dst + 2, (r * k,), generator=g, device="cuda", dtype=torch.int32)  # some dropped
    expert = torch.randint(-1, e + 1, (r, k), generator=g, device="cuda", dtype=torch.int32)          # some no-bias
    variants = [dict(skip1=skip1, skip2=skip2, bias=bias, scales=scales, expert_for_source_row=expert),
                dict(scales=scales),
                dict(skip2=skip2, scales=scales, bias=bias),          # bias without expert ids: ignored
                dict(skip1=skip1, bias=bias, expert_for_source_row=expert[:, :1].contiguous()) if k == 1 else
                dict(skip1=skip1, scales=scales, expert_for_source_row=expert)]
    for kw in variants:
        got = ops.moe_finalize_routing(rows, esdr, drop_pad_mode=mode, **kw)
        okw = {}
        for name, t in kw.items():
            if name == "scales":
                okw["scales"], okw["scale_dtype"] = _to_oracle(t), _code(oracle, t.dtype)
            elif name == "expert_for_source_row":
                okw["expert"] = t.cpu().numpy()
            else:
                okw[name] = _to_oracle(t)
        if "scales" not in kw:
            n = esdr.numel()
            want = oracle.moe_finalize_routing(_to_oracle(rows), esdr.cpu().numpy(), _code(oracle, dtype),
                                               drop_pad_mode=mode, **okw)
            assert got.shape == (n, h)
        else:
            want = oracle.moe_finalize_routing(_to_oracle(rows), esdr.cpu().numpy(), _code(oracle, dtype),
                                               drop_pad_mode=mode, **okw)
        if dtype == torch.float32:
            from helpers import assert_same_f32
            assert_same_f32(got, want, f"mfr {sorted(kw)}")
        else:
            from helpers import assert_same_16
            assert_same_16(bits(got), want, _code(oracle, dtype), f"mfr {sorted(kw)}")


def test_moe_finalize_routing_many_terms_and_combine_equivalence(ops, oracle, backend):
    from cannbench_operator_solutions_b200 import _lib as L

    g = torch.Generator(device="cuda").manual_seed(77)
    # K above the staged batch: accepted for fp32 rows, rejected (clear status) for 16-bit rows
    r, k, h = 4, 200, 64
    rows = torch.randn((r * k, h), generator=g, device="cuda")
    scales = torch.rand((r, k), generator=g, device="cuda")
    esdr = torch.randperm(r * k, generator=g, device="cuda").to(torch.int32)
    got = ops.moe_finalize_routing(rows, esdr, scales=scales, drop_pad_mode=3)
    want = oracle.moe_finalize_routing(rows.cpu().numpy(), esdr.cpu().numpy(), oracle.DT_F32,
                                       scales=scales.cpu().numpy(), drop_pad_mode=3)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    with pytest.raises(RuntimeError, match="limit"):
        ops.moe_finalize_routing(rows.to(torch.bfloat16), esdr, scales=scales, drop_pad_mode=3)
    # the chain's combine step is the scales-only, row-arranged case
    t, topk, h = 40, 8, 512
    rows16 = torch.randn((t * topk, h), generator=g, device="cuda").to(torch.bfloat16)
    probs = torch.rand((t, topk), generator=g, device="cuda")
    pos = torch.randperm(t * topk, generator=g, device="cuda").view(t, topk)
    a = backend.combine(rows16, probs, pos.to(torch.int64))
    b = ops.moe_finalize_routing(rows16, pos.to(torch.int32).reshape(-1), scales=probs, drop_pad_mode=2)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,inner,k", [(37, 8, 2), (1000, 256, 8), (5, 32, 32), (64, 60, 1), (33, 1000, 6),
                                          (9, 1024, 16), (3, 3, 3)])
def test_moe_gating_top_k_softmax_matches_oracle(ops, oracle, dtype, rows, inner, k):
    g = torch.Generator(device="cuda").manual_seed(seed_of(_T[dtype], rows, inner, k))
    x = (torch.randn((rows, inner), generator=g, device="cuda") * 2).to(dtype)
    x[0] = torch.round(x[0])                      # coarse values: many exact ties in the first row
    if rows > 2:
        x[1] = 0.0                                # every probability equal
    fin = torch.rand((rows,), generator=g, device="cuda") < 0.3
    for finished in (None, fin):
        y, ei, ri = ops.moe_gating_top_k_softmax(x, finished, k)
        wy, wei, wri = oracle.moe_gating_top_k_softmax(_to_oracle(x), _code(oracle, dtype), k,
                                                       finished=None if finished is None else fin.cpu().numpy())
        assert y.shape == (rows, k) and ei.dtype == torch.int32 and ri.dtype == torch.int32
        assert np.array_equal(ei.cpu().numpy(), wei)
        assert np.array_equal(ri.cpu().numpy(), wri)
        if dtype == torch.float32:
            from helpers import assert_same_f32
            assert_same_f32(y, wy, "gating y")
        else:
            from helpers import assert_same_16
            assert_same_16(bits(y), wy, _code(oracle, dtype), "gating y")


def test_moe_gating_top_k_softmax_shapes_and_limits(ops):
    x = torch.randn((2, 3, 5, 16), device="cuda")
    y, ei, ri = ops.moe_gating_top_k_softmax(x, k=4)
    assert y.shape == (2, 3, 5, 4) and ri.view(-1, 4)[7].tolist() == [7, 37, 67, 97]
    ref = torch.softmax(x, -1).topk(4, -1)
    assert torch.equal(ei.long(), ref.indices) and torch.allclose(y, ref.values, rtol=1e-5, atol=1e-7)
    with pytest.raises(RuntimeError, match="limit"):
        ops.moe_gating_top_k_softmax(torch.zeros((2, 2048), device="cuda"), k=2)
