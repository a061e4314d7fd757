"""GPU parity of the expert-parallel helper kernels (routing plan, scatter, permute, combine) and of the
whole chain on one GPU, against the CPU oracle."""
import numpy as np
import pytest
import torch

from helpers import bits

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
