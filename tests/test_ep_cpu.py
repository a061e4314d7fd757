"""Host logic of the expert-parallel chain on CPU: index arithmetic, and the whole
chain as world_size-2 gloo processes with a test-supplied backend that computes
each step with the CPU oracle.  The two-rank result must equal the one-rank
result bit for bit (every step is row-wise deterministic)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _from_bits(b, dtype):
    return torch.from_numpy(b.view(np.int16).copy()).view(dtype)


class OracleBackend:
    """CPU stand-in for the CUDA backend, used only to exercise the host logic."""

    def __init__(self):
        from oracle import oracle as O
        self.O = O

    def add_rms_norm_dynamic_quant(self, x1, x2, gamma, eps):
        O = self.O
        y, xo, sc = O.add_rms_norm_dynamic_quant(_bits(x1), _bits(x2), _bits(gamma), eps, O.DT_BF16)
        return torch.from_numpy(y), _from_bits(xo, torch.bfloat16), torch.from_numpy(sc)

    def route_plan(self, expert_idx, num_experts):
        cnt, cum, pos = self.O.route_count(expert_idx.numpy(), num_experts)
        return torch.from_numpy(cnt), torch.from_numpy(cum), torch.from_numpy(pos)

    def scatter_rows(self, src, src_scale, pos, total_rows):
        dst = torch.empty((total_rows, src.shape[1]), dtype=src.dtype)
        dsc = torch.empty((total_rows,), dtype=torch.float32)
        t, topk = pos.shape
        for k in range(topk):
            dst[pos[:, k]] = src
            dsc[pos[:, k]] = src_scale
        return dst, dsc

    def permute_rows(self, src, src_scale, index):
        return src[index].contiguous(), (None if src_scale is None else src_scale[index].contiguous())

    def grouped_matmul_swiglu_quant(self, x, w, w_scale, x_scale, group_list):
        y, ys = self.O.grouped_matmul_swiglu_quant(x.numpy(), w.numpy(), w_scale.numpy(), x_scale.numpy(), group_list)
        return torch.from_numpy(y), torch.from_numpy(ys)

    def grouped_matmul_int8(self, x, w, group_list, x_scale, w_scale):
        O = self.O
        out = O.grouped_matmul(x.numpy(), w.numpy(), group_list, dtype=O.DT_I8, x_scale=x_scale.numpy(),
                               w_scale=w_scale.numpy())
        return _from_bits(out, torch.bfloat16)

    def combine(self, rows, probs, pos):
        out = self.O.combine(_bits(rows), probs.numpy(), pos.numpy(), self.O.DT_BF16)
        return _from_bits(out, torch.bfloat16)


def _problem(seed=0, tokens=48, hidden=64, inter=32, experts=8, topk=2):
    rng = np.random.default_rng(seed)
    f = np.float32
    x = torch.from_numpy(rng.standard_normal((tokens, hidden)).astype(f)).to(torch.bfloat16)
    res = torch.from_numpy(rng.standard_normal((tokens, hidden)).astype(f)).to(torch.bfloat16)
    gamma = torch.from_numpy((1 + 0.1 * rng.standard_normal(hidden)).astype(f)).to(torch.bfloat16)
    logits = rng.standard_normal((tokens, experts)).astype(f)
    p = np.exp(logits - logits.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    idx = np.argsort(-p, axis=1, kind="stable")[:, :topk].astype(np.int32)
    probs = np.take_along_axis(p, idx.astype(np.int64), 1).astype(f)
    w_up = torch.from_numpy(rng.integers(-127, 128, (experts, hidden, 2 * inter)).astype(np.int8))
    s_up = torch.from_numpy(rng.uniform(1e-3, 1e-2, (experts, 2 * inter)).astype(f))
    w_dn = torch.from_numpy(rng.integers(-127, 128, (experts, inter, hidden)).astype(np.int8))
    s_dn = torch.from_numpy(rng.uniform(1e-3, 1e-2, (experts, hidden)).astype(f))
    return x, res, gamma, torch.from_numpy(idx), torch.from_numpy(probs), w_up, s_up, w_dn, s_dn


def _run_chain(rank, world, experts=8):
    from cannbench_operator_solutions_b200.ep import ExpertShard, MoeFfnChain

    x, res, gamma, idx, probs, w_up, s_up, w_dn, s_dn = _problem(experts=experts)
    el = experts // world
    tl = x.shape[0] // world
    sl_e = slice(rank * el, (rank + 1) * el)
    sl_t = slice(rank * tl, (rank + 1) * tl)
    shard = ExpertShard(w_up[sl_e].contiguous(), s_up[sl_e].contiguous(), w_dn[sl_e].contiguous(),
                        s_dn[sl_e].contiguous())
    chain = MoeFfnChain(experts, shard, backend=OracleBackend())
    out, x_out = chain.forward(x[sl_t].contiguous(), res[sl_t].contiguous(), gamma, 1e-6, idx[sl_t].contiguous(),
                               probs[sl_t].contiguous())
    return out, x_out, chain.last_counts


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out, x_out, counts = _run_chain(rank, world)
        ret[rank] = (_bits(out).copy(), _bits(x_out).copy(), counts.copy())
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_regroup_index_matches_rerouting_definition():
    from cannbench_operator_solutions_b200.ep import invert_index, regroup_index

    cnt = np.array([[2, 0, 1], [1, 3, 0]], np.int64)  # 2 ranks x 3 local experts
    src_of_dst, cum = regroup_index(cnt)
    # received buffer (rank-major): r0e0 r0e0 r0e2 | r1e0 r1e1 r1e1 r1e1 ; expert-major: e0: r0,r0,r1  e1: r1x3  e2: r0
    assert src_of_dst.tolist() == [0, 1, 3, 4, 5, 6, 2]
    assert cum.tolist() == [3, 6, 7]
    inv = invert_index(src_of_dst)
    assert inv[src_of_dst].tolist() == list(range(7))
    empty_src, empty_cum = regroup_index(np.zeros((2, 3), np.int64))
    assert empty_src.size == 0 and empty_cum.tolist() == [0, 0, 0]


@pytest.mark.timeout(300)
def test_two_rank_chain_equals_single_rank():
    single_out, single_xout, _ = _run_chain(0, 1)
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    out = np.concatenate([ret[r][0] for r in range(world)], 0)
    x_out = np.concatenate([ret[r][1] for r in range(world)], 0)
    assert np.array_equal(out, _bits(single_out))
    assert np.array_equal(x_out, _bits(single_xout))
    # conservation: every (token, k) pair arrived at exactly one expert
    total = sum(int(ret[r][2].sum()) for r in range(world))
    assert total == 48 * 2


def test_expert_placement_covers_every_row_once_and_balances_tiles():
    """The benchmark's shard of the grouped workload: both placements hand out every expert's rows exactly once;
    the replicating one balances 128-row tiles across ranks and splits experts only at tile boundaries."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench

    rng = np.random.default_rng(0)
    counts = bench.zipf_counts(rng, 131072, 256)
    for world in (1, 2, 4, 8):
        for mode in ("lpt", "replicate"):
            members, loads, replicas = bench.place_experts(counts, world, mode)
            got = np.zeros_like(counts)
            for rank_members in members:
                for e, rows in rank_members:
                    got[e] += rows
            assert np.array_equal(got, counts) and sum(loads) == int(counts.sum())
            if mode == "lpt":
                assert replicas == 0 and all(len(m) == 256 // world for m in members)
            else:
                tiles = [sum(-(-rows // 128) for _, rows in m) for m in members]
                assert max(tiles) - min(tiles) <= 2
                pieces = {}
                for rank_members in members:
                    for e, rows in rank_members:
                        pieces.setdefault(e, []).append(rows)
                for e, parts in pieces.items():     # a split expert: every piece but one is whole tiles
                    assert sum(1 for r in parts if r % 128 != 0) <= 1
    # at 8 ranks whole experts cannot balance (one expert holds more than a rank's share); replication can
    _, loads_lpt, _ = bench.place_experts(counts, 8, "lpt")
    _, loads_rep, replicas = bench.place_experts(counts, 8, "replicate")
    assert max(loads_lpt) / (sum(loads_lpt) / 8) > 1.5
    assert max(loads_rep) / (sum(loads_rep) / 8) < 1.2 and replicas >= 1


@pytest.mark.timeout(300)
def test_four_rank_chain_equals_single_rank():
    """The same check with four ranks (two experts and twelve tokens each)."""
    single_out, single_xout, _ = _run_chain(0, 1)
    world = 4
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    out = np.concatenate([ret[r][0] for r in range(world)], 0)
    x_out = np.concatenate([ret[r][1] for r in range(world)], 0)
    assert np.array_equal(out, _bits(single_out))
    assert np.array_equal(x_out, _bits(single_xout))
    assert sum(int(ret[r][2].sum()) for r in range(world)) == 48 * 2


def _worker_with_absent_peer(rank, world, port, ret):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        if rank == 1:
            ret[rank] = "left before the step"  # never posts its counts
            return
        try:
            _run_chain(rank, world)
            ret[rank] = "completed"
        except Exception as e:  # noqa: BLE001 - whatever the backend raises, it must be raised, not waited out
            ret[rank] = "error: " + type(e).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


@pytest.mark.timeout(240)
def test_a_rank_that_never_joins_the_step_is_an_error_not_a_hang():
    """Failure detection on the host: one rank leaves between steps; the other rank's count exchange ends with an
    exception inside the process group's timeout instead of waiting for ever."""
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker_with_absent_peer, args=(world, port, ret), nprocs=world, join=True)
    assert ret[1] == "left before the step"
    assert str(ret[0]).startswith("error: "), ret[0]
