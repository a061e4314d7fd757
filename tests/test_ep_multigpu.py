"""Expert-parallel chain on two GPUs (skipped when fewer are visible): both transports -- NCCL all-to-all and the
fused peer-memory stores -- must reproduce the single-rank result bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


# the NCCL all-to-all transport; peer stores with host-built tables; peer stores with device-built tables as one call
# of the library's C++ step function (its own NCCL communicator), and as the Python sequence of the same calls
TRANSPORTS = ("nccl", "p2p", "p2p-device-tables", "p2p-device-tables-python")


def _worker(rank, world, port, experts, ret):
    import torch.distributed as dist

    from test_ep_cpu import _bits, _problem

    from cannbench_operator_solutions_b200.ep import ExpertShard, MoeFfnChain

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        x, res, gamma, idx, probs, w_up, s_up, w_dn, s_dn = _problem(seed=9, tokens=512, hidden=512, inter=256,
                                                                     experts=experts, topk=4)
        el, tl = experts // world, x.shape[0] // world
        se, st = slice(rank * el, (rank + 1) * el), slice(rank * tl, (rank + 1) * tl)
        shard = ExpertShard(w_up[se].contiguous().to(dev), s_up[se].contiguous().to(dev),
                            w_dn[se].contiguous().to(dev), s_dn[se].contiguous().to(dev))
        args = (x[st].contiguous().to(dev), res[st].contiguous().to(dev), gamma.to(dev), 1e-6,
                idx[st].contiguous().to(dev), probs[st].contiguous().to(dev))
        out = {}
        for transport in TRANSPORTS:
            chain = MoeFfnChain(experts, shard, transport=transport.split("-")[0],
                                device_tables="device-tables" in transport,
                                native_step=not transport.endswith("python"))
            for _ in range(2):
                o, xo = chain.forward(*args)
            torch.cuda.synchronize()
            chain.check()
            out[transport] = (_bits(o.cpu()).copy(), _bits(xo.cpu()).copy())
        ret[rank] = out
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_gpu_chain_both_transports_equal_single_rank(ops):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from test_ep_cpu import _bits, _problem

    from cannbench_operator_solutions_b200.ep import ExpertShard, MoeFfnChain

    experts = 16
    x, res, gamma, idx, probs, w_up, s_up, w_dn, s_dn = _problem(seed=9, tokens=512, hidden=512, inter=256,
                                                                 experts=experts, topk=4)
    dev = "cuda:0"
    single = MoeFfnChain(experts, ExpertShard(w_up.to(dev), s_up.to(dev), w_dn.to(dev), s_dn.to(dev)))
    want, want_x = single.forward(x.to(dev), res.to(dev), gamma.to(dev), 1e-6, idx.to(dev), probs.to(dev))
    want, want_x = _bits(want.cpu()), _bits(want_x.cpu())

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, experts, ret), nprocs=2, join=True)
    for transport in TRANSPORTS:
        got = np.concatenate([ret[r][transport][0] for r in range(2)], 0)
        got_x = np.concatenate([ret[r][transport][1] for r in range(2)], 0)
        assert np.array_equal(got_x, want_x), transport
        assert np.array_equal(got, want), transport
