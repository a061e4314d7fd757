"""The workspace-free form of grouped_matmul_swiglu_quant.

Callers that cannot allocate device memory where they run the operator (inside
a stream capture, in a serving loop that received all of its memory up front,
behind an interface without an allocator) use
w8a8_grouped_matmul_swiglu_quant_static, which keeps its intermediate results in
memory built into the library.  The test drives it through the C-ABI twice in a
row, with different problems, and expects exactly the bytes the ordinary entry
point produces: int8 outputs and fp32 scales are compared bit for bit, the same
bar the other tensor-core tests use.  The second call is smaller than the first,
so anything it wrongly kept from the first call's scratch contents would show.

This file sorts last on purpose: a run that stops at the first failure has
already been through every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed, m, k, n, e, gl):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.integers(-127, 128, (m, k)).astype(np.int8)).cuda()
    w = torch.from_numpy(rng.integers(-127, 128, (e, k, n)).astype(np.int8)).cuda()
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, (e, n)).astype(np.float32)).cuda()
    xs = torch.from_numpy(rng.uniform(1e-3, 5e-2, m).astype(np.float32)).cuda()
    return x, w, ws, xs, torch.tensor(gl, dtype=torch.int64)


def _run(lib, L, static, x, w, ws, xs, gl_host):
    m, k = x.shape
    e, _, n = w.shape
    y = torch.full((m, n // 2), 77, dtype=torch.int8, device="cuda")
    ysc = torch.full((m,), -1.0, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    if static:
        rc = lib.w8a8_grouped_matmul_swiglu_quant_static(x.data_ptr(), w.data_ptr(), ws.data_ptr(), xs.data_ptr(),
                                                         y.data_ptr(), ysc.data_ptr(), m, k, n, e, gl_host.data_ptr(),
                                                         0, L.W_KN, 0, st)
    else:
        need = lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(m, k, n, e)
        wsb = torch.empty((need,), dtype=torch.uint8, device="cuda")
        rc = lib.w8a8_grouped_matmul_swiglu_quant(x.data_ptr(), w.data_ptr(), ws.data_ptr(), xs.data_ptr(),
                                                  y.data_ptr(), ysc.data_ptr(), m, k, n, e, gl_host.data_ptr(), 0,
                                                  L.W_KN, 0, wsb.data_ptr(), need, st)
    torch.cuda.synchronize()
    return rc, y, ysc


def test_static_entry_point_matches_workspace_entry_point_twice_in_a_row(ops):
    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()
    first = _problem(101, 700, 512, 1024, 6, [100, 100, 356, 357, 699, 700])
    second = _problem(202, 130, 256, 512, 3, [0, 129, 130])  # smaller: stale scratch beyond it must not matter
    for prob in (first, second):
        rc_s, y_s, ys_s = _run(lib, L, True, *prob)
        rc_w, y_w, ys_w = _run(lib, L, False, *prob)
        assert rc_s == 0 and rc_w == 0, (L.status_string(rc_s), L.status_string(rc_w))
        assert torch.equal(y_s, y_w)
        assert torch.equal(ys_s.view(torch.int32), ys_w.view(torch.int32))
        assert not bool((y_s == 77).all())


def test_static_entry_point_rejects_problems_beyond_its_scratch(ops):
    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()
    m, k, n, e = 4096, 256, 4096, 4
    assert lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(m, k, n, e) > L.STATIC_SCRATCH_BYTES
    x, w, ws, xs, gl = _problem(303, 8, k, 64, e, [2, 4, 6, 8])  # tiny buffers: the call must refuse before use
    y = torch.full((8, 32), 5, dtype=torch.int8, device="cuda")
    ysc = torch.zeros((8,), dtype=torch.float32, device="cuda")
    rc = lib.w8a8_grouped_matmul_swiglu_quant_static(x.data_ptr(), w.data_ptr(), ws.data_ptr(), xs.data_ptr(),
                                                     y.data_ptr(), ysc.data_ptr(), m, k, n, e, gl.data_ptr(), 0, L.W_KN,
                                                     0, torch.cuda.current_stream().cuda_stream)
    assert rc == L.ERR_LIMIT
    assert "capacity" in L.status_string(rc)
    torch.cuda.synchronize()
    assert bool((y == 5).all())


def test_static_entry_point_reports_a_bad_device_group_list(ops):
    """A group list that lives on the device is validated there; with this entry point the verdict sits in the
    built-in scratch the caller never sees, so it is read with w8a8_static_scratch_error."""
    from cannbench_operator_solutions_b200 import _lib as L

    lib = L.load()
    x, w, ws, xs, _ = _problem(404, 130, 256, 512, 3, [0, 129, 130])
    st = torch.cuda.current_stream().cuda_stream
    y = torch.full((130, 256), 9, dtype=torch.int8, device="cuda")
    ysc = torch.zeros((130,), dtype=torch.float32, device="cuda")
    bad = torch.tensor([50, 40, 130], dtype=torch.int64, device="cuda")   # decreasing: not a cumulative list
    rc = lib.w8a8_grouped_matmul_swiglu_quant_static(x.data_ptr(), w.data_ptr(), ws.data_ptr(), xs.data_ptr(),
                                                     y.data_ptr(), ysc.data_ptr(), 130, 256, 512, 3, bad.data_ptr(), 1,
                                                     L.W_KN, 0, st)
    assert rc == 0  # nothing is wrong that the host could see
    assert lib.w8a8_static_scratch_error(st) == 1
    assert bool((y == 9).all())  # y left untouched
    good = torch.tensor([0, 129, 130], dtype=torch.int64, device="cuda")
    rc = lib.w8a8_grouped_matmul_swiglu_quant_static(x.data_ptr(), w.data_ptr(), ws.data_ptr(), xs.data_ptr(),
                                                     y.data_ptr(), ysc.data_ptr(), 130, 256, 512, 3, good.data_ptr(), 1,
                                                     L.W_KN, 0, st)
    assert rc == 0 and lib.w8a8_static_scratch_error(st) == 0
    assert not bool((y == 9).all())
    # the dense matmuls' error word (no wait ran out in this process)
    assert lib.w8a8_pipeline_error(st) == 0
