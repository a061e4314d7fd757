"""GPU checks of the tensor-core layer's self-test and measurement entry points: a bounded wait that really runs
out reports error word 2 and leaves the context usable, and the MMA issue probe runs every instruction shape it
accepts without raising its error word."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from cannbench_operator_solutions_b200 import _lib as L

    return L, L.load()


def test_bounded_wait_runs_out_and_reports():
    """A barrier nothing arrives at: the wait helper the matmul kernels use gives up after the given number of SM
    cycles, the kernel ends by itself, error word 2 is set, the CTA-wide abort flag is seen by the other threads, and
    the next kernel on the same context runs normally."""
    L, lib = _lib()
    words = torch.zeros(2, dtype=torch.int32, device="cuda")
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.w8a8_selftest_bounded_wait(1_000_000, words.data_ptr(), torch.cuda.current_stream().cuda_stream)
    t1.record()
    assert rc == 0, L.status_string(rc)
    torch.cuda.synchronize()
    assert words.tolist() == [2, 1]
    assert t0.elapsed_time(t1) < 50.0  # a million cycles is about half a millisecond
    # the context is still usable
    assert int((torch.arange(8, device="cuda") * 2).sum()) == 56


def test_bounded_wait_rejects_bad_arguments():
    L, lib = _lib()
    words = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert lib.w8a8_selftest_bounded_wait(0, words.data_ptr(), None) == L.ERR_INVALID
    assert lib.w8a8_selftest_bounded_wait(1000, None, None) == L.ERR_INVALID


@pytest.mark.parametrize("cg,m,n,a_mn,b_mn,acc", [(1, 128, 256, 0, 1, 1), (1, 128, 128, 0, 0, 2), (1, 64, 64, 0, 1, 4),
                                                   (2, 256, 256, 0, 1, 2), (2, 128, 256, 0, 1, 1), (2, 256, 64, 1, 0, 4),
                                                   (2, 256, 16, 1, 0, 1), (1, 128, 32, 1, 0, 2)])
def test_mma_issue_probe_shapes(cg, m, n, a_mn, b_mn, acc):
    L, lib = _lib()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.w8a8_mma_issue_probe(cg, m, n, a_mn, b_mn, 1, acc, 8, 4, acc % 4, 2000, err.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.status_string(rc)
    torch.cuda.synchronize()
    assert int(err[0]) == 0
    assert lib.w8a8_mma_issue_probe_ops(cg, m, n, 8, 2000) > 0


def test_mma_issue_probe_rejects_bad_shapes():
    L, lib = _lib()
    for cg, m, n in [(1, 256, 256), (2, 64, 64), (3, 128, 128), (1, 128, 264), (1, 128, 8), (2, 256, 24)]:
        assert lib.w8a8_mma_issue_probe(cg, m, n, 0, 1, 0, 1, 4, 4, 0, 10, None, None) == L.ERR_INVALID
    assert lib.w8a8_mma_issue_probe(1, 128, 256, 0, 1, 0, 4, 4, 4, 0, 10, None, None) == L.ERR_INVALID
    assert lib.w8a8_mma_issue_probe(1, 128, 256, 0, 1, 0, 1, 4, 9, 0, 10, None, None) == L.ERR_INVALID


def test_exp_equals_its_defining_sequence_on_every_input():
    """The kernels' exp is an instruction-count-reduced arrangement of the sequence the CPU oracle states; the
    library compares the two on all 2^32 fp32 bit patterns."""
    L, lib = _lib()
    res = torch.zeros(2, dtype=torch.int64, device="cuda")
    rc = lib.w8a8_selftest_exp(res.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.status_string(rc)
    torch.cuda.synchronize()
    bad, first = res.tolist()
    assert bad == 0, f"{bad} patterns differ, the smallest is {first & 0xffffffff:#010x}"
    assert lib.w8a8_selftest_exp(None, None) == L.ERR_INVALID


def test_stream_read_probe_runs_and_checks_its_arguments():
    """The plain-read yardstick: reads a buffer once, writes nothing, rejects sizes and addresses that are not
    multiples of 16."""
    L, lib = _lib()
    buf = torch.randint(0, 255, (1 << 20,), dtype=torch.uint8, device="cuda")
    before = buf.clone()
    st = torch.cuda.current_stream().cuda_stream
    assert lib.w8a8_stream_read_probe(buf.data_ptr(), buf.numel(), None, st) == 0
    assert lib.w8a8_stream_read_probe(buf.data_ptr(), 0, None, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(buf, before)
    assert lib.w8a8_stream_read_probe(buf.data_ptr(), 24, None, st) == L.ERR_INVALID
    assert lib.w8a8_stream_read_probe(buf.data_ptr() + 8, 32, None, st) == L.ERR_INVALID
    assert lib.w8a8_stream_read_probe(None, 32, None, st) == L.ERR_INVALID
