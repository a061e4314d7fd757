"""The torch plugin's Meta implementations (shape functions) run without a GPU: output shapes and dtypes of all nine
schemas on meta tensors, and the shape rules raising as torch errors."""
import pytest
import torch


@pytest.fixture(scope="module")
def cb():
    import cannbench_operator_solutions_b200 as pkg
    from cannbench_operator_solutions_b200 import build

    build.build_library()  # no-ops when the in-tree libraries are up to date
    build.build_plugin()
    pkg.load_torch_plugin()
    return torch.ops.cann_bench


def m(*shape, dt=torch.bfloat16):
    return torch.empty(shape, dtype=dt, device="meta")


I8, I32, F32, F16 = torch.int8, torch.int32, torch.float32, torch.float16


def sig(t):
    return tuple(t.shape), t.dtype


def test_quantising_operators(cb):
    y, s = cb.dynamic_quant(m(4, 5, 8))
    assert sig(y) == ((4, 5, 8), I8) and sig(s) == ((4, 5), F32)
    y, xo, s = cb.add_rms_norm_dynamic_quant(m(3, 16, dt=F16), m(3, 16, dt=F16), m(16, dt=F16), 1e-6)
    assert sig(y) == ((3, 16), I8) and sig(xo) == ((3, 16), F16) and sig(s) == ((3,), F32)
    y, s = cb.dequant_swiglu_quant(m(6, 64, dt=I32), m(64, dt=F32), m(6, dt=F32))
    assert sig(y) == ((6, 32), I8) and sig(s) == ((6,), F32)
    with pytest.raises(RuntimeError, match="rank >= 2"):
        cb.dynamic_quant(m(8))
    with pytest.raises(RuntimeError, match="float16 / bfloat16"):
        cb.dynamic_quant(m(2, 8, dt=F32))
    with pytest.raises(RuntimeError, match="gamma dtype must match"):
        cb.add_rms_norm_dynamic_quant(m(3, 16), m(3, 16), m(16, dt=F16), 1e-6)
    with pytest.raises(RuntimeError, match="gamma must be 1-D"):
        cb.add_rms_norm_dynamic_quant(m(3, 16), m(3, 16), m(8), 1e-6)
    with pytest.raises(RuntimeError, match="share a shape"):
        cb.add_rms_norm_dynamic_quant(m(3, 16), m(4, 16), m(16), 1e-6)
    with pytest.raises(RuntimeError, match="even last dimension"):
        cb.dequant_swiglu_quant(m(6, 63, dt=I32))


def test_matmul_operators(cb):
    out = cb.quant_matmul(m(2, 7, 40, dt=I8), m(2, 40, 24, dt=I8), m(24, dt=F32))
    assert sig(out) == ((2, 7, 24), F16)
    out = cb.quant_matmul(m(7, 40, dt=I8), m(40, 24, dt=I8), m(1, dt=F32), output_dtype="bfloat16")
    assert sig(out) == ((7, 24), torch.bfloat16)
    y, s = cb.grouped_matmul_swiglu_quant(m(10, 32, dt=I8), m(2, 32, 64, dt=I8), m(2, 64, dt=F32), m(10, dt=F32),
                                          [4, 10])
    assert sig(y) == ((10, 32), I8) and sig(s) == ((10,), F32)
    outs = cb.grouped_matmul(m(10, 32), m(3, 32, 48), [4, 4, 10])
    assert [tuple(o.shape) for o in outs] == [(4, 48), (0, 48), (6, 48)] and outs[0].dtype == torch.bfloat16
    outs = cb.grouped_matmul(m(10, 32), m(3, 48, 32), [4, 4, 10], None, 3, True)
    assert [tuple(o.shape) for o in outs] == [(10, 48)]
    outs = cb.grouped_matmul(m(10, 32, dt=I8), m(3, 32, 48, dt=I8), [4, 4, 10], None, 2, False, m(10, dt=F32),
                             m(3, 48, dt=F32))
    assert sig(outs[0]) == ((10, 48), torch.bfloat16)
    with pytest.raises(RuntimeError, match="x1.size\\(-1\\) == x2.size\\(-2\\)"):
        cb.quant_matmul(m(7, 40, dt=I8), m(41, 24, dt=I8), m(24, dt=F32))
    with pytest.raises(RuntimeError, match="N must be even"):
        cb.grouped_matmul_swiglu_quant(m(10, 32, dt=I8), m(2, 32, 63, dt=I8), m(2, 63, dt=F32), m(10, dt=F32), [4, 10])
    with pytest.raises(RuntimeError, match="must equal M"):
        cb.grouped_matmul(m(10, 32), m(3, 32, 48), [4, 4, 9])
    with pytest.raises(RuntimeError, match="x must be 2D"):
        cb.grouped_matmul(m(2, 10, 32), m(3, 32, 48), [4, 4, 10])


def test_routing_operators(cb):
    tok, scale, idx, per_expert = cb.moe_re_routing(m(12, 64, dt=I8), m(2, 3, dt=I32), m(12, dt=F32))
    assert sig(tok) == ((12, 64), I8) and sig(scale) == ((12,), F32) and sig(idx) == ((12,), I32)
    assert sig(per_expert) == ((3,), I32)
    out = cb.moe_finalize_routing(m(40, 64), m(40, dt=I32), scales=m(10, 4, dt=F32))
    assert sig(out) == ((10, 64), torch.bfloat16)
    y, ei, ri = cb.moe_gating_top_k_softmax(m(5, 7, 32, dt=F32), None, 4)
    assert sig(y) == ((5, 7, 4), F32) and sig(ei) == ((5, 7, 4), I32) and sig(ri) == ((5, 7, 4), I32)
    with pytest.raises(RuntimeError, match="tokens must be 2D"):
        cb.moe_re_routing(m(12, dt=I8), m(2, 3, dt=I32))
    with pytest.raises(RuntimeError, match="0 < k <= x.size"):
        cb.moe_gating_top_k_softmax(m(5, 8, dt=F32), None, 9)
    with pytest.raises(RuntimeError, match="bool 'finished'"):
        cb.moe_gating_top_k_softmax(m(5, 8, dt=F32), m(5, dt=I32), 2)
