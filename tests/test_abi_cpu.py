"""The C-ABI library loads without a GPU, exports every symbol the public
header declares, and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from cannbench_operator_solutions_b200 import _lib, build

    build.build_library()
    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "w8a8ffn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(w8a8_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from cannbench_operator_solutions_b200 import _lib

    names = declared_functions()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/w8a8ffn.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_status_strings(lib):
    from cannbench_operator_solutions_b200 import _lib

    assert lib.w8a8_version() >= 100
    for code in (0, -1, -2, -3, -4, -5, -6, -99):
        assert len(_lib.status_string(code)) > 0


def test_argument_validation_needs_no_gpu(lib):
    from cannbench_operator_solutions_b200 import _lib as L

    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 255) & ~255
    # zero rows: successful no-op, as in the reference plugins
    assert lib.w8a8_dynamic_quant(p, p, p, 0, 64, L.DT_BF16, 0, None) == L.OK
    assert lib.w8a8_add_rms_norm_dynamic_quant(p, p, p, p, p, p, 0, 64, 1e-6, L.DT_BF16, 0, None) == L.OK
    # dtype / shape / flag errors
    assert lib.w8a8_dynamic_quant(p, p, p, 4, 64, L.DT_F32, 0, None) == L.ERR_INVALID
    assert lib.w8a8_dynamic_quant(p, p, p, 4, 0, L.DT_BF16, 0, None) == L.ERR_INVALID
    assert lib.w8a8_dynamic_quant(p, p, p, 4, 64, L.DT_BF16, 8, None) == L.ERR_INVALID
    assert lib.w8a8_dynamic_quant(None, p, p, 4, 64, L.DT_BF16, 0, None) == L.ERR_INVALID
    assert lib.w8a8_add_rms_norm_dynamic_quant(p, p, p, p, p, p, 4, 16392, 1e-6, L.DT_BF16, 0, None) == L.ERR_INVALID
    assert lib.w8a8_quant_matmul(p, p, p, None, None, None, p, 1, 0, 16, 16, 0, L.DT_BF16, L.W_KN, 0,
                                 None) == L.ERR_INVALID
    assert lib.w8a8_quant_matmul(p, p, p, None, None, None, p, 1, 16, 24, 16, 0, L.DT_BF16, L.W_KN, 0,
                                 None) == L.ERR_UNSUPPORTED
    assert lib.w8a8_quant_matmul(p, p, p, None, None, None, p, 1, 16, 32, 32, L.QM_HAS_PT, L.DT_BF16, L.W_KN, 0,
                                 None) == L.ERR_INVALID  # pertoken flagged but missing
    assert lib.w8a8_quant_matmul(p + 1, p, p, None, None, None, p, 1, 16, 32, 32, 0, L.DT_BF16, L.W_KN, 0,
                                 None) == L.ERR_ALIGN
    # grouped: N odd, bad group lists (host lists are checked before any CUDA call), small workspace
    gl_ok = (ctypes.c_int64 * 2)(3, 8)
    gl_bad = (ctypes.c_int64 * 2)(5, 3)
    gl_short = (ctypes.c_int64 * 2)(3, 7)
    need = lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(8, 32, 64, 2)
    assert need > 8 * 32 * 4
    assert lib.w8a8_grouped_matmul_swiglu_quant(p, p, p, p, p, p, 8, 32, 63, 2, gl_ok, 0, L.W_KN, 0, p, 1 << 30,
                                                None) == L.ERR_INVALID
    assert lib.w8a8_grouped_matmul_swiglu_quant(p, p, p, p, p, p, 8, 32, 64, 2, gl_ok, 0, L.W_KN, 0, p, need - 1,
                                                None) == L.ERR_WORKSPACE
    assert lib.w8a8_grouped_matmul_swiglu_quant(p, p, p, p, p, p, 8, 32, 64, 2, gl_bad, 0, L.W_KN, 0, p, 1 << 30,
                                                None) == L.ERR_GROUP_LIST
    assert lib.w8a8_grouped_matmul_swiglu_quant(p, p, p, p, p, p, 8, 32, 64, 2, gl_short, 0, L.W_KN, 0, p, 1 << 30,
                                                None) == L.ERR_GROUP_LIST
    assert lib.w8a8_grouped_matmul_swiglu_quant(p, p, p, p, p, p, 0, 32, 64, 2, gl_ok, 0, L.W_KN, 0, None, 0,
                                                None) == L.OK
    assert lib.w8a8_grouped_matmul(p, p, None, p, None, None, 8, 64, 32, 2, gl_ok, 0, L.DT_I8, 0, L.DT_BF16, L.W_KN,
                                   p, 1 << 30, None) == L.ERR_INVALID  # int8 needs scales
    # fp32 operands answer in fp32 only, and need the larger workspace that holds their bf16 pieces
    assert lib.w8a8_grouped_matmul(p, p, None, p, None, None, 8, 64, 32, 2, gl_ok, 0, L.DT_F32, 0, L.DT_BF16, L.W_KN,
                                   p, 1 << 30, None) == L.ERR_INVALID
    small = lib.w8a8_grouped_matmul_workspace_size(8, 64, 32, 2)
    assert lib.w8a8_grouped_matmul_f32_workspace_size(8, 64, 32, 2) > small
    assert lib.w8a8_grouped_matmul(p, p, None, p, None, None, 8, 64, 32, 2, gl_ok, 0, L.DT_F32, 0, L.DT_F32, L.W_KN,
                                   p, small, None) == L.ERR_WORKSPACE
    assert lib.w8a8_grouped_matmul(p, p, None, p, p, p, 8, 64, 32, 2, gl_bad, 0, L.DT_I8, 0, L.DT_BF16, L.W_KN,
                                   p, 1 << 30, None) == L.ERR_GROUP_LIST
    assert lib.w8a8_route_plan(p, 4, 2, 8, p, p, p, p, 16, None) == L.ERR_WORKSPACE
    assert lib.w8a8_moe_re_routing(p, p, None, p, None, p, p, 4, 64, 2, 2, 2, p, 1 << 30, None) == L.ERR_INVALID
    assert lib.w8a8_moe_re_routing(p, p, None, p, None, p, p, 4, 64, 2, 2, 4, p, 16, None) == L.ERR_WORKSPACE
    assert lib.w8a8_moe_re_routing(p, p, None, p, None, p, p, 1 << 31, 64, 2, 2, 4, p, 1 << 40, None) == L.ERR_LIMIT
    assert lib.w8a8_moe_re_routing_workspace_size(4, 2, 2) >= 256 + 5 * 8 + 4 * 8 + 3 * 8 + 3 * 8 + 4 * 8
    assert lib.w8a8_moe_finalize_routing(p, p, None, None, None, None, None, p, 0, 64, 1, 0, 8, 0, L.DT_BF16,
                                         L.DT_F32, None) == L.OK
    assert lib.w8a8_moe_finalize_routing(p, p, None, None, None, None, None, p, 4, 64, 1, 0, 8, 0, L.DT_I8,
                                         L.DT_F32, None) == L.ERR_INVALID
    assert lib.w8a8_moe_finalize_routing(p, p, None, None, None, p, None, p, 4, 64, 2, 0, 8, 0, L.DT_BF16,
                                         L.DT_I8, None) == L.ERR_INVALID
    assert lib.w8a8_moe_finalize_routing(p, p, None, None, None, p, None, p, 4, 64, 129, 0, 8, 0, L.DT_BF16,
                                         L.DT_F32, None) == L.ERR_LIMIT
    assert lib.w8a8_moe_finalize_routing(p + 1, p, None, None, None, None, None, p, 4, 64, 1, 0, 8, 0, L.DT_BF16,
                                         L.DT_F32, None) == L.ERR_ALIGN
    assert lib.w8a8_moe_gating_top_k_softmax(p, None, p, p, p, 0, 64, 2, L.DT_BF16, None) == L.OK
    assert lib.w8a8_moe_gating_top_k_softmax(p, None, p, p, p, 4, 64, 65, L.DT_BF16, None) == L.ERR_INVALID
    assert lib.w8a8_moe_gating_top_k_softmax(p, None, p, p, p, 4, 64, 2, L.DT_I8, None) == L.ERR_INVALID
    assert lib.w8a8_moe_gating_top_k_softmax(p, None, p, p, p, 4, 1025, 2, L.DT_F32, None) == L.ERR_LIMIT
    assert lib.w8a8_dequant_swiglu_quant(p, p, p, None, p, p, 0, 64, L.DT_I32, 0, 0, None) == L.OK
    assert lib.w8a8_dequant_swiglu_quant(p, None, p, None, p, p, 4, 64, L.DT_I32, 0, 0, None) == L.ERR_INVALID
    assert lib.w8a8_dequant_swiglu_quant(p, p, None, None, p, p, 4, 64, L.DT_BF16, 0, 0, None) == L.ERR_INVALID
    assert lib.w8a8_dequant_swiglu_quant(p, None, None, None, p, p, 4, 64, L.DT_F32, 0, 0, None) == L.ERR_INVALID
    assert lib.w8a8_combine(p, p, p, p, 0, 2, 64, L.DT_BF16, None) == L.OK
    assert lib.w8a8_combine(p, p, p, p, 4, 2, 64, L.DT_F32, None) == L.ERR_INVALID


def test_operator_wrappers_validate_like_the_reference_plugins():
    """Shape / dtype checks raise before any device work (CPU tensors suffice to reach them)."""
    import torch

    from cannbench_operator_solutions_b200 import ops

    with pytest.raises(RuntimeError, match="rank >= 2"):
        ops.dynamic_quant(torch.zeros(8, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="float16 / bfloat16"):
        ops.dynamic_quant(torch.zeros(2, 8, dtype=torch.float32))
    with pytest.raises(RuntimeError, match="same shape"):
        ops.add_rms_norm_dynamic_quant(torch.zeros(2, 8, dtype=torch.bfloat16), torch.zeros(2, 4, dtype=torch.bfloat16),
                                       torch.zeros(8, dtype=torch.bfloat16), 1e-6)
    with pytest.raises(RuntimeError, match="int8 x1 and x2"):
        ops.quant_matmul(torch.zeros(2, 8), torch.zeros(8, 8), torch.ones(1))
    with pytest.raises(RuntimeError, match="N must be even"):
        ops.grouped_matmul_swiglu_quant(torch.zeros(2, 16, dtype=torch.int8), torch.zeros(1, 16, 7, dtype=torch.int8),
                                        torch.ones(1, 7), torch.ones(2), [2])
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.dynamic_quant(torch.zeros(2, 8, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="idx_type == 0"):
        ops.moe_re_routing(torch.zeros(2, 8, dtype=torch.int8), torch.zeros(1, 1, dtype=torch.int32), idx_type=1)
    with pytest.raises(RuntimeError, match="must be 2D \\(N, E\\)"):
        ops.moe_re_routing(torch.zeros(2, 8, dtype=torch.int8), torch.zeros(1, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="must be int32"):
        ops.moe_finalize_routing(torch.zeros(4, 8), torch.zeros(4, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="float16 / float32 / bfloat16"):
        ops.moe_finalize_routing(torch.zeros(4, 8, dtype=torch.int8), torch.zeros(4, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="K\\*NUM_ROWS"):
        ops.moe_finalize_routing(torch.zeros(4, 8), torch.zeros(5, dtype=torch.int32), scales=torch.zeros(2, 2))
    with pytest.raises(RuntimeError, match="0 < k <= x.size"):
        ops.moe_gating_top_k_softmax(torch.zeros(4, 8), k=9)
    with pytest.raises(RuntimeError, match="rank >= 2"):
        ops.moe_gating_top_k_softmax(torch.zeros(8), k=1)
    with pytest.raises(RuntimeError, match="even last dimension"):
        ops.dequant_swiglu_quant(torch.zeros(2, 7, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="2D input"):
        ops.dequant_swiglu_quant(torch.zeros(8, dtype=torch.bfloat16))
