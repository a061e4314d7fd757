"""ctypes binding of libw8a8ffn.so (the C-ABI declared in include/w8a8ffn.h).

There is no fallback: if the shared library is missing the import of the
operators fails with instructions to build it.
"""
from __future__ import annotations

import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libw8a8ffn.so")

OK = 0
ERR_INVALID, ERR_ALIGN, ERR_GROUP_LIST, ERR_WORKSPACE, ERR_CUDA, ERR_UNSUPPORTED, ERR_LIMIT = -1, -2, -3, -4, -5, -6, -7
STATIC_SCRATCH_BYTES = (8 << 20) + (64 << 10)
DT_F16, DT_BF16, DT_F32, DT_I8, DT_I32 = 0, 1, 2, 3, 4
F_ROUND_DIRECT = 1
F_STAGE_MATMUL, F_STAGE_REQUANT = 2, 4
W_KN, W_NK = 0, 1

QM_SCALE_PERCHAN = 1 << 0
QM_SCALE_BF16 = 1 << 1
QM_HAS_OFFSET = 1 << 2
QM_OFFSET_PERCHAN = 1 << 3
QM_HAS_PT = 1 << 4
QM_BIAS_SHIFT = 5
QM_BIAS_PERCHAN = 1 << 8
QM_PT_MOD_M = 1 << 9
QM_BIAS_NONE, QM_BIAS_I32, QM_BIAS_F16, QM_BIAS_BF16, QM_BIAS_F32 = 0, 1, 2, 3, 4

# every symbol include/w8a8ffn.h declares: (name, restype, argtypes)
_vp, _i64, _i32, _f32, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
_u64 = ctypes.c_uint64
SIGNATURES = {
    "w8a8_version": (_i32, []),
    "w8a8_kernel_launch_count": (_i64, []),
    "w8a8_status_string": (ctypes.c_char_p, [_i32]),
    "w8a8_dynamic_quant": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "w8a8_add_rms_norm_dynamic_quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32, _i32, _i32, _vp]),
    "w8a8_quant_matmul": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i64,
                                 _vp]),
    "w8a8_matmul_i8_i32": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "w8a8_grouped_matmul_swiglu_quant_workspace_size": (_sz, [_i64, _i64, _i64, _i64]),
    "w8a8_grouped_matmul_swiglu_quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i32,
                                                _i32, _i32, _vp, _sz, _vp]),
    "w8a8_grouped_matmul_swiglu_quant_static": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i32,
                                                       _i32, _i32, _vp]),
    "w8a8_grouped_matmul_workspace_size": (_sz, [_i64, _i64, _i64, _i64]),
    "w8a8_grouped_matmul_f32_workspace_size": (_sz, [_i64, _i64, _i64, _i64]),
    "w8a8_grouped_matmul": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i32, _i32, _i32, _i32,
                                   _i32, _vp, _sz, _vp]),
    "w8a8_workspace_error": (_i32, [_vp, _vp]),
    "w8a8_set_gemm_shape": (_i32, [_i32]),
    "w8a8_set_gmsq_fused_requant": (_i32, [_i32]),
    "w8a8_set_gmsq_epilogue_warps": (_i32, [_i32]),
    "w8a8_pipeline_error": (_i32, [_vp]),
    "w8a8_static_scratch_error": (_i32, [_vp]),
    "w8a8_route_plan_workspace_size": (_sz, [_i64, _i64, _i64]),
    "w8a8_route_plan": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "w8a8_scatter_rows": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "w8a8_permute_rows": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    "w8a8_moe_re_routing_workspace_size": (_sz, [_i64, _i64, _i64]),
    "w8a8_moe_re_routing": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "w8a8_dispatch_rows": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "w8a8_ep_tables": (_i32, [_vp, _i64, _i64, _i64, _vp, _u64, _u64, _u64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp,
                              _vp, _vp, _vp]),
    "w8a8_expand_row_pointers": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "w8a8_grouped_matmul_to_rows": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i32, _i32, _i32,
                                           _i32, _i32, _vp, _sz, _vp]),
    "w8a8_moe_finalize_routing": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32,
                                         _i32, _i32, _vp]),
    "w8a8_moe_gating_top_k_softmax": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "w8a8_dequant_swiglu_quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _vp]),
    "w8a8_combine": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "w8a8_gmsq_host_pipe_device_bytes": (_sz, [_i64, _i64, _i64, _i64]),
    "w8a8_gmsq_host_pipe_create": (_i32, [ctypes.POINTER(_vp), _vp, _vp, _i64, _i64, _i64, _i32, _i64, _vp, _sz]),
    "w8a8_gmsq_host_pipe_run": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _i32, _vp]),
    "w8a8_gmsq_host_pipe_destroy": (_i32, [_vp]),
    "w8a8_ep_unique_id": (_i32, [_vp]),
    "w8a8_ep_comm_create": (_i32, [_vp, _i32, _i32, ctypes.POINTER(_vp)]),
    "w8a8_ep_comm_destroy": (_i32, [_vp]),
    "w8a8_moe_ffn_step_workspace_size": (_sz, [_vp]),
    "w8a8_moe_ffn_step": (_i32, [_vp, _vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp, _vp]),
    "w8a8_moe_ffn_step_status": (_i32, [_vp, _vp]),
    "w8a8_mma_issue_probe": (_i32, [_i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i64, _vp, _vp]),
    "w8a8_mma_issue_probe_ops": (_i64, [_i32, _i32, _i32, _i32, _i64]),
    "w8a8_selftest_bounded_wait": (_i32, [_i64, _vp, _vp]),
    "w8a8_selftest_exp": (_i32, [_vp, _vp]),
    "w8a8_stream_read_probe": (_i32, [_vp, _i64, _vp, _vp]),
}

class MoeFfnStep(ctypes.Structure):
    """W8A8MoeFfnStep of include/w8a8ffn.h."""
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("num_experts", ctypes.c_int32),
                ("topk", ctypes.c_int32), ("dtype", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("tokens", _i64), ("hidden", _i64), ("inter", _i64), ("cap_rows", _i64), ("home_rows", _i64),
                ("peer_base", _vp), ("local_base", _vp), ("off_x", _u64), ("off_s", _u64), ("off_back", _u64),
                ("w_up", _vp), ("s_up", _vp), ("w_down", _vp), ("s_down", _vp), ("comm", _vp), ("workspace", _vp),
                ("workspace_bytes", _sz)]


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m cannbench_operator_solutions_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().w8a8_status_string(status).decode()
