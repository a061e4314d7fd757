"""B200-native W8A8 quantised-FFN operators behind the operator interface of
ai-jiaqian/cannbench-operator-solutions.

``ops`` holds the operator functions (same names and arguments as the
reference's ``torch.ops.cann_bench.*``), ``_lib`` the ctypes view of the C-ABI
library ``libw8a8ffn.so`` (declared in ``include/w8a8ffn.h``), ``build`` the
in-tree nvcc build.  Loading the torch plugin (``load_torch_plugin``)
additionally registers the operators as ``torch.ops.cann_bench.*``.
"""
from . import _lib, ops  # noqa: F401
from .ops import (add_rms_norm_dynamic_quant, dequant_swiglu_quant, dynamic_quant, grouped_matmul,  # noqa: F401
                  grouped_matmul_swiglu_quant, moe_finalize_routing, moe_gating_top_k_softmax,
                  moe_re_routing, quant_matmul)

__all__ = [
    "dynamic_quant", "add_rms_norm_dynamic_quant", "quant_matmul", "grouped_matmul_swiglu_quant", "grouped_matmul",
    "moe_re_routing", "moe_finalize_routing", "moe_gating_top_k_softmax", "dequant_swiglu_quant", "load_torch_plugin",
]


def load_torch_plugin() -> None:
    """Register ``torch.ops.cann_bench.*`` (C++ plugin over the same C-ABI)."""
    import os

    import torch

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libcann_bench_cuda.so")
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: run `python -m cannbench_operator_solutions_b200.build`")
    _lib.load()
    torch.ops.load_library(path)
