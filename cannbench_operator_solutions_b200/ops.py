"""The reference's operator interface, backed by libw8a8ffn.so on B200.

Each function keeps the name, argument order, argument meaning and error
behaviour of the corresponding ``torch.ops.cann_bench.*`` operator of
ai-jiaqian/cannbench-operator-solutions (schemas cited per function; paths
relative to that project).  Validation mirrors the reference plugins'
``TORCH_CHECK``s and raises ``RuntimeError`` like they do.  The work itself is
one call through the C-ABI on the current CUDA stream; PyTorch only provides
device memory and the stream.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import torch

from . import _lib as L


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _status(rc: int, op: str) -> None:
    if rc != L.OK:
        raise RuntimeError(f"{op}: {L.status_string(rc)} (status {rc})")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return L.DT_F16
    if t.dtype == torch.bfloat16:
        return L.DT_BF16
    if t.dtype == torch.float32:
        return L.DT_F32
    if t.dtype == torch.int8:
        return L.DT_I8
    if t.dtype == torch.int32:
        return L.DT_I32
    raise RuntimeError(f"unsupported dtype {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("w8a8ffn operators run on CUDA tensors only (there is no CPU path)")


# ---------------------------------------------------------------------------
def dynamic_quant(x: torch.Tensor, *, round_direct: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``dynamic_quant(Tensor x) -> (Tensor y, Tensor scale)``
    (operators/dynamicquant/csrc/ops/dynamic_quant/op_plugin/dynamic_quant_plugin.cpp:30,33-87)."""
    _check(x.dim() >= 2, "dynamic_quant requires a tensor with rank >= 2.")
    _check(x.dtype in (torch.float16, torch.bfloat16), "dynamic_quant only supports float16 / bfloat16 inputs.")
    _need_cuda(x)
    xc = x.contiguous()
    y = torch.empty_like(xc, dtype=torch.int8)
    scale = torch.empty(xc.shape[:-1], dtype=torch.float32, device=xc.device)
    n = xc.size(-1)
    _check(n > 0, "dynamic_quant requires a non-zero last dimension.")
    m = xc.numel() // n
    if m <= 0:
        return y, scale
    with torch.cuda.device(xc.device):
        rc = L.load().w8a8_dynamic_quant(xc.data_ptr(), y.data_ptr(), scale.data_ptr(), m, n, _dt(xc),
                                         L.F_ROUND_DIRECT if round_direct else 0, _stream())
    _status(rc, "dynamic_quant")
    return y, scale


def add_rms_norm_dynamic_quant(x1: torch.Tensor, x2: torch.Tensor, gamma: torch.Tensor, epsilon: float, *,
                               round_direct: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``add_rms_norm_dynamic_quant(Tensor x1, Tensor x2, Tensor gamma, float epsilon) -> (y, xOut, scaleOut)``
    (operators/addrmsnormdynamicquant/csrc/ops/add_rms_norm_dynamic_quant/op_plugin/add_rms_norm_dynamic_quant_plugin.cpp:32,36-112)."""
    _check(x1.dim() >= 1, "add_rms_norm_dynamic_quant: x1 must have at least one dimension.")
    _check(x1.shape == x2.shape, "add_rms_norm_dynamic_quant: x1 and x2 must have the same shape.")
    _check(gamma.dim() == 1 and gamma.size(0) == x1.size(-1),
           "add_rms_norm_dynamic_quant: gamma must be 1-D with the size of the last dimension.")
    _check(x1.dtype == x2.dtype == gamma.dtype, "add_rms_norm_dynamic_quant: x1, x2 and gamma must share a dtype.")
    _need_cuda(x1, x2, gamma)
    x1c, x2c, gc = x1.contiguous(), x2.contiguous(), gamma.contiguous()
    y = torch.empty_like(x1c, dtype=torch.int8)
    x_out = torch.empty_like(x1c)
    scale = torch.empty(x1c.shape[:-1], dtype=torch.float32, device=x1c.device)
    n = x1c.size(-1)
    if x1c.numel() == 0 or n <= 0:
        return y, x_out, scale
    _check(x1c.dtype in (torch.float16, torch.bfloat16),
           "add_rms_norm_dynamic_quant: only float16/bfloat16 inputs are supported.")
    _check(n <= 16384, "add_rms_norm_dynamic_quant: row length must not exceed 16384.")
    rows = x1c.numel() // n
    with torch.cuda.device(x1c.device):
        rc = L.load().w8a8_add_rms_norm_dynamic_quant(x1c.data_ptr(), x2c.data_ptr(), gc.data_ptr(), y.data_ptr(),
                                                      x_out.data_ptr(), scale.data_ptr(), rows, n, float(epsilon),
                                                      _dt(x1c), L.F_ROUND_DIRECT if round_direct else 0, _stream())
    _status(rc, "add_rms_norm_dynamic_quant")
    return y, x_out, scale


def quant_matmul(x1: torch.Tensor, x2: torch.Tensor, scale: torch.Tensor, *, offset: Optional[torch.Tensor] = None,
                 pertoken_scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                 output_dtype: Optional[str] = None, transpose_x2: bool = False) -> torch.Tensor:
    """``quant_matmul(Tensor x1, Tensor x2, Tensor scale, *, Tensor? offset, Tensor? pertoken_scale, Tensor? bias,
    str? output_dtype) -> Tensor`` (operators/quantmatmul/csrc/ops/quant_matmul/op_plugin/quant_matmul_plugin.cpp:48-49,77-267).

    ``transpose_x2=True`` (not in the reference) takes x2 as [..., N, K]."""
    _check(x1.dtype == torch.int8 and x2.dtype == torch.int8, "quant_matmul requires int8 x1 and x2.")
    _check(x1.is_contiguous() and x2.is_contiguous() and scale.is_contiguous(),
           "quant_matmul requires contiguous x1/x2/scale.")
    _check(scale.dtype in (torch.float32, torch.bfloat16), "quant_matmul requires float32 or bfloat16 scale.")
    _check(x1.dim() >= 2 and x2.dim() >= 2 and x1.dim() == x2.dim(), "quant_matmul expects equal ranks >= 2.")
    k = x1.size(-1)
    m = x1.size(-2)
    n = x2.size(-2) if transpose_x2 else x2.size(-1)
    _check(k == (x2.size(-1) if transpose_x2 else x2.size(-2)), "quant_matmul requires x1.size(-1) == x2.size(-2).")
    _check(k > 0 and m > 0 and n > 0, "quant_matmul requires non-empty shapes.")
    _need_cuda(x1, x2, scale, offset, pertoken_scale, bias)
    batch = 1
    for d in range(x1.dim() - 2):
        _check(x1.size(d) == x2.size(d), "quant_matmul expects matching leading batch dimensions.")
        batch *= x1.size(d)
    bf16out = output_dtype == "bfloat16"
    out = torch.empty(tuple(x1.shape[:-1]) + (n,), dtype=torch.bfloat16 if bf16out else torch.float16,
                      device=x1.device)
    flags = 0
    _check(scale.numel() in (1, n), "quant_matmul expects scale length 1 or n.")
    if scale.numel() > 1:
        flags |= L.QM_SCALE_PERCHAN
    if scale.dtype == torch.bfloat16:
        flags |= L.QM_SCALE_BF16
    if offset is not None:
        _check(offset.dtype == torch.float32 and offset.is_contiguous(),
               "quant_matmul requires float32 contiguous offset.")
        _check(offset.numel() in (1, n), "quant_matmul expects offset length 1 or n.")
        flags |= L.QM_HAS_OFFSET
        if offset.numel() > 1:
            flags |= L.QM_OFFSET_PERCHAN
    if pertoken_scale is not None:
        _check(pertoken_scale.dtype == torch.float32 and pertoken_scale.is_contiguous(),
               "quant_matmul requires float32 contiguous pertoken_scale.")
        _check(pertoken_scale.numel() == m, "quant_matmul expects pertoken_scale length m.")
        flags |= L.QM_HAS_PT
    bias_batch_stride = 0
    if bias is not None:
        _check(bias.is_contiguous(), "quant_matmul requires contiguous bias.")
        kind = {torch.int32: L.QM_BIAS_I32, torch.float16: L.QM_BIAS_F16, torch.bfloat16: L.QM_BIAS_BF16,
                torch.float32: L.QM_BIAS_F32}.get(bias.dtype)
        _check(kind is not None, f"quant_matmul unsupported bias dtype: {bias.dtype}")
        if bias.dim() == 3 and bias.size(1) == 1 and bias.size(2) == n and batch > 1 and bias.size(0) == batch:
            bias_batch_stride = n
            perchan = n > 1
        else:
            _check(bias.numel() in (1, n), "quant_matmul expects bias length 1 or n.")
            perchan = bias.numel() > 1
        flags |= kind << L.QM_BIAS_SHIFT
        if perchan:
            flags |= L.QM_BIAS_PERCHAN
    if batch > 1:
        flags |= L.QM_PT_MOD_M
    with torch.cuda.device(x1.device):
        rc = L.load().w8a8_quant_matmul(x1.data_ptr(), x2.data_ptr(), scale.data_ptr(), _ptr(offset),
                                        _ptr(pertoken_scale), _ptr(bias), out.data_ptr(), batch, m, n, k, flags,
                                        L.DT_BF16 if bf16out else L.DT_F16, L.W_NK if transpose_x2 else L.W_KN,
                                        bias_batch_stride, _stream())
    _status(rc, "quant_matmul")
    return out


GroupList = Union[Sequence[int], torch.Tensor]


def _group_list(group_list: GroupList, e: int, m: int, op: str):
    """Returns (pointer, on_device, keepalive).  A Python sequence is the reference's host attribute and is
    validated here exactly like the plugins do; a CUDA int64 tensor is passed through untouched."""
    if isinstance(group_list, torch.Tensor) and group_list.is_cuda:
        _check(group_list.dtype == torch.int64 and group_list.is_contiguous() and group_list.numel() == e,
               f"{op}: a device group_list must be a contiguous int64 tensor of length E")
        return group_list.data_ptr(), 1, group_list
    vals = [int(v) for v in (group_list.tolist() if isinstance(group_list, torch.Tensor) else group_list)]
    _check(len(vals) == e, f"{op}: group_list length must equal the expert count")
    prev = 0
    for v in vals:
        _check(prev <= v <= m, f"{op}: group_list must be a cumsum <= M")
        prev = v
    _check(prev == m, f"{op}: group_list[-1] must equal M")
    host = torch.tensor(vals, dtype=torch.int64)
    return host.data_ptr(), 0, host


def grouped_matmul_swiglu_quant(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                                x_scale: torch.Tensor, group_list: GroupList, *, transpose_weight: bool = False,
                                round_direct: bool = False,
                                workspace: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``grouped_matmul_swiglu_quant(Tensor x, Tensor weight, Tensor weight_scale, Tensor x_scale, int[] group_list)
    -> (Tensor y, Tensor y_scale)`` (operators/groupedmatmulswigluquant/csrc/ops/grouped_matmul_swiglu_quant/op_plugin/gmsq_plugin.cpp:40-41,67-145).

    Beyond the reference: any expert count (the reference stops at 64), ``group_list`` may be a CUDA int64
    tensor, ``transpose_weight=True`` takes weight as [E, N, K], and a caller-owned ``workspace`` avoids the
    per-call allocation."""
    _check(x.dim() == 2, "grouped_matmul_swiglu_quant: x must be 2D [M, K]")
    _check(weight.dim() == 3, "grouped_matmul_swiglu_quant: weight must be 3D [E, K, N]")
    _check(x.dtype == torch.int8, "grouped_matmul_swiglu_quant: x must be int8")
    _check(weight.dtype == torch.int8, "grouped_matmul_swiglu_quant: weight must be int8")
    _check(weight_scale.dtype == torch.float32, "grouped_matmul_swiglu_quant: weight_scale must be float32")
    _check(x_scale.dtype == torch.float32, "grouped_matmul_swiglu_quant: x_scale must be float32")
    _check((weight.size(1) if transpose_weight else weight.size(2)) % 2 == 0,
           "grouped_matmul_swiglu_quant: N must be even")
    _need_cuda(x, weight, weight_scale, x_scale)
    xc, wc, wsc, xsc = x.contiguous(), weight.contiguous(), weight_scale.contiguous(), x_scale.contiguous()
    m, k = xc.shape
    e = wc.size(0)
    n = wc.size(1) if transpose_weight else wc.size(2)
    y = torch.empty((m, n // 2), dtype=torch.int8, device=xc.device)
    y_scale = torch.empty((m,), dtype=torch.float32, device=xc.device)
    if m == 0 or n == 0 or e == 0:
        return y, y_scale
    _check((wc.size(2) if transpose_weight else wc.size(1)) == k,
           "grouped_matmul_swiglu_quant: K mismatch between x and weight")
    _check(xsc.numel() == m, "grouped_matmul_swiglu_quant: x_scale must have M elements")
    _check(wsc.dim() == 2 and wsc.size(0) == e and wsc.size(1) == n,
           "grouped_matmul_swiglu_quant: weight_scale must be [E, N]")
    gl_ptr, on_dev, keep = _group_list(group_list, e, m, "grouped_matmul_swiglu_quant")
    lib = L.load()
    need = lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(m, k, n, e)
    if workspace is None:
        workspace = torch.empty((need,), dtype=torch.uint8, device=xc.device)
    _check(workspace.is_cuda and workspace.numel() * workspace.element_size() >= need,
           "grouped_matmul_swiglu_quant: workspace too small")
    with torch.cuda.device(xc.device):
        rc = lib.w8a8_grouped_matmul_swiglu_quant(xc.data_ptr(), wc.data_ptr(), wsc.data_ptr(), xsc.data_ptr(),
                                                  y.data_ptr(), y_scale.data_ptr(), m, k, n, e, gl_ptr, on_dev,
                                                  L.W_NK if transpose_weight else L.W_KN,
                                                  L.F_ROUND_DIRECT if round_direct else 0, workspace.data_ptr(),
                                                  workspace.numel() * workspace.element_size(), _stream())
    del keep
    _status(rc, "grouped_matmul_swiglu_quant")
    return y, y_scale


def grouped_matmul(x: torch.Tensor, weight: torch.Tensor, group_list: GroupList,
                   bias: Optional[torch.Tensor] = None, split_item: int = 0, transpose_weight: bool = False, *,
                   x_scale: Optional[torch.Tensor] = None, weight_scale: Optional[torch.Tensor] = None,
                   output_dtype: Optional[torch.dtype] = None,
                   workspace: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """``grouped_matmul(Tensor x, Tensor weight, int[] group_list, Tensor? bias=None, int split_item=0,
    bool transpose_weight=False) -> Tensor[]`` (operators/groupedmatmul/csrc/ops/grouped_matmul/op_plugin/grouped_matmul_plugin.cpp:42-43,120-183).

    ``split_item`` 0/1 returns one view per expert of the joined [M, N] result, 2/3 the joined tensor
    (grouped_matmul_plugin.cpp:65-80).  Beyond the reference: int8 ``x``/``weight`` with ``x_scale`` [M] and
    ``weight_scale`` [E, N] (the quantised down projection; output ``output_dtype``, default bfloat16), any
    expert count, device group lists."""
    _check(x.dim() == 2, "grouped_matmul: x must be 2D [M, K]")
    _check(weight.dim() == 3, "grouped_matmul: weight must be 3D [E, K, N] or [E, N, K]")
    _need_cuda(x, weight, bias, x_scale, weight_scale)
    xc, wc = x.contiguous(), weight.contiguous()
    m, k = xc.shape
    e = wc.size(0)
    _check(e >= 1, "grouped_matmul: weight must contain at least one expert")
    n = wc.size(1) if transpose_weight else wc.size(2)
    _check((wc.size(2) if transpose_weight else wc.size(1)) == k,
           "grouped_matmul: K dimension mismatch between x and weight")
    _check(xc.dtype == wc.dtype, "grouped_matmul: x and weight must share a dtype")
    dt = _dt(xc)
    quant = dt == L.DT_I8
    if quant:
        _check(x_scale is not None and weight_scale is not None,
               "grouped_matmul: int8 inputs need x_scale and weight_scale")
        _check(x_scale.dtype == torch.float32 and x_scale.numel() == m, "grouped_matmul: x_scale must be fp32 [M]")
        _check(weight_scale.dtype == torch.float32 and weight_scale.numel() == e * n,
               "grouped_matmul: weight_scale must be fp32 [E, N]")
        out_dtype = output_dtype or torch.bfloat16
        _check(out_dtype in (torch.bfloat16, torch.float16), "grouped_matmul: output_dtype must be fp16 or bf16")
    else:
        _check(dt in (L.DT_F16, L.DT_BF16, L.DT_F32), "grouped_matmul: unsupported dtype")
        _check(x_scale is None and weight_scale is None, "grouped_matmul: scales are only valid with int8 inputs")
        out_dtype = xc.dtype
    bc = None
    if bias is not None:
        bc = bias.contiguous()
        _check(bc.numel() == e * n, "grouped_matmul: bias must have shape [E, N]")
    gl_ptr, on_dev, keep = _group_list(group_list, e, m, "grouped_matmul")
    y = torch.empty((m, n), dtype=out_dtype, device=xc.device)
    if m > 0:
        lib = L.load()
        need = (lib.w8a8_grouped_matmul_f32_workspace_size(m, n, k, e) if dt == L.DT_F32
                else lib.w8a8_grouped_matmul_workspace_size(m, n, k, e))
        if workspace is None:
            workspace = torch.empty((max(need, 1),), dtype=torch.uint8, device=xc.device)
        _check(workspace.numel() * workspace.element_size() >= need, "grouped_matmul: workspace too small")
        xs = x_scale.contiguous() if x_scale is not None else None
        ws = weight_scale.contiguous() if weight_scale is not None else None
        with torch.cuda.device(xc.device):
            rc = lib.w8a8_grouped_matmul(xc.data_ptr(), wc.data_ptr(), _ptr(bc), y.data_ptr(), _ptr(xs), _ptr(ws), m,
                                         n, k, e, gl_ptr, on_dev, dt, _dt(bc) if bc is not None else dt,
                                         _dt(y), L.W_NK if transpose_weight else L.W_KN, workspace.data_ptr(),
                                         workspace.numel() * workspace.element_size(), _stream())
        _status(rc, "grouped_matmul")
    del keep
    if split_item in (0, 1):
        _check(not (isinstance(group_list, torch.Tensor) and group_list.is_cuda),
               "grouped_matmul: split_item 0/1 needs a host group_list to build the per-expert views")
        ends = [int(v) for v in group_list]
        outs, s = [], 0
        for v in ends:
            outs.append(y.narrow(0, s, v - s))
            s = v
        return outs
    return [y]


def moe_re_routing(tokens: torch.Tensor, expert_token_num_per_rank: torch.Tensor,
                   per_token_scales: Optional[torch.Tensor] = None, expert_token_num_type: int = 1,
                   idx_type: int = 0, *, workspace: Optional[torch.Tensor] = None
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``moe_re_routing(Tensor tokens, Tensor expert_token_num_per_rank, Tensor? per_token_scales=None,
    int expert_token_num_type=1, int idx_type=0) -> (permute_tokens, permute_per_token_scales, permute_token_idx,
    expert_token_num)`` (operators/moererouting/csrc/ops/moe_re_routing/op_plugin/moe_re_routing_plugin.cpp:34-38,
    72-161).

    ``tokens`` [A, H] fp16 / bf16 / int8 in rank-major, expert-minor order (what an all-to-all delivers);
    ``expert_token_num_per_rank`` [N, E] int32 / int64 on the device.  Rows come back expert-major.  As in the
    reference ``expert_token_num_type`` is accepted and ignored (counts are always returned), ``idx_type`` must be
    0, and without ``per_token_scales`` the scale output is allocated but not written.  The whole path runs on the
    device: the count matrix is never read by the host."""
    del expert_token_num_type
    _check(idx_type == 0, "moe_re_routing: only gather index mode (idx_type == 0) is supported.")
    _check(tokens.dim() == 2, "moe_re_routing: tokens must be 2D (A, H).")
    _check(expert_token_num_per_rank.dim() == 2, "moe_re_routing: expert_token_num_per_rank must be 2D (N, E).")
    _need_cuda(tokens, expert_token_num_per_rank, per_token_scales)
    tok = tokens.contiguous()
    cnt = expert_token_num_per_rank.contiguous()
    scl = None
    if per_token_scales is not None:
        scl = per_token_scales.contiguous()
        _check(scl.dtype == torch.float32, "moe_re_routing: per_token_scales must be float32.")
    a, h = tok.shape
    n, e = cnt.shape
    out_tok = torch.empty_like(tok)
    out_scl = torch.empty((a,), dtype=torch.float32, device=tok.device)
    out_idx = torch.empty((a,), dtype=torch.int32, device=tok.device)
    out_num = torch.empty((e,), dtype=cnt.dtype, device=tok.device)
    if a <= 0 or h <= 0 or n <= 0 or e <= 0:
        return out_tok, out_scl, out_idx, out_num
    _check(tok.dtype in (torch.float16, torch.bfloat16, torch.int8), "moe_re_routing: unsupported tokens dtype.")
    _check(cnt.dtype in (torch.int32, torch.int64), "moe_re_routing: unsupported expert_token_num_per_rank dtype.")
    if scl is not None:
        _check(scl.numel() == a, "moe_re_routing: per_token_scales must have A elements.")
    lib = L.load()
    need = lib.w8a8_moe_re_routing_workspace_size(a, n, e)
    if workspace is None:
        workspace = torch.empty((need,), dtype=torch.uint8, device=tok.device)
    _check(workspace.numel() * workspace.element_size() >= need, "moe_re_routing: workspace too small")
    with torch.cuda.device(tok.device):
        rc = lib.w8a8_moe_re_routing(tok.data_ptr(), cnt.data_ptr(), _ptr(scl), out_tok.data_ptr(),
                                     out_scl.data_ptr(), out_idx.data_ptr(), out_num.data_ptr(), a,
                                     h * tok.element_size(), n, e, cnt.element_size(), workspace.data_ptr(),
                                     workspace.numel() * workspace.element_size(), _stream())
    _status(rc, "moe_re_routing")
    return out_tok, out_scl, out_idx, out_num


def moe_finalize_routing(expanded_permuted_rows: torch.Tensor, expanded_src_to_dst_row: torch.Tensor,
                         skip1: Optional[torch.Tensor] = None, skip2: Optional[torch.Tensor] = None,
                         bias: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None,
                         expert_for_source_row: Optional[torch.Tensor] = None, drop_pad_mode: int = 0) -> torch.Tensor:
    """``moe_finalize_routing(Tensor expanded_permuted_rows, Tensor expanded_src_to_dst_row, Tensor? skip1=None,
    Tensor? skip2=None, Tensor? bias=None, Tensor? scales=None, Tensor? expert_for_source_row=None,
    int drop_pad_mode=0) -> Tensor out``
    (operators/moefinalizerouting/csrc/ops/moe_finalize_routing/op_plugin/moe_finalize_routing_plugin.cpp:31-36,
    40-58 for the shape rules, 96-215 for the checks).

    ``out[i] = skip1[i] + skip2[i] + sum_k scales[i, k] * (rows[p(i, k)] + bias[expert[i, k]])``; K is
    ``scales.size(1)`` (1 without scales), ``num_rows = expanded_src_to_dst_row.numel() / K``; ``drop_pad_mode`` is
    clamped to 0..3 (0/1: index arranged [K, num_rows], 2/3: [num_rows, K]); bias is only applied together with
    ``expert_for_source_row``."""
    epr = expanded_permuted_rows
    _check(epr.dtype in (torch.float16, torch.float32, torch.bfloat16),
           "moe_finalize_routing: expanded_permuted_rows must be float16 / float32 / bfloat16.")
    _check(epr.dim() >= 2, "moe_finalize_routing: expanded_permuted_rows must have rank >= 2.")
    _check(expanded_src_to_dst_row.dtype == torch.int32,
           "moe_finalize_routing: expanded_src_to_dst_row must be int32.")
    h = epr.size(-1)
    nk = expanded_src_to_dst_row.numel()
    k = 1
    if scales is not None:
        _check(scales.dim() == 2, "moe_finalize_routing: scales must be 2-D (NUM_ROWS, K).")
        k = scales.size(1)
    _check(k > 0, "moe_finalize_routing: K must be positive.")
    _check(nk % k == 0, "moe_finalize_routing: expanded_src_to_dst_row length must be K*NUM_ROWS.")
    num_rows = nk // k
    _need_cuda(epr, expanded_src_to_dst_row, skip1, skip2, bias, scales, expert_for_source_row)
    out = torch.empty((num_rows, h), dtype=epr.dtype, device=epr.device)
    if num_rows <= 0 or h <= 0:
        return out
    eprc = epr.contiguous()
    esdr = expanded_src_to_dst_row.contiguous()
    has_bias = bias is not None and expert_for_source_row is not None
    if has_bias:
        _check(bias.size(1) == h, "moe_finalize_routing: bias head dim must equal H.")
    for name, t in (("skip1", skip1), ("skip2", skip2), ("bias", bias if has_bias else None)):
        _check(t is None or t.dtype == epr.dtype, f"moe_finalize_routing: {name} must have the rows' dtype.")
    if scales is not None:
        _check(scales.dtype in (torch.float16, torch.float32, torch.bfloat16),
               "moe_finalize_routing: unsupported dtype combination for expanded_permuted_rows / scales.")
    if expert_for_source_row is not None:
        _check(expert_for_source_row.dtype == torch.int32, "moe_finalize_routing: expert_for_source_row must be int32.")
    mode = min(max(int(drop_pad_mode), 0), 3)
    s1 = skip1.contiguous() if skip1 is not None else None
    s2 = skip2.contiguous() if skip2 is not None else None
    bs = bias.contiguous() if has_bias else None
    sc = scales.contiguous() if scales is not None else None
    ex = expert_for_source_row.contiguous() if expert_for_source_row is not None else None
    with torch.cuda.device(epr.device):
        rc = L.load().w8a8_moe_finalize_routing(eprc.data_ptr(), esdr.data_ptr(), _ptr(s1), _ptr(s2), _ptr(bs), _ptr(sc),
                                                _ptr(ex) if has_bias else None, out.data_ptr(), num_rows, h, k,
                                                bs.size(0) if has_bias else 0, eprc.numel() // h, mode, _dt(eprc),
                                                _dt(sc) if sc is not None else _dt(eprc), _stream())
    _status(rc, "moe_finalize_routing")
    return out


def moe_gating_top_k_softmax(x: torch.Tensor, finished: Optional[torch.Tensor] = None, k: int = 1
                             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``moe_gating_top_k_softmax(Tensor x, Tensor? finished=None, int k=1) -> (Tensor y, Tensor expert_idx,
    Tensor row_idx)`` (operators/moegatingtopksoftmax/csrc/ops/moe_gating_top_k_softmax/op_plugin/
    moe_gating_plugin.cpp:28-53 for the schema and shape rules, 60-88 for the checks).

    Softmax over the last dimension in fp32, the ``k`` largest probabilities per row in ``x``'s dtype, their
    expert columns (int32; ``x.size(-1)`` for rows whose ``finished`` flag is set) and ``row_idx = j * rows + r``."""
    _check(x.dtype in (torch.float32, torch.float16, torch.bfloat16),
           "cann_bench.moe_gating_top_k_softmax only supports float32, float16 and bfloat16 inputs.")
    _check(x.dim() >= 2, "cann_bench.moe_gating_top_k_softmax requires a tensor with rank >= 2.")
    inner = x.size(-1)
    _check(inner > 0, "cann_bench.moe_gating_top_k_softmax requires a non-empty last dimension.")
    _check(0 < k <= inner, "cann_bench.moe_gating_top_k_softmax requires 0 < k <= x.size(-1).")
    if finished is not None:
        _check(finished.dtype == torch.bool, "cann_bench.moe_gating_top_k_softmax requires a bool 'finished' tensor.")
    _need_cuda(x, finished)
    xc = x.contiguous()
    rows = xc.numel() // inner
    _check(rows > 0, "cann_bench.moe_gating_top_k_softmax requires at least one row.")
    shape = tuple(xc.shape[:-1]) + (k,)
    y = torch.empty(shape, dtype=xc.dtype, device=xc.device)
    ei = torch.empty(shape, dtype=torch.int32, device=xc.device)
    ri = torch.empty(shape, dtype=torch.int32, device=xc.device)
    fin = None
    if finished is not None:
        fin = finished.contiguous()
        _check(fin.numel() == rows, "cann_bench.moe_gating_top_k_softmax: finished must have numel == rows.")
    with torch.cuda.device(xc.device):
        rc = L.load().w8a8_moe_gating_top_k_softmax(xc.data_ptr(), _ptr(fin), y.data_ptr(), ei.data_ptr(),
                                                    ri.data_ptr(), rows, inner, k, _dt(xc), _stream())
    _status(rc, "moe_gating_top_k_softmax")
    return y, ei, ri


def dequant_swiglu_quant(x: torch.Tensor, weight_scale: Optional[torch.Tensor] = None,
                         activation_scale: Optional[torch.Tensor] = None, quant_scale: Optional[torch.Tensor] = None,
                         activate_left: bool = False, *, round_direct: bool = False
                         ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``dequant_swiglu_quant(Tensor x, Tensor? weight_scale=None, Tensor? activation_scale=None,
    Tensor? quant_scale=None, bool activate_left=False) -> (Tensor y, Tensor scale)``
    (operators/dequantswigluquant/csrc/ops/dequant_swiglu_quant/op_plugin/dqsq_plugin.cpp:31-56 for the schema and
    shapes, 62-111 for the checks).

    ``x`` [TokensNum, 2H] int32 (then both scales are required) or float16 / bfloat16 (then both must be None);
    returns int8 ``y`` [TokensNum, H] and float32 ``scale`` [TokensNum]."""
    _check(x.dim() == 2, "dequant_swiglu_quant requires a 2D input [TokensNum, 2H].")
    m, n2 = x.shape
    _check(n2 % 2 == 0, "dequant_swiglu_quant requires an even last dimension.")
    h = n2 // 2
    _need_cuda(x, weight_scale, activation_scale, quant_scale)
    _check(x.is_contiguous(), "dequant_swiglu_quant requires a contiguous input.")
    y = torch.empty((m, h), dtype=torch.int8, device=x.device)
    scale = torch.empty((m,), dtype=torch.float32, device=x.device)
    if m <= 0 or n2 <= 0:
        return y, scale
    if x.dtype == torch.int32:
        _check(weight_scale is not None, "weight_scale is required when x is int32.")
        _check(activation_scale is not None, "activation_scale is required when x is int32.")
        _check(weight_scale.dtype == torch.float32, "weight_scale must be float32.")
        _check(activation_scale.dtype == torch.float32, "activation_scale must be float32.")
        _check(weight_scale.is_contiguous() and activation_scale.is_contiguous(),
               "weight_scale / activation_scale must be contiguous.")
        _check(weight_scale.numel() == n2, "weight_scale must have 2H elements.")
        _check(activation_scale.numel() == m, "activation_scale must have TokensNum elements.")
    else:
        _check(x.dtype in (torch.float16, torch.bfloat16),
               "dequant_swiglu_quant supports int32 / float16 / bfloat16 inputs.")
        _check(weight_scale is None, "weight_scale must be None for float16 / bfloat16 inputs.")
        _check(activation_scale is None, "activation_scale must be None for float16 / bfloat16 inputs.")
    if quant_scale is not None:
        _check(quant_scale.dtype == torch.float32, "quant_scale must be float32.")
        _check(quant_scale.is_contiguous(), "quant_scale must be contiguous.")
        _check(quant_scale.numel() == h, "quant_scale must have H elements.")
    with torch.cuda.device(x.device):
        rc = L.load().w8a8_dequant_swiglu_quant(x.data_ptr(), _ptr(weight_scale), _ptr(activation_scale),
                                                _ptr(quant_scale), y.data_ptr(), scale.data_ptr(), m, h, _dt(x),
                                                1 if activate_left else 0, L.F_ROUND_DIRECT if round_direct else 0,
                                                _stream())
    _status(rc, "dequant_swiglu_quant")
    return y, scale
