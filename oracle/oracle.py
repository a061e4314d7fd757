"""ctypes loader for the CPU oracle (test infrastructure only).

Only tests, the smoke check and the benchmark's CPU legs import this module;
the product package never does.  The shared object is built by
``oracle/Makefile`` into ``oracle/_ref/``; :func:`load` builds it on demand
when it is missing (gcc is the only requirement).

Arrays are numpy: bf16 and fp16 tensors travel as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libw8a8_oracle.so")

DT_F16, DT_BF16, DT_F32, DT_I8, DT_I32 = 0, 1, 2, 3, 4
ROUND_AS_WRITTEN, ROUND_DIRECT = 0, 1
SUM_CANONICAL, SUM_FP64 = 0, 1
EXP_CANONICAL, EXP_LIBM = 0, 1

QM_SCALE_PERCHAN = 1 << 0
QM_SCALE_BF16 = 1 << 1
QM_HAS_OFFSET = 1 << 2
QM_OFFSET_PERCHAN = 1 << 3
QM_HAS_PT = 1 << 4
QM_BIAS_SHIFT = 5
QM_BIAS_PERCHAN = 1 << 8
QM_PT_MOD_M = 1 << 9
QM_BIAS_NONE, QM_BIAS_I32, QM_BIAS_F16, QM_BIAS_BF16, QM_BIAS_F32 = 0, 1, 2, 3, 4

_lib: Optional[ctypes.CDLL] = None


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile; returns the path of the library."""
    src_time = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("w8a8_oracle.c", "w8a8_oracle.h"))
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < src_time:
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    build()
    lib = ctypes.CDLL(_SO)
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    lib.oracle_bf16_to_f32.restype = f32
    lib.oracle_bf16_to_f32.argtypes = [ctypes.c_uint16]
    lib.oracle_f16_to_f32.restype = f32
    lib.oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
    lib.oracle_f32_to_bf16.restype = ctypes.c_uint16
    lib.oracle_f32_to_bf16.argtypes = [f32]
    lib.oracle_f32_to_f16.restype = ctypes.c_uint16
    lib.oracle_f32_to_f16.argtypes = [f32]
    lib.oracle_narrow_i8.restype = ctypes.c_int8
    lib.oracle_narrow_i8.argtypes = [f32, i32]
    lib.oracle_expf.restype = f32
    lib.oracle_expf.argtypes = [f32]
    lib.oracle_silu.restype = f32
    lib.oracle_silu.argtypes = [f32, i32]
    lib.oracle_dynamic_quant.restype = i32
    lib.oracle_dynamic_quant.argtypes = [vp, vp, vp, i64, i64, i32, i32]
    lib.oracle_add_rms_norm_dynamic_quant.restype = i32
    lib.oracle_add_rms_norm_dynamic_quant.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, f32, i32, i32, i32]
    lib.oracle_quant_matmul.restype = i32
    lib.oracle_quant_matmul.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i32, i32, vp]
    lib.oracle_grouped_matmul_swiglu_quant.restype = i32
    lib.oracle_grouped_matmul_swiglu_quant.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, i32, vp]
    lib.oracle_grouped_matmul.restype = i32
    lib.oracle_grouped_matmul.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, i32, i32]
    lib.oracle_route_count.restype = i32
    lib.oracle_route_count.argtypes = [vp, i64, i64, i64, vp, vp, vp]
    lib.oracle_gather_rows.restype = i32
    lib.oracle_gather_rows.argtypes = [vp, vp, vp, i64, i64]
    lib.oracle_combine.restype = i32
    lib.oracle_combine.argtypes = [vp, vp, vp, vp, i64, i64, i64, i32]
    lib.oracle_moe_re_routing.restype = i32
    lib.oracle_moe_re_routing.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64]
    lib.oracle_moe_finalize_routing.restype = i32
    lib.oracle_moe_finalize_routing.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i32, i32, i32]
    lib.oracle_moe_gating_top_k_softmax.restype = i32
    lib.oracle_moe_gating_top_k_softmax.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i32]
    lib.oracle_dequant_swiglu_quant.restype = i32
    lib.oracle_dequant_swiglu_quant.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, vp]
    lib.oracle_num_threads.restype = i32
    _lib = lib
    return lib


def _p(a: Optional[np.ndarray]):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(load().oracle_num_threads())


# --------------------------------------------------------------------------
# scalar helpers
# --------------------------------------------------------------------------
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Vectorised fp32 -> bf16 bit patterns (RNE), same rule as the oracle."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r)
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


def f32_to_f16_bits(a: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.ascontiguousarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


def bits_to_f32(b: np.ndarray, dtype: int) -> np.ndarray:
    return bf16_bits_to_f32(b) if dtype == DT_BF16 else f16_bits_to_f32(b)


def f32_to_bits(a: np.ndarray, dtype: int) -> np.ndarray:
    return f32_to_bf16_bits(a) if dtype == DT_BF16 else f32_to_f16_bits(a)


# --------------------------------------------------------------------------
# operators
# --------------------------------------------------------------------------
def dynamic_quant(x_bits: np.ndarray, dtype: int, round_mode: int = ROUND_AS_WRITTEN):
    """x_bits: uint16 [..., N] -> (y int8 [..., N], scale fp32 [...])."""
    x_bits = _c(x_bits, np.uint16)
    n = x_bits.shape[-1]
    m = x_bits.size // n if n else 0
    y = np.empty(x_bits.shape, np.int8)
    scale = np.empty(x_bits.shape[:-1], np.float32)
    rc = load().oracle_dynamic_quant(_p(x_bits), _p(y), _p(scale), m, n, dtype, round_mode)
    if rc != 0:
        raise ValueError("oracle_dynamic_quant rejected the arguments")
    return y, scale


def add_rms_norm_dynamic_quant(x1_bits, x2_bits, gamma_bits, eps: float, dtype: int,
                               round_mode: int = ROUND_AS_WRITTEN, sum_order: int = SUM_CANONICAL):
    x1_bits = _c(x1_bits, np.uint16)
    x2_bits = _c(x2_bits, np.uint16)
    gamma_bits = _c(gamma_bits, np.uint16)
    n = x1_bits.shape[-1]
    rows = x1_bits.size // n if n else 0
    y = np.empty(x1_bits.shape, np.int8)
    x_out = np.empty(x1_bits.shape, np.uint16)
    scale = np.empty(x1_bits.shape[:-1], np.float32)
    rc = load().oracle_add_rms_norm_dynamic_quant(_p(x1_bits), _p(x2_bits), _p(gamma_bits), _p(y), _p(x_out),
                                                  _p(scale), rows, n, eps, dtype, round_mode, sum_order)
    if rc != 0:
        raise ValueError("oracle_add_rms_norm_dynamic_quant rejected the arguments")
    return y, x_out, scale


def quant_matmul(x1, x2, scale, *, offset=None, pertoken=None, bias=None, flags: int, out_dtype: int,
                 batch: int = 1, x2_transposed: bool = False, want_acc: bool = False):
    """x1 int8 [batch*M, K]; x2 int8 [batch, K, N] (or [batch, N, K] when transposed)."""
    x1 = _c(x1, np.int8)
    x2 = _c(x2, np.int8)
    k = x1.shape[-1]
    m = x1.size // k // batch
    n = x2.shape[-2] if x2_transposed else x2.shape[-1]
    out = np.empty((batch * m, n), np.uint16)
    acc = np.empty((batch * m, n), np.int32) if want_acc else None
    rc = load().oracle_quant_matmul(_p(x1), _p(x2), _p(scale), _p(offset), _p(pertoken), _p(bias), _p(out),
                                    batch, m, n, k, flags, out_dtype, int(x2_transposed), _p(acc))
    if rc != 0:
        raise ValueError("oracle_quant_matmul rejected the arguments")
    return (out, acc) if want_acc else out


def grouped_matmul_swiglu_quant(x, w, w_scale, x_scale, group_list: Sequence[int], *,
                                w_transposed: bool = False, round_mode: int = ROUND_AS_WRITTEN,
                                exp_kind: int = EXP_CANONICAL, want_act: bool = False):
    x = _c(x, np.int8)
    w = _c(w, np.int8)
    w_scale = _c(w_scale, np.float32)
    x_scale = _c(x_scale, np.float32)
    gl = _c(np.asarray(group_list), np.int64)
    m, k = x.shape
    e = w.shape[0]
    n = w.shape[1] if w_transposed else w.shape[2]
    y = np.empty((m, n // 2), np.int8)
    ys = np.empty((m,), np.float32)
    act = np.empty((m, n // 2), np.float32) if want_act else None
    rc = load().oracle_grouped_matmul_swiglu_quant(_p(x), _p(w), _p(w_scale), _p(x_scale), _p(gl), _p(y), _p(ys),
                                                   m, k, n, e, int(w_transposed), round_mode, exp_kind, _p(act))
    if rc != 0:
        raise ValueError("oracle_grouped_matmul_swiglu_quant rejected the arguments")
    return (y, ys, act) if want_act else (y, ys)


def grouped_matmul(x, w, group_list: Sequence[int], *, dtype: int, bias=None, bias_dtype: int = DT_F32,
                   x_scale=None, w_scale=None, out_dtype: int = DT_BF16, w_transposed: bool = False):
    gl = _c(np.asarray(group_list), np.int64)
    m, k = x.shape
    e = w.shape[0]
    n = w.shape[1] if w_transposed else w.shape[2]
    if dtype == DT_I8:
        y = np.empty((m, n), np.uint16)
    elif dtype == DT_F32:
        y = np.empty((m, n), np.float32)
    else:
        y = np.empty((m, n), np.uint16)
    rc = load().oracle_grouped_matmul(_p(np.ascontiguousarray(x)), _p(np.ascontiguousarray(w)), _p(bias), _p(y),
                                      _p(x_scale), _p(w_scale), _p(gl), m, n, k, e, dtype, bias_dtype, out_dtype,
                                      int(w_transposed))
    if rc != 0:
        raise ValueError("oracle_grouped_matmul rejected the arguments")
    return y


def route_count(expert_idx: np.ndarray, num_experts: int):
    """expert_idx int32 [T, topk] -> (count[E], cumsum[E], expanded_pos[T, topk]) as int64."""
    expert_idx = _c(expert_idx, np.int32)
    t, topk = expert_idx.shape
    cnt = np.empty((num_experts,), np.int64)
    cum = np.empty((num_experts,), np.int64)
    pos = np.empty((t, topk), np.int64)
    rc = load().oracle_route_count(_p(expert_idx), t, topk, num_experts, _p(cnt), _p(cum), _p(pos))
    if rc != 0:
        raise ValueError("oracle_route_count rejected the arguments")
    return cnt, cum, pos


def gather_rows(src: np.ndarray, src_row: np.ndarray) -> np.ndarray:
    src = np.ascontiguousarray(src)
    src_row = _c(src_row, np.int64)
    row_bytes = src.strides[0] if src.ndim > 1 else src.itemsize
    dst = np.empty((src_row.size,) + src.shape[1:], src.dtype)
    load().oracle_gather_rows(_p(src), _p(dst), _p(src_row), src_row.size, row_bytes)
    return dst


def combine(rows_bits: np.ndarray, probs: np.ndarray, expanded_pos: np.ndarray, dtype: int) -> np.ndarray:
    rows_bits = np.ascontiguousarray(rows_bits)
    probs = _c(probs, np.float32)
    expanded_pos = _c(expanded_pos, np.int64)
    t, topk = probs.shape
    h = rows_bits.shape[1]
    out = np.empty((t, h), rows_bits.dtype)
    rc = load().oracle_combine(_p(rows_bits), _p(probs), _p(expanded_pos), _p(out), t, topk, h, dtype)
    if rc != 0:
        raise ValueError("oracle_combine rejected the arguments")
    return out


def moe_re_routing(tokens: np.ndarray, counts: np.ndarray, scales: Optional[np.ndarray] = None):
    """tokens [A, H] (any element type), counts [N, E] -> (permute_tokens, permute_scales, permute_token_idx,
    expert_token_num)."""
    tokens = np.ascontiguousarray(tokens)
    cnt = _c(counts, np.int64)
    a = tokens.shape[0]
    n, e = cnt.shape
    out = np.zeros_like(tokens)
    out_s = np.zeros((a,), np.float32)
    idx = np.zeros((a,), np.int32)
    num = np.zeros((e,), np.int64)
    sc = None if scales is None else _c(scales, np.float32)
    rc = load().oracle_moe_re_routing(_p(tokens), _p(cnt), _p(sc), _p(out), _p(out_s), _p(idx), _p(num), a,
                                      int(np.prod(tokens.shape[1:])) * tokens.itemsize, n, e)
    if rc != 0:
        raise ValueError("oracle_moe_re_routing rejected the arguments")
    return out, out_s, idx, num


def moe_finalize_routing(rows, esdr, dtype: int, *, skip1=None, skip2=None, bias=None, scales=None,
                         scale_dtype: int = DT_F32, expert=None, drop_pad_mode: int = 0):
    """rows [num_dst, H] as uint16 bit patterns (F16 / BF16) or float32 (F32); esdr int32 [K * R]; scales [R, K] in
    scale_dtype's representation.  Returns out [R, H] in rows' representation."""
    np_t = np.float32 if dtype == DT_F32 else np.uint16
    rows = _c(rows, np_t)
    esdr = _c(esdr, np.int32)
    h = rows.shape[-1]
    num_dst = rows.size // h
    k = 1
    sc = None
    if scales is not None:
        sc = _c(scales, np.float32 if scale_dtype == DT_F32 else np.uint16)
        k = sc.shape[1]
    r = esdr.size // k
    s1 = None if skip1 is None else _c(skip1, np_t)
    s2 = None if skip2 is None else _c(skip2, np_t)
    bs = None if bias is None else _c(bias, np_t)
    ex = None if expert is None else _c(expert, np.int32)
    e = 0 if bs is None else bs.shape[0]
    out = np.empty((r, h), np_t)
    rc = load().oracle_moe_finalize_routing(_p(rows), _p(esdr), _p(s1), _p(s2), _p(bs), _p(sc), _p(ex), _p(out), r, h,
                                            k, e, num_dst, drop_pad_mode, dtype, scale_dtype)
    if rc != 0:
        raise ValueError("oracle_moe_finalize_routing rejected the arguments")
    return out


def moe_gating_top_k_softmax(x, dtype: int, k: int, finished=None):
    """x [..., inner] as uint16 bit patterns (F16 / BF16) or float32 -> (y, expert_idx, row_idx), each [..., k]."""
    np_t = np.float32 if dtype == DT_F32 else np.uint16
    x = _c(x, np_t)
    inner = x.shape[-1]
    rows = x.size // inner
    shape = x.shape[:-1] + (k,)
    y = np.empty(shape, np_t)
    ei = np.empty(shape, np.int32)
    ri = np.empty(shape, np.int32)
    fin = None if finished is None else _c(finished, np.uint8)
    rc = load().oracle_moe_gating_top_k_softmax(_p(x), _p(fin), _p(y), _p(ei), _p(ri), rows, inner, k, dtype)
    if rc != 0:
        raise ValueError("oracle_moe_gating_top_k_softmax rejected the arguments")
    return y, ei, ri


def dequant_swiglu_quant(x, x_dtype: int, *, weight_scale=None, activation_scale=None, quant_scale=None,
                         activate_left: bool = False, round_mode: int = ROUND_AS_WRITTEN, want_out: bool = False):
    """x [M, 2H]: int32 (DT_I32) or uint16 bit patterns (DT_F16 / DT_BF16) -> (y int8 [M, H], scale fp32 [M])."""
    x = _c(x, np.int32 if x_dtype == DT_I32 else np.uint16)
    m, n2 = x.shape
    h = n2 // 2
    y = np.empty((m, h), np.int8)
    sc = np.empty((m,), np.float32)
    out = np.empty((m, h), np.float32) if want_out else None
    ws = None if weight_scale is None else _c(weight_scale, np.float32)
    a_s = None if activation_scale is None else _c(activation_scale, np.float32)
    qs = None if quant_scale is None else _c(quant_scale, np.float32)
    rc = load().oracle_dequant_swiglu_quant(_p(x), _p(ws), _p(a_s), _p(qs), _p(y), _p(sc), m, h, x_dtype,
                                            1 if activate_left else 0, round_mode, _p(out))
    if rc != 0:
        raise ValueError("oracle_dequant_swiglu_quant rejected the arguments")
    return (y, sc, out) if want_out else (y, sc)
