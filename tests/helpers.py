"""Conversions between torch CUDA tensors and the oracle's numpy bit patterns."""
import numpy as np
import torch

from oracle import oracle as O


def seed_of(*args) -> int:
    """Deterministic seed from the test parameters."""
    import zlib

    return zlib.crc32(repr(args).encode())


def dt_code(dtype: torch.dtype) -> int:
    return {torch.float16: O.DT_F16, torch.bfloat16: O.DT_BF16, torch.float32: O.DT_F32}[dtype]


def bits(t: torch.Tensor) -> np.ndarray:
    """16-bit float tensor -> uint16 bit patterns on the host."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_bits(b: np.ndarray, dtype: torch.dtype, device="cuda") -> torch.Tensor:
    return torch.from_numpy(b.view(np.int16).copy()).view(dtype).to(device)


def f32_bits(a) -> np.ndarray:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_same_f32(a, b, what=""):
    """Bit-exact fp32 comparison that treats every NaN as equal."""
    a = np.asarray(a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else a, dtype=np.float32)
    b = np.asarray(b.detach().cpu().numpy() if isinstance(b, torch.Tensor) else b, dtype=np.float32)
    an, bn = np.isnan(a), np.isnan(b)
    assert np.array_equal(an, bn), f"{what}: NaN positions differ"
    ok = (a.view(np.uint32) == b.view(np.uint32)) | an
    assert ok.all(), f"{what}: {np.count_nonzero(~ok)} of {ok.size} fp32 values differ"


def assert_same_16(a_bits, b_bits, dtype_code, what=""):
    """Bit-exact 16-bit float comparison that treats every NaN as equal."""
    fa, fb = O.bits_to_f32(a_bits, dtype_code), O.bits_to_f32(b_bits, dtype_code)
    an, bn = np.isnan(fa), np.isnan(fb)
    assert np.array_equal(an, bn), f"{what}: NaN positions differ"
    ok = (a_bits == b_bits) | an
    assert ok.all(), f"{what}: {np.count_nonzero(~ok)} of {ok.size} values differ"


def zipf_group_list(rng, rows: int, experts: int, s: float = 1.1) -> np.ndarray:
    """Cumulative group list from a Zipf(s)-skewed multinomial."""
    p = np.arange(1, experts + 1, dtype=np.float64) ** (-s)
    p /= p.sum()
    counts = rng.multinomial(rows, p)
    return np.cumsum(counts).astype(np.int64)
