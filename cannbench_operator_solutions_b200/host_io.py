"""Host-buffer front ends: operators whose inputs start and whose results end in pinned host memory.

An operator of this library takes a few milliseconds on the device while its operands take tens of milliseconds
to cross PCIe, so a call made with host buffers is bound by the copies.  These front ends cut the rows into chunks
and keep three streams busy at once -- chunk i+1 going up, chunk i computing, chunk i-1 coming back -- so the call
costs about as long as the slower copy direction instead of the sum of all three.  The arithmetic is the library's
own operator on every chunk (rows are independent in all of them), so results equal a single whole-tensor call bit
for bit.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib as L


class GroupedSwigluQuantFromHost:
    """``grouped_matmul_swiglu_quant`` for int8 rows and fp32 row scales that live in pinned host memory.

    A binding of the library's C++ front end (``w8a8_gmsq_host_pipe_*``): weights and their scales stay on the
    device, ``chunk_rows`` rows travel and compute at a time over a copy-in stream, the current stream and a
    copy-out stream; a chunk may start and end inside an expert's rows."""

    def __init__(self, weight: torch.Tensor, weight_scale: torch.Tensor, chunk_rows: int = 4096,
                 transpose_weight: bool = False):
        import ctypes

        if not (weight.is_cuda and weight_scale.is_cuda):
            raise RuntimeError("GroupedSwigluQuantFromHost: weight and weight_scale must be CUDA tensors")
        if weight.dtype != torch.int8 or weight_scale.dtype != torch.float32 or weight.dim() != 3:
            raise RuntimeError("GroupedSwigluQuantFromHost: weight must be int8 [E, K, N], weight_scale float32 [E, N]")
        self.w = weight.contiguous()
        self.ws = weight_scale.contiguous()
        self.e = self.w.size(0)
        self.k = self.w.size(2) if transpose_weight else self.w.size(1)
        self.n = self.w.size(1) if transpose_weight else self.w.size(2)
        if self.n % 2 != 0:
            raise RuntimeError("GroupedSwigluQuantFromHost: N must be even")
        self.dev = self.w.device
        self.lib = L.load()
        need = self.lib.w8a8_gmsq_host_pipe_device_bytes(self.k, self.n, self.e, int(chunk_rows))
        self.device_mem = torch.empty((need,), dtype=torch.uint8, device=self.dev)
        self.pipe = ctypes.c_void_p(None)
        with torch.cuda.device(self.dev):
            rc = self.lib.w8a8_gmsq_host_pipe_create(ctypes.byref(self.pipe), self.w.data_ptr(), self.ws.data_ptr(),
                                                     self.k, self.n, self.e, L.W_NK if transpose_weight else L.W_KN,
                                                     int(chunk_rows), self.device_mem.data_ptr(), need)
        if rc != L.OK:
            raise RuntimeError(f"GroupedSwigluQuantFromHost: {L.status_string(rc)} (status {rc})")

    def __del__(self):
        pipe = getattr(self, "pipe", None)
        if pipe is not None and pipe.value:
            self.lib.w8a8_gmsq_host_pipe_destroy(pipe)
            self.pipe = None

    def __call__(self, x: torch.Tensor, x_scale: torch.Tensor, group_list: Sequence[int],
                 y: Optional[torch.Tensor] = None, y_scale: Optional[torch.Tensor] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
        if x.is_cuda or x_scale.is_cuda:
            raise RuntimeError("GroupedSwigluQuantFromHost: x and x_scale are host tensors (use the plain operator)")
        if x.dtype != torch.int8 or x_scale.dtype != torch.float32 or x.dim() != 2 or x.size(1) != self.k:
            raise RuntimeError("GroupedSwigluQuantFromHost: x must be int8 [M, K] and x_scale float32 [M]")
        m = x.size(0)
        ends = torch.tensor([int(v) for v in group_list], dtype=torch.int64)
        if ends.numel() != self.e or x_scale.numel() != m:
            raise RuntimeError("GroupedSwigluQuantFromHost: group_list must have E entries ending at M = len(x_scale)")
        if y is None:
            y = torch.empty((m, self.n // 2), dtype=torch.int8).pin_memory()
        if y_scale is None:
            y_scale = torch.empty((m,), dtype=torch.float32).pin_memory()
        xc, xsc = x.contiguous(), x_scale.contiguous()
        if not (y.is_contiguous() and y_scale.is_contiguous()):
            raise RuntimeError("GroupedSwigluQuantFromHost: result buffers must be contiguous")
        with torch.cuda.device(self.dev):
            rc = self.lib.w8a8_gmsq_host_pipe_run(self.pipe, xc.data_ptr(), xsc.data_ptr(), ends.data_ptr(), m,
                                                  y.data_ptr(), y_scale.data_ptr(), 0,
                                                  torch.cuda.current_stream().cuda_stream)
        if rc == L.ERR_GROUP_LIST:
            raise RuntimeError("GroupedSwigluQuantFromHost: group_list must be a cumsum <= M")
        if rc != L.OK:
            raise RuntimeError(f"GroupedSwigluQuantFromHost: {L.status_string(rc)} (status {rc})")
        return y, y_scale


class RowQuantFromHost:
    """``dynamic_quant`` / ``add_rms_norm_dynamic_quant`` for 16-bit rows that live in pinned host memory.

    ``fused=False``: x -> (y int8, scale).  ``fused=True``: (x1, x2) with a device-resident gamma ->
    (y int8, x_out, scale).  Rows travel and compute ``chunk_rows`` at a time over a copy-in stream, the current
    stream and a copy-out stream, with double-buffered device staging."""

    def __init__(self, n: int, dtype: torch.dtype, device, *, fused: bool, gamma: Optional[torch.Tensor] = None,
                 epsilon: float = 1e-6, chunk_rows: int = 1024):
        if dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError("RowQuantFromHost: rows must be float16 or bfloat16")
        if fused and (gamma is None or not gamma.is_cuda or gamma.dtype != dtype or gamma.numel() != n):
            raise RuntimeError("RowQuantFromHost: the fused form needs a CUDA gamma of the rows' dtype and length")
        self.n, self.dtype, self.fused, self.eps, self.chunk = n, dtype, fused, float(epsilon), int(chunk_rows)
        self.gamma = gamma.contiguous() if fused else None
        self.dev = torch.device(device)
        self.code = L.DT_BF16 if dtype == torch.bfloat16 else L.DT_F16
        self.lib = L.load()
        with torch.cuda.device(self.dev):
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            mk = lambda dt, *shape: [torch.empty(shape, dtype=dt, device=self.dev) for _ in range(2)]
            self.x1 = mk(dtype, self.chunk, n)
            self.x2 = mk(dtype, self.chunk, n) if fused else None
            self.y = mk(torch.int8, self.chunk, n)
            self.xo = mk(dtype, self.chunk, n) if fused else None
            self.sc = mk(torch.float32, self.chunk)

    def __call__(self, x1: torch.Tensor, x2: Optional[torch.Tensor] = None, out: Optional[Sequence[torch.Tensor]] = None):
        rows = x1.size(0)
        if x1.is_cuda or x1.dtype != self.dtype or x1.dim() != 2 or x1.size(1) != self.n:
            raise RuntimeError("RowQuantFromHost: x must be a host tensor [rows, N] of the configured dtype")
        if self.fused and (x2 is None or x2.shape != x1.shape or x2.dtype != self.dtype or x2.is_cuda):
            raise RuntimeError("RowQuantFromHost: the fused form needs a second host tensor of the same shape")
        if out is None:
            out = [torch.empty((rows, self.n), dtype=torch.int8).pin_memory()]
            if self.fused:
                out.append(torch.empty((rows, self.n), dtype=self.dtype).pin_memory())
            out.append(torch.empty((rows,), dtype=torch.float32).pin_memory())
        y_h, sc_h = out[0], out[-1]
        xo_h = out[1] if self.fused else None
        if rows == 0:
            return tuple(out)
        lib = self.lib
        with torch.cuda.device(self.dev):
            main = torch.cuda.current_stream()
            start = torch.cuda.Event()
            start.record(main)
            self.s_in.wait_event(start)
            self.s_out.wait_event(start)
            computed: List[torch.cuda.Event] = []
            returned: List[torch.cuda.Event] = []
            for i, r0 in enumerate(range(0, rows, self.chunk)):
                r1 = min(rows, r0 + self.chunk)
                b, m = i % 2, r1 - r0
                with torch.cuda.stream(self.s_in):
                    if i >= 2:
                        self.s_in.wait_event(computed[i - 2])
                    self.x1[b][:m].copy_(x1[r0:r1], non_blocking=True)
                    if self.fused:
                        self.x2[b][:m].copy_(x2[r0:r1], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(self.s_in)
                main.wait_event(arrived)
                if i >= 2:
                    main.wait_event(returned[i - 2])
                if self.fused:
                    rc = lib.w8a8_add_rms_norm_dynamic_quant(self.x1[b].data_ptr(), self.x2[b].data_ptr(),
                                                             self.gamma.data_ptr(), self.y[b].data_ptr(),
                                                             self.xo[b].data_ptr(), self.sc[b].data_ptr(), m, self.n,
                                                             self.eps, self.code, 0, main.cuda_stream)
                else:
                    rc = lib.w8a8_dynamic_quant(self.x1[b].data_ptr(), self.y[b].data_ptr(), self.sc[b].data_ptr(), m,
                                                self.n, self.code, 0, main.cuda_stream)
                if rc != L.OK:
                    raise RuntimeError(f"RowQuantFromHost: {L.status_string(rc)} (status {rc})")
                done = torch.cuda.Event()
                done.record(main)
                computed.append(done)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(done)
                    y_h[r0:r1].copy_(self.y[b][:m], non_blocking=True)
                    if self.fused:
                        xo_h[r0:r1].copy_(self.xo[b][:m], non_blocking=True)
                    sc_h[r0:r1].copy_(self.sc[b][:m], non_blocking=True)
                    back = torch.cuda.Event()
                    back.record(self.s_out)
                returned.append(back)
            main.wait_event(returned[-1])
            if len(returned) > 1:
                main.wait_event(returned[-2])
        return tuple(out)
