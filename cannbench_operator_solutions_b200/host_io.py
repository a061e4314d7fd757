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

    Weights and their scales stay on the device.  ``chunk_rows`` rows travel and compute at a time; a chunk may
    start and end inside an expert's rows (the chunk's own cumulative group list is cut from the caller's)."""

    def __init__(self, weight: torch.Tensor, weight_scale: torch.Tensor, chunk_rows: int = 16384,
                 transpose_weight: bool = False):
        if not (weight.is_cuda and weight_scale.is_cuda):
            raise RuntimeError("GroupedSwigluQuantFromHost: weight and weight_scale must be CUDA tensors")
        if weight.dtype != torch.int8 or weight_scale.dtype != torch.float32 or weight.dim() != 3:
            raise RuntimeError("GroupedSwigluQuantFromHost: weight must be int8 [E, K, N], weight_scale float32 [E, N]")
        self.w = weight.contiguous()
        self.ws = weight_scale.contiguous()
        self.transposed = transpose_weight
        self.e = self.w.size(0)
        self.k = self.w.size(2) if transpose_weight else self.w.size(1)
        self.n = self.w.size(1) if transpose_weight else self.w.size(2)
        if self.n % 2 != 0:
            raise RuntimeError("GroupedSwigluQuantFromHost: N must be even")
        self.chunk = int(chunk_rows)
        dev = self.w.device
        self.dev = dev
        self.lib = L.load()
        with torch.cuda.device(dev):
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            self.xbuf = [torch.empty((self.chunk, self.k), dtype=torch.int8, device=dev) for _ in range(2)]
            self.xsbuf = [torch.empty((self.chunk,), dtype=torch.float32, device=dev) for _ in range(2)]
            self.ybuf = [torch.empty((self.chunk, self.n // 2), dtype=torch.int8, device=dev) for _ in range(2)]
            self.ysbuf = [torch.empty((self.chunk,), dtype=torch.float32, device=dev) for _ in range(2)]
            need = self.lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(self.chunk, self.k, self.n, self.e)
            self.workspace = torch.empty((need,), dtype=torch.uint8, device=dev)

    def _chunks(self, ends: Sequence[int], m: int) -> List[Tuple[int, int, int, List[int]]]:
        """(first row, last row, first expert, local cumulative list) per chunk."""
        out = []
        e0 = 0
        for r0 in range(0, m, self.chunk):
            r1 = min(m, r0 + self.chunk)
            while e0 < self.e and ends[e0] <= r0:
                e0 += 1
            local, e1 = [], e0
            while True:
                local.append(min(ends[e1], r1) - r0)
                if ends[e1] >= r1:
                    break
                e1 += 1
            out.append((r0, r1, e0, local))
        return out

    def __call__(self, x: torch.Tensor, x_scale: torch.Tensor, group_list: Sequence[int],
                 y: Optional[torch.Tensor] = None, y_scale: Optional[torch.Tensor] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
        if x.is_cuda or x_scale.is_cuda:
            raise RuntimeError("GroupedSwigluQuantFromHost: x and x_scale are host tensors (use the plain operator)")
        if x.dtype != torch.int8 or x_scale.dtype != torch.float32 or x.dim() != 2 or x.size(1) != self.k:
            raise RuntimeError("GroupedSwigluQuantFromHost: x must be int8 [M, K] and x_scale float32 [M]")
        m = x.size(0)
        ends = [int(v) for v in group_list]
        prev = 0
        for v in ends:
            if not prev <= v <= m:
                raise RuntimeError("GroupedSwigluQuantFromHost: group_list must be a cumsum <= M")
            prev = v
        if len(ends) != self.e or prev != m or x_scale.numel() != m:
            raise RuntimeError("GroupedSwigluQuantFromHost: group_list must have E entries ending at M = len(x_scale)")
        if y is None:
            y = torch.empty((m, self.n // 2), dtype=torch.int8).pin_memory()
        if y_scale is None:
            y_scale = torch.empty((m,), dtype=torch.float32).pin_memory()
        if m == 0:
            return y, y_scale
        lib = self.lib
        layout = L.W_NK if self.transposed else L.W_KN
        with torch.cuda.device(self.dev):
            main = torch.cuda.current_stream()
            start = torch.cuda.Event()
            start.record(main)
            self.s_in.wait_event(start)
            self.s_out.wait_event(start)
            computed: List[torch.cuda.Event] = []
            returned: List[torch.cuda.Event] = []
            for i, (r0, r1, e0, local) in enumerate(self._chunks(ends, m)):
                b, rows = i % 2, r1 - r0
                with torch.cuda.stream(self.s_in):
                    if i >= 2:
                        self.s_in.wait_event(computed[i - 2])       # the staging buffer's last reader is done
                    self.xbuf[b][:rows].copy_(x[r0:r1], non_blocking=True)
                    self.xsbuf[b][:rows].copy_(x_scale[r0:r1], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(self.s_in)
                main.wait_event(arrived)
                if i >= 2:
                    main.wait_event(returned[i - 2])                # the result buffer has been copied out
                gl = torch.tensor(local, dtype=torch.int64)
                w = self.w[e0:e0 + len(local)]
                ws = self.ws[e0:e0 + len(local)]
                rc = lib.w8a8_grouped_matmul_swiglu_quant(
                    self.xbuf[b].data_ptr(), w.data_ptr(), ws.data_ptr(), self.xsbuf[b].data_ptr(),
                    self.ybuf[b].data_ptr(), self.ysbuf[b].data_ptr(), rows, self.k, self.n, len(local),
                    gl.data_ptr(), 0, layout, 0, self.workspace.data_ptr(), self.workspace.numel(), main.cuda_stream)
                if rc != L.OK:
                    raise RuntimeError(f"GroupedSwigluQuantFromHost: {L.status_string(rc)} (status {rc})")
                done = torch.cuda.Event()
                done.record(main)
                computed.append(done)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(done)
                    y[r0:r1].copy_(self.ybuf[b][:rows], non_blocking=True)
                    y_scale[r0:r1].copy_(self.ysbuf[b][:rows], non_blocking=True)
                    back = torch.cuda.Event()
                    back.record(self.s_out)
                returned.append(back)
            main.wait_event(returned[-1])
            if len(returned) > 1:
                main.wait_event(returned[-2])
        return y, y_scale
