"""Expert-parallel W8A8 MoE FFN chain over torch.distributed.

One process per GPU; rank r owns experts [r*E/P, (r+1)*E/P) and T/P tokens.

    add_rms_norm_dynamic_quant                      (tokens -> int8 + fp32 scale)
    route plan + scatter into expert-major order    (send buffer is grouped by destination rank for free,
                                                     because experts are sharded in contiguous blocks)
    all-to-all of the count matrix, then of the int8 rows and their fp32 scales  (dispatch)
    regroup rank-major -> expert-major              (MoeReRouting's permutation)
    grouped_matmul_swiglu_quant -> grouped_matmul (int8 down projection, bf16 out)
    inverse regroup, all-to-all back                (combine transport)
    weighted sum over the top-k copies              (MoeFinalizeRouting's arithmetic)

The compute steps go through a backend object: `CudaBackend` (the product:
libw8a8ffn.so through the C-ABI) or, in the CPU tests of this host logic, a
backend the test supplies.  The collectives are `all_to_all_single` on the
default process group (NCCL over NVLink on the GPU box, gloo in the CPU tests).

Layout contracts follow the reference catalog: the received buffer is
rank-major / expert-minor and the regroup is MoeReRouting's
(operators/moererouting/csrc/ops/moe_re_routing/op_kernel/moe_re_routing_launch.h:15-21);
the combine is MoeFinalizeRouting's fp32 ascending-k sum
(operators/moefinalizerouting/csrc/ops/moe_finalize_routing/op_kernel/moe_finalize_routing_kernel.cpp:15-25).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------
# host-side index arithmetic (tiny: P x E/P integers)
# ---------------------------------------------------------------------------
def regroup_index(recv_counts: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """recv_counts[i, j] = rows received from rank i for local expert j (rank-major, expert-minor buffer).

    Returns (src_of_dst, group_cumsum): src_of_dst[d] is the row of the received buffer that lands at row d of
    the expert-major buffer; group_cumsum is the cumulative group list of the local experts.  Same mapping as
    MoeReRouting: srcStart(i,j) = sum_{i'<i} rowSum(i') + sum_{j'<j} cnt[i][j'];
    dstStart(i,j) = sum_{j'<j} colSum(j') + sum_{i'<i} cnt[i'][j].
    """
    cnt = np.asarray(recv_counts, dtype=np.int64)
    p, e = cnt.shape
    row_sum = cnt.sum(1)
    col_sum = cnt.sum(0)
    src_start = (np.concatenate([[0], np.cumsum(row_sum)[:-1]])[:, None] +
                 np.concatenate([np.zeros((p, 1), np.int64), np.cumsum(cnt, 1)[:, :-1]], 1))
    dst_start = (np.concatenate([[0], np.cumsum(col_sum)[:-1]])[None, :] +
                 np.concatenate([np.zeros((1, e), np.int64), np.cumsum(cnt, 0)[:-1, :]], 0))
    total = int(cnt.sum())
    src_of_dst = np.empty((total,), np.int64)
    for i in range(p):
        for j in range(e):
            c = int(cnt[i, j])
            if c:
                src_of_dst[dst_start[i, j]:dst_start[i, j] + c] = np.arange(src_start[i, j], src_start[i, j] + c)
    return src_of_dst, np.cumsum(col_sum).astype(np.int64)


def invert_index(src_of_dst: np.ndarray) -> np.ndarray:
    inv = np.empty_like(src_of_dst)
    inv[src_of_dst] = np.arange(src_of_dst.size, dtype=np.int64)
    return inv


# ---------------------------------------------------------------------------
# compute backend
# ---------------------------------------------------------------------------
class CudaBackend:
    """The product path: every step is one C-ABI call on the current CUDA stream."""

    def __init__(self):
        from . import _lib, ops
        self.L, self.ops = _lib, ops
        self.lib = _lib.load()

    def _st(self):
        return torch.cuda.current_stream().cuda_stream

    def add_rms_norm_dynamic_quant(self, x1, x2, gamma, eps):
        return self.ops.add_rms_norm_dynamic_quant(x1, x2, gamma, eps)

    def route_plan(self, expert_idx: torch.Tensor, num_experts: int):
        t, topk = expert_idx.shape
        dev = expert_idx.device
        count = torch.empty((num_experts,), dtype=torch.int64, device=dev)
        cumsum = torch.empty((num_experts,), dtype=torch.int64, device=dev)
        pos = torch.empty((t, topk), dtype=torch.int64, device=dev)
        need = self.lib.w8a8_route_plan_workspace_size(t, topk, num_experts)
        ws = torch.empty((need,), dtype=torch.uint8, device=dev)
        rc = self.lib.w8a8_route_plan(expert_idx.data_ptr(), t, topk, num_experts, count.data_ptr(), cumsum.data_ptr(),
                                      pos.data_ptr(), ws.data_ptr(), need, self._st())
        if rc != 0:
            raise RuntimeError(f"route_plan: {self.L.status_string(rc)}")
        return count, cumsum, pos

    def scatter_rows(self, src, src_scale, pos, total_rows):
        t, topk = pos.shape
        dst = torch.empty((total_rows, src.shape[1]), dtype=src.dtype, device=src.device)
        dst_scale = torch.empty((total_rows,), dtype=torch.float32, device=src.device)
        rc = self.lib.w8a8_scatter_rows(src.data_ptr(), src_scale.data_ptr(), dst.data_ptr(), dst_scale.data_ptr(),
                                        pos.data_ptr(), t, topk, src.shape[1] * src.element_size(), self._st())
        if rc != 0:
            raise RuntimeError(f"scatter_rows: {self.L.status_string(rc)}")
        return dst, dst_scale

    def permute_rows(self, src, src_scale, index):
        rows = index.numel()
        dst = torch.empty((rows, src.shape[1]), dtype=src.dtype, device=src.device)
        dst_scale = torch.empty((rows,), dtype=torch.float32, device=src.device) if src_scale is not None else None
        rc = self.lib.w8a8_permute_rows(src.data_ptr(), None if src_scale is None else src_scale.data_ptr(),
                                        dst.data_ptr(), None if dst_scale is None else dst_scale.data_ptr(),
                                        index.data_ptr(), rows, src.shape[1] * src.element_size(), self._st())
        if rc != 0:
            raise RuntimeError(f"permute_rows: {self.L.status_string(rc)}")
        return dst, dst_scale

    def grouped_matmul_swiglu_quant(self, x, w, w_scale, x_scale, group_list):
        return self.ops.grouped_matmul_swiglu_quant(x, w, w_scale, x_scale, group_list)

    def grouped_matmul_int8(self, x, w, group_list, x_scale, w_scale):
        return self.ops.grouped_matmul(x, w, group_list, None, 3, False, x_scale=x_scale, weight_scale=w_scale)[0]

    def combine(self, rows, probs, pos):
        t, topk = probs.shape
        out = torch.empty((t, rows.shape[1]), dtype=rows.dtype, device=rows.device)
        code = self.L.DT_BF16 if rows.dtype == torch.bfloat16 else self.L.DT_F16
        rc = self.lib.w8a8_combine(rows.data_ptr(), probs.data_ptr(), pos.data_ptr(), out.data_ptr(), t, topk,
                                   rows.shape[1], code, self._st())
        if rc != 0:
            raise RuntimeError(f"combine: {self.L.status_string(rc)}")
        return out


# ---------------------------------------------------------------------------
@dataclass
class ExpertShard:
    """This rank's experts: up projection [E/P, hidden, 2*inter] + scales, down projection [E/P, inter, hidden]."""
    w_up: torch.Tensor
    s_up: torch.Tensor
    w_down: torch.Tensor
    s_down: torch.Tensor


class MoeFfnChain:
    def __init__(self, num_experts: int, shard: ExpertShard, backend=None, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world != 0:
            raise ValueError("the expert count must be divisible by the number of ranks")
        self.E = num_experts
        self.e_local = num_experts // self.world
        if shard.w_up.shape[0] != self.e_local or shard.w_down.shape[0] != self.e_local:
            raise ValueError("expert shard does not match E / world_size")
        self.shard = shard
        self.backend = backend if backend is not None else CudaBackend()
        self.last_counts: Optional[np.ndarray] = None

    # -- collectives --------------------------------------------------------
    def _all_to_all(self, send: torch.Tensor, send_rows: List[int], recv_rows: List[int]) -> torch.Tensor:
        out = torch.empty((sum(recv_rows),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        if self.world == 1:
            out.copy_(send)
            return out
        dist.all_to_all_single(out, send, output_split_sizes=recv_rows, input_split_sizes=send_rows, group=self.group)
        return out

    def _exchange_counts(self, count: torch.Tensor) -> np.ndarray:
        """count[E] (rows this rank sends to every global expert) -> recv_counts[P, E/P] on the host."""
        if self.world == 1:
            return count.cpu().numpy().reshape(1, self.e_local)
        send = count.reshape(self.world, self.e_local).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv.cpu().numpy()

    # -- the chain ----------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float,
                expert_idx: torch.Tensor, probs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x, residual [T_local, hidden] fp16/bf16; expert_idx int32 [T_local, topk]; probs fp32 [T_local, topk].
        Returns (ffn_out [T_local, hidden], residual_out [T_local, hidden])."""
        b = self.backend
        t, topk = expert_idx.shape
        xq, x_out, xs = b.add_rms_norm_dynamic_quant(x, residual, gamma, eps)
        count, _cumsum, pos = b.route_plan(expert_idx, self.E)
        send_rows_t, send_scale = b.scatter_rows(xq, xs, pos, t * topk)

        recv_counts = self._exchange_counts(count)                      # one small all-to-all + host read
        send_per_rank = count.cpu().numpy().reshape(self.world, self.e_local).sum(1)
        send_rows = [int(v) for v in send_per_rank]
        recv_rows = [int(v) for v in recv_counts.sum(1)]
        self.last_counts = recv_counts

        got = self._all_to_all(send_rows_t, send_rows, recv_rows)       # dispatch: int8 rows
        got_scale = self._all_to_all(send_scale, send_rows, recv_rows)  #           fp32 scales

        src_of_dst, group_cumsum = regroup_index(recv_counts)
        idx = torch.from_numpy(src_of_dst).to(x.device)
        xe, xe_scale = b.permute_rows(got, got_scale, idx)              # rank-major -> expert-major
        gl = [int(v) for v in group_cumsum]

        h, hs = b.grouped_matmul_swiglu_quant(xe, self.shard.w_up, self.shard.s_up, xe_scale, gl)
        y = b.grouped_matmul_int8(h, self.shard.w_down, gl, hs, self.shard.s_down)

        inv = torch.from_numpy(invert_index(src_of_dst)).to(x.device)
        y_rank_major, _ = b.permute_rows(y, None, inv)                  # expert-major -> rank-major
        back = self._all_to_all(y_rank_major, recv_rows, send_rows)     # combine transport: bf16 rows
        out = b.combine(back, probs, pos)
        return out, x_out
