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

Two transports for the two exchanges:

    "nccl"  pack -> all_to_all_single -> regroup kernel on the way in; un-permute kernel -> all_to_all_single on
            the way back.  Works on any backend (gloo in the CPU tests).
    "p2p"   the exchanges are fused into the kernels on either side of them: the dispatch kernel stores every
            quantised row directly at its final expert-major position in the owning rank's buffer, and the down
            projection's epilogue stores every output row directly where its home rank's combine reads it.  The
            stores are plain peer stores over NVLink into symmetric buffers (torch symmetric memory supplies the
            peer pointers); the only collectives left are the small count all-gather and two stream barriers.

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

    def dispatch_rows(self, src, src_scale, expert_idx, pos, row_dst, scale_dst, my_base):
        t, topk = pos.shape
        rc = self.lib.w8a8_dispatch_rows(src.data_ptr(), src_scale.data_ptr(), expert_idx.data_ptr(), pos.data_ptr(),
                                         row_dst.data_ptr(), scale_dst.data_ptr(), my_base.data_ptr(), t, topk,
                                         src.shape[1] * src.element_size(), self._st())
        if rc != 0:
            raise RuntimeError(f"dispatch_rows: {self.L.status_string(rc)}")

    def expand_row_pointers(self, seg_first, seg_ptr, rows, row_bytes):
        out = torch.empty((max(rows, 1),), dtype=torch.int64, device=seg_first.device)
        rc = self.lib.w8a8_expand_row_pointers(seg_first.data_ptr(), seg_ptr.data_ptr(), seg_ptr.numel(), rows,
                                               row_bytes, out.data_ptr(), self._st())
        if rc != 0:
            raise RuntimeError(f"expand_row_pointers: {self.L.status_string(rc)}")
        return out

    def grouped_matmul_int8_to_rows(self, x, w, group_list, x_scale, w_scale, out_row_ptrs, out_dtype):
        m, k = x.shape
        e, _, n = w.shape
        lib, L = self.lib, self.L
        need = lib.w8a8_grouped_matmul_workspace_size(m, n, k, e)
        ws = torch.empty((max(need, 1),), dtype=torch.uint8, device=x.device)
        gl = torch.tensor([int(v) for v in group_list], dtype=torch.int64)
        code = L.DT_BF16 if out_dtype == torch.bfloat16 else L.DT_F16
        rc = lib.w8a8_grouped_matmul_to_rows(x.data_ptr(), w.data_ptr(), None, out_row_ptrs.data_ptr(),
                                             x_scale.data_ptr(), w_scale.data_ptr(), m, n, k, e, gl.data_ptr(), 0,
                                             L.DT_I8, L.DT_F32, code, L.W_KN, ws.data_ptr(), need, self._st())
        if rc != 0:
            raise RuntimeError(f"grouped_matmul_to_rows: {L.status_string(rc)}")

    # -- forms that take their row count from a device list (no host readback) ---------------------------
    def ep_tables(self, gathered, rank, peer_base, off_x, off_s, off_back, row_bytes, back_row_bytes, cap_rows, out):
        p, e = gathered.shape
        rc = self.lib.w8a8_ep_tables(gathered.data_ptr(), p, e, rank, peer_base.data_ptr(), off_x, off_s, off_back,
                                     row_bytes, back_row_bytes, cap_rows, out["row_dst"].data_ptr(),
                                     out["scale_dst"].data_ptr(), out["my_base"].data_ptr(),
                                     out["group_list"].data_ptr(), out["seg_first"].data_ptr(),
                                     out["seg_ptr"].data_ptr(), out["status"].data_ptr(), self._st())
        if rc != 0:
            raise RuntimeError(f"ep_tables: {self.L.status_string(rc)}")

    def grouped_matmul_swiglu_quant_capacity(self, x, w, w_scale, x_scale, group_list_dev, y, y_scale, workspace):
        """x, x_scale, y, y_scale hold `capacity` rows; the device list says how many of them exist."""
        cap, k = x.shape
        e, _, n = w.shape
        L = self.L
        rc = self.lib.w8a8_grouped_matmul_swiglu_quant(x.data_ptr(), w.data_ptr(), w_scale.data_ptr(),
                                                       x_scale.data_ptr(), y.data_ptr(), y_scale.data_ptr(), cap, k,
                                                       n, e, group_list_dev.data_ptr(), 2, L.W_KN, 0,
                                                       workspace.data_ptr(), workspace.numel(), self._st())
        if rc != 0:
            raise RuntimeError(f"grouped_matmul_swiglu_quant: {L.status_string(rc)}")

    def grouped_matmul_int8_to_rows_capacity(self, x, w, group_list_dev, x_scale, w_scale, out_row_ptrs, out_dtype,
                                             workspace):
        cap, k = x.shape
        e, _, n = w.shape
        L = self.L
        code = L.DT_BF16 if out_dtype == torch.bfloat16 else L.DT_F16
        rc = self.lib.w8a8_grouped_matmul_to_rows(x.data_ptr(), w.data_ptr(), None, out_row_ptrs.data_ptr(),
                                                  x_scale.data_ptr(), w_scale.data_ptr(), cap, n, k, e,
                                                  group_list_dev.data_ptr(), 2, L.DT_I8, L.DT_F32, code, L.W_KN,
                                                  workspace.data_ptr(), workspace.numel(), self._st())
        if rc != 0:
            raise RuntimeError(f"grouped_matmul_to_rows: {L.status_string(rc)}")

    def expand_row_pointers_into(self, seg_first, seg_ptr, nseg, rows, row_bytes, out):
        rc = self.lib.w8a8_expand_row_pointers(seg_first.data_ptr(), seg_ptr.data_ptr(), nseg, rows, row_bytes,
                                               out.data_ptr(), self._st())
        if rc != 0:
            raise RuntimeError(f"expand_row_pointers: {self.L.status_string(rc)}")

    def workspace_bytes(self, cap, hidden, inter):
        lib = self.lib
        return max(lib.w8a8_grouped_matmul_swiglu_quant_workspace_size(cap, hidden, 2 * inter, 1 << 10),
                   lib.w8a8_grouped_matmul_workspace_size(cap, hidden, inter, 1 << 10))

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


def _align(v: int, a: int = 256) -> int:
    return (v + a - 1) // a * a


class PeerBuffers:
    """One symmetric allocation per rank holding the expert-major receive buffer (int8 rows + fp32 scales) and
    the combine receive buffer (16-bit rows), plus every rank's pointer to it."""

    def __init__(self, cap_rows: int, hidden: int, home_rows: int, device, world: int, group):
        self.cap_rows, self.hidden, self.home_rows = cap_rows, hidden, home_rows
        self.off_x = 0
        self.off_s = _align(cap_rows * hidden)
        self.off_back = self.off_s + _align(cap_rows * 4)
        total = self.off_back + _align(home_rows * hidden * 2)
        if world == 1:
            self.buf = torch.empty((total,), dtype=torch.uint8, device=device)
            self.ptrs = [self.buf.data_ptr()]
        else:
            import os

            import torch.distributed._symmetric_memory as symm_mem

            # plain peer loads / stores only: no NVLink multicast object is bound to these buffers
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            self.buf = symm_mem.empty((total,), dtype=torch.uint8, device=device)
            name = group.group_name if group is not None else dist.group.WORLD.group_name
            self.handle = symm_mem.rendezvous(self.buf, name)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.xe = self.buf[self.off_x:self.off_x + cap_rows * hidden].view(torch.int8).view(cap_rows, hidden)
        self.xs = self.buf[self.off_s:self.off_s + cap_rows * 4].view(torch.float32)


class MoeFfnChain:
    def __init__(self, num_experts: int, shard: ExpertShard, backend=None, group=None, transport: str = "nccl",
                 capacity_rows: Optional[int] = None, device_tables: Optional[bool] = None,
                 native_step: Optional[bool] = None):
        self.group = group
        if transport not in ("nccl", "p2p"):
            raise ValueError("transport must be 'nccl' or 'p2p'")
        self.transport = transport
        self.capacity_rows = capacity_rows
        # p2p transport only: build the address tables on the device from the gathered counts, so that a step has
        # no host readback at all (the row counts then exist only on the device and the grouped matmuls are
        # launched on the buffers' capacity with a device list that says how many rows exist)
        self._dev_state = None
        self.peer: Optional[PeerBuffers] = None
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        # Default: tables built on the device at every rank count, so that no step ever waits for the host (with
        # the host readback the step was 4 % slower on 8 GPUs and equal within noise on 1 and 2).
        self.device_tables = True if device_tables is None else bool(device_tables)
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world != 0:
            raise ValueError("the expert count must be divisible by the number of ranks")
        self.E = num_experts
        self.e_local = num_experts // self.world
        if shard.w_up.shape[0] != self.e_local or shard.w_down.shape[0] != self.e_local:
            raise ValueError("expert shard does not match E / world_size")
        self.shard = shard
        self.backend = backend if backend is not None else CudaBackend()
        # p2p transport with device-built tables: the whole step is ONE call of the library's C++ step function
        # (w8a8_moe_ffn_step, with its own NCCL communicator for the count all-gather and the barriers); the
        # Python sequence of the same calls stays for injected backends (the CPU tests) and for comparison
        self.native_step = (backend is None) if native_step is None else bool(native_step)
        self._native = None
        self.last_counts: Optional[np.ndarray] = None
        # measurement hook: called with a phase name after each phase of a step has been enqueued (the benchmark
        # records a CUDA event there); None in normal use
        self.phase_hook = None

    def _mark(self, name: str) -> None:
        if self.phase_hook is not None:
            self.phase_hook(name)

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
    def _barrier(self, device) -> None:
        """All ranks' kernels issued so far are complete, stream-ordered (no host synchronisation)."""
        if self.world > 1:
            token = torch.zeros((1,), dtype=torch.int32, device=device)
            dist.all_reduce(token, group=self.group)

    def _forward_p2p(self, x, residual, gamma, eps, expert_idx, probs):
        b = self.backend
        dev = x.device
        t, topk = expert_idx.shape
        hidden = x.shape[1]
        xq, x_out, xs = b.add_rms_norm_dynamic_quant(x, residual, gamma, eps)
        self._mark("add_rms_norm_dynamic_quant")
        count, _cumsum, pos = b.route_plan(expert_idx, self.E)
        self._mark("route_plan")

        # every rank learns every rank's per-expert counts (P x E integers), then all index arithmetic is local
        if self.world > 1:
            gathered = torch.empty((self.world, self.E), dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(gathered, count, group=self.group)
            C = gathered.cpu().numpy()
        else:
            C = count.cpu().numpy().reshape(1, self.E)
        self._mark("count_all_gather_and_host_tables")
        self.last_counts = C[:, self.rank * self.e_local:(self.rank + 1) * self.e_local]
        col = C.sum(0)                                               # rows per expert over all ranks
        base_of_rank = np.cumsum(C, 1) - C                            # [P, E]: rank i's own expert-major positions
        owner = np.arange(self.E) // self.e_local
        ex_incl = np.cumsum(col.reshape(self.world, self.e_local), 1)
        ex_base = (ex_incl - col.reshape(self.world, self.e_local)).reshape(-1)   # expert's first row at its owner
        before_me = C[:self.rank].sum(0)                              # rows of lower ranks inside each expert
        rows_on = ex_incl[:, -1]                                      # rows each owner receives
        if self.peer is None:
            cap = self.capacity_rows
            if cap is None:
                # room for 1.5x a balanced share; routing more skewed than that needs an explicit capacity
                cap = int(1.5 * t * topk) + 1024
            self.peer = PeerBuffers(cap, hidden, t * topk, dev, self.world, self.group)
        pb = self.peer
        if int(rows_on.max()) > pb.cap_rows or t * topk > pb.home_rows:
            raise RuntimeError("expert-parallel receive buffer too small for this routing: raise capacity_rows")

        dst_row = ex_base + before_me
        ptrs = np.asarray(pb.ptrs, dtype=np.uint64)
        row_dst = ptrs[owner] + np.uint64(pb.off_x) + dst_row.astype(np.uint64) * np.uint64(hidden)
        scale_dst = ptrs[owner] + np.uint64(pb.off_s) + dst_row.astype(np.uint64) * np.uint64(4)
        tables = np.stack([row_dst.view(np.int64), scale_dst.view(np.int64), base_of_rank[self.rank].astype(np.int64)])
        tables_dev = torch.from_numpy(tables).to(dev)

        # No barrier is needed before the stores: the count all-gather above has completed on this rank, so every
        # other rank's stream has reached its own all-gather of this step, which it enqueued after everything
        # that read its buffers in the previous step.
        b.dispatch_rows(xq, xs, expert_idx, pos, tables_dev[0], tables_dev[1], tables_dev[2])
        self._mark("dispatch_stores")
        self._barrier(dev)   # every rank's rows have landed
        self._mark("barrier_after_dispatch")

        mine = slice(self.rank * self.e_local, (self.rank + 1) * self.e_local)
        rows_me = int(rows_on[self.rank])
        gl = [int(v) for v in ex_incl[self.rank]]
        xe = pb.xe[:rows_me]
        h, hs = b.grouped_matmul_swiglu_quant(xe, self.shard.w_up, self.shard.s_up, pb.xs[:rows_me], gl)
        self._mark("grouped_matmul_swiglu_quant")

        # one segment per (local expert, source rank): where its rows start here, and where they go home
        cm = C[:, mine]                                               # [P, E_loc]
        seg_len = cm.T.reshape(-1)                                    # ordered (expert, source rank)
        seg_first = np.concatenate([[0], np.cumsum(seg_len)]).astype(np.int64)
        home = base_of_rank[:, mine].T.reshape(-1).astype(np.uint64)  # row in the source rank's send order
        src_rank = np.tile(np.arange(self.world), self.e_local)
        elem = x.element_size()
        seg_ptr = ptrs[src_rank] + np.uint64(pb.off_back) + home * np.uint64(hidden * elem)
        seg_dev = torch.from_numpy(np.concatenate([seg_first, seg_ptr.view(np.int64)])).to(dev)
        nseg = seg_len.size
        out_ptrs = b.expand_row_pointers(seg_dev[:nseg + 1], seg_dev[nseg + 1:], rows_me, hidden * elem)
        if rows_me > 0:
            b.grouped_matmul_int8_to_rows(h, self.shard.w_down, gl, hs, self.shard.s_down, out_ptrs, x.dtype)
        self._mark("down_projection_with_peer_stores")
        self._barrier(dev)   # every rank's output rows have landed at home
        self._mark("barrier_after_down_projection")

        back = pb.buf[pb.off_back:pb.off_back + t * topk * hidden * elem].view(x.dtype).view(t * topk, hidden)
        out = b.combine(back, probs, pos)
        self._mark("combine")
        return out, x_out

    # -- the step as one C++ call ---------------------------------------------------------------------------
    def _native_state(self, x, expert_idx):
        """Peer buffers, the library's NCCL communicator, the step descriptor and its workspace (made once)."""
        from . import _lib as L
        import ctypes

        t, topk = expert_idx.shape
        hidden = x.shape[1]
        dev = x.device
        key = (t, topk, hidden, x.dtype)
        if self._native is not None and self._native["key"] == key:
            return self._native
        lib = L.load()
        if self.peer is None:
            cap = self.capacity_rows
            if cap is None:
                cap = int(1.5 * t * topk) + 1024
            self.peer = PeerBuffers(cap, hidden, t * topk, dev, self.world, self.group)
        pb = self.peer
        comm = ctypes.c_void_p(None)
        if self.world > 1:
            if self._native is not None:
                comm = self._native["comm"]
            else:
                ident = torch.zeros((128,), dtype=torch.uint8, device=dev)
                if self.rank == 0:
                    raw = (ctypes.c_uint8 * 128)()
                    rc = lib.w8a8_ep_unique_id(raw)
                    if rc != 0:
                        raise RuntimeError(f"ep_unique_id: {L.status_string(rc)}")
                    ident.copy_(torch.tensor(list(raw), dtype=torch.uint8))
                src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
                dist.broadcast(ident, src=src, group=self.group)
                raw = (ctypes.c_uint8 * 128)(*ident.cpu().tolist())
                with torch.cuda.device(dev):
                    rc = lib.w8a8_ep_comm_create(raw, self.world, self.rank, ctypes.byref(comm))
                if rc != 0:
                    raise RuntimeError(f"ep_comm_create: {L.status_string(rc)}")
        peer_base = torch.tensor([int(p) for p in pb.ptrs], dtype=torch.int64, device=dev)
        step = L.MoeFfnStep()
        step.world, step.rank, step.num_experts, step.topk = self.world, self.rank, self.E, topk
        step.dtype = L.DT_BF16 if x.dtype == torch.bfloat16 else L.DT_F16
        step.tokens, step.hidden, step.inter = t, hidden, self.shard.w_down.shape[1]
        step.cap_rows, step.home_rows = pb.cap_rows, pb.home_rows
        step.peer_base, step.local_base = peer_base.data_ptr(), pb.buf.data_ptr()
        step.off_x, step.off_s, step.off_back = pb.off_x, pb.off_s, pb.off_back
        step.w_up, step.s_up = self.shard.w_up.data_ptr(), self.shard.s_up.data_ptr()
        step.w_down, step.s_down = self.shard.w_down.data_ptr(), self.shard.s_down.data_ptr()
        step.comm = comm
        step.workspace, step.workspace_bytes = None, 0
        need = lib.w8a8_moe_ffn_step_workspace_size(ctypes.byref(step))
        if need == 0:
            raise RuntimeError("moe_ffn_step: invalid step description")
        ws = torch.zeros((need,), dtype=torch.uint8, device=dev)
        step.workspace, step.workspace_bytes = ws.data_ptr(), need
        self._native = {"key": key, "step": step, "workspace": ws, "peer_base": peer_base, "comm": comm, "lib": lib,
                        "L": L}
        return self._native

    def _forward_native(self, x, residual, gamma, eps, expert_idx, probs):
        import ctypes

        st = self._native_state(x, expert_idx)
        for tns in (x, residual, gamma, expert_idx, probs):
            if not tns.is_contiguous():
                raise ValueError("the step takes contiguous tensors")
        out = torch.empty_like(x)
        x_out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            rc = st["lib"].w8a8_moe_ffn_step(ctypes.byref(st["step"]), x.data_ptr(), residual.data_ptr(),
                                             gamma.data_ptr(), float(eps), expert_idx.data_ptr(), probs.data_ptr(),
                                             out.data_ptr(), x_out.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"moe_ffn_step: {st['L'].status_string(rc)}")
        return out, x_out

    def _forward_p2p_device_tables(self, x, residual, gamma, eps, expert_idx, probs):
        """The p2p step with no host readback: count all-gather -> ep_tables kernel -> dispatch -> grouped matmuls
        on the capacity with a device group list -> combine.  `check()` reads the overflow flag when asked."""
        b = self.backend
        dev = x.device
        t, topk = expert_idx.shape
        hidden = x.shape[1]
        elem = x.element_size()
        inter = self.shard.w_down.shape[1]
        if self.peer is None:
            cap = self.capacity_rows
            if cap is None:
                cap = int(1.5 * t * topk) + 1024
            self.peer = PeerBuffers(cap, hidden, t * topk, dev, self.world, self.group)
        pb = self.peer
        if t * topk > pb.home_rows:
            raise RuntimeError("expert-parallel return buffer too small for this batch: raise capacity_rows")
        cap = pb.cap_rows
        nseg = self.e_local * self.world
        if self._dev_state is None:
            i64 = dict(dtype=torch.int64, device=dev)
            self._dev_state = {
                "peer_base": torch.tensor([int(p) for p in pb.ptrs], dtype=torch.int64, device=dev),
                "gathered": torch.empty((self.world, self.E), **i64),
                "row_dst": torch.empty((self.E,), **i64), "scale_dst": torch.empty((self.E,), **i64),
                "my_base": torch.empty((self.E,), **i64), "group_list": torch.empty((self.e_local,), **i64),
                "seg_first": torch.empty((nseg + 1,), **i64), "seg_ptr": torch.empty((nseg,), **i64),
                "status": torch.zeros((4,), dtype=torch.int32, device=dev),
                "h": torch.empty((cap, inter), dtype=torch.int8, device=dev),
                "hs": torch.empty((cap,), dtype=torch.float32, device=dev),
                "out_ptrs": torch.empty((cap,), **i64),
                "workspace": torch.empty((b.workspace_bytes(cap, hidden, inter),), dtype=torch.uint8, device=dev),
            }
        st = self._dev_state
        xq, x_out, xs = b.add_rms_norm_dynamic_quant(x, residual, gamma, eps)
        self._mark("add_rms_norm_dynamic_quant")
        count, _cumsum, pos = b.route_plan(expert_idx, self.E)
        self._mark("route_plan")
        if self.world > 1:
            dist.all_gather_into_tensor(st["gathered"], count, group=self.group)
        else:
            st["gathered"].copy_(count.view(1, self.E))
        b.ep_tables(st["gathered"], self.rank, st["peer_base"], pb.off_x, pb.off_s, pb.off_back, hidden,
                    hidden * elem, cap, st)
        self._mark("count_all_gather_and_device_tables")
        # No barrier is needed before the stores: the count all-gather above has completed on this rank, so every
        # other rank's stream has reached its own all-gather of this step, which it enqueued after everything
        # that read its buffers in the previous step.
        b.dispatch_rows(xq, xs, expert_idx, pos, st["row_dst"], st["scale_dst"], st["my_base"])
        self._mark("dispatch_stores")
        self._barrier(dev)   # every rank's rows have landed
        self._mark("barrier_after_dispatch")
        b.grouped_matmul_swiglu_quant_capacity(pb.xe, self.shard.w_up, self.shard.s_up, pb.xs, st["group_list"],
                                               st["h"], st["hs"], st["workspace"])
        self._mark("grouped_matmul_swiglu_quant")
        b.expand_row_pointers_into(st["seg_first"], st["seg_ptr"], nseg, cap, hidden * elem, st["out_ptrs"])
        b.grouped_matmul_int8_to_rows_capacity(st["h"], self.shard.w_down, st["group_list"], st["hs"],
                                               self.shard.s_down, st["out_ptrs"], x.dtype, st["workspace"])
        self._mark("down_projection_with_peer_stores")
        self._barrier(dev)   # every rank's output rows have landed at home
        self._mark("barrier_after_down_projection")
        back = pb.buf[pb.off_back:pb.off_back + t * topk * hidden * elem].view(x.dtype).view(t * topk, hidden)
        out = b.combine(back, probs, pos)
        self._mark("combine")
        return out, x_out

    def close(self) -> None:
        """Releases the C++ step's NCCL communicator (every rank must call it, or none)."""
        if self._native is not None and self._native["comm"].value:
            rc = self._native["lib"].w8a8_ep_comm_destroy(self._native["comm"])
            self._native = None
            if rc != 0:
                raise RuntimeError("ep_comm_destroy failed")
        self._native = None

    def check(self) -> None:
        """Device-table mode: raises if any step since the last check routed more rows to a rank than its buffers
        hold (the flag is sticky on the device and cleared here; reading it synchronises, so call it when that is
        acceptable)."""
        if self._dev_state is not None and int(self._dev_state["status"][0].item()) != 0:
            self._dev_state["status"].zero_()
            raise RuntimeError("expert-parallel receive buffer too small for this routing: raise capacity_rows")
        if self._native is not None:
            import ctypes

            with torch.cuda.device(self._native["workspace"].device):
                rc = self._native["lib"].w8a8_moe_ffn_step_status(ctypes.byref(self._native["step"]),
                                                                  torch.cuda.current_stream().cuda_stream)
            if rc == 1:
                raise RuntimeError("expert-parallel receive buffer too small for this routing: raise capacity_rows")
            if rc != 0:
                raise RuntimeError(f"moe_ffn_step_status: {self._native['L'].status_string(rc)}")

    def forward(self, x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float,
                expert_idx: torch.Tensor, probs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x, residual [T_local, hidden] fp16/bf16; expert_idx int32 [T_local, topk]; probs fp32 [T_local, topk].
        Returns (ffn_out [T_local, hidden], residual_out [T_local, hidden])."""
        if self.transport == "p2p":
            if self.device_tables:
                if self.native_step and self.phase_hook is None:
                    return self._forward_native(x, residual, gamma, eps, expert_idx, probs)
                return self._forward_p2p_device_tables(x, residual, gamma, eps, expert_idx, probs)
            return self._forward_p2p(x, residual, gamma, eps, expert_idx, probs)
        b = self.backend
        t, topk = expert_idx.shape
        xq, x_out, xs = b.add_rms_norm_dynamic_quant(x, residual, gamma, eps)
        self._mark("add_rms_norm_dynamic_quant")
        count, _cumsum, pos = b.route_plan(expert_idx, self.E)
        self._mark("route_plan")
        send_rows_t, send_scale = b.scatter_rows(xq, xs, pos, t * topk)
        self._mark("scatter_rows")

        recv_counts = self._exchange_counts(count)                      # one small all-to-all + host read
        send_per_rank = count.cpu().numpy().reshape(self.world, self.e_local).sum(1)
        send_rows = [int(v) for v in send_per_rank]
        recv_rows = [int(v) for v in recv_counts.sum(1)]
        self.last_counts = recv_counts
        self._mark("count_exchange_and_host_read")

        got = self._all_to_all(send_rows_t, send_rows, recv_rows)       # dispatch: int8 rows
        got_scale = self._all_to_all(send_scale, send_rows, recv_rows)  #           fp32 scales
        self._mark("dispatch_all_to_all")

        src_of_dst, group_cumsum = regroup_index(recv_counts)
        idx = torch.from_numpy(src_of_dst).to(x.device)
        xe, xe_scale = b.permute_rows(got, got_scale, idx)              # rank-major -> expert-major
        gl = [int(v) for v in group_cumsum]
        self._mark("regroup_rows")

        h, hs = b.grouped_matmul_swiglu_quant(xe, self.shard.w_up, self.shard.s_up, xe_scale, gl)
        self._mark("grouped_matmul_swiglu_quant")
        y = b.grouped_matmul_int8(h, self.shard.w_down, gl, hs, self.shard.s_down)
        self._mark("down_projection")

        inv = torch.from_numpy(invert_index(src_of_dst)).to(x.device)
        y_rank_major, _ = b.permute_rows(y, None, inv)                  # expert-major -> rank-major
        self._mark("inverse_regroup")
        back = self._all_to_all(y_rank_major, recv_rows, send_rows)     # combine transport: bf16 rows
        self._mark("combine_all_to_all")
        out = b.combine(back, probs, pos)
        self._mark("combine")
        return out, x_out
