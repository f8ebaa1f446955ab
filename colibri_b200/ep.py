"""Expert-parallel MoE layer: one process per GPU, experts sharded, tokens data-parallel.

The reference places whole experts on devices and moves rows host -> device per
call (c/colibri.c:8367-8417, 4819-4839); it has no collective library. Here rank
r owns experts [r*E/G, (r+1)*E/G), every rank routes its own M/G rows, and rows
travel to the owning rank and back with two all-to-all exchanges
(torch.distributed: NCCL over NVLink on GPUs, gloo in the CPU tests):

  1. route locally                          -> idx [m,K], w [m,K], keff [m]
  2. plan: entries (row, kk<keff) sorted by (owner rank, expert, row order)
  3. all-to-all of the per-expert row counts (G*E/G ints per rank)
  4. all-to-all of the rows (f32, so that results do not depend on G)
  5. expert FFN on the received rows, grouped per local expert
  6. all-to-all of the results back along the same plan
  7. out[row] = sum over kk in selection order of w[row,kk] * y[entry] (+ shared expert)

Step 7 adds in the row's selection order and every expert sees its rows one by
one, so the result of this layer is bit-identical for every G. The shared
expert is replicated and applied to the local rows.

The layer is written against two callbacks so that the host logic (steps 2-4,
6, 7) runs unchanged on CPU tensors in the gloo tests:
  route(x)                      -> idx, w, keff            (int64/float32/int64 tensors)
  experts(rows_per_expert, x)   -> y                       (local experts, rows in call order)
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class DispatchPlan:
    """Where every (row, kk) entry goes and how to put the answers back."""

    def __init__(self, idx: torch.Tensor, keff: torch.Tensor, E: int, world: int):
        m, K = idx.shape
        self.m, self.K, self.E, self.world = m, K, E, world
        self.e_loc = E // world
        dev = idx.device
        kk = torch.arange(K, device=dev).unsqueeze(0)
        valid = (kk < keff.view(m, 1)).reshape(-1)
        # dead entries (kk >= keff) get the key E and sort behind every live one; the stable sort
        # makes experts ascend (so owner ranks ascend) and keeps row order inside an expert
        key = torch.where(valid, idx.reshape(-1), torch.full_like(idx.reshape(-1), E))
        order = torch.sort(key, stable=True).indices           # sorted position -> flat (row*K + kk)
        pos = torch.empty(m * K, dtype=torch.int64, device=dev)
        pos[order] = torch.arange(m * K, device=dev)
        self.entry_of = torch.where(valid, pos, torch.full_like(pos, -1)).view(m, K)   # (row, kk) -> send position
        counts = torch.bincount(key, minlength=E + 1)[:E]
        self.counts = counts.view(world, self.e_loc)           # [dest rank, local expert]
        self.counts_host = self.counts.tolist()                # the one host synchronisation of the plan
        self.send_splits = [int(sum(r)) for r in self.counts_host]
        self.n = int(sum(self.send_splits))
        self.send_rows = torch.div(order[:self.n], K, rounding_mode="floor")   # source row of every sent entry


def _all_to_all_rows(send: torch.Tensor, send_splits, recv_splits, group):
    recv = send.new_empty((int(sum(recv_splits)),) + tuple(send.shape[1:]))
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(recv, send, output_split_sizes=list(recv_splits),
                               input_split_sizes=list(send_splits), group=group)
    else:
        recv.copy_(send)
    return recv


def _combine_torch(got, entry_of, w, keff, ys):
    """Step 7 with tensor ops (CPU tests): selection order, shared expert last."""
    m, K = entry_of.shape
    out = torch.zeros((m, got.shape[1]), dtype=got.dtype, device=got.device)
    for kk in range(K):
        ent = entry_of[:, kk]
        live = ent >= 0
        contrib = got.index_select(0, ent.clamp(min=0)) * w[:, kk].unsqueeze(1)
        out = out + torch.where(live.unsqueeze(1), contrib, torch.zeros_like(contrib))
    return out if ys is None else out + ys


def ep_moe_layer(x: torch.Tensor, route, experts, shared, E: int, group=None, combine=None):
    """One expert-parallel MoE layer for this rank's rows x [m, D]. Returns out [m, D]
    and the routing (idx, w, keff). combine(got, entry_of, w, keff, ys) -> out replaces
    the tensor-op combine (the CUDA layer passes its kernel)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    m, D = x.shape
    idx, w, keff = route(x)
    plan = DispatchPlan(idx, keff, E, world)
    # 4. rows out, grouped by (dest rank, expert, row order)
    send_x = x.index_select(0, plan.send_rows)
    if world == 1:
        # one rank: the send buffer already is the expert-order buffer
        got = experts(plan.counts_host[0], send_x)
    else:
        # 3. counts: recv_counts[src, local expert]
        send_counts = plan.counts.to(torch.int64).contiguous()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts.view(-1), send_counts.view(-1), group=group)
        rc_host = recv_counts.tolist()                             # [src][local expert]
        recv_splits = [int(sum(r)) for r in rc_host]
        recv_x = _all_to_all_rows(send_x, plan.send_splits, recv_splits, group)
        # received rows are ordered (source rank, local expert, row order); the expert call wants
        # (local expert, source rank, row order)
        src_n, e_n = len(rc_host), len(rc_host[0])
        seg_start, acc = [[0] * e_n for _ in range(src_n)], 0
        for s_ in range(src_n):
            for e_ in range(e_n):
                seg_start[s_][e_] = acc
                acc += rc_host[s_][e_]
        n_recv = acc
        starts, lengths = [], []
        for e_ in range(e_n):
            for s_ in range(src_n):
                starts.append(seg_start[s_][e_]); lengths.append(rc_host[s_][e_])
        lengths_t = torch.tensor(lengths, dtype=torch.int64, device=x.device)
        starts_t = torch.tensor(starts, dtype=torch.int64, device=x.device)
        dst_start = torch.cumsum(lengths_t, 0) - lengths_t
        perm = (torch.repeat_interleave(starts_t - dst_start, lengths_t, output_size=n_recv) +
                torch.arange(n_recv, device=x.device))            # expert-order position -> recv position
        rows_per_expert = [sum(rc_host[s_][e_] for s_ in range(src_n)) for e_ in range(e_n)]
        xe = recv_x.index_select(0, perm)
        # 5. local experts
        ye = experts(rows_per_expert, xe)
        # 6. results back along the same plan
        back = torch.empty_like(ye)
        back[perm] = ye
        got = _all_to_all_rows(back, recv_splits, plan.send_splits, group)   # [n, D] in send-buffer order
    # 7. weighted combine in selection order, shared expert last
    ys = shared(x) if shared is not None else None
    out = (combine or _combine_torch)(got, plan.entry_of, w, keff, ys)
    return out, (idx, w, keff)


class CudaEpLayer:
    """The callbacks of ep_moe_layer on one GPU: routing and expert FFN by the
    CUDA backend (device pointers of torch tensors), experts [lo, hi) resident here.
    All work is enqueued on the backend's stream, a blocking stream, so it orders
    with torch's default stream and with the NCCL exchanges torch issues."""

    def __init__(self, be, device, cfg, gates, ups, downs, shared, bias, lo, routed_scale=2.5):
        import ctypes as C
        from .backend import Backend
        self.C = C
        self.be, self.device, self.cfg, self.lo = be, device, cfg, lo
        self.n_loc = len(gates)
        self.g, self.u, self.d = Backend.handle_array(gates), Backend.handle_array(ups), Backend.handle_array(downs)
        self.shared = shared
        if shared is not None:
            self.sg, self.su, self.sd = (Backend.handle_array([h]) for h in shared)
        self.bias = bias                     # torch tensor on the device or None
        self.scale = routed_scale
        self.logits = None                   # set per call by the driver

    def route(self, x):
        cfg, C = self.cfg, self.C
        m = x.shape[0]
        K, E = cfg["K"], cfg["E"]
        idx = torch.empty((m, K), dtype=torch.int32, device=x.device)
        w = torch.empty((m, K), dtype=torch.float32, device=x.device)
        keff = torch.empty((m,), dtype=torch.int32, device=x.device)
        ok = self.be.route_topk_dev(self.device, self.logits.data_ptr(),
                                    self.bias.data_ptr() if self.bias is not None else None, m, E, K,
                                    cfg["gating"], cfg["norm_topk"], C.c_float(self.scale), C.c_float(0.0),
                                    idx.data_ptr(), w.data_ptr(), keff.data_ptr())
        if not ok:
            raise RuntimeError("coli_cuda_route_topk_dev failed")
        return idx.to(torch.int64), w, keff.to(torch.int64)

    def _group(self, g, u, d, rows, xe):
        import numpy as np
        y = torch.empty_like(xe)
        if xe.shape[0] == 0:
            return y
        r = np.ascontiguousarray(rows, np.int32)
        ok = self.be.expert_group_dev(g, u, d, r.ctypes.data_as(self.C.POINTER(self.C.c_int)), len(r),
                                      y.data_ptr(), xe.data_ptr())
        if not ok:
            raise RuntimeError("coli_cuda_expert_group_dev failed")
        return y

    def experts(self, rows, xe):
        return self._group(self.g, self.u, self.d, rows, xe.contiguous())

    def combine(self, got, entry_of, w, keff, ys):
        out = torch.empty((entry_of.shape[0], got.shape[1]), dtype=torch.float32, device=got.device)
        if got.shape[0] == 0:
            got = out                        # no live entry: the pointer is never read
        ok = self.be.moe_combine_dev(self.device, out.data_ptr(), got.data_ptr(), entry_of.data_ptr(),
                                     w.data_ptr(), keff.data_ptr(), ys.data_ptr() if ys is not None else None,
                                     entry_of.shape[0], entry_of.shape[1], got.shape[1])
        if not ok:
            raise RuntimeError("coli_cuda_moe_combine_dev failed")
        return out

    def shared_fn(self, x):
        return self._group(self.sg, self.su, self.sd, [x.shape[0]], x.contiguous())
