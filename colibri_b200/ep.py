"""Expert-parallel MoE layer: one process per GPU, experts sharded, tokens data-parallel.

The reference places whole experts on devices by heat rank and moves rows host -> device
per call (c/colibri.c:8367-8417, 4819-4839); it has no collective library. Here every
rank routes its own M/G rows, an `ExpertMap` says which rank owns which expert (equal
blocks, or balanced by a routing histogram: the reference's heat-driven placement turned
into a load balancer), and rows travel to the owning rank and back with two all-to-all
exchanges (torch.distributed: NCCL over NVLink on GPUs, gloo in the CPU tests):

  1. route locally                          -> idx [m,K], w [m,K], keff [m]
  2. plan: live entries (row, kk < keff) ordered by (owner rank, expert slot on that rank, row order)
  3. all-to-all of the per-(rank, slot) entry counts
  4. all-to-all of the rows (bf16 when the activations are exact in bf16, else f32)
  5. expert FFN on the received rows, grouped per local expert
  6. all-to-all of the results (f32) back along the same plan
  7. out[row] = sum over kk in selection order of w[row,kk] * y[entry] (+ shared expert)

Step 7 adds in the row's selection order and every expert sees its rows one by one, so the
result is bit-identical for every G and every placement. The shared expert is replicated
and applied to the local rows while the dispatch is in flight.

Two implementations of the same plan:
  * `ep_moe_layer`  tensor ops + callbacks, device-agnostic: the host logic under test in
                    the gloo CPU tests (routing and expert FFN supplied by the CPU oracle);
  * `CudaEpLayer`   the GPU path: plan, packing, regrouping and combine are kernels of the
                    backend (coli_cuda_ep_plan_dev, coli_cuda_ep_expert_group_dev,
                    coli_cuda_ep_combine_dev); the host reads back one small table of
                    counts per layer (the split sizes of the all-to-all).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


class ExpertMap:
    """Placement of E experts on G ranks: dest[e] = owning rank, slot[e] = index among that
    rank's experts, local[r] = that rank's experts in slot order, slots = max per rank."""

    def __init__(self, E: int, G: int, dest=None):
        self.E, self.G = E, G
        if dest is None:
            per = (E + G - 1) // G
            dest = [e // per for e in range(E)]
        self.dest = [int(d) for d in dest]
        assert len(self.dest) == E and all(0 <= d < G for d in self.dest)
        self.local = [[e for e in range(E) if self.dest[e] == r] for r in range(G)]
        self.slot = [0] * E
        for r in range(G):
            for j, e in enumerate(self.local[r]):
                self.slot[e] = j
        self.slots = max(1, max(len(l) for l in self.local))

    @staticmethod
    def balanced(load, G: int) -> "ExpertMap":
        """Experts in descending load to the least-loaded rank that still has a free slot
        (every rank holds at most ceil(E/G) experts, so memory stays even). Ties go to the
        lower expert id and the lower rank: the map is a pure function of `load`."""
        load = [float(v) for v in load]
        E = len(load)
        cap = (E + G - 1) // G
        order = sorted(range(E), key=lambda e: (-load[e], e))
        tot, cnt, dest = [0.0] * G, [0] * G, [0] * E
        for e in order:
            r = min((r for r in range(G) if cnt[r] < cap), key=lambda r: (tot[r], r))
            dest[e] = r
            tot[r] += load[e]
            cnt[r] += 1
        return ExpertMap(E, G, dest)

    def rank_load(self, load):
        return [sum(float(load[e]) for e in self.local[r]) for r in range(self.G)]

    def imbalance(self, load) -> float:
        """max over ranks / mean over ranks of the rows a rank's experts receive."""
        rl = self.rank_load(load)
        mean = sum(rl) / len(rl)
        return max(rl) / mean if mean > 0 else 1.0


class DispatchPlan:
    """Where every (row, kk) entry goes and how to put the answers back (tensor ops)."""

    def __init__(self, idx: torch.Tensor, keff: torch.Tensor, emap: ExpertMap):
        m, K = idx.shape
        self.m, self.K = m, K
        G, slots = emap.G, emap.slots
        dev = idx.device
        nb = G * slots
        bucket_of = torch.tensor([emap.dest[e] * slots + emap.slot[e] for e in range(emap.E)], dtype=torch.int64, device=dev)
        kk = torch.arange(K, device=dev).unsqueeze(0)
        valid = (kk < keff.view(m, 1)).reshape(-1)
        # dead entries (kk >= keff) get the key nb and sort behind every live one; the stable sort
        # makes buckets ascend (owner rank, then slot) and keeps row order inside a bucket
        key = torch.where(valid, bucket_of[idx.reshape(-1)], torch.full((m * K,), nb, dtype=torch.int64, device=dev))
        order = torch.sort(key, stable=True).indices           # sorted position -> flat (row*K + kk)
        pos = torch.empty(m * K, dtype=torch.int64, device=dev)
        pos[order] = torch.arange(m * K, device=dev)
        self.entry_of = torch.where(valid, pos, torch.full_like(pos, -1)).view(m, K)   # (row, kk) -> send position
        counts = torch.bincount(key, minlength=nb + 1)[:nb]
        self.counts = counts.view(G, slots)                    # [dest rank, slot]
        self.counts_host = self.counts.tolist()
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


def _regroup(rc_host, device):
    """Receive order is (source rank, slot, row); the expert call wants (slot, source rank,
    row). -> (rows per slot, perm: expert-order position -> receive position)."""
    src_n, e_n = len(rc_host), len(rc_host[0])
    seg_start, acc = [[0] * e_n for _ in range(src_n)], 0
    for s_ in range(src_n):
        for e_ in range(e_n):
            seg_start[s_][e_] = acc
            acc += rc_host[s_][e_]
    perm = []
    for e_ in range(e_n):
        for s_ in range(src_n):
            perm.extend(range(seg_start[s_][e_], seg_start[s_][e_] + rc_host[s_][e_]))
    rows = [sum(rc_host[s_][e_] for s_ in range(src_n)) for e_ in range(e_n)]
    return rows, torch.tensor(perm, dtype=torch.int64, device=device)


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


def ep_moe_layer(x: torch.Tensor, route, experts, shared, emap: ExpertMap, group=None):
    """One expert-parallel MoE layer for this rank's rows x [m, D] with tensor ops.
    route(x) -> idx, w, keff (int64 / float32 / int64); experts(rows_per_slot, x) -> y for this
    rank's experts in slot order, rows in call order; shared(x) -> y or None.
    Returns out [m, D] and the routing."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    assert world == emap.G
    idx, w, keff = route(x)
    plan = DispatchPlan(idx, keff, emap)
    send_x = x.index_select(0, plan.send_rows)
    if world == 1:
        rc_host = [plan.counts_host[0]]
        recv_splits = plan.send_splits
        recv_x = send_x
    else:
        send_counts = plan.counts.to(torch.int64).contiguous()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts.view(-1), send_counts.view(-1), group=group)
        rc_host = recv_counts.tolist()                             # [src][slot]
        recv_splits = [int(sum(r)) for r in rc_host]
        recv_x = _all_to_all_rows(send_x, plan.send_splits, recv_splits, group)
    rows_per_slot, perm = _regroup(rc_host, x.device)
    ye = experts(rows_per_slot, recv_x.index_select(0, perm))
    back = torch.empty_like(ye)
    back[perm] = ye
    got = back if world == 1 else _all_to_all_rows(back, recv_splits, plan.send_splits, group)
    ys = shared(x) if shared is not None else None
    return _combine_torch(got, plan.entry_of, w, keff, ys), (idx, w, keff)


class PeerExchangeUnavailable(RuntimeError):
    """Raised on EVERY rank when some rank could not export or map the peer buffers (the ranks
    agree on it with a collective), so that a caller can build the layer with exchange="nccl"."""


class CudaEpLayer:
    """One expert-parallel MoE layer on this rank's GPU through the backend's device-pointer
    entries. `gates/ups/downs` are the handles of this rank's experts in slot order.

    Streams: the backend's kernels run on its own stream, the exchanges on a side stream of
    torch's, ordered by events, so the shared expert's GEMM (enqueued right after the packing)
    runs while the rows are in flight. The host waits once per layer, for the table of counts
    that gives the exchange its sizes.

    exchange: "nccl" moves the rows with all_to_all_single; "peer" (several ranks on one NVLink
    domain) pushes every block straight into the receiver's buffer with device-to-device copies
    over peer memory (copy engines, so they need no SM; about twice
    NCCL's all-to-all rate between two B200s), with a 4-byte all-reduce as the "everybody's rows
    have landed" barrier. Both give the same bits. max_rows must be the same on every rank."""

    def __init__(self, be, device, cfg, emap: ExpertMap, rank, gates, ups, downs, shared, bias,
                 routed_scale=2.5, max_rows=2048, payload="bf16", group=None, exchange="nccl"):
        import ctypes as C
        from .backend import Backend
        self.C, self.be, self.device, self.cfg, self.emap, self.rank, self.group = C, be, device, cfg, emap, rank, group
        self.dev = torch.device("cuda", device)
        self.n_loc = len(gates)
        assert self.n_loc == len(emap.local[rank])
        # slots beyond this rank's experts (uneven maps) never receive rows: pad with the first handle
        pad = lambda hs: list(hs) + [hs[0]] * (emap.slots - len(hs))
        self.g, self.u, self.d = (Backend.handle_array(pad(h)) for h in (gates, ups, downs))
        self.shared = shared
        if shared is not None:
            self.sg, self.su, self.sd = (Backend.handle_array([h]) for h in shared)
        self.bias = bias                     # torch tensor on the device or None
        self.scale = routed_scale
        self.bf16 = payload == "bf16"
        D, K, G, slots = cfg["D"], cfg["K"], emap.G, emap.slots
        i32 = dict(dtype=torch.int32, device=self.dev)
        self.dest = torch.tensor(emap.dest, **i32)
        self.slot = torch.tensor(emap.slot, **i32)
        self.idx = torch.empty((max_rows, K), **i32)
        self.w = torch.empty((max_rows, K), dtype=torch.float32, device=self.dev)
        self.keff = torch.empty((max_rows,), **i32)
        self.entry_of = torch.empty((max_rows * K,), **i32)
        self.counts = torch.zeros((2, G * slots), **i32)           # [0] sent per (dest, slot), [1] received per (src, slot)
        self.counts_pin = torch.zeros((2, G * slots), dtype=torch.int32).pin_memory()
        self.inexact = torch.zeros((1,), **i32)
        self.send = torch.empty((max_rows * K, D), dtype=torch.bfloat16 if self.bf16 else torch.float32, device=self.dev)
        self.ys = torch.empty((max_rows, D), dtype=torch.float32, device=self.dev) if shared is not None else None
        self.max_rows = max_rows
        self.bstream = torch.cuda.ExternalStream(be.stream(device), device=self.dev)
        self.cstream = torch.cuda.Stream(device=self.dev)
        self.timing = None                   # optional dict of event pairs (bench)
        self.exchange = exchange if G > 1 else "nccl"
        assert self.exchange in ("nccl", "peer")
        if self.exchange == "peer":
            self._open_peers(max_rows, D, K, G)

    def _open_peers(self, max_rows, D, K, G):
        """Receive buffer (rows from every rank, worst case all of them) and answer buffer (one row
        per own entry) in memory other ranks can map; everybody's handles, opened."""
        C, be = self.C, self.be
        esz = 2 if self.bf16 else 4
        self.recv_bytes = max_rows * G * K * D * esz
        self.got_bytes = max_rows * K * D * 4
        self.recv_buf = be.pipe_alloc(self.device, self.recv_bytes)
        self.got_buf = be.pipe_alloc(self.device, self.got_bytes)
        why = "" if self.recv_buf and self.got_buf else "peer buffers: allocation refused"
        mine = []
        for ptr in (self.recv_buf, self.got_buf):
            h = (C.c_ubyte * 64)()
            if not why and not be.pipe_ipc_export(self.device, ptr, h):
                why = "coli_cuda_pipe_ipc_export refused"
            mine.append(bytes(h))
        every = [None] * G
        dist.all_gather_object(every, (mine, why), group=self.group)
        self.peer_recv, self.peer_got = [None] * G, [None] * G
        self.peer_recv[self.rank], self.peer_got[self.rank] = self.recv_buf, self.got_buf
        if not any(w for _, w in every):
            for r in range(G):
                if r == self.rank:
                    continue
                ptrs = [be.pipe_ipc_open(self.device, (C.c_ubyte * 64).from_buffer_copy(hb)) for hb in every[r][0]]
                if not all(ptrs):
                    why = f"rank {self.rank} cannot map rank {r}'s buffers (coli_cuda_pipe_ipc_open)"
                self.peer_recv[r], self.peer_got[r] = ptrs
        # every rank learns whether all of them succeeded
        answers = [None] * G
        dist.all_gather_object(answers, why, group=self.group)
        bad = [w for w in answers if w] + [w for _, w in every if w]
        if bad:
            for r in range(G):
                if r != self.rank:
                    for q in (self.peer_recv[r], self.peer_got[r]):
                        if q:
                            be.pipe_ipc_close(self.device, q)
            for q in (self.recv_buf, self.got_buf):
                if q:
                    be.pipe_free(self.device, q)
            self.exchange = "nccl"
            raise PeerExchangeUnavailable("; ".join(sorted(set(bad))))
        self.flag = torch.zeros((1,), dtype=torch.int32, device=self.dev)
        self.counts_all = torch.zeros((G, G * self.emap.slots), dtype=torch.int32, device=self.dev)
        self.counts_all_pin = torch.zeros((G, G * self.emap.slots), dtype=torch.int32).pin_memory()
        self.e_comb = None
        self.cnt_np = self.counts_all_pin.numpy().reshape(G, G, self.emap.slots)      # [src][dest][slot], pinned
        dist.barrier(group=self.group)

    def close(self):
        """Unmaps the peers' buffers and frees this rank's (collective: every rank calls it)."""
        if self.exchange != "peer":
            return
        torch.cuda.synchronize(self.dev)
        for r in range(self.emap.G):
            if r != self.rank:
                self.be.pipe_ipc_close(self.device, self.peer_recv[r])
                self.be.pipe_ipc_close(self.device, self.peer_got[r])
        dist.barrier(group=self.group)
        self.be.pipe_free(self.device, self.recv_buf)
        self.be.pipe_free(self.device, self.got_buf)
        self.exchange = "nccl"

    def _check(self, ok, what):
        if not ok:
            raise RuntimeError(f"{what} failed")

    def route(self, logits, m):
        cfg, C = self.cfg, self.C
        self._check(self.be.route_topk_dev(self.device, logits.data_ptr(),
                                           self.bias.data_ptr() if self.bias is not None else None, m, cfg["E"],
                                           cfg["K"], cfg["gating"], cfg["norm_topk"], C.c_float(self.scale),
                                           C.c_float(0.0), self.idx.data_ptr(), self.w.data_ptr(),
                                           self.keff.data_ptr()), "coli_cuda_route_topk_dev")

    def __call__(self, x: torch.Tensor, logits: torch.Tensor):
        """x [m, D] f32 and logits [m, E] f32 on this rank's GPU, produced on the backend's
        stream or earlier. -> out [m, D] f32 (valid on the backend's stream)."""
        be, C, cfg, emap = self.be, self.C, self.cfg, self.emap
        m, D = x.shape
        K, G, slots, E = cfg["K"], emap.G, emap.slots, cfg["E"]
        assert m <= self.max_rows
        bs, cs = self.bstream, self.cstream
        ev = lambda: torch.cuda.Event(enable_timing=self.timing is not None)
        marks = {}
        if self.timing is not None:
            marks["t0"] = ev(); marks["t0"].record(bs)
        # 1-2. route, plan and pack on the backend's stream
        self.route(logits, m)
        self._check(be.ep_plan_dev(self.device, x.data_ptr(), m, D, K, self.idx.data_ptr(), self.keff.data_ptr(),
                                   self.dest.data_ptr(), self.slot.data_ptr(), E, G, slots, int(self.bf16),
                                   self.counts[0].data_ptr(), self.entry_of.data_ptr(), self.send.data_ptr(),
                                   self.inexact.data_ptr()), "coli_cuda_ep_plan_dev")
        e_pack = ev(); e_pack.record(bs)
        # the shared expert does not depend on the exchange: its GEMM runs while the rows travel
        if self.shared is not None:
            rows = (C.c_int * 1)(m)
            self._check(be.expert_group_dev(self.sg, self.su, self.sd, rows, 1, self.ys.data_ptr(), x.data_ptr()),
                        "coli_cuda_expert_group_dev (shared expert)")
        if self.exchange == "peer":
            return self._forward_peer(x, logits, m, D, K, G, slots, e_pack, marks, ev)
        # 3. counts exchange and the one read-back of the layer
        with torch.cuda.stream(cs):
            cs.wait_event(e_pack)
            if G > 1:
                dist.all_to_all_single(self.counts[1], self.counts[0], group=self.group)
            else:
                self.counts[1].copy_(self.counts[0])
            self.counts_pin.copy_(self.counts, non_blocking=True)
            e_cnt = ev(); e_cnt.record(cs)
        e_cnt.synchronize()
        cp = self.counts_pin.numpy()
        send_splits = cp[0].reshape(G, slots).sum(axis=1).tolist()
        recv_counts = np.ascontiguousarray(cp[1])                 # [src][slot]
        recv_splits = recv_counts.reshape(G, slots).sum(axis=1).tolist()
        n_send, n_recv = int(sum(send_splits)), int(sum(recv_splits))
        # 4. rows out
        with torch.cuda.stream(cs):
            if G > 1:
                recv_x = torch.empty((n_recv, D), dtype=self.send.dtype, device=self.dev)
                dist.all_to_all_single(recv_x, self.send[:n_send], output_split_sizes=recv_splits,
                                       input_split_sizes=send_splits, group=self.group)
            else:
                recv_x = self.send[:n_send]
            e_recv = ev(); e_recv.record(cs)
        # 5. local experts on the received rows, results in receive order
        bs.wait_event(e_recv)
        y = torch.empty((n_recv, D), dtype=torch.float32, device=self.dev)
        if self.timing is not None:
            marks["g0"] = ev(); marks["g0"].record(bs)
        if n_recv:
            self._check(be.ep_expert_group_dev(self.g, self.u, self.d, slots,
                                               recv_counts.ctypes.data_as(C.POINTER(C.c_int)), G, y.data_ptr(),
                                               recv_x.data_ptr(), int(self.bf16)), "coli_cuda_ep_expert_group_dev")
        e_gemm = ev(); e_gemm.record(bs)
        # 6. results back
        with torch.cuda.stream(cs):
            cs.wait_event(e_gemm)
            if G > 1:
                got = torch.empty((n_send, D), dtype=torch.float32, device=self.dev)
                dist.all_to_all_single(got, y, output_split_sizes=send_splits, input_split_sizes=recv_splits,
                                       group=self.group)
            else:
                got = y
            e_back = ev(); e_back.record(cs)
        # 7. combine
        bs.wait_event(e_back)
        out = torch.empty((m, D), dtype=torch.float32, device=self.dev)
        self._check(be.ep_combine_dev(self.device, out.data_ptr(), (got if n_send else out).data_ptr(),
                                      self.entry_of.data_ptr(), self.w.data_ptr(), self.keff.data_ptr(),
                                      self.ys.data_ptr() if self.ys is not None else None, m, K, D),
                    "coli_cuda_ep_combine_dev")
        for t in (recv_x, y, got, x, logits):        # keep the allocator from recycling them under queued work
            t.record_stream(bs); t.record_stream(cs)
        if self.timing is not None:
            marks["t1"] = ev(); marks["t1"].record(bs)
            marks.update(pack=e_pack, recv=e_recv, gemm=e_gemm, back=e_back)
            self.timing.setdefault("layers", []).append(marks)
        self.last = dict(n_send=n_send, n_recv=n_recv, send_splits=send_splits, recv_splits=recv_splits)
        return out

    def _forward_peer(self, x, logits, m, D, K, G, slots, e_pack, marks, ev):
        """Steps 3-7 over peer memory. The receive buffer holds the blocks in [source][slot] order
        and the answer buffer the rows in this rank's send order, exactly as the all-to-all
        leaves them, so the GEMM and the combine are the same calls."""
        be, C, me = self.be, self.C, self.rank
        bs, cs = self.bstream, self.cstream
        esz = 2 if self.bf16 else 4
        csh = C.c_void_p(cs.cuda_stream)

        def fan_out(jobs):
            """jobs: (peer, dst, src, bytes), one after the other on the exchange stream: they all
            leave through this GPU's NVLink ports, which one copy already fills (streams per peer
            were measured: no faster, and their events cost host time)."""
            for _, dst, src, nbytes in jobs:
                self._check(be.pipe_copy_async(self.device, C.c_void_p(dst), C.c_void_p(src), C.c_size_t(nbytes), csh),
                            "coli_cuda_pipe_copy_async")
        # 3. every rank's table of counts, and the one read-back of the layer
        with torch.cuda.stream(cs):
            cs.wait_event(e_pack)
            if self.e_comb is not None:
                cs.wait_event(self.e_comb)        # the previous call's combine has read the answer buffer
            dist.all_gather_into_tensor(self.counts_all.view(-1), self.counts[0], group=self.group)
            self.counts_all_pin.copy_(self.counts_all, non_blocking=True)
            e_cnt = ev(); e_cnt.record(cs)
        e_cnt.synchronize()
        mat = self.cnt_np.sum(axis=2)                                           # [src][dest] rows
        send_splits = mat[me].tolist()
        recv_counts = np.ascontiguousarray(self.cnt_np[:, me, :])               # [src][slot]
        recv_splits = mat[:, me].tolist()
        n_send, n_recv = int(sum(send_splits)), int(sum(recv_splits))
        assert n_recv * D * esz <= self.recv_bytes and n_send * D * 4 <= self.got_bytes
        send_off = np.concatenate(([0], np.cumsum(mat[me])))                   # my blocks in my send buffer
        recv_off = np.concatenate(([0], np.cumsum(mat[:, me])))                # sources' blocks in my receive buffer
        # 4. rows out: block (me -> d) goes behind the blocks of the ranks below me in d's buffer
        with torch.cuda.stream(cs):
            fan_out([(d, self.peer_recv[d] + int(mat[:me, d].sum()) * D * esz,
                      self.send.data_ptr() + int(send_off[d]) * D * esz, int(mat[me, d]) * D * esz)
                     for d in range(G) if mat[me, d]])
            dist.all_reduce(self.flag, group=self.group)       # every rank's copies were enqueued before it joined
            e_recv = ev(); e_recv.record(cs)
        # 5. local experts on the received rows, results in receive order
        bs.wait_event(e_recv)
        y = torch.empty((max(n_recv, 1), D), dtype=torch.float32, device=self.dev)
        if self.timing is not None:
            marks["g0"] = ev(); marks["g0"].record(bs)
        if n_recv:
            self._check(be.ep_expert_group_dev(self.g, self.u, self.d, slots,
                                               recv_counts.ctypes.data_as(C.POINTER(C.c_int)), G, y.data_ptr(),
                                               C.c_void_p(self.recv_buf), int(self.bf16)), "coli_cuda_ep_expert_group_dev")
        e_gemm = ev(); e_gemm.record(bs)
        # 6. results back: block (s -> me) returns to where s keeps its block for me
        with torch.cuda.stream(cs):
            cs.wait_event(e_gemm)
            fan_out([(s, self.peer_got[s] + int(mat[s, :me].sum()) * D * 4,
                      y.data_ptr() + int(recv_off[s]) * D * 4, int(mat[s, me]) * D * 4)
                     for s in range(G) if mat[s, me]])
            dist.all_reduce(self.flag, group=self.group)
            e_back = ev(); e_back.record(cs)
        # 7. combine
        bs.wait_event(e_back)
        out = torch.empty((m, D), dtype=torch.float32, device=self.dev)
        self._check(be.ep_combine_dev(self.device, out.data_ptr(), C.c_void_p(self.got_buf),
                                      self.entry_of.data_ptr(), self.w.data_ptr(), self.keff.data_ptr(),
                                      self.ys.data_ptr() if self.ys is not None else None, m, K, D),
                    "coli_cuda_ep_combine_dev")
        self.e_comb = torch.cuda.Event(); self.e_comb.record(bs)
        for t in (y, x, logits):
            t.record_stream(bs); t.record_stream(cs)
        if self.timing is not None:
            marks["t1"] = ev(); marks["t1"].record(bs)
            marks.update(pack=e_pack, recv=e_recv, gemm=e_gemm, back=e_back)
            self.timing.setdefault("layers", []).append(marks)
        self.last = dict(n_send=n_send, n_recv=n_recv, send_splits=send_splits, recv_splits=recv_splits)
        return out

    def check_exact(self):
        """Raises if a bf16 payload rounded a value (the caller must use payload='f32' then)."""
        if self.bf16 and int(self.inexact.item()) != 0:
            raise RuntimeError("activations are not exact in bf16: use payload='f32'")
