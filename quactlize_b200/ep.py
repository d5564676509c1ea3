"""Expert-parallel MoE FFN over the GPUs of one node, one process per GPU, with no host round trip inside a step.

Experts are sharded contiguously (rank r owns experts [r*E/W, (r+1)*E/W), leading-axis views of every artifact tensor);
tokens stay where they are.  One step, all on the current stream:

  plan      per-expert route counts (one small kernel); `ep_sync` stores them into every rank's table through mapped
            memory and lets the ranks meet (epoch words, bounded wait); from the table a single-CTA kernel gives every
            route its final row in its owner's EXPERT-MAJOR receive buffer -- nothing is copied to the host
            (`plan_routes` states the same plan in torch index arithmetic; the tests hold the kernel to it);
  dispatch  `ep_dispatch`: every routed token row is stored straight into the owner's receive buffer at that row
            (NVLink peer stores into IPC-mapped buffers), with a tag saying where its result must come back to;
  meeting   `ep_sync` again orders those stores before the owners' reads (sync="nccl": a one-element all_reduce, and an
            all_gather for the counts above);
  compute   gate/up grouped GEMM (tensor cores) -> silu(gate)*up -> down grouped GEMM whose EPILOGUE stores every output
            row at its return address, i.e. directly into the sender's combine buffer (`out_rows` of the plane GEMM);
  meeting   a third one, then each rank sums its tokens' top-k rows with the router weights.

With the default sync="peer" a step contains no collective at all; NCCL serves the set-up (IPC handle exchange).

So the regrouping permutations of an all_to_all formulation do not exist: rows land expert-major, results land in the
order of the sender's own routes.  The receive buffers hold `capacity` rows (every rank could be sent everything); the
GEMMs are launched for that capacity and find their real row count in the device-side offsets.

`transport="nccl"` keeps the same step on NCCL all_to_all with host-known split sizes (one device->host copy per step)
for boxes where IPC peer mapping is unavailable.  The reference has no multi-device code for this path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
import torch.distributed as dist

import quactlize_b200 as qb
from . import _lib


def plan_routes(expert_of_route: torch.Tensor, counts_all: torch.Tensor, rank: int):
    """Where each of this rank's routes goes.  expert_of_route int64 [R] (any order); counts_all int [W, E] = every rank's
    routes per global expert.  Returns (order, dst_rank, dst_pos, local_offsets):

      order          int64 [R]  this rank's routes sorted by expert (stable): route `order[i]` is sent as item i
      dst_rank       int32 [R]  owner of item i's expert
      dst_pos        int32 [R]  its row in the owner's receive buffer: experts in order, and inside an expert the
                                sources in rank order, each source's rows in its own sorted order
      local_offsets  int32 [E/W + 1]  cumulative rows per LOCAL expert of this rank (what its grouped GEMM reads)

    Pure index arithmetic on the tensors' device; no communication, no host copy."""
    world, experts = counts_all.shape
    per = experts // world
    counts_all = counts_all.to(torch.int64)
    order = torch.argsort(expert_of_route, stable=True)
    es = expert_of_route[order]
    tot = counts_all.sum(0)                                               # rows per global expert
    blk = tot.view(world, per)
    base = (blk.cumsum(1) - blk).reshape(-1)                              # first row of expert e in its owner's buffer
    src_off = (counts_all.cumsum(0) - counts_all)[rank]                   # rows of lower ranks inside expert e
    mine = counts_all[rank]
    local_start = mine.cumsum(0) - mine                                   # first item of expert e among my sorted routes
    idx = torch.arange(es.numel(), device=es.device, dtype=torch.int64)
    dst_pos = (base + src_off)[es] + (idx - local_start[es])
    dst_rank = es // per
    lo = rank * per
    local = torch.zeros(per + 1, dtype=torch.int64, device=es.device)
    local[1:] = tot[lo:lo + per].cumsum(0)
    return order, dst_rank.to(torch.int32), dst_pos.to(torch.int32), local.to(torch.int32)


class _Array:
    """A device buffer owned outside torch, visible to torch through the CUDA array interface."""
    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


class PeerBuffers:
    """This rank's receive buffers (rows, return addresses, combine rows) and the mapped buffers of every peer."""

    def __init__(self, capacity: int, row_elems: int, routes_capacity: int, out_elems: int, group=None, experts: int = 0):
        self.group, self.L = group, _lib.lib()
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        sync_bytes = self.L.quactlize_b200_ep_sync_bytes(self.world, experts)
        if sync_bytes <= 0:
            raise RuntimeError(f"no sync area for {self.world} ranks and {experts} experts")
        sizes = {"rows": capacity * row_elems * 2, "ret": capacity * 8, "comb": routes_capacity * out_elems * 2, "sync": sync_bytes}
        self.own, handles = {}, {}
        for name, nbytes in sizes.items():
            p, h = C.c_void_p(), C.create_string_buffer(64)
            rc = self.L.quactlize_b200_peer_alloc(nbytes, C.byref(p), h)
            if rc:
                raise RuntimeError(f"peer buffer allocation failed (rc={rc})")
            self.own[name], handles[name] = p.value, h.raw
        everyone = [None] * self.world
        dist.all_gather_object(everyone, handles, group=group)
        self.mapped, self.ptrs = [], {n: [] for n in sizes}
        for r, hs in enumerate(everyone):
            for name in sizes:
                if r == self.rank:
                    self.ptrs[name].append(self.own[name])
                    continue
                p = C.c_void_p()
                rc = self.L.quactlize_b200_peer_open(hs[name], C.byref(p))
                if rc:
                    raise RuntimeError(f"mapping rank {r}'s {name} buffer failed (rc={rc}): IPC peer access is unavailable")
                self.mapped.append(p.value)
                self.ptrs[name].append(p.value)
        as_dev = lambda xs: torch.tensor([int(x) for x in xs], dtype=torch.int64, device=dev)
        self.peer_rows, self.peer_ret, self.peer_comb = as_dev(self.ptrs["rows"]), as_dev(self.ptrs["ret"]), as_dev(self.ptrs["comb"])
        self.rows = torch.as_tensor(_Array(self.own["rows"], (capacity, row_elems), "<i2"), device=dev).view(torch.bfloat16)
        self.ret = torch.as_tensor(_Array(self.own["ret"], (capacity,), "<i8"), device=dev)
        self.comb = torch.as_tensor(_Array(self.own["comb"], (routes_capacity, out_elems), "<i2"), device=dev).view(torch.bfloat16)
        self.comb_base, self.comb_row_bytes = self.own["comb"], out_elems * 2
        self.peer_sync = as_dev(self.ptrs["sync"])
        self.sync = torch.as_tensor(_Array(self.own["sync"], (sync_bytes // 4,), "<i4"), device=dev)
        self.sync.zero_()                                    # epochs start at zero everywhere before anybody posts
        self.counts_all = self.sync[256:256 + self.world * experts].view(self.world, experts) if experts else None
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def close(self):
        torch.cuda.synchronize()
        dist.barrier(group=self.group)                       # nobody still writes into a buffer that is about to go
        for p in self.mapped:
            self.L.quactlize_b200_peer_close(p)
        self.rows = self.ret = self.comb = self.sync = self.counts_all = None
        for p in self.own.values():
            self.L.quactlize_b200_peer_free(p)
        self.mapped, self.own = [], {}


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def silu_mul(gate_up: torch.Tensor, rows_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = silu(gate_up[r, :f]) * gate_up[r, f:], bf16; rows_dev (int32 [1], device) bounds the rows that exist."""
    rows, f2 = gate_up.shape
    out = torch.empty((rows, f2 // 2), dtype=torch.bfloat16, device=gate_up.device)
    rc = _lib.lib().quactlize_b200_silu_mul_dev_v1(_p(gate_up), _p(out), _p(rows_dev), rows, f2 // 2,
                                                   C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc:
        raise RuntimeError(f"silu_mul failed (rc={rc})")
    return out


def _gemm(a, art, bits, gs, offsets, out=None, out_rows=None):
    low, scale, zero = art
    e, n, k = low.shape[0], low.shape[1], a.shape[1]
    if out is None and out_rows is None:
        out = torch.empty((a.shape[0], n), dtype=a.dtype, device=a.device)
    rc = _lib.lib().quactlize_b200_gemm_plane_dev_v2(_p(a), _p(low), None, _p(scale), _p(zero), _p(out), a.shape[0], n, k, bits, 0, gs, 0,
                                                     1 if a.dtype == torch.bfloat16 else 0, e, _p(offsets), _p(out_rows),
                                                     C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc:
        raise RuntimeError(f"grouped GEMM failed (rc={rc})")
    return out


def local_ffn(rows: torch.Tensor, offsets: torch.Tensor, gate_up, down, bits: int, gs: int, out_rows=None):
    """gate/up GEMM -> silu*mul -> down GEMM over rows grouped by the experts of `gate_up` / `down` (plane artifacts
    (low, scale, zero) with a leading expert axis); offsets int32 [E+1] on the device, rows.shape[0] may be a capacity."""
    gu = _gemm(rows, gate_up, bits, gs, offsets)
    act = silu_mul(gu, offsets[-1:])
    return _gemm(act, down, bits, gs, offsets, out_rows=out_rows)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def combine(comb: torch.Tensor, item_of_route: torch.Tensor, weights: torch.Tensor, tokens: int, top_k: int) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * comb[item_of_route[t*top_k + j]] (fp32 in route order) -> bf16 [tokens, hidden]."""
    h = comb.shape[1]
    out = torch.empty((tokens, h), dtype=torch.bfloat16, device=comb.device)
    w = weights.to(torch.float32).contiguous()
    rc = _lib.lib().quactlize_b200_ep_combine_dev_v1(_p(comb), _p(item_of_route), _p(w), _p(out), tokens, top_k, h, _stream())
    if rc:
        raise RuntimeError(f"combine failed (rc={rc})")
    return out


class Plan:
    """Device-side plan of one step (see ep_plan in the C header): per item the token, owner rank and row in the owner's
    buffer; per route its item; the cumulative rows per local expert."""
    __slots__ = ("item_token", "item_rank", "item_pos", "item_of_route", "local_off", "local_total", "counts", "counts_flat",
                 "counts_all", "routes")


class ExpertParallelFFN:
    """The MoE FFN of one layer, experts sharded over the process group (see the module text).

    gate_up / down: this rank's plane artifacts (low uint8 [E_local, n, k*bits/8], scale fp16, zero fp16 [E_local, k/gs, n]);
    capacity: rows the receive buffer holds (the routes of ALL ranks is always enough)."""

    def __init__(self, gate_up, down, experts: int, top_k: int, bits: int, group_size: int, capacity: int, max_local_routes: int,
                 transport: str = "peer", group=None, sync: str = "peer"):
        self.gate_up, self.down, self.experts, self.top_k, self.bits, self.gs = gate_up, down, experts, top_k, bits, group_size
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        if experts % self.world:
            raise ValueError(f"{experts} experts do not divide over {self.world} ranks")
        self.hidden, self.ffn = gate_up[0].shape[2] * 8 // bits, down[0].shape[2] * 8 // bits
        self.capacity, self.transport = capacity, transport
        self.buf = PeerBuffers(capacity, self.hidden, max_local_routes, self.hidden, group, experts) if transport == "peer" else None
        # how the ranks meet inside a step: "peer" = epoch words in mapped memory (one small kernel per meeting, no collective
        # in the step at all), "nccl" = all_gather of the counts and one-element all_reduces
        self.sync = sync if transport == "peer" else "nccl"
        dev = gate_up[0].device
        self._flag = torch.zeros(1, device=dev)
        self._plans = {}
        self._addr = torch.zeros(capacity, dtype=torch.int64, device=dev) if transport == "peer" else None

    def close(self):
        if self.buf is not None:
            self.buf.close()
            self.buf = None

    def _barrier(self, which: int):
        if self.sync == "peer":
            rc = _lib.lib().quactlize_b200_ep_sync_dev_v1(_p(self.buf.peer_sync), self.rank, self.world, which, None, 0, _stream())
            if rc:
                raise RuntimeError(f"rendezvous failed (rc={rc})")
        else:
            dist.all_reduce(self._flag, group=self.group)    # stream-ordered: peers' stores before this, reads after it

    def plan(self, routes: torch.Tensor) -> Plan:
        """ep_count -> all_gather of the counts -> ep_plan: three launches, nothing copied to the host."""
        L = _lib.lib()
        flat = routes.reshape(-1)
        if flat.dtype != torch.int64 or not flat.is_contiguous():
            flat = flat.to(torch.int64).contiguous()
        r, dev = flat.numel(), flat.device
        p = self._plans.get(r)
        if p is None:                                        # the buffers of a plan are reused by every step of this size
            p = Plan()
            p.routes = r
            p.item_token, p.item_rank, p.item_pos, p.item_of_route = (torch.empty(max(r, 1), dtype=torch.int32, device=dev) for _ in range(4))
            p.local_off = torch.empty(self.experts // self.world + 1, dtype=torch.int32, device=dev)
            p.local_total = p.local_off[-1:]
            p.counts = torch.empty(self.experts, dtype=torch.int32, device=dev)
            p.counts_flat = torch.empty(self.world * self.experts, dtype=torch.int32, device=dev)
            p.counts_all = p.counts_flat.view(self.world, self.experts)
            self._plans[r] = p
        rc = L.quactlize_b200_ep_count_dev_v1(_p(flat), r, self.experts, _p(p.counts), _stream())
        if self.sync == "peer":                              # every rank's counts land in every rank's table, then a meeting
            rc = rc or L.quactlize_b200_ep_sync_dev_v1(_p(self.buf.peer_sync), self.rank, self.world, 0, _p(p.counts), self.experts, _stream())
            table = self.buf.counts_all
        else:
            dist.all_gather_into_tensor(p.counts_flat, p.counts, group=self.group)
            table = p.counts_flat
        rc = rc or L.quactlize_b200_ep_plan_dev_v1(_p(flat), _p(table), self.rank, self.world, self.experts, r, self.top_k,
                                                   _p(p.item_token), _p(p.item_rank), _p(p.item_pos), _p(p.item_of_route),
                                                   _p(p.local_off), _stream())
        if rc:
            raise RuntimeError(f"expert-parallel plan failed (rc={rc})")
        return p

    def __call__(self, x: torch.Tensor, routes: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """x bf16 [T, hidden]; routes int64 [T, top_k] expert ids; weights [T, top_k] -> bf16 [T, hidden]."""
        L = _lib.lib()
        p = self.plan(routes)
        x = x.contiguous()
        if self.transport == "peer":
            b = self.buf
            rc = L.quactlize_b200_ep_dispatch_dev_v1(_p(x), _p(p.item_token), _p(p.item_rank), _p(p.item_pos), _p(b.peer_rows),
                                                     _p(b.peer_ret), self.rank, p.routes, self.hidden * 2, _stream())
            if rc:
                raise RuntimeError(f"dispatch failed (rc={rc})")
            self._barrier(1)
            rc = L.quactlize_b200_ep_return_addr_dev_v1(_p(b.ret), _p(b.peer_comb), self.world, _p(p.local_total), self.capacity,
                                                        self.hidden * 2, _p(self._addr), _stream())
            if rc:
                raise RuntimeError(f"return addresses failed (rc={rc})")
            local_ffn(b.rows, p.local_off, self.gate_up, self.down, self.bits, self.gs, out_rows=self._addr)
            self._barrier(2)
            comb = b.comb
        else:
            comb = self._nccl_step(x, p)
        return combine(comb, p.item_of_route, weights, x.shape[0], self.top_k)

    def _nccl_step(self, x, p: Plan):
        """The same step on NCCL all_to_all with host-known split sizes: one device->host copy of the counts."""
        per = self.experts // self.world
        c = p.counts_all.cpu().to(torch.int64)                            # [W, E]
        send = c[self.rank].view(self.world, per).sum(1).tolist()
        recv = c[:, self.rank * per:(self.rank + 1) * per].sum(1).tolist()
        rows = x[p.item_token[:p.routes].long()].contiguous()             # item order = expert order = destination-rank order
        got = rows.new_empty((sum(recv), self.hidden))
        dist.all_to_all_single(got, rows, output_split_sizes=recv, input_split_sizes=send, group=self.group)
        # received source-major (s, e); the grouped GEMM wants expert-major (e, s)
        blocks = c[:, self.rank * per:(self.rank + 1) * per]              # [W, per]
        dst_start = (blocks.t().reshape(-1).cumsum(0) - blocks.t().reshape(-1)).view(per, self.world)
        perm = torch.cat([torch.arange(int(blocks[s, j]), dtype=torch.int64) + int(dst_start[j, s])
                          for s in range(self.world) for j in range(per)]).to(x.device)
        grouped = torch.empty_like(got)
        grouped[perm] = got
        out = local_ffn(grouped, p.local_off, self.gate_up, self.down, self.bits, self.gs)
        back = out[perm].contiguous()
        comb = back.new_empty((rows.shape[0], self.hidden))
        dist.all_to_all_single(comb, back, output_split_sizes=send, input_split_sizes=recv, group=self.group)
        return comb
