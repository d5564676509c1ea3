"""Multi-GPU forms of the two shapes the path shards into, one process per GPU over torch.distributed.

The reference has no multi-device code for this path; these wrappers stay in host code and call the single-GPU
device-pointer entries, as the raw-pointer ABI intends (quactlize/include/quactlize_ppu_device.h:12-14: the caller owns
streams and ordering).

* Dense weights: COLUMN PARALLEL over the output dimension n.  Rank r owns output rows [lo, hi) of the weight -- a
  contiguous run of raw blocks (row-major by output row, quactlize/routes.py:19-23) or the same slice of every plane
  along its n axis.  The activation is replicated, outputs are disjoint, so the data path has NO collective; an
  optional all_gather assembles y.
* MoE weights: EXPERT PARALLEL.  Experts are the leading axis of every artifact tensor
  (quactlize/csrc/preprocess/thop/gguf_prepass_ops.cpp:836-841), so rank r owns experts [r*E/W, (r+1)*E/W) as views.
  One exchange each way: all_to_all of per-expert row counts, all_to_all(v) of the gathered token rows to the ranks
  that own their experts, the local ragged grouped kernel, all_to_all(v) of the results back.

Everything here works on any backend: NCCL on GPUs, gloo on CPU tensors for the host-side logic.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------------------------------------------------
# column-parallel dense
# ---------------------------------------------------------------------------------------------------------------------

def column_range(n: int, rank: int, world: int, multiple: int = 1) -> Tuple[int, int]:
    """Output rows [lo, hi) of rank `rank`: n/multiple units dealt as evenly as possible, contiguous, in rank order."""
    if n % multiple:
        raise ValueError(f"n={n} is not a multiple of {multiple}")
    units = n // multiple
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * multiple, hi * multiple


def shard_blocks(blocks: torch.Tensor, n: int, k: int, rank: int, world: int, multiple: int = 1) -> torch.Tensor:
    """Raw GGUF blocks [n*k/256, type_size] -> this rank's rows, a view."""
    bpr = k // 256
    if blocks.dim() != 2 or blocks.shape[0] != n * bpr:
        raise ValueError(f"blocks should be [{n * bpr}, type_size], got {tuple(blocks.shape)}")
    lo, hi = column_range(n, rank, world, multiple)
    return blocks[lo * bpr:hi * bpr]


def shard_planes(tensors: Sequence[Optional[torch.Tensor]], n_axes: Sequence[int], n: int, rank: int, world: int,
                 multiple: int = 1) -> List[Optional[torch.Tensor]]:
    """Slice every artifact tensor along its n axis: planes [E,n,bytes] (axis 1), fp16 scale/zero [E,k/gs,n] (axis 2),
    packed units [E,U,n,bytes] (axis 2).  Empty tensors (an absent high plane) pass through."""
    lo, hi = column_range(n, rank, world, multiple)
    out = []
    for t, ax in zip(tensors, n_axes):
        if t is None or t.numel() == 0:
            out.append(t)
            continue
        if t.shape[ax] != n:
            raise ValueError(f"axis {ax} of a tensor shaped {tuple(t.shape)} is not n={n}")
        out.append(t.narrow(ax, lo, hi - lo).contiguous())
    return out


def gather_columns(y_local: torch.Tensor, n: int, multiple: int = 1, group=None) -> torch.Tensor:
    """all_gather of the disjoint output slices [m, n_local] -> [m, n] on every rank."""
    world = dist.get_world_size(group)
    widths = [column_range(n, r, world, multiple) for r in range(world)]
    parts = [y_local.new_empty((y_local.shape[0], hi - lo)) for lo, hi in widths]
    if len({hi - lo for lo, hi in widths}) == 1:
        dist.all_gather(parts, y_local.contiguous(), group=group)
    else:                                             # uneven slices: one broadcast per owner
        for r, p in enumerate(parts):
            if r == dist.get_rank(group):
                p.copy_(y_local)
            dist.broadcast(p, src=dist.get_global_rank(group, r) if group is not None else r, group=group)
    return torch.cat(parts, dim=1)


# ---------------------------------------------------------------------------------------------------------------------
# expert-parallel MoE
# ---------------------------------------------------------------------------------------------------------------------

def expert_range(experts: int, rank: int, world: int) -> Tuple[int, int]:
    """Experts [lo, hi) owned by `rank` (contiguous; experts must divide evenly so every rank runs the same kernels)."""
    if experts % world:
        raise ValueError(f"{experts} experts do not divide over {world} ranks")
    per = experts // world
    return rank * per, (rank + 1) * per


def shard_experts(tensors: Sequence[Optional[torch.Tensor]], experts: int, rank: int, world: int):
    """Leading-axis views of every artifact tensor for the experts this rank owns."""
    lo, hi = expert_range(experts, rank, world)
    out = []
    for t in tensors:
        if t is None or t.numel() == 0:
            out.append(t)
            continue
        if t.shape[0] != experts:
            raise ValueError(f"leading axis of a tensor shaped {tuple(t.shape)} is not the expert count {experts}")
        out.append(t[lo:hi])
    return out


@dataclass
class DispatchPlan:
    """Where every row goes and comes back from, for one step.  All small host tensors."""
    send_rows: List[int]            # rows this rank sends to each rank
    recv_rows: List[int]            # rows this rank receives from each rank
    recv_counts: torch.Tensor       # int64 [world, E_local]: rows from source rank s for local expert j
    perm: torch.Tensor              # int64 [R]: received (source-major) position -> expert-major position
    offsets: torch.Tensor           # int32 [E_local+1]: cumulative rows per local expert after the permutation
    max_rows: int


def plan_dispatch(rows_per_expert: torch.Tensor, experts: int, group=None) -> DispatchPlan:
    """rows_per_expert: this rank's gathered rows per GLOBAL expert (rows are sorted by expert).  Exchanges the counts
    (one all_to_all of world*E_local integers) and derives splits, the regrouping permutation and local offsets."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    per = experts // world
    if rows_per_expert.numel() != experts:
        raise ValueError(f"rows_per_expert has {rows_per_expert.numel()} entries, expected {experts}")
    mine = rows_per_expert.detach().to(device="cpu", dtype=torch.int64).reshape(world, per).contiguous()
    if bool((mine < 0).any()):
        raise ValueError("rows_per_expert must be nonnegative")
    dev = _comm_device(group)
    theirs = torch.empty_like(mine, device=dev)
    dist.all_to_all_single(theirs, mine.to(dev), group=group)
    theirs = theirs.cpu()
    send_rows = mine.sum(dim=1).tolist()
    recv_rows = theirs.sum(dim=1).tolist()
    # received layout: for s in ranks: for j in local experts: theirs[s, j] rows.  Wanted: for j: for s.
    src_start = torch.zeros(world * per + 1, dtype=torch.int64)
    src_start[1:] = theirs.reshape(-1).cumsum(0)                      # start of block (s, j) in the received buffer
    dst_counts = theirs.t().contiguous()                               # [per, world]
    dst_start = torch.zeros(world * per + 1, dtype=torch.int64)
    dst_start[1:] = dst_counts.reshape(-1).cumsum(0)                   # start of block (j, s) after regrouping
    total = int(theirs.sum())
    perm = torch.empty(total, dtype=torch.int64)
    for s in range(world):
        for j in range(per):
            c = int(theirs[s, j])
            if c:
                a, b = int(src_start[s * per + j]), int(dst_start[j * world + s])
                perm[a:a + c] = torch.arange(b, b + c)
    per_expert = theirs.sum(dim=0)
    offsets = torch.zeros(per + 1, dtype=torch.int32)
    offsets[1:] = per_expert.cumsum(0).to(torch.int32)
    return DispatchPlan(send_rows, recv_rows, theirs, perm, offsets, int(per_expert.max()) if per else 0)


def _comm_device(group=None) -> torch.device:
    return torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")


def expert_parallel_apply(a: torch.Tensor, rows_per_expert: torch.Tensor, experts: int, n_out: int,
                          compute: Callable[[torch.Tensor, torch.Tensor, int], torch.Tensor], group=None,
                          plan: Optional[DispatchPlan] = None) -> torch.Tensor:
    """One expert-parallel grouped matmul.

    a                 this rank's gathered rows [R, k], sorted by global expert
    rows_per_expert   this rank's rows per global expert, int [experts]
    compute(rows, offsets, max_rows) -> [rows, n_out]: the single-GPU ragged kernel over this rank's experts
                      (rows grouped by local expert, cumulative int32 offsets [E_local+1] on the rows' device)
    Returns the outputs of this rank's own rows, in their original order, [R, n_out] in compute's dtype.
    """
    if plan is None:
        plan = plan_dispatch(rows_per_expert, experts, group)
    if a.shape[0] != sum(plan.send_rows):
        raise ValueError(f"rows_per_expert sums to {sum(plan.send_rows)}, activation has {a.shape[0]} rows")
    total = sum(plan.recv_rows)
    recv = a.new_empty((total, a.shape[1]))
    dist.all_to_all_single(recv, a.contiguous(), output_split_sizes=plan.recv_rows, input_split_sizes=plan.send_rows, group=group)
    perm = plan.perm.to(a.device)
    grouped = torch.empty_like(recv)
    grouped[perm] = recv                                              # source-major -> expert-major
    out_grouped = compute(grouped, plan.offsets.to(a.device), plan.max_rows)
    if out_grouped.shape != (total, n_out):
        raise ValueError(f"compute returned {tuple(out_grouped.shape)}, expected {(total, n_out)}")
    back = out_grouped[perm].contiguous()                             # expert-major -> source-major
    out = back.new_empty((a.shape[0], n_out))
    dist.all_to_all_single(out, back, output_split_sizes=plan.send_rows, input_split_sizes=plan.recv_rows, group=group)
    return out


def imbalance(plan: DispatchPlan, group=None) -> Tuple[int, float]:
    """(rows this rank computes, max-over-ranks / mean) -- what the expert-parallel step time follows."""
    dev = _comm_device(group)
    mine = torch.tensor([float(sum(plan.recv_rows))], device=dev)
    mx, sm = mine.clone(), mine.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(sm, op=dist.ReduceOp.SUM, group=group)
    mean = float(sm) / dist.get_world_size(group)
    return int(mine), (float(mx) / mean if mean else 1.0)
