"""Tensor- and expert-parallel sharding of the quantized-matmul path (one process per GPU).

Collectives happen only at shard boundaries and go through `torch.distributed` (NCCL on GPUs; the
same code runs on the `gloo` backend with CPU tensors, which is how the host logic is tested):

    ColumnParallelLinear   shard N (q/k/v, gate/up): no communication, optional all-gather
    RowParallelLinear      shard K in multiples of 32 (o, down): all-reduce(sum) of the partial outputs
    VocabParallelHead      shard the vocabulary: greedy decode exchanges one (max, argmax) pair per rank
    ExpertParallelMoE      experts E/world per rank, tokens stay data-parallel: all-to-all of routed rows
                           to the owning rank, grouped experts there, all-to-all back, weighted combine

Every class takes *callables* for the compute (`QuantLinear`, `MoEExperts.experts`, the permute /
gather / combine kernels), so the communication logic is independent of where the math runs.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


def _world(group=None):
    return dist.get_world_size(group), dist.get_rank(group)


class ColumnParallelLinear:
    """y_local = x . W[rank*N/world : (rank+1)*N/world]^T ; gather_output concatenates along N."""

    def __init__(self, linear: Callable, gather_output: bool = False, group=None):
        self.linear, self.gather_output, self.group = linear, gather_output, group

    def __call__(self, x):
        y = self.linear(x)
        if not self.gather_output:
            return y
        world, _ = _world(self.group)
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


class RowParallelLinear:
    """x is this rank's K slice (K/world columns, a multiple of 32); partial outputs are summed."""

    def __init__(self, linear: Callable, group=None):
        self.linear, self.group = linear, group

    def __call__(self, x_local):
        y = self.linear(x_local)
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y


class VocabParallelHead:
    """Vocabulary-sharded lm_head.  `head(x)` -> local logits [M, V/world]."""

    def __init__(self, head: Callable, vocab_local: int, group=None, comm=None):
        # comm: an ops.PeerComm; the (max, argmax) pairs then travel through peer memory instead of the process group
        self.head, self.vocab_local, self.group, self.comm = head, vocab_local, group, comm

    def logits(self, x):
        return ColumnParallelLinear(self.head, gather_output=True, group=self.group)(x)

    def greedy(self, x):
        """Global argmax ids (ties -> lower id) exchanging 2 numbers per row and rank."""
        if self.comm is not None:              # one launch sequence in the library: head, local arg-max, pair exchange
            return self.comm.greedy_head(self.head, x, self.comm.rank * self.vocab_local)
        world, rank = _world(self.group)
        local = self.head(x).float()
        mx, am = local.max(dim=-1)
        pair = torch.stack([mx, (am + rank * self.vocab_local).to(mx.dtype)], dim=-1).contiguous()   # [M, 2]
        pairs = [torch.empty_like(pair) for _ in range(world)]
        dist.all_gather(pairs, pair, group=self.group)
        allp = torch.stack(pairs, dim=0)                     # [world, M, 2]
        vals, ids = allp[..., 0], allp[..., 1]
        best = vals.max(dim=0).values
        # lowest id among the ranks that hold the maximum
        cand = torch.where(vals == best.unsqueeze(0), ids, torch.full_like(ids, float("inf")))
        return cand.min(dim=0).values.to(torch.int64)


class MoEBackend:
    """The five MoE kernels as callables (defaults: the CUDA ones from chadslab_b200.ops)."""

    def __init__(self, route=None, permute=None, gather=None, combine=None):
        from . import ops
        self.route = route or ops.moe_route
        self.permute = permute or ops.moe_permute
        self.gather = gather or ops.moe_gather
        self.combine = combine or ops.moe_combine


class ExpertParallelMoE:
    """router (replicated) -> top-k -> sort by global expert -> all-to-all rows to the owning rank ->
    local sort by local expert -> grouped experts -> inverse -> all-to-all back -> weighted combine.

    router:      callable x[T,H] -> logits[T,E]           (replicated weights)
    experts:     callable (xp[P,H], offsets[E_local+1]) -> out[P,H] float32   (this rank's experts)

    With `ep` (an ops.PeerEP) and `local_moe` (the ops.MoEExperts holding this rank's experts) both exchanges run
    on the device through peer memory -- no collective call, no host synchronisation, graph-capturable; the route
    through `torch.distributed` below is what the CPU (gloo) tests exercise.
    """

    def __init__(self, router: Callable, experts: Callable, n_experts: int, top_k: int, backend: Optional[MoEBackend] = None,
                 renormalise: bool = True, group=None, act_dtype=torch.bfloat16, ep=None, local_moe=None):
        self.router, self.experts, self.E, self.top_k = router, experts, n_experts, top_k
        self.backend = backend or MoEBackend()
        self.renormalise, self.group, self.act_dtype = renormalise, group, act_dtype
        self.ep, self.local_moe = ep, local_moe
        world, _ = (ep.world, ep.rank) if ep is not None else _world(group)
        if n_experts % world:
            raise ValueError(f"{n_experts} experts do not divide over {world} ranks")
        self.E_local = n_experts // world

    def __call__(self, x):
        be, k = self.backend, self.top_k
        El = self.E_local
        xb = x if x.dtype == self.act_dtype else x.to(self.act_dtype)
        if self.ep is not None and hasattr(self.router, "pw"):                  # router matmul + softmax + top-k in one launch
            from . import ops
            idx, w = ops.moe_route_linear(self.router, xb, k, self.renormalise)
        else:
            idx, w = be.route(self.router(xb), k, self.renormalise)            # [T,k]
        perm, inv, offsets = be.permute(idx, self.E)                            # sorted by global expert
        if self.ep is not None:
            self.ep.dispatch(xb.contiguous(), idx, perm, offsets)               # rows land in their owners' buffers
            self.local_moe.experts_received(self.ep, rows_hint=xb.shape[0] * k)  # balanced routing: ~T*k rows per rank
            return self.ep.combine(inv, w)
        world, rank = _world(self.group)
        xp = be.gather(xb, perm, k)                                             # [T*k, H], grouped by owner rank
        # rows per (destination rank, local expert) and the counts exchange
        counts = (offsets[1:] - offsets[:-1]).to(torch.int64).reshape(world, El)        # what I send
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts.contiguous(), group=self.group)       # [src, local expert]
        send_rows = counts.sum(dim=1).tolist()
        recv_rows = recv_counts.sum(dim=1).tolist()
        xr = torch.empty((int(sum(recv_rows)), xp.shape[1]), dtype=xp.dtype, device=xp.device)
        dist.all_to_all_single(xr, xp.contiguous(), output_split_sizes=recv_rows, input_split_sizes=send_rows,
                               group=self.group)
        # received rows are ordered (source rank, local expert); regroup by local expert, sources in rank order
        eid = torch.repeat_interleave(torch.arange(El, device=xr.device).repeat(world), recv_counts.reshape(-1))
        lperm, linv, loffsets = be.permute(eid.to(torch.int32).reshape(-1, 1), El)
        xl = be.gather(xr, lperm, 1)
        out_l = self.experts(xl, loffsets)                                      # float32 [P_local, H]
        out_r = out_l[linv.long()] if out_l.shape[0] else out_l                 # back to (source, expert) order
        out_p = torch.empty((xp.shape[0], out_r.shape[1]), dtype=out_r.dtype, device=out_r.device)
        dist.all_to_all_single(out_p, out_r.contiguous(), output_split_sizes=send_rows, input_split_sizes=recv_rows,
                               group=self.group)
        return be.combine(out_p, inv, w)


def ep_layout(counts, rank: int):
    """The row bookkeeping of the device-side expert-parallel exchange (csrc/ep.cu, ep_layout_kernel), restated on
    the host with numpy-style integer arithmetic.  counts[s][x] = rows source rank s routes to global expert x
    (every rank knows the whole matrix after the counts exchange).  Returns for `rank`:
      dest_base[x]     row in the owner's receive buffer where this rank's rows of expert x start
      loffsets[El+1]   row ranges of this rank's local experts in its receive buffer
      blk_start[El*world+1]  first received row of block (local expert, source); last entry = rows received
      blk_src[El*world]      position of that block's first row in the source's sorted order
    Rows of one local expert are contiguous on the owner, sources in rank order."""
    import numpy as np
    C = np.asarray(counts, dtype=np.int64)
    world, E = C.shape
    El = E // world
    tot = C.sum(axis=0)
    seg = np.zeros(E, dtype=np.int64)                       # first row of expert x in its owner's buffer
    for x in range(E):
        first = (x // El) * El
        seg[x] = tot[first:x].sum()
    dest_base = seg + C[:rank].sum(axis=0)
    mine = slice(rank * El, (rank + 1) * El)
    loffsets = np.concatenate([seg[mine], [seg[mine][-1] + tot[mine][-1]]])
    src_pos = np.cumsum(C, axis=1) - C                      # position of expert x in source s's sorted order
    blk_start, blk_src = [], []
    for le in range(El):
        x = rank * El + le
        run = seg[x]
        for s_ in range(world):
            blk_start.append(run)
            blk_src.append(src_pos[s_, x])
            run += C[s_, x]
    blk_start.append(loffsets[-1])
    return (dest_base.astype(np.int32), loffsets.astype(np.int32), np.asarray(blk_start, dtype=np.int32),
            np.asarray(blk_src, dtype=np.int32))


def shard_experts(items: Sequence, rank: int, world: int):
    """The contiguous block of experts a rank owns."""
    n = len(items)
    if n % world:
        raise ValueError(f"{n} experts do not divide over {world} ranks")
    per = n // world
    return list(items[rank * per:(rank + 1) * per])
