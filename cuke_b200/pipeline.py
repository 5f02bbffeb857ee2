"""One forward+backward step of the KGE scorers over a (possibly row-partitioned) entity table.

Inspector-executor per step and rank:
  1. inspector over the batch's entity ids [h | t | neg]  -> sorted distinct ids, inverse map, segments
  2. stage every distinct row once into a compact buffer:
        1 GPU : gather from the local table
        N GPUs: the table is row-partitioned (owner = id // rows_per_rank); distinct ids are already sorted, so
                each owner's ids are one contiguous range -> all-to-all of ids, owners gather the requested
                rows, all-to-all of rows (NCCL over NVLink); everything lands in local HBM before it is read
  3. score forward, loss, score backward against the compact buffer through the inverse map
  4. segmented reduction: per-slot gradient rows -> one row per distinct id (fixed order, no atomics)
  5. N GPUs: gradient rows travel back to their owners (all-to-all), who sum the contributions of all ranks
     with the same inspector + segmented reduction (the "reduce-scatter"); relation gradients are all-reduced.

The reference has no counterpart of steps 2 and 5 (single GPU, `cuda:0`, apps/kge/data/data_init.py:6-15) and
only the relation half of step 1 (apps/kge/kge.py:249-271).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import scoring
from .scoring import Inspection, Scorer


class RowExchange:
    """The row-partition protocol of steps 2 and 5, independent of where the kernels run.

    `ops` supplies inspect / owner_counts / gather_rows / segment_reduce with the signatures of
    cuke_b200.scoring (the CUDA kernels); tests drive the same protocol on CPU ranks over gloo with a
    numpy stand-in, which is how the multi-rank bookkeeping is checked without GPUs."""

    def __init__(self, ent_local: torch.Tensor, n_ent: int, rank: int, world: int, group=None, ops=scoring):
        self.ent_local, self.n_ent, self.rank, self.world, self.group, self.ops = ent_local, int(n_ent), rank, world, group, ops
        self.rows_per_rank = (self.n_ent + world - 1) // world
        self.dim = ent_local.shape[1]
        self.need = self.serve = None
        self.req_ids = None
        self.owner_insp = None        # inspection of the ids this rank serves, shared by every gradient return of a step

    def stage(self, insp: Inspection) -> torch.Tensor:
        """Compact buffer holding row uniq[u] of the global table at position u (u < U)."""
        import torch.distributed as dist
        dev = self.ent_local.device
        counts = self.ops.owner_counts(insp, self.rows_per_rank, self.world)       # ids I need from each owner
        wanted = torch.empty_like(counts)                                           # ids each rank needs from me
        dist.all_to_all_single(wanted, counts, group=self.group)
        both = torch.stack((counts, wanted)).cpu()                                  # the one host read: split sizes
        self.need, self.serve = both[0].tolist(), both[1].tolist()
        U, S = sum(self.need), sum(self.serve)
        self.req_ids = torch.empty(max(S, 1), dtype=torch.int64, device=dev)
        dist.all_to_all_single(self.req_ids[:S], insp.uniq[:U], output_split_sizes=self.serve,
                               input_split_sizes=self.need, group=self.group)
        if S:
            send_rows = self.ops.gather_rows(self.ent_local, self.req_ids[:S], first_row=self.rank * self.rows_per_rank)
        else:
            send_rows = torch.empty((0, self.dim), dtype=self.ent_local.dtype, device=dev)
        self.owner_insp = None
        staged = torch.empty((max(U, 1), self.dim), dtype=self.ent_local.dtype, device=dev)
        dist.all_to_all_single(staged[:U], send_rows, output_split_sizes=self.need, input_split_sizes=self.serve,
                               group=self.group)
        return staged

    def return_grads(self, grad_rows: torch.Tensor):
        """grad_rows[u] belongs to uniq[u] of the last stage().  Returns (ids, n_rows, rows): one summed gradient
        row per distinct OWNED id that any rank touched; ids int64 sorted, first n_rows entries valid."""
        import torch.distributed as dist
        U, S = sum(self.need), sum(self.serve)
        recv = torch.empty((max(S, 1), self.dim), dtype=torch.float32, device=grad_rows.device)
        dist.all_to_all_single(recv[:S], grad_rows[:U].contiguous(), output_split_sizes=self.serve,
                               input_split_sizes=self.need, group=self.group)
        if S == 0:
            return self.req_ids[:0], torch.zeros(1, dtype=torch.int64, device=grad_rows.device), recv[:0]
        if self.owner_insp is None:
            self.owner_insp = self.ops.inspect(self.req_ids[:S], self.n_ent)
        oinsp = self.owner_insp
        return oinsp.uniq, oinsp.n_unique, self.ops.segment_reduce(recv[:S], oinsp)


@dataclass
class StepOutput:
    loss: Dict[str, torch.Tensor] = field(default_factory=dict)        # model -> (1,) fp32
    pos: Dict[str, torch.Tensor] = field(default_factory=dict)         # model -> (B,) fp32
    ent_ids: Optional[torch.Tensor] = None       # (n,) int64: ids of the entity gradient rows (first n_ent_rows valid)
    n_ent_rows: Optional[torch.Tensor] = None    # (1,) int64 device
    ent_grad: Dict[str, torch.Tensor] = field(default_factory=dict)    # model -> (n, dim) fp32 rows aligned with ent_ids
    rel_grad: Dict[str, torch.Tensor] = field(default_factory=dict)    # model -> (n_rel, dim) dense fp32
    n_staged: Optional[torch.Tensor] = None      # (1,) distinct entity rows this rank touched
    done: Optional[torch.cuda.Event] = None      # N GPUs, step(..., wait=False): recorded after the last gradient return

    def wait(self) -> None:
        """Make the current stream wait until the entity / relation gradients of this step have arrived."""
        if self.done is not None:
            torch.cuda.current_stream().wait_event(self.done)


class KgeStep:
    """models: scorers sharing one entity table; rel: model -> relation table (n_rel, dim).

    ent_local holds rows [rank * rows_per_rank, ...) of the global (n_ent, dim) table (the whole table when
    world == 1).  `group` is a torch.distributed process group (NCCL) when world > 1."""

    def __init__(self, models: List[str], ent_local: torch.Tensor, rel: Dict[str, torch.Tensor], n_ent: int,
                 neg_mode: str, n_neg_head: int = 0, chunk: int = 0, rank: int = 0, world: int = 1, group=None,
                 precision: str = "fp32", fused: bool = True):
        self.models, self.ent_local, self.rel = list(models), ent_local, rel
        self.fused = fused                    # use the fused forward+loss+backward call where the scorer supports it
        self.n_ent, self.rank, self.world, self.group = int(n_ent), int(rank), int(world), group
        self.neg_mode, self.n_neg_head, self.chunk, self.precision = neg_mode, n_neg_head, chunk, precision
        self.dim = ent_local.shape[1]
        self.n_rel = {m: rel[m].shape[0] for m in self.models}
        for m in self.models:
            if m in ("TransH", "TransR", "RESCAL"):
                raise NotImplementedError("KgeStep covers the vector-relation scorers (TransE, DistMult, ComplEx, TransF)")
        self.exchange = RowExchange(ent_local, n_ent, rank, world, group) if world > 1 else None
        # gradient rows travel home on a side stream while the next scorer computes
        self.comm_stream = torch.cuda.Stream(device=ent_local.device) if world > 1 else None

    def step(self, h: torch.Tensor, r: torch.Tensor, t: torch.Tensor, neg: torch.Tensor, backward: bool = True,
             wait: bool = True) -> StepOutput:
        """One step.  With several GPUs and wait=False the call returns while the last scorer's gradient rows are still
        travelling to their owners (side stream); `StepOutput.wait()` orders a consumer after them.  The next step's
        inspector then overlaps that return; its staging exchange runs on the same side stream, i.e. after it."""
        import torch.distributed as dist
        out = StepOutput()
        B = h.numel()
        insp = scoring.inspect(scoring.entity_id_list(h, t, neg), self.n_ent)
        out.n_staged = insp.n_unique
        r32 = r.to(torch.int32)
        rinsp = None
        if self.exchange is None:
            staged = scoring.gather_rows(self.ent_local, insp.uniq, n_dev=insp.n_unique)
        else:
            # the staging exchange (three collectives and one host read of the split sizes) runs on the side stream;
            # the relation-side inspector needs no entity row and is queued on the main stream first, so it runs meanwhile
            main = torch.cuda.current_stream()
            ready = torch.cuda.Event()
            ready.record(main)
            if backward:
                rinsp = scoring.inspect(r32, self.n_rel[self.models[0]])
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                staged = self.exchange.stage(insp)
            main.wait_stream(self.comm_stream)
            staged.record_stream(main)
        sh, st = insp.inverse[:B], insp.inverse[B:2 * B]
        sneg = insp.inverse[2 * B:].view(neg.shape)
        for m in self.models:
            sc = Scorer(m, staged, self.rel[m], None, self.neg_mode, self.n_neg_head, self.chunk, self.precision)
            if backward and self.fused and sc.supports_fused_step(sneg.shape[-1]):
                # one call: the scores of the negatives become loss terms and gradient weights inside the tile kernel
                pos, loss, sg = sc.loss_backward(sh, r32, st, sneg)
                out.loss[m], out.pos[m] = loss, pos
            else:
                pos, negs, _ = sc.forward(sh, r32, st, sneg)
                loss, dpos, dneg = scoring.logistic_loss(pos, negs)
                out.loss[m], out.pos[m] = loss, pos
                if not backward:
                    continue
                sg = sc.backward(sh, r32, st, sneg, pos, negs, dpos, dneg)
            grad_rows = scoring.segment_reduce(sg.ent_slots, insp, zero_tail=False)     # aligned with insp.uniq
            if self.exchange is None:
                out.ent_ids, out.n_ent_rows, out.ent_grad[m] = insp.uniq, insp.n_unique, grad_rows
            else:
                # the entity rows start their way home before the relation-side reduction is queued
                main = torch.cuda.current_stream()
                ready = torch.cuda.Event()
                ready.record(main)
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(ready)
                    grad_rows.record_stream(self.comm_stream)
                    out.ent_ids, out.n_ent_rows, out.ent_grad[m] = self.exchange.return_grads(grad_rows)
            if rinsp is None:
                rinsp = scoring.inspect(r32, self.n_rel[m])
            rel_rows = scoring.segment_reduce(sg.rel_slots, rinsp, zero_tail=False)
            dense_rel = torch.zeros((self.n_rel[m], self.dim), dtype=torch.float32, device=staged.device)
            scoring.scatter_rows(rel_rows, rinsp.uniq, dense_rel, n_dev=rinsp.n_unique)
            if self.exchange is not None:
                ready2 = torch.cuda.Event()
                ready2.record(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(ready2)
                    dense_rel.record_stream(self.comm_stream)
                    dist.all_reduce(dense_rel, group=self.group)
            out.rel_grad[m] = dense_rel
        if self.exchange is not None and backward:
            out.done = torch.cuda.Event()
            out.done.record(self.comm_stream)
            if wait:
                out.wait()
        return out


def sharded_selfcheck(rank: int, world: int, group, precision: str = "tensor", d: int = 64, chunk: int = 256, n_neg: int = 160,
                      n_chunks: int = 2, n_ent: int = 5003, n_rel: int = 13) -> dict:
    """Row-partitioned step against the same step on one GPU, on a small seeded problem (GPU against GPU; no CPU code).

    Every rank scores its own batch against its shard of the table; rank 0 then recomputes all ranks' batches with the
    whole table and compares: each rank's losses must be bit-equal (same kernels, same operand values, same order), the
    summed entity / relation gradients must agree to 1e-5 (the owner-side sum adds the ranks' contributions in another
    order than a single GPU would) and every rank must return gradients of rows it owns only.  Collective: call it on
    every rank of `group`.  Returns {"ok", "world", "precision", "loss_bit_equal", "max_entity_err", "max_relation_err"}
    on rank 0 and {"ok": None} elsewhere."""
    import numpy as np
    import torch.distributed as dist
    dev = torch.device("cuda", torch.cuda.current_device())
    g = np.random.Generator(np.random.PCG64(77))
    E = (g.standard_normal((n_ent, d)) / np.sqrt(d)).astype(np.float32)
    models = ["TransE", "DistMult"]
    rel = {m: torch.from_numpy((g.standard_normal((n_rel, d)) / np.sqrt(d)).astype(np.float32)).to(dev) for m in models}
    w = np.arange(1, n_ent + 1, dtype=np.float64) ** -1.1
    B = chunk * n_chunks

    def batch(rk):
        gi = np.random.Generator(np.random.PCG64(1000 + rk))
        ids = lambda size: torch.from_numpy(gi.choice(n_ent, size=size, p=w / w.sum()).astype(np.int64)).to(dev)
        return ids(B), torch.from_numpy(gi.integers(0, n_rel, B)).to(dev), ids(B), ids((n_chunks, n_neg))

    rpr = (n_ent + world - 1) // world
    local = torch.from_numpy(E[rank * rpr: min(n_ent, (rank + 1) * rpr)]).to(dev).contiguous()
    step = KgeStep(models, local, rel, n_ent, "chunk_shared", 0, chunk, rank, world, group, precision=precision)
    out = step.step(*batch(rank))
    k = int(out.n_ent_rows.item())
    mine = {m: (out.ent_ids[:k].cpu(), out.ent_grad[m][:k].cpu(), out.rel_grad[m].cpu(), out.loss[m].cpu()) for m in models}
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, mine, group=group)
    else:
        gathered = [mine]
    res = {"ok": None}
    if rank == 0:
        full = KgeStep(models, torch.from_numpy(E).to(dev), rel, n_ent, "chunk_shared", 0, chunk, precision=precision)
        dense = {m: torch.zeros((n_ent, d), dtype=torch.float64) for m in models}
        drel = {m: torch.zeros((n_rel, d), dtype=torch.float64) for m in models}
        loss_equal, owned = True, True
        for rk in range(world):
            o = full.step(*batch(rk))
            u = int(o.n_ent_rows.item())
            for m in models:
                dense[m][o.ent_ids[:u].cpu()] += o.ent_grad[m][:u].double().cpu()
                drel[m] += o.rel_grad[m].double().cpu()
                loss_equal = loss_equal and bool(torch.equal(o.loss[m].cpu(), gathered[rk][m][3]))
        err = rerr = 0.0
        for m in models:
            got = torch.zeros((n_ent, d), dtype=torch.float64)
            for rk in range(world):
                ids, rows, _, _ = gathered[rk][m]
                owned = owned and bool(torch.all((ids >= rk * rpr) & (ids < (rk + 1) * rpr)))
                got[ids] += rows.double()
            err = max(err, float((got - dense[m]).abs().max() / dense[m].abs().max()))
            rerr = max(rerr, float((gathered[0][m][2].double() - drel[m]).abs().max() / drel[m].abs().max()))
        res = {"ok": bool(loss_equal and owned and err < 1e-5 and rerr < 1e-5), "world": world, "precision": precision,
               "loss_bit_equal": loss_equal, "rows_owned_only": owned, "max_entity_err": err, "max_relation_err": rerr,
               "case": f"TransE+DistMult, {B} triples/rank, {n_neg} shared negatives per {chunk}-chunk, dim {d}, {n_ent} rows"}
    if world > 1:
        dist.barrier(group=group)
    return res
