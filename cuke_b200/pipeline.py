"""One training step of the KGE scorers over a (possibly row-partitioned) entity table.

Inspector-executor per step and rank:
  1. inspector over the batch's entity ids [h | t | neg]  -> sorted distinct ids, inverse map, segments
     (and over r -> relation grouping)
  2. stage every distinct row once into a compact buffer:
        1 GPU : gather from the local table
        N GPUs: the table is row-partitioned (owner = id // rows_per_rank); distinct ids are already sorted, so
                each owner's ids are one contiguous range -> all-to-all of ids, owners gather the requested
                rows, all-to-all of rows (NCCL over NVLink); everything lands in local HBM before it is read
  3. score forward, loss, score backward against the compact buffer through the inverse map
  4. segmented reduction: per-slot gradient rows -> one row per distinct id (fixed order, no atomics)
  5. N GPUs: gradient rows travel back to their owners (all-to-all), who sum the contributions of all ranks
     with the same inspector + segmented reduction (the "reduce-scatter"); relation gradients are all-reduced.
  6. optional sparse optimizer (SGD / Adagrad) on exactly the rows the step touched.

Steps 1 and the id half of 2 depend on the ids only, not on the tables: `step(..., prefetch=next_batch)` runs them for
the NEXT batch on a side stream (and its own communicator) while this step computes, so the next step starts at the
row exchange and never waits for the host to read split sizes.

Micro-batches (`KgeStep(micro=k)`): the batch is cut into k runs of whole chunks, each with its own plan, staging buffer and
gradient return.  All k row exchanges are queued at the head of the step, all against the tables as they were when the
step began; micro-batch j then computes while the rows of j+1 are still arriving and the gradient rows of j-1 travel
home, so of the 2k exchanges of a step only the first and the last are not covered by compute.  The step's result is the
one of the whole batch (the loss is a sum over triples); an optimizer sees each micro-batch's gradient as its own update.

The reference has no counterpart of steps 2, 5 and 6 (single GPU, `cuda:0`, apps/kge/data/data_init.py:6-15; its
backward_* functions stop at per-triple pieces, apps/kge/kge.py:393-515) and only the relation half of step 1
(apps/kge/kge.py:249-271).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from . import scoring
from ._lib import MATRIX_MODELS
from .scoring import Inspection, Scorer


@dataclass
class StepPlan:
    """Everything about a batch that depends on its ids only."""
    batch: Tuple[torch.Tensor, ...]            # (h, r, t, neg) as given (kept alive: the plan is matched by identity)
    ids: torch.Tensor                          # [h | t | neg]
    insp: Inspection                           # over ids
    r32: torch.Tensor                          # relation ids as int32
    rinsp: Inspection                          # over r32
    need: Optional[List[int]] = None           # N GPUs: distinct ids I need from each owner
    serve: Optional[List[int]] = None          #         ids each rank needs from me
    req_ids: Optional[torch.Tensor] = None     #         the ids I serve, grouped by requesting rank
    owner_insp: Optional[Inspection] = None    #         inspection of req_ids (the owner-side sum of returned gradients)
    ready: Optional[torch.cuda.Event] = None   # N GPUs: recorded after the copy of the split sizes to the host
    counts_host: Optional[torch.Tensor] = None   # pinned (2, world) int64: need / serve, valid once `ready` has passed
    done: Optional[torch.cuda.Event] = None    # prefetched plans: recorded on the side stream after their last kernel
    first: int = 0                             # first triple of this micro-batch within the step's batch
    sub: Optional[Tuple[torch.Tensor, ...]] = None   # this micro-batch's own (h, r, t, neg): views of `batch`
    inspected: Optional[torch.cuda.Event] = None     # recorded after the inspections, before the count exchange
    wanted: Optional[torch.Tensor] = None      # N GPUs, device (world, 2) int64: per requesting rank, how many of my rows it needs
                                               # and where they start in its own sorted distinct ids
    src_start: Optional[torch.Tensor] = None   # device (world + 1,): positions of each rank's ids within req_ids


class RowExchange:
    """The row-partition protocol of steps 2 and 5, independent of where the kernels run.

    `ops` supplies inspect / owner_counts / gather_rows / segment_reduce with the signatures of
    cuke_b200.scoring (the CUDA kernels); tests drive the same protocol on CPU ranks over gloo with a
    numpy stand-in, which is how the multi-rank bookkeeping is checked without GPUs."""

    def __init__(self, ent_local: torch.Tensor, n_ent: int, rank: int, world: int, group=None, ops=scoring, plan_group=None,
                 peers=None):
        self.ent_local, self.n_ent, self.rank, self.world, self.group, self.ops = ent_local, int(n_ent), rank, world, group, ops
        self.peers = peers            # cuke_b200.peer.PeerTable: stage rows by reading the owners' shards in place
        self.insp = None              # inspection of the batch whose rows are staged (peer staging reads its uniq)
        self.wanted = self.src_start = None
        self.plan_group = plan_group if plan_group is not None else group       # communicator of the id-only collectives
        self.rows_per_rank = (self.n_ent + world - 1) // world
        self.dim = ent_local.shape[1]
        self.need = self.serve = None
        self.req_ids = None
        self.owner_insp = None        # inspection of the ids this rank serves, shared by every gradient return of a step

    # -- id half: depends on the batch's ids only ------------------------------------------------------------------
    def plan_counts(self, insp: Inspection):
        """Queues the count exchange; returns a (2, world) int64 host tensor (pinned on CUDA) holding need / serve once the
        current stream has passed this point."""
        import torch.distributed as dist
        counts = self.ops.owner_counts(insp, self.rows_per_rank, self.world)       # ids I need from each owner
        # each owner also learns where its range starts in my sorted distinct ids (it reads my gradient rows there)
        mine = torch.stack((counts, torch.cumsum(counts, 0) - counts), dim=1).contiguous()
        wanted2 = torch.empty_like(mine)                                            # per rank: ids it needs from me, its offset
        dist.all_to_all_single(wanted2, mine, group=self.plan_group)
        self.wanted = wanted2
        wanted = wanted2[:, 0]
        both = torch.stack((counts, wanted))
        if both.is_cuda:
            host = torch.empty(both.shape, dtype=both.dtype, pin_memory=True)
            host.copy_(both, non_blocking=True)
            return host
        return both

    def plan_ids(self, insp: Inspection, counts_host: torch.Tensor):
        """With the split sizes on the host: the id exchange and the owner-side inspection.  Sets need / serve / req_ids."""
        import torch.distributed as dist
        dev = self.ent_local.device
        self.need, self.serve = counts_host[0].tolist(), counts_host[1].tolist()
        U, S = sum(self.need), sum(self.serve)
        self.req_ids = torch.empty(max(S, 1), dtype=torch.int64, device=dev)
        dist.all_to_all_single(self.req_ids[:S], insp.uniq[:U], output_split_sizes=self.serve,
                               input_split_sizes=self.need, group=self.plan_group)
        self.owner_insp = self.ops.inspect(self.req_ids[:S], self.n_ent) if S else None
        if self.wanted is not None:
            self.src_start = torch.cat((torch.zeros(1, dtype=torch.int64, device=self.wanted.device), torch.cumsum(self.wanted[:, 0], 0)))

    def adopt(self, need, serve, req_ids, owner_insp, insp=None, wanted=None, src_start=None):
        self.need, self.serve, self.req_ids, self.owner_insp, self.insp = need, serve, req_ids, owner_insp, insp
        self.wanted, self.src_start = wanted, src_start

    def return_grads_pull(self, grad_map, sgd_lr: Optional[float] = None):
        """The owner-side sum of return_grads with the ranks' gradient rows read in place (grad_map: cuke_b200.peer.PeerMap
        of the buffers that hold every rank's rows, in the order of its own sorted distinct ids).  The caller has put a
        barrier among the ranks between the writes of those buffers and this call.  sgd_lr: apply the owner's plain SGD step
        to the local shard (fp32) in the same kernel."""
        S = sum(self.serve)
        dev = self.ent_local.device
        out = torch.empty((max(S, 1), self.dim), dtype=torch.float32, device=dev)
        if S == 0:
            return self.req_ids[:0], torch.zeros(1, dtype=torch.int64, device=dev), out[:0]
        oinsp = self.owner_insp
        src_off = self.wanted[:, 1].contiguous()
        scoring.check(scoring._lib.lib().kge_pull_reduce(grad_map.ptrs.data_ptr(), src_off.data_ptr(), self.src_start.data_ptr(), self.world,
                                                         self.dim, oinsp.perm.data_ptr(), oinsp.seg.data_ptr(), oinsp.n_unique.data_ptr(), S,
                                                         out.data_ptr(), None if sgd_lr is None else self.ent_local.data_ptr(),
                                                         oinsp.uniq.data_ptr(), self.rank * self.rows_per_rank,
                                                         0.0 if sgd_lr is None else float(sgd_lr), scoring._stream()))
        return oinsp.uniq, oinsp.n_unique, out

    # -- row half: depends on the tables -------------------------------------------------------------------------------
    def stage_rows(self, staged: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Owners gather the requested rows, all-to-all of rows - or, with peer access, one gather kernel that reads the
        owners' shards in place.  Returns the compact buffer (row u = row uniq[u])."""
        import torch.distributed as dist
        dev = self.ent_local.device
        if self.peers is not None:
            # the number of distinct rows is known on the device only: room for one row per slot, the kernel stops at n_unique
            cap = max(self.insp.n, 1)
            if staged is None or staged.shape[0] < cap:
                staged = torch.empty((cap, self.dim), dtype=self.ent_local.dtype, device=dev)
            return self.peers.gather(self.insp.uniq, cap, self.insp.n_unique, staged)
        U, S = sum(self.need), sum(self.serve)
        if S:
            send_rows = self.ops.gather_rows(self.ent_local, self.req_ids[:S], first_row=self.rank * self.rows_per_rank)
        else:
            send_rows = torch.empty((0, self.dim), dtype=self.ent_local.dtype, device=dev)
        if staged is None or staged.shape[0] < max(U, 1):
            staged = torch.empty((max(U, 1), self.dim), dtype=self.ent_local.dtype, device=dev)
        dist.all_to_all_single(staged[:U], send_rows, output_split_sizes=self.need, input_split_sizes=self.serve,
                               group=self.group)
        return staged

    def stage(self, insp: Inspection) -> torch.Tensor:
        """Whole staging in one call (id half, host read of the split sizes, row half)."""
        host = self.plan_counts(insp)
        if host.is_pinned():
            torch.cuda.current_stream().synchronize()                                # the one host read: split sizes
        self.plan_ids(insp, host)
        return self.stage_rows()

    def return_grads(self, grad_rows: torch.Tensor):
        """grad_rows[u] belongs to uniq[u] of the staged batch.  Returns (ids, n_rows, rows): one summed gradient
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
    rel2_grad: Dict[str, torch.Tensor] = field(default_factory=dict)   # TransH: (n_rel, dim) dense; TransR / RESCAL: (groups, dim, dim)
    rel2_ids: Optional[torch.Tensor] = None      # TransR / RESCAL: relation id of each group of rel2_grad (first n_rel2_groups valid)
    n_rel2_groups: Optional[torch.Tensor] = None
    n_staged: Optional[torch.Tensor] = None      # (1,) distinct entity rows this rank touched
    done: Optional[torch.cuda.Event] = None      # N GPUs, step(..., wait=False): recorded after the last gradient return
    parts: Optional[List["StepOutput"]] = None   # micro > 1: one output per micro-batch (entity gradients live there; loss,
                                                 # pos and the relation-side gradients of the whole batch are in this object)

    def wait(self) -> None:
        """Make the current stream wait until the entity / relation gradients of this step have arrived."""
        if self.done is None:
            return
        cur = torch.cuda.current_stream()
        cur.wait_event(self.done)
        # the travelling results were allocated on the side stream: tell the allocator that this stream reads them too
        for o in [self] + (self.parts or []):
            for x in [o.ent_ids, o.n_ent_rows] + list(o.ent_grad.values()) + list(o.rel_grad.values()) + list(o.rel2_grad.values()):
                if x is not None and x.is_cuda:
                    x.record_stream(cur)


class KgeStep:
    """models: scorers sharing one entity table; rel: model -> relation table (n_rel, dim) (absent for RESCAL);
    rel2: model -> TransH normals (n_rel, dim) or TransR / RESCAL matrices (n_rel, dim, dim).

    ent_local holds rows [rank * rows_per_rank, ...) of the global (n_ent, dim) table (the whole table when
    world == 1).  `group` is a torch.distributed process group (NCCL) when world > 1; relation tables are replicated.
    optimizer: None (gradients are returned, tables untouched), ("sgd", lr) or ("adagrad", lr, eps): applied to the touched
    rows at their owner at the end of the step (each scorer's gradient as its own update).
    relation_partitioned: every rank's batches hold only relations that no other rank sees (see cuke_b200.partition):
    relation-side gradients stay local (no all-reduce), which is what makes TransR / RESCAL usable on several GPUs.
    micro: number of micro-batches a step is cut into (runs of whole chunks; see the module text).
    peer_staging: several GPUs of one node: the rows of a batch are staged by one kernel that reads the owners' shards in
    place over NVLink (cuke_b200.peer.PeerTable) instead of an all-to-all; gradients still travel by all-to-all.  After
    changing the local shard outside of step() (an optimizer of the caller's), call publish() before the next step."""

    def __init__(self, models: List[str], ent_local: torch.Tensor, rel: Dict[str, torch.Tensor], n_ent: int,
                 neg_mode: str, n_neg_head: int = 0, chunk: int = 0, rank: int = 0, world: int = 1, group=None,
                 precision: str = "fp32", fused: bool = True, rel2: Optional[Dict[str, torch.Tensor]] = None,
                 optimizer: Optional[tuple] = None, relation_partitioned: bool = False, micro: int = 1,
                 peer_staging: bool = False):
        self.micro = max(1, int(micro))
        self.models, self.ent_local, self.rel, self.rel2 = list(models), ent_local, rel, rel2 or {}
        self.fused = fused                    # use the fused forward+loss+backward call where the scorer supports it
        self.n_ent, self.rank, self.world, self.group = int(n_ent), int(rank), int(world), group
        self.neg_mode, self.n_neg_head, self.chunk, self.precision = neg_mode, n_neg_head, chunk, precision
        self.dim = ent_local.shape[1]
        self.n_rel = {m: (rel[m] if m in rel else self.rel2[m]).shape[0] for m in self.models}
        if len(set(self.n_rel.values())) != 1:
            raise ValueError("the scorers of a step share one relation id space")
        # relation_partitioned: the batches were split by relation (cuke_b200.partition), so every relation's triples are
        # scored by ONE rank; relation-side gradients then need no all-reduce and each rank updates only its own relations
        self.relation_partitioned = bool(relation_partitioned)
        for m in self.models:
            if m in MATRIX_MODELS and world > 1 and not self.relation_partitioned:
                raise NotImplementedError("relation-matrix scorers on several GPUs need relation-partitioned batches "
                                          "(relation_partitioned=True): their dim x dim gradients are not all-reduced")
            if m in MATRIX_MODELS and self.micro > 1:
                raise NotImplementedError("relation-matrix scorers run with micro = 1 (their per-group gradients are not merged "
                                          "across micro-batches)")
            if m in ("TransH", "TransR", "RESCAL") and m not in self.rel2:
                raise ValueError(f"{m} needs rel2[{m!r}]")
        self.optimizer = optimizer
        self.state = {}
        if optimizer is not None:
            if optimizer[0] not in ("sgd", "adagrad"):
                raise ValueError("optimizer is ('sgd', lr) or ('adagrad', lr, eps)")
            if optimizer[0] == "adagrad":
                z = lambda t: torch.zeros(t.shape, dtype=torch.float32, device=t.device)
                self.state = {"ent": z(ent_local), **{("rel", m): z(rel[m]) for m in rel}, **{("rel2", m): z(self.rel2[m]) for m in self.rel2}}
        dev = ent_local.device
        self.plan_group = None
        if world > 1:
            import torch.distributed as dist
            self.plan_group = dist.new_group(backend="nccl") if group is not None and dist.get_backend(group) == "nccl" else group
        self.peers = None
        self.peer_note = None          # why peer access is off although it was asked for
        if world > 1 and peer_staging:
            from .peer import PeerTable, PeerUnavailable
            try:
                self.peers = PeerTable(ent_local, n_ent, rank, world, group)
            except PeerUnavailable as e:           # raised on every rank alike: all of them take the all-to-all path
                self.peer_note = str(e)
        self.exchange = RowExchange(ent_local, n_ent, rank, world, group, plan_group=self.plan_group, peers=self.peers) if world > 1 else None
        self._token = torch.zeros(1, dtype=torch.float32, device=dev) if self.peers is not None else None
        self._grad_maps = {}
        self._pull = self.peers is not None
        self._fenced = False
        # gradient rows travel home on a side stream while the next scorer computes; plans of the next batch on another
        self.comm_stream = torch.cuda.Stream(device=dev) if world > 1 else None
        self.plan_stream = torch.cuda.Stream(device=dev)
        self._planned: Optional[List[StepPlan]] = None

    # -- the id-only part of a step ---------------------------------------------------------------------------------------
    def _make_plan(self, h, r, t, neg, ids=None, finish: bool = True) -> StepPlan:
        """Inspections of the batch (current stream).  N GPUs: also the count exchange; with finish=True the host then
        reads the split sizes (a synchronisation of the current stream) and the id exchange follows."""
        if ids is None:
            ids = scoring.entity_id_list(h, t, neg)
        insp = scoring.inspect(ids, self.n_ent)
        r32 = r if r.dtype == torch.int32 else r.to(torch.int32)
        rinsp = scoring.inspect(r32, self.n_rel[self.models[0]])
        plan = StepPlan((h, r, t, neg), ids, insp, r32, rinsp)
        if self.exchange is not None:
            plan.inspected = torch.cuda.Event()
            plan.inspected.record()
            plan.counts_host = self.exchange.plan_counts(insp)
            plan.wanted = self.exchange.wanted
            plan.ready = torch.cuda.Event()
            plan.ready.record()
            if finish:
                self._finish_plan(plan)
        return plan

    def _finish_plan(self, plan: StepPlan) -> None:
        """N GPUs: the host reads the split sizes, then the id exchange and the owner-side inspection are queued on the
        current stream."""
        if self.exchange is None or plan.need is not None:
            return
        plan.ready.synchronize()
        self.exchange.wanted = plan.wanted
        self.exchange.plan_ids(plan.insp, plan.counts_host)
        plan.need, plan.serve = self.exchange.need, self.exchange.serve
        plan.req_ids, plan.owner_insp, plan.src_start = self.exchange.req_ids, self.exchange.owner_insp, self.exchange.src_start

    def _split(self, h, r, t, neg, ids=None):
        """The micro-batches of a batch: runs of whole rows of `neg` (chunks, or triples with per-triple negatives)."""
        k = self.micro
        if k == 1 or neg is None:
            return [(0, h, r, t, neg, ids)]
        rows = neg.shape[0]
        per = h.numel() // rows                      # triples per row of neg: the chunk, or 1
        k = min(k, rows)
        parts = []
        for j in range(k):
            a, b = rows * j // k, rows * (j + 1) // k
            parts.append((a * per, h[a * per:b * per], r[a * per:b * per], t[a * per:b * per], neg[a:b], None))
        return parts

    def _make_plans(self, h, r, t, neg, ids, finish: bool) -> List[StepPlan]:
        plans = []
        for first, hh, rr, tt, nn, ii in self._split(h, r, t, neg, ids):
            plan = self._make_plan(hh, rr, tt, nn, ii, finish=finish)
            plan.first, plan.sub = first, plan.batch
            plan.batch = (h, r, t, neg)              # the step's batch is matched by the identity of its tensors
            plans.append(plan)
        return plans

    def prefetch(self, h, r, t, neg, ids=None) -> None:
        """Queues the plan(s) of a coming batch on the side stream.  The tensors must be the very objects later passed to
        step().  N GPUs: the host read of the split sizes is left to finish_prefetch()."""
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)                                # the batch tensors were produced on the current stream
        with torch.cuda.stream(self.plan_stream):
            self.plan_stream.wait_event(ev)
            plans = self._make_plans(h, r, t, neg, ids, finish=False)
            done = torch.cuda.Event()
            done.record(self.plan_stream)
            for plan in plans:
                plan.done = done
        self._planned = plans

    def finish_prefetch(self) -> None:
        """N GPUs: completes the queued plans (host read of their split sizes, then the id exchanges on the side stream).
        step() calls it after launching its own work, when the device has long passed the few kernels the read waits for."""
        plans = self._planned
        if plans is None or self.exchange is None or self.peers is not None or all(p.need is not None for p in plans):
            return
        with torch.cuda.stream(self.plan_stream):
            for plan in plans:
                self._finish_plan(plan)
            done = torch.cuda.Event()
            done.record(self.plan_stream)
            for plan in plans:
                plan.done = done

    def _take_plans(self, h, r, t, neg, ids) -> List[StepPlan]:
        plans, self._planned = self._planned, None
        main = torch.cuda.current_stream()
        if plans is None or not all(a is b for a, b in zip(plans[0].batch, (h, r, t, neg))):
            plans = self._make_plans(h, r, t, neg, ids, finish=self.peers is None)
        elif self.peers is not None:
            # rows are staged by peer loads from the inspection alone; the id exchange (split sizes on the host, ids to their
            # owners, owner-side inspection) serves the gradient return only and is completed there (_finish_late)
            for plan in plans:
                main.wait_event(plan.inspected)
        else:
            self._planned = plans
            self.finish_prefetch()
            self._planned = None
            main.wait_event(plans[0].done)
        for plan in plans:
            self._hold(plan, main)
        return plans

    def _finish_late(self, plan: StepPlan, main) -> None:
        """Peer staging: the id half of the exchange, queued on the plan stream when the first gradient return of the
        micro-batch is about to be queued.  The host read of the split sizes waits for an event that the device passed
        during the previous step (prefetched plans) or a few kernels ago."""
        if plan.need is not None:
            return
        with torch.cuda.stream(self.plan_stream):
            self.plan_stream.wait_event(plan.inspected)
            self._finish_plan(plan)
            plan.done = torch.cuda.Event()
            plan.done.record(self.plan_stream)
        self._hold(plan, main)

    def _hold(self, plan: StepPlan, main) -> None:
        """The plan's tensors are read on streams other than the one they were allocated on."""
        held = [plan.ids, plan.r32, plan.req_ids, plan.wanted, plan.src_start]
        for ins in (plan.insp, plan.rinsp, plan.owner_insp):
            if ins is not None:
                held += [ins.uniq, ins.inverse, ins.perm, ins.seg, ins.n_unique]
        for x in held:
            if x is not None and x.is_cuda:
                x.record_stream(main)
                if self.comm_stream is not None:
                    x.record_stream(self.comm_stream)

    # -- optimizer --------------------------------------------------------------------------------------------------------
    def _apply(self, table: torch.Tensor, key, grad_rows: torch.Tensor, ids=None, n_dev=None, first_row: int = 0) -> None:
        """table and grad_rows as 2-D (rows, width) views; ids None = row i."""
        if self.optimizer[0] == "sgd":
            scoring.apply_sgd(table, grad_rows, self.optimizer[1], ids, n_dev, first_row)
        else:
            eps = self.optimizer[2] if len(self.optimizer) > 2 else 1e-10
            scoring.apply_adagrad(table, self.state[key].view(table.shape), grad_rows, self.optimizer[1], eps, ids, n_dev, first_row)

    def _allreduce(self, dense: torch.Tensor, main) -> None:
        """N GPUs: sum of a replicated table's dense gradient over the ranks, on the side stream."""
        if self.exchange is None or self.relation_partitioned:
            return
        import torch.distributed as dist
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            dense.record_stream(self.comm_stream)
            dist.all_reduce(dense, group=self.group)
        self._fenced = True

    def close(self) -> None:
        """Peer access: unmaps the other ranks' shards and gradient buffers.  Call it on every rank, after a barrier, once no
        rank will step again."""
        torch.cuda.synchronize()
        for gm in self._grad_maps.values():
            gm.close()
        self._grad_maps = {}
        self._fenced = False
        if self.peers is not None:
            self.peers.close()

    def publish(self) -> None:
        """Peer staging: a barrier among the ranks on the side stream, behind the updates queued there so far.  A rank's next
        staging gather is queued behind it, so it reads every owner's rows as updated."""
        if self.peers is None:
            return
        import torch.distributed as dist
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            dist.all_reduce(self._token, group=self.group)

    def _update(self, table, key, rows, ids=None, n_dev=None, first_row: int = 0) -> None:
        """Applies one gradient on the stream where it became ready (the side stream when it travelled)."""
        if self.exchange is not None:
            with torch.cuda.stream(self.comm_stream):
                self._apply(table, key, rows, ids, n_dev, first_row)
        else:
            self._apply(table, key, rows, ids, n_dev, first_row)

    # -- the step ---------------------------------------------------------------------------------------------------------
    def step(self, h: torch.Tensor, r: torch.Tensor, t: torch.Tensor, neg: torch.Tensor, backward: bool = True,
             wait: bool = True, ids: Optional[torch.Tensor] = None, prefetch: Optional[tuple] = None,
             update: bool = True) -> StepOutput:
        """One step.  `ids`: the list [h | t | neg] if the caller already holds it contiguously (h, t, neg being views;
        used with micro = 1).  `prefetch`: the next batch (h, r, t, neg[, ids]) - its inspection (and id exchange) is queued
        on a side stream while this step computes.  With several GPUs and wait=False the call returns while the last
        gradient rows are still travelling to their owners; `StepOutput.wait()` orders a consumer after them.  With an
        optimizer the touched rows are updated before the call's work ends (update=False: the tables stay as they are).

        Order of table accesses within a step: the entity table is read by the staging gathers only, all of them queued
        before the first update; a scorer's relation tables are read by that scorer only and updated after its last
        micro-batch; each update is queued after the kernels that produced its gradient - so every scorer and every
        micro-batch sees the tables as they were when the step began."""
        plans = self._take_plans(h, r, t, neg, ids)
        main = torch.cuda.current_stream()
        first_row = 0
        # staging of every micro-batch, in order, before anything else touches the entity table
        staged, arrived = [], []
        if self.exchange is None:
            for plan in plans:
                staged.append(scoring.gather_rows(self.ent_local, plan.insp.uniq, n_dev=plan.insp.n_unique))
                arrived.append(None)
        else:
            first_row = self.rank * self.exchange.rows_per_rank
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                for plan in plans:
                    self.exchange.adopt(plan.need, plan.serve, plan.req_ids, plan.owner_insp, plan.insp)
                    rows = self.exchange.stage_rows()
                    rows.record_stream(main)
                    ev = torch.cuda.Event()
                    ev.record(self.comm_stream)
                    staged.append(rows)
                    arrived.append(ev)
        if prefetch is not None:
            self.prefetch(*prefetch)
        do_update = backward and update and self.optimizer is not None
        outs = [StepOutput() for _ in plans]
        rel_acc: Dict[tuple, torch.Tensor] = {}        # (key, model) -> dense relation-side gradient summed over the micro-batches
        for j, plan in enumerate(plans):
            if arrived[j] is not None:
                main.wait_event(arrived[j])
            self._run_part(plan, staged[j], outs[j], first_row, backward, do_update, j == len(plans) - 1, rel_acc, main, j)
        out = outs[0]
        if len(outs) > 1:
            out = StepOutput(parts=outs)
            for m in self.models:
                out.loss[m] = torch.stack([o.loss[m] for o in outs]).sum(0)
                out.pos[m] = torch.cat([o.pos[m] for o in outs])
            last = outs[-1]
            out.rel_grad, out.rel2_grad = last.rel_grad, last.rel2_grad
            out.rel2_ids, out.n_rel2_groups = last.rel2_ids, last.n_rel2_groups
            out.n_staged = outs[0].n_staged
        if backward and self.peers is not None and not self._fenced:
            # behind the updates; also: every owner has read this step's gradient buffers.  (When the last thing queued on
            # the side stream after the last shard access was the relation-gradient all-reduce, that collective already is
            # this barrier: no rank enters it before its own reads and updates are done.)
            self.publish()
        if self.exchange is not None and backward:
            out.done = torch.cuda.Event()
            out.done.record(self.comm_stream)
            if wait or do_update:                      # an updated table must be complete before the next step gathers from it
                out.wait()
        self.finish_prefetch()
        return out

    def _grad_map(self, model: str, part: int, rows: int):
        """Peer access: the buffer that holds this rank's entity-gradient rows of (scorer, micro-batch), mapped into every
        process.  Made on first use - a collective, reached by every rank at the same point of its first step."""
        key = (model, part)
        if not self._pull:
            return None
        gm = self._grad_maps.get(key)
        if gm is None or gm.local.shape[0] < rows:
            from .peer import PeerMap, PeerUnavailable
            if gm is not None:
                torch.cuda.synchronize()
                gm.close()
            buf = torch.empty((rows, self.dim), dtype=torch.float32, device=self.ent_local.device)
            try:
                gm = PeerMap(buf, self.rank, self.world, self.group)
            except PeerUnavailable as e:           # every rank alike: gradients travel by all-to-all from now on
                self._pull, self.peer_note = False, str(e)
                self._grad_maps.pop(key, None)
                return None
            self._grad_maps[key] = gm
        return gm

    def _run_part(self, plan: StepPlan, staged: torch.Tensor, out: StepOutput, first_row: int, backward: bool, do_update: bool,
                  last: bool, rel_acc: Dict[tuple, torch.Tensor], main, part: int = 0) -> None:
        """Scorers, reductions, gradient return and entity updates of one micro-batch; the relation-side gradients are
        accumulated in rel_acc and all-reduced / applied with the last micro-batch."""
        h, r, t, neg = plan.sub
        insp, rinsp, r32 = plan.insp, plan.rinsp, plan.r32
        B = h.numel()
        out.n_staged = insp.n_unique
        sh, st = insp.inverse[:B], insp.inverse[B:2 * B]
        sneg = insp.inverse[2 * B:].view(neg.shape)
        for m in self.models:
            nnh = 0 if m == "RESCAL" else self.n_neg_head
            sc = Scorer(m, staged, self.rel.get(m), self.rel2.get(m), self.neg_mode, nnh, self.chunk, self.precision)
            if backward and self.fused and sc.supports_fused_step(sneg.shape[-1]):
                # one call: the scores of the negatives become loss terms and gradient weights inside the tile kernel
                pos, loss, sg = sc.loss_backward(sh, r32, st, sneg, rel_insp=rinsp)
                out.loss[m], out.pos[m] = loss, pos
            else:
                pos, negs, _ = sc.forward(sh, r32, st, sneg, rinsp)
                loss, dpos, dneg = scoring.logistic_loss(pos, negs)
                out.loss[m], out.pos[m] = loss, pos
                if not backward:
                    continue
                sg = sc.backward(sh, r32, st, sneg, pos, negs, dpos, dneg, rinsp)
            gmap = self._grad_map(m, part, insp.n) if self.peers is not None else None
            ent_updated = False
            self._fenced = False          # this scorer's reads of peer buffers and shard updates follow
            grad_rows = scoring.segment_reduce(sg.ent_slots, insp, out=None if gmap is None else gmap.local,
                                               zero_tail=False)                           # aligned with insp.uniq
            if self.exchange is None:
                out.ent_ids, out.n_ent_rows, out.ent_grad[m] = insp.uniq, insp.n_unique, grad_rows
            elif gmap is not None:
                # peer access: every owner reads the rows it owns out of the ranks' buffers and sums them in one kernel
                # (no all-to-all, no receive buffer); the barrier says that every rank's rows of this scorer are complete
                import torch.distributed as dist
                ready = torch.cuda.Event()
                ready.record(main)
                self._finish_late(plan, main)
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(ready)
                    if plan.done is not None:
                        self.comm_stream.wait_event(plan.done)
                    dist.all_reduce(self._token, group=self.group)
                    self.exchange.adopt(plan.need, plan.serve, plan.req_ids, plan.owner_insp, plan.insp, plan.wanted, plan.src_start)
                    fused_sgd = do_update and self.optimizer[0] == "sgd" and self.ent_local.dtype == torch.float32
                    out.ent_ids, out.n_ent_rows, out.ent_grad[m] = self.exchange.return_grads_pull(
                        gmap, self.optimizer[1] if fused_sgd else None)
                    ent_updated = fused_sgd
            else:
                # the entity rows start their way home before the relation-side reduction is queued
                ready = torch.cuda.Event()
                ready.record(main)
                self._finish_late(plan, main)
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(ready)
                    if plan.done is not None:
                        self.comm_stream.wait_event(plan.done)
                    grad_rows.record_stream(self.comm_stream)
                    self.exchange.adopt(plan.need, plan.serve, plan.req_ids, plan.owner_insp, plan.insp)
                    out.ent_ids, out.n_ent_rows, out.ent_grad[m] = self.exchange.return_grads(grad_rows)
            if do_update and not ent_updated:
                self._update(self.ent_local, "ent", out.ent_grad[m], out.ent_ids, out.n_ent_rows, first_row)
            for slots, table, key, dest in ((sg.rel_slots, self.rel.get(m), ("rel", m), out.rel_grad),
                                            (sg.rel2_slots, self.rel2.get(m), ("rel2", m), out.rel2_grad)):
                if slots is None:
                    continue
                rows = scoring.segment_reduce(slots, rinsp, zero_tail=False)
                dense = torch.zeros((self.n_rel[m], self.dim), dtype=torch.float32, device=staged.device)
                scoring.scatter_rows(rows, rinsp.uniq, dense, n_dev=rinsp.n_unique)
                if key in rel_acc:
                    dense.add_(rel_acc[key])
                rel_acc[key] = dense
                if last:
                    self._allreduce(dense, main)
                    dest[m] = dense
                    if do_update:
                        self._update(table, key, dense)
            if sg.rel2_groups is not None:              # TransR / RESCAL: one summed (dim, dim) gradient per relation group
                out.rel2_grad[m], out.rel2_ids, out.n_rel2_groups = sg.rel2_groups, rinsp.uniq, rinsp.n_unique
                if do_update:
                    d2 = self.dim * self.dim
                    self._update(self.rel2[m].view(-1, d2), ("rel2", m), sg.rel2_groups.view(-1, d2), rinsp.uniq, rinsp.n_unique)


def sharded_selfcheck(rank: int, world: int, group, precision: str = "tensor", d: int = 64, chunk: int = 256, n_neg: int = 160,
                      n_chunks: int = 2, n_ent: int = 5003, n_rel: int = 13, micro: int = 1,
                      peer_staging: bool = False) -> dict:
    """Row-partitioned step against the same step on one GPU, on a small seeded problem (GPU against GPU; no CPU code).

    Every rank scores its own batch against its shard of the table; rank 0 then recomputes all ranks' batches with the
    whole table and compares: each rank's losses must be bit-equal (same kernels, same operand values, same order), the
    summed entity / relation gradients must agree to 1e-5 (the owner-side sum adds the ranks' contributions in another
    order than a single GPU would) and every rank must return gradients of rows it owns only.  With micro > 1 the sharded
    step runs in micro-batches (the single-GPU step does not): its loss is then a sum of per-micro-batch losses and is
    compared to 1e-6 instead of bit for bit.  Collective: call it on every rank of `group`.  Returns {"ok", "world", "precision", "loss_bit_equal", "max_entity_err", "max_relation_err"}
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
    step = KgeStep(models, local, rel, n_ent, "chunk_shared", 0, chunk, rank, world, group, precision=precision, micro=micro,
                   peer_staging=peer_staging)
    out = step.step(*batch(rank))
    parts = out.parts or [out]
    ks = [int(o.n_ent_rows.item()) for o in parts]
    mine = {m: ([(o.ent_ids[:k].cpu(), o.ent_grad[m][:k].cpu()) for o, k in zip(parts, ks)], out.rel_grad[m].cpu(), out.loss[m].cpu())
            for m in models}
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
                a, b = o.loss[m].cpu(), gathered[rk][m][2]
                loss_equal = loss_equal and bool(torch.equal(a, b) if micro == 1 else (a - b).abs().max() <= 1e-6 * a.abs().max())
        err = rerr = 0.0
        for m in models:
            got = torch.zeros((n_ent, d), dtype=torch.float64)
            for rk in range(world):
                for ids, rows in gathered[rk][m][0]:
                    owned = owned and bool(torch.all((ids >= rk * rpr) & (ids < (rk + 1) * rpr)))
                    got[ids] += rows.double()
            err = max(err, float((got - dense[m]).abs().max() / dense[m].abs().max()))
            rerr = max(rerr, float((gathered[0][m][1].double() - drel[m]).abs().max() / drel[m].abs().max()))
        res = {"ok": bool(loss_equal and owned and err < 1e-5 and rerr < 1e-5), "world": world, "precision": precision, "micro": micro, "peer_staging": peer_staging,
               "loss_bit_equal" if micro == 1 else "loss_equal_1e-6": loss_equal, "rows_owned_only": owned, "max_entity_err": err, "max_relation_err": rerr,
               "case": f"TransE+DistMult, {B} triples/rank, {n_neg} shared negatives per {chunk}-chunk, dim {d}, {n_ent} rows"}
    if world > 1:
        dist.barrier(group=group)
    step.close()
    return res


def sharded_traincheck(rank: int, world: int, group, precision: str = "tensor", d: int = 64, chunk: int = 128, n_neg: int = 96,
                       n_chunks: int = 2, n_ent: int = 3001, n_rel: int = 11, steps: int = 4, lr: float = 0.02,
                       peer_staging: bool = True, micro: int = 1) -> dict:
    """Several training steps (sparse SGD inside the step) on a row-partitioned table against the same steps on one GPU over
    the ranks' batches joined: after the last step every rank's shard must equal the single-GPU table's rows to 1e-5 of the
    largest update, and so must the replicated relation tables.  A stale read of a peer's rows, an update that overtakes a
    peer's gather or a gradient buffer overwritten before its owner has read it would all show up here.  Collective.
    Returns {"ok", "max_entity_err", "max_relation_err", ...} on rank 0 and {"ok": None} elsewhere."""
    import numpy as np
    import torch.distributed as dist
    dev = torch.device("cuda", torch.cuda.current_device())
    g = np.random.Generator(np.random.PCG64(91))
    E = (g.standard_normal((n_ent, d)) / np.sqrt(d)).astype(np.float32)
    models = ["TransE", "DistMult"]
    R = {m: (g.standard_normal((n_rel, d)) / np.sqrt(d)).astype(np.float32) for m in models}
    w = np.arange(1, n_ent + 1, dtype=np.float64) ** -1.1
    B = chunk * n_chunks

    def batch(step, rk):
        gi = np.random.Generator(np.random.PCG64(5000 + 97 * step + rk))
        ids = lambda size: torch.from_numpy(gi.choice(n_ent, size=size, p=w / w.sum()).astype(np.int64)).to(dev)
        return ids(B), torch.from_numpy(gi.integers(0, n_rel, B)).to(dev), ids(B), ids((n_chunks, n_neg))

    rpr = (n_ent + world - 1) // world
    lo, hi = rank * rpr, min(n_ent, (rank + 1) * rpr)
    local = torch.from_numpy(E[lo:hi]).to(dev).contiguous()
    rel = {m: torch.from_numpy(R[m]).to(dev) for m in models}
    st = KgeStep(models, local, rel, n_ent, "chunk_shared", 0, chunk, rank, world, group, precision=precision,
                 optimizer=("sgd", lr), peer_staging=peer_staging, micro=micro)
    mine = [batch(s, rank) for s in range(steps)]
    for s in range(steps):
        st.step(*mine[s], prefetch=mine[s + 1] if s + 1 < steps else None)
    torch.cuda.synchronize()
    shards = [None] * world
    got = (local.cpu(), {m: rel[m].cpu() for m in models})
    if world > 1:
        dist.all_gather_object(shards, got, group=group)
    else:
        shards = [got]
    res = {"ok": None}
    if rank == 0:
        full_E = torch.from_numpy(E).to(dev)
        full_rel = {m: torch.from_numpy(R[m]).to(dev) for m in models}
        ref = KgeStep(models, full_E, full_rel, n_ent, "chunk_shared", 0, chunk, precision=precision, optimizer=("sgd", lr))
        for s in range(steps):
            parts = [batch(s, rk) for rk in range(world)]
            ref.step(*(torch.cat([p[i] for p in parts]) for i in range(4)))
        torch.cuda.synchronize()
        moved = float((full_E.cpu() - torch.from_numpy(E)).abs().max())
        err = max(float((shards[rk][0] - full_E[rk * rpr: min(n_ent, (rk + 1) * rpr)].cpu()).abs().max()) for rk in range(world)) / moved
        rmoved = max(float((full_rel[m].cpu() - torch.from_numpy(R[m])).abs().max()) for m in models)
        rerr = max(float((shards[rk][1][m] - full_rel[m].cpu()).abs().max()) for rk in range(world) for m in models) / rmoved
        res = {"ok": bool(err < 1e-4 and rerr < 1e-4 and moved > 0), "world": world, "steps": steps, "peer_staging": peer_staging, "micro": micro,
               "max_entity_err": err, "max_relation_err": rerr, "largest_entity_update": moved,
               "case": f"TransE+DistMult, SGD lr {lr}, {steps} steps of {B} triples/rank, dim {d}, {n_ent} rows"}
    if world > 1:
        dist.barrier(group=group)
    st.close()
    return res
