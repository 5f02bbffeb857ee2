#!/usr/bin/env python
"""Benchmark of the KGE scoring hot path: scored triples/sec, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --config c1|c2|c3|c4          (side measurements of the parity configurations, 1 GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Workload (default c5): TransE and DistMult scored on the same batch, fp32, entity table 4,000,000 x 400 rows
row-partitioned over the N GPUs, relations 1000 x 400 replicated, 65,536 triples per GPU per step, 1,024 shared
negatives per 1,024-triple chunk, Zipf(1.1) entity ids.  A step = inspector, staging of distinct rows, forward,
logistic loss, backward, segmented gradient reduction, the way back to the rows' owners and the sparse SGD update,
for BOTH scorers.  When N > 1 rows and gradient rows move by kernels that read the other GPUs' memory over NVLink
(`--no-peer-staging`: by NCCL all-to-all); `--micro k` cuts a step into k micro-batches; `--precision` selects the
operand split of the tensor-core contractions (tensor = bf16 pairs, tensor_tf32 = tf32 pairs) or the fp32 CUDA-core
path.  Scored triples per step per GPU = 2 scorers x (65,536 + 64 x 1,024 x 1,024).

One JSON line is printed by rank 0.  `value` is measured with the step's ids already on the device; `e2e` includes
the pinned-host -> device copy of the ids and the device -> host read of the losses every step (consumed by the host
one step late, the last one inside the timed region).  64 untimed settle steps precede the W warm-up steps of runs
with K >= 10.  `--impl reference`
times the reference's own CPU path (cuke's generated OpenMP C++, oracle/_ref) on a bounded sample.
Beside the contract's keys the line carries
  spread    the same K-step region repeated (every region's ms per step, median, min, max, host time to queue a step);
  roofline  the dominant kernel timed live (useful TFLOP/s against the measured bf16 peak), the ncu DRAM traffic of
            its launches read from profiles/, and under "hbm" the compulsory bytes of the WHOLE step over the step time;
  parity    computed outside the timed regions: at N = 1 one whole chunk of the timed batch through the timed KgeStep
            object against the CPU oracle (loss, entity and relation gradients); at N > 1 the row-partitioned step
            against the same step on one GPU (losses bit-equal, gradients 1e-5);
  side      (N = 1) configurations c1-c4 and c4 over bf16 tables, one record per scorer, each with its roofline view
            and the reference's OpenMP C++ on a bounded sample (`--no-side` skips them).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "scored_triples_per_sec_fwd_bwd"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c5")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel-only", action="store_true",
                    help="profiling aid: run forward+backward of the scorers 3 times on a reduced case (--chunks chunks, "
                         "entity table scaled down to fit a few GB) and exit; meant to be run under ncu -k <kernel>")
    ap.add_argument("--chunks", type=int, default=32)
    ap.add_argument("--micro", type=int, default=1,
                    help="micro-batches per step (runs of whole chunks; with k > 1 the row exchanges of one micro-batch travel while "
                         "another computes - measured slower than 1 at c5, where half-size contractions lose more than the overlap gains)")
    ap.add_argument("--no-peer-staging", action="store_true",
                    help="N GPUs: stage rows by all-to-all (NCCL) instead of reading the owners' shards in place over NVLink")
    ap.add_argument("--precision", default="tensor", choices=["fp32", "tensor", "tensor_tf32"],
                    help="fp32: CUDA-core arithmetic; tensor: 3xTF32 tcgen05 contractions where available (same tolerance)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="CPU work budget per scorer for cpu_baseline")
    ap.add_argument("--no-optimizer", action="store_true", help="return gradients only (no sparse SGD update in the step)")
    ap.add_argument("--no-prefetch", action="store_true", help="inspect every batch inside its own step")
    ap.add_argument("--no-side", action="store_true", help="skip the c1-c4 side measurements appended to the c5 line")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def settle(self, samples: int = 3, limit_s: float = 8.0):
        """Returns once nvidia-smi has printed a few samples: its start-up (driver queries that can stall the GPU for
        milliseconds) then lies before the timed region, not inside its first steps."""
        t0 = time.time()
        while self.proc is not None and len(self.lines) < samples and time.time() - t0 < limit_s and self.proc.poll() is None:
            time.sleep(0.05)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------------
# reference (CPU) arm and cpu_baseline
# ---------------------------------------------------------------------------------------------------------
def cpu_reference_rate(cfg, models, seconds: float, steps: int = 1, warmup: int = 0):
    """Scored triples/s of cuke's generated OpenMP C++ (forward: the reference's only complete path) on a bounded
    sample of the workload, flattened the way the reference flattens negatives (apps/kge/data/data_init.py:55-61):
    chunk-shared configurations take the first m triples of each of the first nc chunks against their chunk's shared
    negatives, per-triple configurations the first m triples with their own negatives.  Tables are compact copies
    holding exactly the rows the sample touches (fp32: the reference has no bf16 path)."""
    import torch
    from cuke_b200 import synth
    from oracle import oracle
    kind = "reference" if all(oracle.have_ref(m, omp=True) for m in models) else "port"
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    h, r, t, neg = synth.make_batch(cfg, 0, 0)
    n_neg = neg.shape[1]
    shared = cfg.neg_mode == "chunk_shared"
    g = np.random.Generator(np.random.PCG64(synth.BASE_SEED + 5))

    def sample(m, nc=1):
        hs, rs, ts = [], [], []
        if shared:
            for c in range(nc):
                lo = c * cfg.chunk
                hh, rr, tt = h[lo:lo + m], r[lo:lo + m], t[lo:lo + m]
                fh, fr, ft = oracle.flatten(hh, rr, tt, neg[c:c + 1], "chunk_shared", 0, m)
                hs += [hh, fh]; rs += [rr, fr]; ts += [tt, ft]
        else:
            hh, rr, tt = h[:m], r[:m], t[:m]
            fh, fr, ft = oracle.flatten(hh, rr, tt, neg[:m], "per_triple", cfg.n_neg_head)
            hs += [hh, fh]; rs += [rr, fr]; ts += [tt, ft]
        fh, fr, ft = np.concatenate(hs), np.concatenate(rs), np.concatenate(ts)
        ue, inv = np.unique(np.concatenate([fh, ft]), return_inverse=True)
        ur, rinv = np.unique(fr, return_inverse=True)
        tabs = {}
        for model in models:
            d = synth.row_floats(cfg, model)
            E = (g.standard_normal((len(ue), d)) / np.sqrt(d)).astype(np.float32)
            R = None if model == "RESCAL" else (g.standard_normal((len(ur), d)) / np.sqrt(d)).astype(np.float32)
            P2 = None
            if model == "TransH":
                w = g.standard_normal((len(ur), d))
                P2 = (w / np.linalg.norm(w, axis=1, keepdims=True)).astype(np.float32)
            if model in ("TransR", "RESCAL"):
                P2 = (g.standard_normal((len(ur), d, d)) / np.sqrt(d)).astype(np.float32)
            tabs[model] = (E, R, P2)
        return tabs, inv[: len(fh)].astype(np.int32), rinv.astype(np.int32), inv[len(fh):].astype(np.int32)

    def run(model, tabs, fh, fr, ft):
        E, R, P2 = tabs[model]
        if kind == "reference":
            tt = lambda a: None if a is None else torch.from_numpy(a)
            out = oracle.ref_run(model, tt(E), tt(R), tt(P2), tt(fh), tt(fr), tt(ft), omp=True)
            if model in oracle.VECTOR_MODELS:
                out = -torch.linalg.vector_norm(out, dim=1)      # the norm the reference leaves to its caller
            return out
        return oracle.flat_scores(model, E, R, P2, fh, fr, ft)

    # size the sample: probe with 8 triples x n_neg, then scale to the time budget
    tabs, fh, fr, ft = sample(8)
    probe = 1e9
    for _ in range(2):
        t0 = time.perf_counter()
        for model in models:
            run(model, tabs, fh, fr, ft)
        probe = min(probe, time.perf_counter() - t0)
    per_triple = probe / len(fh)                                                     # all scorers, per flattened triple
    want = seconds / max(steps + warmup, 1) / max(per_triple, 1e-9) / (n_neg + 1)     # triples per step
    if shared:
        m = int(max(8, min(cfg.chunk, want)))
        nc = int(max(1, min(cfg.batch // cfg.chunk, 8, want // cfg.chunk)))
    else:
        m, nc = int(max(8, min(cfg.batch, want))), 1
    tabs, fh, fr, ft = sample(m, nc)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for model in models:
            run(model, tabs, fh, fr, ft)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    scored = len(fh) * len(models)
    best = min(times)
    what = (f"{m} triples of each of the first {nc} chunks x {n_neg} shared negatives + positives" if shared
            else f"the first {m} triples x {n_neg} negatives + positives")
    return {"value": scored / best, "unit": "triples/s", "cores": cores if kind == "reference" else 1, "kind": kind,
            "sample": f"forward only (the reference has no aggregated backward): {what}, flattened ({len(fh)} triples) "
                      f"x {len(models)} scorer(s), compact fp32 tables, best of {len(times)}",
            "ms_per_step": statistics.mean(times) * 1e3, "scored_per_step": scored}


def reference_arm(args, cfg, models):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    res = cpu_reference_rate(cfg, models, seconds=max(20.0, 4.0 * (args.steps + args.warmup)), steps=args.steps, warmup=args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": res["scored_per_step"] / (res["ms_per_step"] * 1e-3),
            "unit": "triples/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(cfg, models, args.gpus),
            "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}}
    line["cpu_baseline"]["value"] = line["value"]
    line["e2e"] = {"value": line["value"], "unit": "triples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    print(json.dumps(line), flush=True)


def staging_note(stepper, world):
    """How rows and gradient rows moved in this run (the peer path falls back to collectives on every rank alike if any
    rank could not map a peer's memory; the reason is reported)."""
    if world == 1:
        return "local gather"
    rows = "rows: one gather kernel over the owners' shards" if stepper.peers is not None else "rows: all-to-all of ids and rows (NCCL)"
    grads = ("gradients: one owner-side sum over the ranks' buffers" if getattr(stepper, "_pull", False)
             else "gradients: all-to-all + owner-side segmented sum (NCCL)")
    how = " (CUDA IPC mappings, NVLink peer loads); NCCL for ids, counts and barriers" if stepper.peers is not None else ""
    note = f"; peer access unavailable: {stepper.peer_note}" if getattr(stepper, "peer_note", None) else ""
    return f"{rows}; {grads}{how}{note}"


def workload_config(cfg, models, n_gpus):
    return {"workload": f"{cfg.name}: {'+'.join(models)} fwd+bwd fp32, entities {cfg.n_ent}x{cfg.dim} row-partitioned over "
                        f"{n_gpus} GPU(s), relations {cfg.n_rel}x{cfg.dim}, {cfg.batch} triples/GPU, {cfg.n_neg} shared negatives "
                        f"per {cfg.chunk}-triple chunk, Zipf(1.1) entity ids",
            "scorers": models, "triples_per_gpu": cfg.batch, "neg_mode": cfg.neg_mode, "n_neg": cfg.n_neg, "chunk": cfg.chunk,
            "dim": cfg.dim, "n_ent": cfg.n_ent, "n_rel": cfg.n_rel, "parallelism": f"dp{n_gpus}+row-sharded-entities",
            "step": "inspector, staging (row exchange), forward + logistic loss + backward, segmented gradient reduction (owner-side sum), "
                    "sparse SGD update of the touched rows, for both scorers",
            "pipelining": "the inspection of batch i+1 (N>1: and its id exchange) runs on a side stream during step i; N>1: a step "
                          "is cut into micro-batches (`micro_batches`) whose row exchanges travel while another micro-batch "
                          "computes; the timed region ends after the last update",
            "l2": "inputs larger than L2 (6.4 GB table, 76 MB staged rows, 2 x 268 MB of split gradient weights per scorer; "
                  "the 268 MB score matrix is consumed inside the tile kernel); no flush"}


# ---------------------------------------------------------------------------------------------------------
# side measurements: the parity configurations c1-c4, one scorer at a time, single GPU
# ---------------------------------------------------------------------------------------------------------
def reference_gpu_anchor(cfg, sc, h, r, t, neg, flush, steps):
    """GPU against GPU on c1's flattened batch (positives + flattened negatives, the reference's own layout,
    apps/kge/data/data_init.py:55-61): the kernel the reference's generator emits for TransE without relation reuse
    (apps/kge/test_cuke.py:27-54; built ahead of time for sm_100 by oracle/build_ref.py --cuda-anchor) beside this
    library's drop-in forward producing the same (batch, dim) vectors.  Both are timed as bare calls with CUDA events
    (the reference's own timing loop also pays a file compare and a module lookup per call, pycuke1/run/gpu.py:4-19)."""
    import torch
    from oracle import oracle
    if not oracle.have_ref_cuda():
        return {"unavailable": "oracle/_ref/ref_transE_cuda.so was not built (needs the reference checkout and nvcc)"}
    try:
        mod = oracle.load_ref_cuda()
        fh, fr, ft = oracle.flatten(h.cpu().numpy(), r.cpu().numpy(), t.cpu().numpy(), neg.cpu().numpy(), "per_triple", 0)
        dev = h.device
        ah = torch.cat([h, torch.from_numpy(fh).to(dev)]); ar = torch.cat([r, torch.from_numpy(fr).to(dev)])
        at = torch.cat([t, torch.from_numpy(ft).to(dev)])
        n, d = ah.numel(), sc.dim
        assert n % 16 == 0
        call_ref = lambda: mod.run(n, d, sc.ent.shape[0], sc.ent, ah, at, sc.rel.shape[0], sc.rel, ar)
        call_ours = lambda: sc.ref_forward(ah, ar, at)
        same = bool(torch.allclose(call_ref(), call_ours(), rtol=1e-6, atol=1e-7))

        def timed(fn, cold):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            tot = 0.0
            for _ in range(max(steps, 5)):
                if cold:
                    flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record()
                torch.cuda.synchronize()
                tot += e0.elapsed_time(e1)
            return tot / max(steps, 5)
        res = {"triples": n, "outputs_equal": same,
               "reference_ms_cold_l2": timed(call_ref, True), "reference_ms_warm_l2": timed(call_ref, False),
               "ours_ms_cold_l2": timed(call_ours, True), "ours_ms_warm_l2": timed(call_ours, False),
               "what": "(batch, dim) vectors h - t + r of the flattened batch; reference = cuke's generated kernel (grid batch/16, "
                       "block 32x16, scalar loads), ours = kge_ref_forward"}
        res["speedup_cold_l2"] = res["reference_ms_cold_l2"] / res["ours_ms_cold_l2"]
        return res
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {e}"}


def side_measure(cname, steps, warmup, precision, cpu_seconds=0.0):
    """Times forward (and backward + gradient reduction where the configuration has one) of a parity configuration on
    one GPU, one scorer at a time; returns one record per scorer with the HBM view of the roofline and, if
    cpu_seconds > 0, the reference's OpenMP C++ on a bounded sample.  Not the headline metric: the tables of c1-c3 fit
    in L2, so a 384 MB buffer is written between timed iterations (cold-L2 figure) and the warm-L2 figure is reported
    beside it."""
    import torch
    from cuke_b200 import scoring, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = synth.CONFIGS[cname]
    hbm_gbs, _, peak_kind = peaks()
    flush = torch.empty(384 << 20, dtype=torch.uint8, device=dev)
    out = []
    for model in (cfg.model,) + tuple(cfg.extra_models):
        ent, rel, rel2 = synth.make_tables(cfg, model)
        to = lambda a: None if a is None else torch.from_numpy(a).to(dev).to(torch.bfloat16 if cfg.dtype == "bf16" else torch.float32).contiguous()
        sc = scoring.Scorer(model, to(ent), to(rel), to(rel2), cfg.neg_mode, cfg.n_neg_head if model != "RESCAL" else 0, cfg.chunk,
                            precision)
        del ent, rel, rel2
        h, r, t, neg = (torch.from_numpy(x).to(dev) for x in synth.make_batch(cfg, 0, 0))
        backward = cfg.backward
        d = synth.row_floats(cfg, model)
        ids = scoring.entity_id_list(h, t, neg)

        # fwd+bwd configurations run through the same step pipeline as the headline workload (inspector, dedup staging,
        # forward + loss + backward - fused where the scorer has a fused call -, entity- and relation-side reductions);
        # the forward-only configuration c1 is the bare scoring call
        stepper = None
        if backward:
            from cuke_b200.pipeline import KgeStep
            stepper = KgeStep([model], sc.ent, {} if sc.rel is None else {model: sc.rel}, cfg.n_ent, cfg.neg_mode,
                              cfg.n_neg_head, cfg.chunk, precision=precision, rel2={} if sc.rel2 is None else {model: sc.rel2})

        def step(bwd=True):
            if stepper is not None:
                return stepper.step(h, r, t, neg, backward=bwd, ids=ids)
            return sc.forward(h, r, t, neg)[0]

        def timed(cold, bwd=True):
            for _ in range(max(warmup, 3)):
                step(bwd)
            torch.cuda.synchronize()
            tot = 0.0
            for _ in range(steps):
                if cold:
                    flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); step(bwd); e1.record()
                torch.cuda.synchronize()
                tot += e0.elapsed_time(e1)
            return tot / steps

        ms_cold, ms_warm, ms_fwd = timed(True), timed(False), timed(True, False)
        S = synth.scored_triples(cfg)
        U_e = int(torch.unique(ids).numel()); U_r = int(torch.unique(r).numel())
        es = 2 if cfg.dtype == "bf16" else 4
        relrow = {"TransH": 2 * d * es, "TransR": (d + d * d) * es, "RESCAL": d * d * es}.get(model, d * es)
        bytes_fwd = U_e * d * es + U_r * relrow + 8 * (3 * cfg.batch + neg.numel()) + 4 * S
        bytes_bwd = (4 * S + U_e * d * 4 + U_r * relrow * 4 // es + U_e * d * es + U_r * relrow) if backward else 0
        bytes_alg = bytes_fwd + bytes_bwd
        rec = {"metric": METRIC if backward else "scored_triples_per_sec_fwd", "side_measurement": True,
               "value": S / (ms_cold * 1e-3), "value_warm_l2": S / (ms_warm * 1e-3), "unit": "triples/s", "n_gpus": 1,
               "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms_cold, "ms_per_step_warm_l2": ms_warm, "ms_fwd_only": ms_fwd,
               "dtype": cfg.dtype, "data": "synthetic", "precision": precision,
               "config": {"workload": f"{cfg.name}: {model} {'fwd+bwd' if backward else 'fwd'}, entities {cfg.n_ent}x{d}, "
                                      f"batch {cfg.batch}, {cfg.n_neg} negatives ({cfg.neg_mode})",
                          "l2": "384 MB written between timed iterations (cold L2); warm figure beside it"},
               "roofline": {"bound": "hbm", "achieved": bytes_alg / (ms_cold * 1e-3) / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                            "frac": bytes_alg / (ms_cold * 1e-3) / 1e9 / hbm_gbs, "bytes_alg": bytes_alg,
                            "gathered_bytes": S * 2 * d * es, "peak_source": f"MEASURED_PEAKS.json ({peak_kind})",
                            "traffic": None}}
        if model in ("TransR", "RESCAL"):
            # contraction scorers: useful flops of the relation-matrix products beside the HBM view
            # one d x d projection per scored triple (TransR, difference rows) or per positive (RESCAL); backward = 2 more
            flops = 2.0 * d * d * (S if model == "TransR" else cfg.batch) * (3 if backward else 1)
            _, bf16_peak, _ = peaks()
            rec["roofline"]["tensor"] = {"useful_flops": flops, "achieved": flops / (ms_cold * 1e-3) / 1e12, "peak": bf16_peak,
                                         "unit": "TFLOP/s", "frac": flops / (ms_cold * 1e-3) / 1e12 / bf16_peak}
        if cname == "c1":
            rec["reference_gpu_kernel"] = reference_gpu_anchor(cfg, sc, h, r, t, neg, flush, steps)
        if cpu_seconds > 0:
            try:
                res = cpu_reference_rate(cfg, [model], seconds=cpu_seconds, steps=2, warmup=1)
                rec["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
            except Exception as e:
                rec["cpu_baseline"] = {"value": None, "unit": "triples/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        out.append(rec)
        del sc
        torch.cuda.empty_cache()
    return out


def side_config(args):
    import torch
    torch.cuda.set_device(0)
    for rec in side_measure(args.config, args.steps, args.warmup, args.precision, 0.0 if args.no_cpu_baseline else args.cpu_seconds):
        print(json.dumps(rec), flush=True)


# ---------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------
def profile_traffic():
    """DRAM read + write of the tile kernel's launches as captured by ncu (profiles/umma_pair_c5_32chunks_ncu_full.txt:
    one 'DRAM read' and one 'DRAM write' line per captured launch, in MB, at 32 of the bench's 64 chunks).  Returns
    (bytes per launch averaged over the captured launches, launches captured, file) or None if the summary is absent."""
    path = os.path.join(ROOT, "profiles", "umma_pair_c5_32chunks_ncu_full.txt")
    if not os.path.exists(path):
        return None
    rd, wr = [], []
    for ln in open(path):
        f = ln.split()
        if len(f) >= 4 and f[0] == "DRAM" and f[1] in ("read", "write") and f[-1] == "Mbyte":
            (rd if f[1] == "read" else wr).append(float(f[2]) * 1e6)
    if not rd or len(rd) != len(wr):
        return None
    return (sum(rd) + sum(wr)) / len(rd), len(rd), os.path.relpath(path, ROOT)


def parity_single_gpu(cfg, models, stepper, ent_local, rel, devb, dev):
    """One whole chunk of the bench's own batch (1,024 triples x 1,024 shared negatives x dim 400) through the same
    KgeStep object the timed region uses, against the CPU oracle: loss, every entity gradient row, relation gradients.
    Outside the timed region.  The oracle sees a compact copy of exactly the rows the chunk touches."""
    import torch
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle
    h, r, t, neg = devb[0]
    c, nn = cfg.chunk, cfg.n_neg
    hs, rs, ts, ns = h[:c].contiguous(), r[:c].contiguous(), t[:c].contiguous(), neg[:1].contiguous()
    out = stepper.step(hs, rs, ts, ns, update=False)
    U = int(out.n_ent_rows.item())
    ids = out.ent_ids[:U]
    E = ent_local[ids].cpu().numpy()                               # rows of the distinct ids, ascending
    remap = lambda x: np.searchsorted(ids.cpu().numpy(), x.cpu().numpy())
    hh, tt, ng, rr = remap(hs), remap(ts), remap(ns), rs.cpu().numpy()
    sp = lambda x: np.maximum(x, 0.0) + np.log1p(np.exp(-np.abs(x)))
    sg = lambda x: 1.0 / (1.0 + np.exp(-x))
    oracle.lib()

    def one(m):
        R = rel[m].cpu().numpy()
        pos, negs = oracle.scores(m, E, R, None, hh, rr, tt, ng, "chunk_shared", 0, c)
        p64, n64 = pos.astype(np.float64), negs.astype(np.float64)
        loss = sp(-p64).sum() + sp(n64).sum() / nn
        gE, gR, _ = oracle.grads(m, E, R, None, hh, rr, tt, (-sg(-p64)).astype(np.float32), ng, (sg(n64) / nn).astype(np.float32),
                                 "chunk_shared", 0, c)
        rel_err = lambda a, b: float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
        return {"loss_rel_err": abs(out.loss[m].item() - loss) / abs(loss),
                "pos_rel_err": rel_err(out.pos[m].double().cpu().numpy(), p64),
                "entity_grad_rel_err": rel_err(out.ent_grad[m][:U].double().cpu().numpy(), gE),
                "relation_grad_rel_err": rel_err(out.rel_grad[m].double().cpu().numpy(), gR)}
    with ThreadPoolExecutor(max_workers=len(models)) as ex:
        res = dict(zip(models, ex.map(one, models)))
    worst = max(v for m in models for v in res[m].values())
    return {"ok": bool(worst < 1e-4), "tolerance": 1e-4, "against": "CPU oracle (oracle/kge_oracle.c, pinned to the reference's generated C++)",
            "case": f"chunk 0 of the timed batch: {c} triples x {nn} shared negatives, dim {cfg.dim}, {U} distinct rows, "
                    f"through the timed KgeStep object", "scorers": res}


def main():
    args = parse()
    from cuke_b200 import synth
    if args.config != "c5":
        if args.impl == "reference" or args.gpus != 1:
            raise SystemExit("only c5 has a reference arm and a multi-GPU run; c1-c4 are single-GPU side measurements")
        side_config(args)
        return
    cfg = synth.CONFIGS[args.config]
    models = ["TransE", "DistMult"]
    if args.impl == "reference":
        reference_arm(args, cfg, models)
        return

    import torch
    import torch.distributed as dist
    from cuke_b200 import _lib, scoring
    from cuke_b200.pipeline import KgeStep, sharded_selfcheck

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    _lib.lib()          # fail loudly if the CUDA library is missing

    if args.kernel_only:
        cfg = cfg.scaled(ent=0.1, batch=args.chunks * cfg.chunk / cfg.batch)
    d = synth.row_floats(cfg, models[0])
    rows_per_rank = (cfg.n_ent + world - 1) // world
    my_rows = max(0, min(cfg.n_ent, (rank + 1) * rows_per_rank) - rank * rows_per_rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(synth.BASE_SEED + 1000 * cfg.cid + 1 + 100000 * rank)
    ent_local = torch.randn((my_rows, d), generator=gen, device=dev, dtype=torch.float32) * (1.0 / np.sqrt(d))
    rel = {}
    for mi, m in enumerate(models):
        g = np.random.Generator(np.random.PCG64(synth.BASE_SEED + 1000 * cfg.cid + 2 + mi))
        rel[m] = torch.from_numpy((g.standard_normal((cfg.n_rel, d)) / np.sqrt(d)).astype(np.float32)).to(dev)
    # a training step: sparse SGD on the rows the step touched (entity rows at their owner, relation tables everywhere)
    # (the loss is a SUM over 65,536 random triples per step, so the hottest Zipf row collects ~10^4 gradient terms: the
    # learning rate is set so that the few hundred steps of a benchmark run leave the table in its initial distribution;
    # the update's memory traffic and launches do not depend on its value)
    optimizer = None if args.no_optimizer else ("sgd", 1e-8)
    micro = max(1, args.micro)
    stepper = KgeStep(models, ent_local, rel, cfg.n_ent, cfg.neg_mode, cfg.n_neg_head, cfg.chunk, rank, world, group,
                      precision=args.precision, optimizer=optimizer, micro=micro,
                      peer_staging=world > 1 and not args.no_peer_staging)

    nb = 4
    host = []
    for s in range(nb):
        h, r, t, neg = synth.make_batch(cfg, s, rank)
        host.append(tuple(torch.from_numpy(x).pin_memory() for x in (h, r, t, neg)))
    devb = [tuple(x.to(dev) for x in b) for b in host]
    h2d_bytes = sum(x.numel() * x.element_size() for x in host[0])

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        tns = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tns, op=dist.ReduceOp.MAX, group=group)
        return float(tns.item())

    host_ms = []        # per timed region: host time to queue its steps (no synchronisation inside), per step

    def timed(fn, steps, warmup, after=None):
        for i in range(warmup):
            fn(i)
        if after is not None:
            after()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        if after is not None:
            after()
        e1.record()
        host_ms.append((time.perf_counter() - t0) * 1e3 / steps)
        sync_all()
        return max_over_ranks(e0.elapsed_time(e1)) / steps

    scored_per_gpu = synth.scored_triples(cfg) * len(models)
    if args.kernel_only:
        for i in range(3):
            stepper.step(*devb[i % nb])
        torch.cuda.synchronize()
        print(json.dumps({"kernel_only": True, "chunks": args.chunks, "n_ent": cfg.n_ent, "batch": cfg.batch}))
        return

    # ---- value: ids resident on the device ------------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.settle()
    if world > 1:
        dist.barrier(group=group)
    # N GPUs: the last scorer's gradient return of step i may overlap the inspector of step i+1 (wait=False); the last
    # timed step waits for its own return, so the timed region covers all the work of its K steps
    w_main = max(args.warmup, 3)
    # settle: allocator pools, clocks and the NCCL channels reach their steady state before the W warm-up steps begin
    # (a fixed number of steps: every rank must make the same calls)
    for i_settle in range(64 if args.steps >= 10 else 0):      # (short runs are profiling runs: every launch costs there)
        stepper.step(*devb[i_settle % nb], prefetch=None if args.no_prefetch else devb[(i_settle + 1) % nb])
        if i_settle % 8 == 7:
            torch.cuda.synchronize()
    sync_all()
    launches0 = _lib.lib().kge_launch_count()
    # the next batch's inspection (N GPUs: and its id exchange) is queued on a side stream while a step computes
    nxt = (lambda i: devb[(i + 1) % nb]) if not args.no_prefetch else (lambda i: None)
    ms_step = timed(lambda i: stepper.step(*devb[i % nb], wait=(i == w_main + args.steps - 1), prefetch=nxt(i)), args.steps, w_main)
    launches = (_lib.lib().kge_launch_count() - launches0) // (args.steps + max(args.warmup, 3))
    value = scored_per_gpu * world / (ms_step * 1e-3)
    # the same K-step region four more times: the spread of a 50-60 ms measurement
    regions = [ms_step] + [timed(lambda i: stepper.step(*devb[i % nb], wait=(i == args.steps - 1), prefetch=nxt(i)), args.steps, 0)
                           for _ in range(4)]
    clocks = sampler.stop() if rank == 0 else None
    spread = {"regions": len(regions), "steps_each": args.steps, "ms_per_step_regions": regions,
              "host_queue_ms_per_step": host_ms[:len(regions)], "ms_per_step_median": statistics.median(regions),
              "ms_per_step_min": min(regions), "ms_per_step_max": max(regions),
              "note": "`value` and `ms_per_step` are the first region (W warm-up steps, then exactly K timed steps)"}

    ms_fwd = timed(lambda i: stepper.step(*devb[i % nb], backward=False, prefetch=nxt(i)), max(3, args.steps // 2), 2)

    # ---- e2e: host ids in, losses out, every step --------------------------------------------------------------
    sink = []

    uploaded = {}

    def upload(i):          # pinned host ids -> device, once per step, inside the timed region
        if i not in uploaded:
            uploaded[i] = tuple(x.to(dev, non_blocking=True) for x in host[i % nb])
        return uploaded[i]

    # every step's losses travel to pinned host memory right behind the step; the host consumes them one step later, so it
    # queues step i + 1 while step i computes instead of draining the device once per step
    loss_host = torch.empty((2, len(models)), dtype=torch.float32, pin_memory=True)
    loss_ev = [torch.cuda.Event(), torch.cuda.Event()]
    pending = []

    def consume():
        while pending:
            k = pending.pop(0)
            loss_ev[k].synchronize()
            sink.append(float(loss_host[k].sum()))

    def e2e_step(i):
        b = upload(i)
        ahead = None if args.no_prefetch else upload(i + 1)        # the next step's ids travel while this step computes
        out = stepper.step(*b, wait=(i == 2 + args.steps - 1), prefetch=ahead)
        consume()                                                  # the previous step's losses, long since on the host
        k = i & 1
        loss_host[k].copy_(torch.cat([out.loss[m] for m in models]), non_blocking=True)     # device -> host read of the step's result
        loss_ev[k].record()
        pending.append(k)
        uploaded.pop(i, None)

    ms_e2e = timed(e2e_step, args.steps, 2, after=consume)
    e2e = {"value": scored_per_gpu * world / (ms_e2e * 1e-3), "unit": "triples/s", "h2d_bytes_per_step": h2d_bytes,
           "d2h_bytes_per_step": 4 * len(models), "ms_per_step": ms_e2e,
           "api": "cuke_b200.pipeline.KgeStep.step (pinned host ids -> device every step; every step's losses copied to pinned host "
                  "memory behind the step and consumed by the host one step later, the last one inside the timed region)"}

    # ---- parity, outside the timed regions -------------------------------------------------------------------------
    parity = None
    try:
        if world == 1:
            parity = parity_single_gpu(cfg, models, stepper, ent_local, rel, devb, dev)
        else:
            parity = sharded_selfcheck(rank, world, group, precision=args.precision, n_chunks=2 * micro, micro=micro,
                                       peer_staging=not args.no_peer_staging)
            if rank == 0:
                parity["against"] = "the same step on one GPU with the whole table (GPU against GPU)"
    except Exception as e:          # reported, never hidden
        parity = {"ok": False, "error": f"{type(e).__name__}: {e}"}

    # ---- roofline of the dominant kernel, timed live (no collectives here: rank 0 only) ----------------------------
    hbm_gbs, bf16_peak, peak_kind = peaks()
    roof = None
    if rank == 0:
        import ctypes as C
        h, r, t, neg = devb[0]
        insp = scoring.inspect(scoring.entity_id_list(h, t, neg), cfg.n_ent)
        U = insp.count()
        # any rows do for timing when the table is sharded: the kernels only see the compact staging buffer
        staged = scoring.gather_rows(ent_local, insp.uniq, n_dev=insp.n_unique) if world == 1 else \
            torch.randn((insp.n, d), device=dev) * (1.0 / np.sqrt(d))
        B = h.numel()
        sh, st, sneg = insp.inverse[:B], insp.inverse[B:2 * B], insp.inverse[2 * B:].view(neg.shape)
        r32 = r.to(torch.int32)
        pairs = (B // cfg.chunk) * cfg.chunk * cfg.n_neg
        U_r = int(torch.unique(r).numel())
        n_ids = 3 * B + neg.numel()
        # compulsory HBM traffic of the WHOLE step: every distinct row once (the staging copy serves both scorers), ids
        # once, one gradient row per distinct entity / relation row and scorer; the score matrix and its gradient are
        # consumed inside the tile kernel (fused loss), so they contribute nothing.  Forward rows are read again by the
        # backward only from the compact staging buffer, counted once more.
        fused = args.precision != "fp32"
        S1 = synth.scored_triples(cfg)
        bytes_fwd = U * d * 4 + len(models) * U_r * d * 4 + 8 * n_ids + (0 if fused else len(models) * 4 * S1)
        bytes_bwd = len(models) * (U * d * 4 + U_r * d * 4) + U * d * 4 + (0 if fused else len(models) * 4 * S1)
        step_bytes = bytes_fwd + bytes_bwd
        hbm_step = {"bound": "hbm", "scope": "whole step, compulsory bytes", "bytes_alg": step_bytes,
                    "achieved": step_bytes / (ms_step * 1e-3) / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                    "frac": step_bytes / (ms_step * 1e-3) / 1e9 / hbm_gbs, "peak_source": f"MEASURED_PEAKS.json ({peak_kind})",
                    "distinct_entity_rows": U, "distinct_relation_rows": U_r,
                    "note": "c5 with chunk-shared negatives is bound by the contraction, not by HBM: this fraction is small by construction"}
        L = _lib.lib()
        if args.precision != "fp32":
            # the six contractions of a step (forward S with the loss epilogue, backward GA and GX, for both scorers) are
            # launches of ONE kernel; the same calls as KgeStep.step makes
            def fwd_bwd():
                for m in models:
                    sc = scoring.Scorer(m, staged, rel[m], None, cfg.neg_mode, cfg.n_neg_head, cfg.chunk, args.precision)
                    if sc.supports_fused_step(sneg.shape[-1]):
                        sc.loss_backward(sh, r32, st, sneg)
                    else:
                        pos, negs, _ = sc.forward(sh, r32, st, sneg)
                        loss, dpos, dneg = scoring.logistic_loss(pos, negs)
                        sc.backward(sh, r32, st, sneg, pos, negs, dpos, dneg)
            for _ in range(2):
                fwd_bwd()
            torch.cuda.synchronize()
            L.kge_profile_gemm(1)
            reps = 5
            for _ in range(reps):
                fwd_bwd()
            ms, n, fl = C.c_double(0), C.c_int64(0), C.c_double(0)
            _lib.check(L.kge_profile_gemm_read(C.byref(ms), C.byref(n), C.byref(fl)))
            L.kge_profile_gemm(0)
            t_k = ms.value * 1e-3 / max(n.value, 1)
            flops = fl.value / max(n.value, 1)
            ach = flops / t_k / 1e12
            per_step = n.value // reps
            traffic, traffic_note = None, "no ncu summary found under profiles/"
            pt = profile_traffic()
            if pt is not None:
                scale = (B // cfg.chunk) / 32.0
                traffic = pt[0] * scale
                traffic_note = (f"dram__bytes_read.sum + dram__bytes_write.sum per launch, mean of the {pt[1]} launches of one step captured by "
                                f"ncu at 32 chunks ({pt[2]}), x {scale:g} for this run's {B // cfg.chunk} chunks (traffic grows with the chunk count)")
            split = "two-term bf16 split, three kind::f16 MMAs per product" if args.precision == "tensor" else "3xTF32"
            pipe_x = 3 if args.precision == "tensor" else 6
            roof = {"kernel": f"umma_pair_kernel (tcgen05 cta_group::2, {split}; average over the step's contraction launches: "
                              "per scorer the forward product with the fused loss epilogue and two backward products)",
                    "bound": "tensor", "achieved": ach, "peak": bf16_peak, "unit": "TFLOP/s", "frac": ach / bf16_peak,
                    "peak_source": f"MEASURED_PEAKS.json bf16 dense, burst ({peak_kind})",
                    "note": "achieved counts useful fp32 flops (2MNK); each is 3 MMAs (bf16 split: at the bf16 rate; tf32 split: "
                            f"at half of it), so the tensor pipe does {pipe_x}x this many bf16-equivalent flops",
                    "tensor_pipe_equiv_frac": pipe_x * ach / bf16_peak, "launches_timed": n.value, "launches_per_step": per_step,
                    "ms": t_k * 1e3, "share_of_step": per_step * t_k * 1e3 / ms_step,
                    "traffic": traffic, "traffic_note": traffic_note,
                    "traffic_per_step": None if traffic is None else traffic * per_step,
                    "traffic_over_step_bytes_alg": None if traffic is None else traffic * per_step / step_bytes,
                    "hbm": hbm_step}
        else:
            sc = scoring.Scorer(models[0], staged, rel[models[0]], None, cfg.neg_mode, cfg.n_neg_head, cfg.chunk)
            for _ in range(3):
                sc.forward(sh, r32, st, sneg)
            torch.cuda.synchronize()
            reps = 10
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                sc.forward(sh, r32, st, sneg)
            e1.record()
            torch.cuda.synchronize()
            t_k = e0.elapsed_time(e1) * 1e-3 / reps
            flop_per = 3 if models[0] == "TransE" else 2
            flops = flop_per * d * (pairs + B)
            fma_peak = scoring.fma_peak_tflops(dev)
            roof = {"kernel": f"pair_fwd_kernel<{models[0]}> (+ positives kernel, <2% of the time)", "bound": "fp32_fma",
                    "achieved": flops / t_k / 1e12, "peak": fma_peak, "unit": "TFLOP/s", "frac": flops / t_k / 1e12 / fma_peak,
                    "peak_source": "kge_probe_fma microbenchmark on this GPU (2 flop per FMA)",
                    "pipe_slot_frac": (2 * d * (pairs + B) if models[0] == "TransE" else d * (pairs + B)) / t_k / (fma_peak * 1e12 / 2),
                    "traffic": None, "ms": t_k * 1e3, "hbm": hbm_step}
        del staged

    cpu = None
    side = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            res = cpu_reference_rate(cfg, models, seconds=args.cpu_seconds, steps=2, warmup=1)
            cpu = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as e:          # the baseline is reported, never required
            cpu = {"value": None, "unit": "triples/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    if rank == 0 and world == 1 and not args.no_side:
        # the parity configurations c1-c4, after the timed c5 regions: one record per scorer (cold- and warm-L2 figures,
        # HBM view of the roofline, the reference's OpenMP C++ on a bounded sample)
        del stepper, devb
        torch.cuda.empty_cache()
        side = []
        for cname in ("c1", "c2", "c3", "c4", "c4_bf16"):
            try:
                side += side_measure(cname, 5, 3, args.precision, 0.0 if args.no_cpu_baseline else min(args.cpu_seconds, 3.0))
            except Exception as e:
                side.append({"config": {"workload": cname}, "error": f"{type(e).__name__}: {e}"})

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "triples/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": dict(workload_config(cfg, models, world), micro_batches=micro,
                                                                                         staging=staging_note(stepper, world),
                                                                                         arithmetic=(
                    "fp32 storage and accumulation; contractions on the tensor cores over a two-term bf16 split of each fp32 "
                    "operand (three MMAs per product, error-compensated; see the parity block for the measured error)"
                    if args.precision == "tensor" else
                    "fp32 storage and accumulation; contractions as 3xTF32 on the tensor cores (error-compensated)"
                    if args.precision == "tensor_tf32" else "fp32 CUDA cores")),
                "spread": spread,
                "value_fwd_only": scored_per_gpu * world / (ms_fwd * 1e-3), "ms_per_step_fwd_only": ms_fwd,
                "e2e": e2e, "gpu_launches": int(launches) * args.steps, "gpu_launches_per_step": int(launches),
                "clocks": clocks, "roofline": roof, "cpu_baseline": cpu, "parity": parity, "side": side}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier(group=group)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
