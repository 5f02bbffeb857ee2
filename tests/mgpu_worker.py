"""Worker of tests/test_gpu_pipeline.py::test_sharded_step_equals_single_gpu (launched under torchrun, one rank per GPU).
Every rank scores its own batch against a row-partitioned table; rank 0 then recomputes all ranks' batches on one
GPU with the whole table and compares: losses per rank, and the summed entity / relation gradients."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np
import torch
import torch.distributed as dist

from cuke_b200.pipeline import KgeStep


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    ne, d, B, chunk, nn, nr = 5003, 64, 256, 64, 96, 13
    g = np.random.Generator(np.random.PCG64(77))
    E = (g.standard_normal((ne, d)) / np.sqrt(d)).astype(np.float32)
    models = ["TransE", "DistMult"]
    rel = {m: torch.from_numpy((g.standard_normal((nr, d)) / np.sqrt(d)).astype(np.float32)).to(dev) for m in models}
    w = np.arange(1, ne + 1, dtype=np.float64) ** -1.1

    def batch(rk):
        gi = np.random.Generator(np.random.PCG64(1000 + rk))
        ids = lambda size: torch.from_numpy(gi.choice(ne, size=size, p=w / w.sum()).astype(np.int64)).to(dev)
        return ids(B), torch.from_numpy(gi.integers(0, nr, B)).to(dev), ids(B), ids((B // chunk, nn))

    rpr = (ne + world - 1) // world
    local = torch.from_numpy(E[rank * rpr: min(ne, (rank + 1) * rpr)]).to(dev).contiguous()
    step = KgeStep(models, local, rel, ne, "chunk_shared", 0, chunk, rank, world, dist.group.WORLD)
    out = step.step(*batch(rank))
    k = int(out.n_ent_rows.item())
    mine = {m: (out.ent_ids[:k].cpu(), out.ent_grad[m][:k].cpu(), out.rel_grad[m].cpu(), out.loss[m].cpu()) for m in models}
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        full = KgeStep(models, torch.from_numpy(E).to(dev), rel, ne, "chunk_shared", 0, chunk)
        dense = {m: torch.zeros((ne, d), dtype=torch.float64) for m in models}
        drel = {m: torch.zeros((nr, d), dtype=torch.float64) for m in models}
        for rk in range(world):
            o = full.step(*batch(rk))
            u = int(o.n_ent_rows.item())
            for m in models:
                dense[m][o.ent_ids[:u].cpu()] += o.ent_grad[m][:u].double().cpu()
                drel[m] += o.rel_grad[m].double().cpu()
                assert torch.equal(o.loss[m].cpu(), gathered[rk][m][3]), "loss differs between sharded and single-GPU run"
        for m in models:
            got = torch.zeros((ne, d), dtype=torch.float64)
            for rk in range(world):
                ids, rows, _, _ = gathered[rk][m]
                assert torch.all((ids >= rk * rpr) & (ids < (rk + 1) * rpr)), "a rank returned gradients of rows it does not own"
                got[ids] += rows.double()
            err = (got - dense[m]).abs().max() / dense[m].abs().max()
            rerr = (gathered[0][m][2].double() - drel[m]).abs().max() / drel[m].abs().max()
            assert err < 1e-5 and rerr < 1e-5, (m, float(err), float(rerr))
        print("SHARDED_OK", world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
