"""Worker of tests/test_gpu_pipeline.py::test_sharded_step_equals_single_gpu (launched under torchrun, one rank per GPU).
Every rank scores its own batch against a row-partitioned table; rank 0 then recomputes all ranks' batches on one
GPU with the whole table and compares (cuke_b200.pipeline.sharded_selfcheck): losses per rank bit-equal, the summed
entity / relation gradients to 1e-5.  Run on the tensor-core path (fused step; CTA-pair and one-CTA tile shapes) and
once on the fp32 CUDA-core path, then with the sharded step cut into micro-batches and with the rows staged by peer loads instead of an all-to-all."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from cuke_b200.pipeline import sharded_selfcheck, sharded_traincheck


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    cases = [dict(precision="tensor", d=64, chunk=256, n_neg=160, n_chunks=2),       # CTA-pair tiles
             dict(precision="tensor", d=40, chunk=64, n_neg=96, n_chunks=4),         # one-CTA tiles
             dict(precision="fp32", d=64, chunk=64, n_neg=96, n_chunks=4),
             dict(precision="tensor", d=64, chunk=256, n_neg=160, n_chunks=4, micro=2),   # two micro-batches per step
             dict(precision="tensor", d=40, chunk=64, n_neg=96, n_chunks=5, micro=3),     # uneven micro-batches
             dict(precision="tensor", d=64, chunk=256, n_neg=160, n_chunks=2, peer_staging=True),   # rows read in place over NVLink
             dict(precision="fp32", d=36, chunk=64, n_neg=96, n_chunks=4, micro=2, peer_staging=True)]
    ok = True
    for c in cases:
        res = sharded_selfcheck(rank, world, dist.group.WORLD, **c)
        if rank == 0:
            print("selfcheck", c, res, flush=True)
            ok = ok and res["ok"]
    # several steps with the optimizer inside the step: the order of peer reads, updates and barriers across steps
    for c in (dict(peer_staging=True), dict(peer_staging=False), dict(peer_staging=True, micro=2, n_chunks=4)):
        res = sharded_traincheck(rank, world, dist.group.WORLD, **c)
        if rank == 0:
            print("traincheck", c, res, flush=True)
            ok = ok and res["ok"]
    if rank == 0:
        assert ok, "sharded step differs from the single-GPU step"
        print("SHARDED_OK", world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
