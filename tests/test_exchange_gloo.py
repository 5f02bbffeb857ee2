"""The row-partition exchange protocol (ids out, rows back, gradients home, owner-side sum) on CPU ranks over
gloo, world sizes 2 and 3.  The kernels are replaced by a numpy stand-in with the same signatures; what is
checked is the multi-rank bookkeeping of cuke_b200.pipeline.RowExchange."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys
    sys.path.insert(0, %r)
    import numpy as np, torch, torch.distributed as dist
    from oracle import oracle
    from cuke_b200.pipeline import RowExchange
    from cuke_b200.scoring import Inspection

    class CpuOps:      # numpy stand-ins for the CUDA kernels, same signatures as cuke_b200.scoring
        @staticmethod
        def inspect(ids, id_space):
            u, inv, perm, seg = oracle.inspect(ids.numpy())
            n = ids.numel()
            uniq = torch.zeros(max(n, 1), dtype=torch.int64); uniq[:len(u)] = torch.from_numpy(u)
            return Inspection(uniq, torch.from_numpy(inv), torch.from_numpy(perm), torch.from_numpy(seg),
                              torch.tensor([len(u)], dtype=torch.int64), n)
        @staticmethod
        def owner_counts(insp, rpr, world):
            U = int(insp.n_unique)
            own = torch.clamp(insp.uniq[:U] // rpr, max=world - 1)
            return torch.bincount(own, minlength=world).to(torch.int64)
        @staticmethod
        def gather_rows(table, ids, n_dev=None, first_row=0, out=None):
            return table[ids - first_row].contiguous()
        @staticmethod
        def segment_reduce(rows, insp, out=None, n_out=None):
            res = torch.zeros((insp.n, rows.shape[1]), dtype=torch.float32)
            res.index_add_(0, insp.inverse.long(), rows)
            return res

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    n_ent, d, n = 103, 6, 400
    g = np.random.Generator(np.random.PCG64(5))
    table = torch.from_numpy(g.standard_normal((n_ent, d)).astype(np.float32))      # same on every rank
    rpr = (n_ent + world - 1) // world
    local = table[rank * rpr: min(n_ent, (rank + 1) * rpr)].contiguous()
    gi = np.random.Generator(np.random.PCG64(100 + rank))
    w = np.arange(1, n_ent + 1, dtype=np.float64) ** -1.1
    ids = torch.from_numpy(gi.choice(n_ent, size=n, p=w / w.sum()))
    if rank == world - 1:
        ids = ids[ids >= rpr]            # one rank asks nothing of rank 0's shard: zero-length splits
    insp = CpuOps.inspect(ids, n_ent)
    U = int(insp.n_unique)
    ex = RowExchange(local, n_ent, rank, world, None, ops=CpuOps)
    staged = ex.stage(insp)
    assert torch.equal(staged[:U], table[insp.uniq[:U]]), "staged rows differ from the global table"
    # gradient rows home: every rank contributes grad[u] = (rank + 1) * one-hot-ish row of its distinct ids
    grad = torch.zeros((max(U, 1), d)); grad[:U] = (rank + 1) * (insp.uniq[:U, None].float() + torch.arange(d)[None, :])
    oid, on, orows = ex.return_grads(grad)
    # reference: gather everyone's (ids, grads) and sum per owned id
    all_ids = [None] * world; all_g = [None] * world
    dist.all_gather_object(all_ids, insp.uniq[:U].tolist()); dist.all_gather_object(all_g, grad[:U].tolist())
    dense = np.zeros((n_ent, d))
    for ii, gg in zip(all_ids, all_g):
        if ii:
            dense[np.array(ii)] += np.array(gg)
    lo, hi = rank * rpr, min(n_ent, (rank + 1) * rpr)
    touched = sorted({i for ii in all_ids for i in ii if lo <= i < hi})
    k = int(on)
    assert oid[:k].tolist() == touched, "owner-side distinct ids"
    assert np.allclose(orows[:k].numpy(), dense[touched], rtol=1e-6), "owner-side gradient sums"
    # The peer-memory form of the return (kge_pull_reduce): the owner reads every rank's gradient rows in place.  Its index
    # arithmetic - where my rows start in rank r's buffer (sent along with the counts), where rank r's ids start in the
    # concatenated request list - is restated here over all-gathered buffers: position pos of rank r in the request list
    # is row src_off[r] + pos - src_start[r] of r's buffer.
    S = sum(ex.serve)
    if S:
        src_off, src_start = ex.wanted[:, 1].tolist(), ex.src_start.tolist()
        oi = ex.owner_insp
        pulled = np.zeros((k, d))
        for u in range(k):
            for p in range(int(oi.seg[u]), int(oi.seg[u + 1]) if u + 1 < k else S):
                pos = int(oi.perm[p])
                r = max(rr for rr in range(world) if src_start[rr] <= pos)
                assert pos < src_start[r + 1]
                pulled[u] += np.array(all_g[r][src_off[r] + pos - src_start[r]])
        assert np.allclose(pulled, orows[:k].numpy(), rtol=1e-6), "peer-pull index arithmetic"
        assert ex.wanted[:, 0].tolist() == ex.serve
    dist.barrier()
    if rank == 0:
        print("EXCHANGE_OK", world)
    dist.destroy_process_group()
''') % ROOT


@pytest.mark.parametrize("world", [2, 3, 4])
def test_row_exchange_over_gloo(world, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = 29600 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert f"EXCHANGE_OK {world}" in r.stdout
