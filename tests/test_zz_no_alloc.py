"""kge_segment_reduce_static: the segmented reduction whose scratch is a fixed array inside the library, for hosts
that cannot allocate device memory once they are running.  Collected last on purpose (file name), so a run that
stops at the first failure has already run every other test.

Checked through the C ABI against kge_segment_reduce (caller-provided workspace) on two calls in a row with
different inputs: the second call finds the first call's leftovers in the shared scratch and must not be
affected by them.  Same kernels and summation order, so the tolerance of the segmented-reduction tests (1e-5
relative) is met with room to spare."""
import numpy as np
import pytest
import torch

from tests.kge_testlib import rel_err, to_dev

pytestmark = pytest.mark.gpu


def _case(seed, n, space, d):
    g = np.random.Generator(np.random.PCG64(seed))
    w = np.arange(1, space + 1, dtype=np.float64) ** -1.1
    ids = g.choice(space, size=n, p=w / w.sum())
    rows = g.standard_normal((n, d)).astype(np.float32)
    return to_dev(ids), to_dev(rows)


def test_static_scratch_matches_workspace_version_twice():
    from cuke_b200 import scoring
    for seed, n, space, d in [(1, 6000, 500, 200), (2, 4500, 40, 64)]:      # long, window-crossing segments
        ids, rows = _case(seed, n, space, d)
        insp = scoring.inspect(ids, space)
        ref = scoring.segment_reduce(rows, insp)
        out = torch.full_like(ref, float("nan"))
        scoring.segment_reduce_static(rows, insp, out)
        torch.cuda.synchronize()
        assert rel_err(out.cpu().numpy(), ref.cpu().numpy()) < 1e-5
        assert torch.equal(out, ref)


def test_static_scratch_rejects_oversize():
    from cuke_b200 import scoring
    from cuke_b200._lib import KgeError
    n, d = 40000, 1024                     # ceil(n/32) * dim = 1,280,000 > 1,048,576
    ids = torch.zeros(n, dtype=torch.int64, device="cuda")
    insp = scoring.inspect(ids, 4)
    rows = torch.zeros((n, d), dtype=torch.float32, device="cuda")
    out = torch.zeros((8, d), dtype=torch.float32, device="cuda")
    with pytest.raises(KgeError) as e:
        scoring.segment_reduce_static(rows, insp, out)
    assert e.value.code == -6 and "built-in scratch" in str(e.value)
