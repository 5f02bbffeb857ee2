"""kge_segment_reduce_static: the segmented reduction whose scratch is a fixed array inside the library, for hosts
that cannot allocate device memory once they are running.  Collected last on purpose (file name), so a run that
stops at the first failure has already run every other test.

Checked through the C ABI against kge_segment_reduce (caller-provided workspace) on two calls in a row with
different inputs: the second call finds the first call's leftovers in the shared scratch and must not be
affected by them.  Same kernels and summation order, so the tolerance of the segmented-reduction tests (1e-5
relative) is met with room to spare.  A second test takes the numpy inspector model and a float64 scatter-add
as the reference, a third the argument checks (no output buffer, too large a problem)."""
import numpy as np
import pytest
import torch

from oracle import oracle
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


def test_static_scratch_matches_float64_scatter_add():
    """out[u] = sum of the rows whose id is uniq[u], against np.add.at in float64 over the numpy inspector's uniq order;
    rows past the distinct count are zero-filled up to n_out."""
    from cuke_b200 import scoring
    seed, n, space, d = 3, 5000, 300, 96
    ids, rows = _case(seed, n, space, d)
    uniq, inverse, perm, seg = oracle.inspect(ids.cpu().numpy())
    ref = np.zeros((len(uniq), d), dtype=np.float64)
    np.add.at(ref, inverse, rows.cpu().numpy().astype(np.float64))
    insp = scoring.inspect(ids, space)
    assert int(insp.n_unique.item()) == len(uniq)
    assert np.array_equal(insp.uniq[:len(uniq)].cpu().numpy(), uniq)
    n_out = len(uniq) + 7
    out = torch.full((n_out, d), float("nan"), dtype=torch.float32, device="cuda")
    scoring.segment_reduce_static(rows, insp, out)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert rel_err(got[:len(uniq)], ref) < 1e-5
    assert not got[len(uniq):].any()


def test_static_scratch_rejects_missing_output():
    """rows to reduce but no output buffer: KGE_E_NULL before anything is launched, also when n_out is 0."""
    from cuke_b200 import _lib, scoring
    ids, rows = _case(4, 256, 16, 32)
    insp = scoring.inspect(ids, 16)
    for n_out in (0, 16):
        rc = _lib.lib().kge_segment_reduce_static(rows.data_ptr(), 32, 256, insp.perm.data_ptr(), insp.seg.data_ptr(),
                                                  insp.n_unique.data_ptr(), None, n_out, None)
        assert rc == -1, rc                # KGE_E_NULL
    torch.cuda.synchronize()
    assert scoring.device_flags() == 0


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
