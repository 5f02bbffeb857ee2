"""Host-side logic of the training step that needs no GPU: how a batch is cut into micro-batches."""
from types import SimpleNamespace

import pytest
import torch

from cuke_b200.pipeline import KgeStep


@pytest.mark.parametrize("micro,rows,per", [(1, 5, 64), (2, 4, 256), (3, 5, 64), (4, 3, 16), (2, 7, 1)])
def test_micro_batches_are_runs_of_whole_chunks(micro, rows, per):
    B = rows * per
    h, r, t = torch.arange(B), torch.arange(B) + 1000, torch.arange(B) + 2000
    neg = torch.arange(rows * 6).view(rows, 6)
    parts = KgeStep._split(SimpleNamespace(micro=micro), h, r, t, neg)
    assert len(parts) == min(micro, rows)
    assert parts[0][0] == 0
    seen_rows, seen = 0, 0
    for first, hh, rr, tt, nn, ids in parts:
        assert first == seen and first % per == 0                 # consecutive, starting on a chunk boundary
        assert hh.numel() == rr.numel() == tt.numel() == nn.shape[0] * per and nn.shape[0] >= 1
        assert torch.equal(hh, h[first:first + hh.numel()]) and torch.equal(rr, r[first:first + hh.numel()])
        assert torch.equal(tt, t[first:first + hh.numel()]) and torch.equal(nn, neg[seen_rows:seen_rows + nn.shape[0]])
        seen += hh.numel()
        seen_rows += nn.shape[0]
    assert seen == B and seen_rows == rows
    if micro == 1:
        assert parts[0][1] is h and parts[0][4] is neg            # the whole batch, the caller's own tensors
