"""Selection encoding of the decomposed graph primitives (host logic, CPU tensors)."""
import pytest
import torch

from ateniaengine_b200 import graph_ops as go


def test_round_trip_and_layout():
    idx = torch.tensor([[1, 3], [0, 2]], dtype=torch.int32)
    w = torch.tensor([[0.25, 0.75], [0.5, 0.5]], dtype=torch.float32)
    sel = go.encode_selection(idx, w)
    assert sel.tolist() == [[1.0, 0.25, 3.0, 0.75], [0.0, 0.5, 2.0, 0.5]]  # [idx0, w0, idx1, w1]
    i2, w2 = go.decode_selection(sel)
    assert torch.equal(i2, idx) and torch.equal(w2, w)
    assert go.expert_weight_in_selection(sel[0], 3) == 0.75
    assert go.expert_weight_in_selection(sel[0], 2) is None


def test_validation_follows_the_reference():
    with pytest.raises(ValueError):
        go.decode_selection(torch.zeros((1, 3)))
    with pytest.raises(ValueError):
        go.decode_selection(torch.tensor([[-1.0, 0.5]]))
    with pytest.raises(ValueError):
        go.decode_selection(torch.tensor([[float("nan"), 0.5]]))
