"""The general (any row length) graph builder called with a topology that lives on the GPU: it works on the CPU copy
and returns the graph on the topology's device, identical to the CPU call."""
import pytest
import torch

from budgetformer_b200.graph.builder import build_attn_graph
from tests.helpers import random_topology

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kwargs,budgets", [({}, (None, None)), ({"fanout": [3, 2]}, (3, 4)), ({}, (40, 40))])
def test_general_builder_from_a_gpu_topology(kwargs, budgets):
    topo, _ = random_topology(500, 4000, hub_out=40, seed=5)
    want = build_attn_graph(topo, budgets[0], budgets[1], 2, 3, 17, **kwargs)
    got = build_attn_graph(topo.to("cuda"), budgets[0], budgets[1], 2, 3, 17, **kwargs)
    assert got.rowptr.is_cuda and got.col.is_cuda
    assert torch.equal(got.rowptr.cpu(), want.rowptr) and torch.equal(got.col.cpu(), want.col)
    assert (got.n_real, got.n_rw) == (want.n_real, want.n_rw)
