"""CPU oracle: plain float32 PyTorch / NumPy restatements of the reference's mathematics, written against the
reference's own data layout (int64 COO ``edge_index`` with row 0 = key node, row 1 = query node) and independent of
the framework's containers, kernels and model classes.  Tests compare the CUDA kernels and the fused layer path against
these functions; nothing here is on a training path.

``attention``    edge-list attention of the four model families (models/*_dist_node_level.py sparse paths)
``layers``       one encoder layer of each model from a plain dict of weights
``graph``        per-query hash sampling, random-walk edge emission, merge, virtual-node index maps
``reducer``      the reducer's mean of per-rank means and the per-rank loss rule
``schedules``    the two learning-rate schedules in closed form
"""
from . import attention, graph, layers, reducer, schedules  # noqa: F401
