"""Import-only stand-in for DGL.  The reference imports ``dgl`` at module load (gt_sp/utils.py:9) and tries it
first for CPU random walks inside a try/except that falls through to ``torch_cluster`` on any error
(gt_sp/utils.py:1396-1442); every entry point here raises so that this fall-through is taken."""


class _Unavailable(RuntimeError):
    pass


def _raise(*a, **k):
    raise _Unavailable("DGL is not installed; the baseline harness provides an import-only stand-in")


seed = from_csr = graph = metis_partition_assignment = to_bidirected = _raise


class sampling:  # noqa: N801
    random_walk = staticmethod(_raise)
    sample_neighbors = staticmethod(_raise)
